// moc_decode_global_static: the global-MoC decode FFN for callers that cannot provide scratch memory.
//
// Some hosts of this library may not allocate device memory at the point where they need an FFN
// evaluated: code running under a memory budget that was handed out completely at start-up, a
// serving loop whose allocator is frozen once the weights and caches are placed, or a plugin that is
// only given input and output buffers by its runtime. moc_decode_global needs up to about ten megabytes
// of scratch (gate scores, histograms, one partial output vector per SM and batch row) from such a
// caller; this variant keeps that scratch inside the library instead, in a fixed array in device
// memory that every GPU loading the library holds until the process exits.
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/moc_b200.h"
#include "common.cuh"
#include "internal.h"

namespace {

constexpr int64_t kStaticMaxBatch = 8;
constexpr int64_t kStaticMaxD = 4096;
constexpr int64_t kStaticMaxDffn = 8192;
constexpr size_t kStaticScratchBytes = 12u << 20;   // 12 MiB per GPU

// The scratch itself. In host code this name is only a stand-in for the symbol, not a device address;
// the address is obtained once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

// First call on a device: look up the device address of the scratch array with that device current.
int scratch_for_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return moc::check_last("cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) {
    moc::set_error("moc_decode_global_static: device ordinal %d out of range", dev);
    return moc::kErrUnsupported;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      moc::set_error("moc_decode_global_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return moc::kErrCuda;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return moc::kOk;
}

}  // namespace

extern "C" {

int64_t moc_decode_static_max_batch(void) { return kStaticMaxBatch; }
int64_t moc_decode_static_max_d(void) { return kStaticMaxD; }
int64_t moc_decode_static_max_d_ffn(void) { return kStaticMaxDffn; }

int moc_decode_global_static(int64_t batch, int64_t d, int64_t d_ffn, int64_t k, const void* x, const void* w_gate,
                             const void* w_up, const void* w_down_t, void* y, void* stream) {
  if (!x || !w_gate || !w_up || !w_down_t || !y) {
    moc::set_error("moc_decode_global_static: null pointer");
    return moc::kErrInvalidArg;
  }
  if (batch < 0 || batch > kStaticMaxBatch || d <= 0 || d > kStaticMaxD || d_ffn <= 0 || d_ffn > kStaticMaxDffn ||
      moc::decode_workspace_bytes(batch, d, d_ffn) > static_cast<int64_t>(kStaticScratchBytes)) {
    moc::set_error("moc_decode_global_static: batch=%lld d=%lld d_ffn=%lld exceed the built-in scratch "
                   "(batch <= %lld, d <= %lld, d_ffn <= %lld); use moc_decode_global with a caller workspace",
                   (long long)batch, (long long)d, (long long)d_ffn, (long long)kStaticMaxBatch,
                   (long long)kStaticMaxD, (long long)kStaticMaxDffn);
    return moc::kErrUnsupported;
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != moc::kOk) return rc;
  // Every buffer carved from the scratch is fully rewritten before it is read inside one call, so nothing
  // has to be cleared between calls.
  return moc::decode_global(batch, d, d_ffn, k, 0, x, nullptr, w_gate, w_up, w_down_t, y, scratch,
                            static_cast<int64_t>(kStaticScratchBytes), reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
