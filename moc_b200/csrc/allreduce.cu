// In-place sum (or mean) of the weight-gradient bucket over the ranks of one node, over NVLink: every rank holds
// the bucket in a symmetric allocation that its peers have mapped, and one small kernel per rank reduces the
// rank's own 1/W slice and writes the result to every rank:
//
//   multicast form  - the slice is read with multimem.ld_reduce (the NVSwitch adds the W replicas in fp32 and
//                     returns one vector) and written back with multimem.st (the switch stores it to all W
//                     replicas): each byte crosses this GPU's links once per direction and the SMs only move data;
//   peer form       - plain 16-byte loads from each peer's buffer, summed in fp32 in rank order, plain stores to
//                     each peer (for allocations without a multicast mapping).
//
// The kernel is meant to run with few CTAs beside the dX GEMM of the backward pass (which leaves that many SMs
// free), so the reduction needs no separate phase of the step. Ranks meet twice through flag words that live in
// a second symmetric allocation: before the first read (every rank's gradients are final) and after the last
// write (every slice has arrived everywhere). The flags carry the number of the call, which only grows, so they
// are never reset. Every wait is bounded: on a time-out the kernel sets its status word, releases its own CTAs
// and returns, leaving the bucket's contents unspecified.
//
// No multicast LOAD of the TMA kind is used anywhere: multimem.* are plain load/store/reduce instructions on a
// multicast address.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moc_b200.h"
#include "common.cuh"
#include "internal.h"

namespace moc {

constexpr int kArMaxWorld = 8;
constexpr int kArThreads = 512;
// flag words (uint32) of one rank's flag allocation
constexpr int kArEntry = 0;      // [W] call number published by rank r before it reads
constexpr int kArExit = 32;      // [W] call number published by rank r after its last write
constexpr int kArGo = 64;        // local: CTA 0 -> the other CTAs of this rank
constexpr int kArDone = 65;      // local: CTAs of this rank that have finished their share
constexpr int kArStatus = 66;    // local: nonzero after a time-out
constexpr uint32_t kArAbortBit = 0x80000000u;   // in the go word: this call gave up (call numbers stay below 2^31)

struct ArArgs {
  void* mc;                           // multicast address of the buffer, or null
  void* peer[kArMaxWorld];            // every rank's buffer as mapped here
  uint32_t* flags[kArMaxWorld];       // every rank's flag words as mapped here
  int64_t vecs;                       // 16-byte vectors in the buffer
  long long wait_cycles;
  uint32_t call;                      // number of this call on this communicator, from 1
  int rank, world;
  float scale;                        // 1 or 1 / world
};

__device__ __forceinline__ void ar_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ar_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ar_st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ar_ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// waits until *p >= want (call numbers only grow); false when the limit ran out
__device__ __forceinline__ bool ar_wait_sys(const uint32_t* p, uint32_t want, long long limit) {
  const long long t0 = clock64();
  while (true) {
    if (ar_ld_acquire_sys(p) >= want) return true;
    if (clock64() - t0 > limit) return false;
    __nanosleep(100);
  }
}

template <typename T> struct ArVec;
template <> struct ArVec<__nv_bfloat16> {
  __device__ __forceinline__ static uint4 mc_load_sum(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  __device__ __forceinline__ static void unpack(const uint4& q, float (&f)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[2 * j] = __uint_as_float(w[j] << 16);
      f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static constexpr int kElems = 8;
};
template <> struct ArVec<float> {
  __device__ __forceinline__ static uint4 mc_load_sum(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  __device__ __forceinline__ static void unpack(const uint4& q, float (&f)[4]) {
    f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static constexpr int kElems = 4;
};

__device__ __forceinline__ void ar_mc_store(void* p, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ar_peer_load(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ar_peer_store(void* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kArThreads) symm_allreduce_kernel(const ArArgs a) {
  __shared__ int ok_s;
  const int tid = threadIdx.x;
  uint32_t* mine = a.flags[a.rank];
  if (tid == 0) ok_s = 1;
  __syncthreads();

  // ---- all ranks' gradients are final ----
  if (blockIdx.x == 0) {
    if (tid < a.world) {
      ar_st_release_sys(a.flags[tid] + kArEntry + a.rank, a.call);
      if (!ar_wait_sys(mine + kArEntry + tid, a.call, a.wait_cycles)) {
        ok_s = 0;
        atomicCAS(reinterpret_cast<unsigned*>(mine + kArStatus), 0u, 0x01000000u | static_cast<unsigned>(tid));
      }
    }
    __syncthreads();
    if (tid == 0) ar_st_release_gpu(mine + kArGo, ok_s ? a.call : (a.call | kArAbortBit));
  } else {
    if (tid == 0) {
      const long long t0 = clock64();
      while (true) {
        const uint32_t v = ar_ld_acquire_gpu(mine + kArGo);
        if ((v & ~kArAbortBit) >= a.call) {
          if (v & kArAbortBit) ok_s = 0;
          break;
        }
        if (clock64() - t0 > 2 * a.wait_cycles) {
          ok_s = 0;
          atomicCAS(reinterpret_cast<unsigned*>(mine + kArStatus), 0u, 0x02000000u);
          break;
        }
        __nanosleep(100);
      }
    }
    __syncthreads();
  }
  const bool ok = ok_s != 0;

  // ---- this rank's slice ----
  if (ok) {
    const int64_t begin = a.vecs * a.rank / a.world, end = a.vecs * (a.rank + 1) / a.world;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kArThreads;
    constexpr int kUnroll = 8;
    if (a.mc) {
      uint8_t* mc = static_cast<uint8_t*>(a.mc);
      for (int64_t i0 = begin + static_cast<int64_t>(blockIdx.x) * kArThreads + tid; i0 < end; i0 += stride * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (i0 + u * stride < end) v[u] = ArVec<T>::mc_load_sum(mc + (i0 + u * stride) * 16);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (i0 + u * stride < end) {
            if (a.scale != 1.0f) {
              float f[ArVec<T>::kElems];
              ArVec<T>::unpack(v[u], f);
#pragma unroll
              for (int e = 0; e < ArVec<T>::kElems; ++e) f[e] *= a.scale;
              v[u] = ArVec<T>::pack(f);
            }
            ar_mc_store(mc + (i0 + u * stride) * 16, v[u]);
          }
        }
      }
    } else {
      for (int64_t i = begin + static_cast<int64_t>(blockIdx.x) * kArThreads + tid; i < end; i += stride) {
        uint4 v[kArMaxWorld];
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r)
          if (r < a.world) v[r] = ar_peer_load(static_cast<const uint8_t*>(a.peer[r]) + i * 16);
        float acc[ArVec<T>::kElems];
#pragma unroll
        for (int e = 0; e < ArVec<T>::kElems; ++e) acc[e] = 0.0f;
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r) {
          if (r < a.world) {
            float f[ArVec<T>::kElems];
            ArVec<T>::unpack(v[r], f);
#pragma unroll
            for (int e = 0; e < ArVec<T>::kElems; ++e) acc[e] += f[e];
          }
        }
#pragma unroll
        for (int e = 0; e < ArVec<T>::kElems; ++e) acc[e] *= a.scale;
        const uint4 out = ArVec<T>::pack(acc);
#pragma unroll
        for (int r = 0; r < kArMaxWorld; ++r)
          if (r < a.world) ar_peer_store(static_cast<uint8_t*>(a.peer[r]) + i * 16, out);
      }
    }
  }

  // ---- every slice has arrived everywhere ----
  __threadfence_system();
  __syncthreads();
  __shared__ int last_s;
  if (tid == 0) {
    const unsigned prev = atomicAdd(reinterpret_cast<unsigned*>(mine + kArDone), 1u);
    last_s = prev == gridDim.x - 1 ? 1 : 0;
  }
  __syncthreads();
  if (last_s) {
    if (tid == 0) mine[kArDone] = 0u;     // ready for the next call
    if (ok && tid < a.world) {
      __threadfence_system();
      ar_st_release_sys(a.flags[tid] + kArExit + a.rank, a.call);
      if (!ar_wait_sys(mine + kArExit + tid, a.call, a.wait_cycles))
        atomicCAS(reinterpret_cast<unsigned*>(mine + kArStatus), 0u, 0x03000000u | static_cast<unsigned>(tid));
    }
  }
}

}  // namespace moc

using namespace moc;

extern "C" {

int moc_symm_allreduce(int dtype, int rank, int world, void* const* peer_buffers, void* multicast_buffer,
                       void* const* peer_flags, int64_t bytes, int average, uint32_t call, int ctas, void* stream_) {
  if (dtype != kBF16 && dtype != kF32) {
    set_error("moc_symm_allreduce: unsupported dtype code %d", dtype);
    return kErrInvalidArg;
  }
  if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world || !peer_buffers || !peer_flags || bytes < 0 ||
      call == 0 || call >= kArAbortBit) {
    set_error("moc_symm_allreduce: bad rank / world (at most %d ranks) / call number or null pointer table", kArMaxWorld);
    return kErrInvalidArg;
  }
  if (bytes % 16 != 0) {
    set_error("moc_symm_allreduce: the buffer size must be a multiple of 16 bytes, got %lld", (long long)bytes);
    return kErrInvalidArg;
  }
  if (ctas < 1 || ctas > 1024) {
    set_error("moc_symm_allreduce: ctas=%d is outside 1..1024", ctas);
    return kErrInvalidArg;
  }
  ArArgs a = {};
  for (int r = 0; r < world; ++r) {
    if (!peer_buffers[r] || !peer_flags[r] || (reinterpret_cast<uintptr_t>(peer_buffers[r]) & 15u) != 0) {
      set_error("moc_symm_allreduce: buffer or flag pointer of rank %d is null or not 16-byte aligned", r);
      return kErrInvalidArg;
    }
    a.peer[r] = peer_buffers[r];
    a.flags[r] = static_cast<uint32_t*>(peer_flags[r]);
  }
  a.mc = multicast_buffer;
  a.vecs = bytes / 16;
  a.wait_cycles = 2000000000LL;   // about one second
  a.call = call;
  a.rank = rank;
  a.world = world;
  a.scale = average ? 1.0f / static_cast<float>(world) : 1.0f;
  if (bytes == 0) return kOk;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype == kBF16)
    symm_allreduce_kernel<__nv_bfloat16><<<ctas, kArThreads, 0, stream>>>(a);
  else
    symm_allreduce_kernel<float><<<ctas, kArThreads, 0, stream>>>(a);
  return check_last("moc_symm_allreduce");
}

int64_t moc_symm_allreduce_flag_bytes(void) { return 512; }

int moc_symm_allreduce_status(const void* flags, void* stream_) {
  if (!flags) {
    set_error("moc_symm_allreduce_status: null flags");
    return kErrInvalidArg;
  }
  uint32_t word = 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (cudaMemcpyAsync(&word, static_cast<const uint32_t*>(flags) + kArStatus, sizeof(word), cudaMemcpyDeviceToHost,
                      stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return check_last("moc_symm_allreduce_status");
  if (word != 0) {
    set_error("moc_symm_allreduce: a wait for another rank timed out (phase %u, peer %u)", word >> 24, word & 0xFFu);
    return kErrDeviceTimeout;
  }
  return kOk;
}

}  // extern "C"
