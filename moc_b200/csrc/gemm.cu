// Host-side GEMM dispatch: builds the TMA descriptors, picks the core (tcgen05 for bf16,
// CUDA cores for fp32) and instantiates the epilogue functors.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "epilogues.cuh"
#include "gemm_simt.cuh"
#include "gemm_tcgen05.cuh"
#include "gemm_tcgen05_pair.cuh"
#include "internal.h"

namespace moc {

// ---- error text (thread-local, read through moc_last_error) ---------------------------------
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* last_error_text() { return g_err; }

int check_last(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return kErrCuda;
  }
  return kOk;
}

// ---- optional per-kernel event profile ---------------------------------------------------------
struct Profile {
  cudaEvent_t* events = nullptr;
  int capacity = 0;
  int count = 0;
  int tags[4096];
};
// process-wide (PyTorch runs backward passes on its own autograd threads)
static Profile g_prof;
static std::mutex g_prof_mutex;

void prof_mark(int tag, cudaStream_t stream) {
  if (!g_prof.events) return;
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  if (!g_prof.events || g_prof.count >= g_prof.capacity || g_prof.count >= 4096) return;
  if (cudaEventRecord(g_prof.events[g_prof.count], stream) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  g_prof.tags[g_prof.count++] = tag;
}
void profile_begin(cudaEvent_t* events, int capacity) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  g_prof.events = events;
  g_prof.capacity = capacity;
  g_prof.count = 0;
}
int profile_end(int* tags_out, int capacity) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  const int n = g_prof.count;
  for (int i = 0; i < n && i < capacity; ++i) tags_out[i] = g_prof.tags[i];
  g_prof.events = nullptr;
  g_prof.capacity = 0;
  g_prof.count = 0;
  return n;
}

// ---- driver entry point for tensor-map encoding (no link-time dependency on libcuda) -----------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// bf16 operand of extent [mn_extent, k_extent]; tile_mn = rows of the CTA tile it feeds.
static int make_operand_map(CUtensorMap* tm, const MatOperand& op, int64_t mn_extent, int64_t k_extent, int tile_mn) {
  auto encode = get_encode_fn();
  if (!encode) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return kErrCuda;
  }
  if ((reinterpret_cast<uintptr_t>(op.ptr) & 15u) != 0 || (op.ld * 2) % 16 != 0) {
    set_error("GEMM operand needs a 16-byte aligned base and a leading dimension that is a multiple of 8 "
              "(ptr=%p ld=%lld)", op.ptr, static_cast<long long>(op.ld));
    return kErrUnsupported;
  }
  cuuint64_t dims[2], strides[1];
  cuuint32_t box[2], estr[2] = {1, 1};
  if (!op.mn_major) {
    dims[0] = static_cast<cuuint64_t>(k_extent);
    dims[1] = static_cast<cuuint64_t>(mn_extent);
    box[0] = kBlockK;
    box[1] = static_cast<cuuint32_t>(tile_mn);
  } else {
    dims[0] = static_cast<cuuint64_t>(mn_extent);
    dims[1] = static_cast<cuuint64_t>(k_extent);
    box[0] = 64;
    box[1] = kBlockK;
  }
  strides[0] = static_cast<cuuint64_t>(op.ld) * 2;
  const CUresult r = encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(op.ptr), dims, strides, box,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (dims %llu x %llu, ld %lld)", static_cast<int>(r),
              static_cast<unsigned long long>(dims[0]), static_cast<unsigned long long>(dims[1]),
              static_cast<long long>(op.ld));
    return kErrTensorMap;
  }
  return kOk;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <class Epi>
static int launch_tcgen05(const GemmProblem& p, const Epi& epi, cudaStream_t stream) {
  if (!p.status) {
    set_error("tcgen05 GEMM needs a device status word");
    return kErrInvalidArg;
  }
  GemmMaps maps;
  memset(&maps, 0, sizeof(maps));
  const int nmaps = p.k1 > 0 ? 2 : p.groups;
  // products with few columns (decode: N = batch rows): the MMA and the B tile are as narrow as N allows
  const int mma_n = (!p.b[0].mn_major && p.n <= kBlockN / 2) ? (p.n + 15) / 16 * 16 : kBlockN;
  int rc;
  for (int i = 0; i < nmaps; ++i) {
    const int kext = (p.k1 > 0 && i == 1) ? p.k1 : p.k0;
    if ((rc = make_operand_map(&maps.a[i], p.a[i], p.m, kext, kBlockM)) != kOk) return rc;
    if ((rc = make_operand_map(&maps.b[i], p.b[i], p.n, kext, mma_n)) != kOk) return rc;
    if (p.a[i].mn_major != p.a[0].mn_major || p.b[i].mn_major != p.b[0].mn_major) {
      set_error("all K segments / groups of one launch must use the same operand majors");
      return kErrUnsupported;
    }
  }
  GemmShape sh;
  sh.m = p.m;
  sh.n = p.n;
  sh.kb0 = ceil_div_i(p.k0, kBlockK);
  sh.kb1 = p.k1 > 0 ? ceil_div_i(p.k1, kBlockK) : 0;
  sh.groups = p.groups;
  sh.a_mn = p.a[0].mn_major;
  sh.b_mn = p.b[0].mn_major;
  sh.tiles_m = ceil_div_i(p.m, kBlockM);
  sh.tiles_n = ceil_div_i(p.n, kBlockN);
  sh.status = p.status;
  sh.tile_counter = nullptr;
  sh.k_splits = p.k_splits > 1 ? p.k_splits : 1;
  sh.mma_n = mma_n;
  if (sh.k_splits > 1 && (p.k1 > 0 || sh.k_splits > sh.kb0 ||
                          ceil_div_i(sh.kb0, sh.k_splits) * (sh.k_splits - 1) >= sh.kb0)) {
    set_error("split-K needs a single K segment and at least one k-block per split");
    return kErrInvalidArg;
  }
  auto kern = gemm_tcgen05_kernel<Epi>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes) != cudaSuccess)
    return check_last("gemm smem attribute");
  const int tiles = sh.tiles_m * sh.tiles_n * sh.groups * sh.k_splits;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  if (!p.no_prof) prof_mark(kProfGemmTc, stream);
  kern<<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(maps, sh, epi);
  return check_last("gemm_tcgen05");
}

// CTA-pair variant (cta_group::2): 256 x 256 tiles per cluster of two CTAs.
template <class Epi>
static int launch_tcgen05_pair(const GemmProblem& p, const Epi& epi, cudaStream_t stream) {
  GemmMaps maps;
  memset(&maps, 0, sizeof(maps));
  const int nmaps = p.k1 > 0 ? 2 : p.groups;
  int rc;
  for (int i = 0; i < nmaps; ++i) {
    const int kext = (p.k1 > 0 && i == 1) ? p.k1 : p.k0;
    if ((rc = make_operand_map(&maps.a[i], p.a[i], p.m, kext, kBlockM)) != kOk) return rc;
    if ((rc = make_operand_map(&maps.b[i], p.b[i], p.n, kext, kBlockN / 2)) != kOk) return rc;
    if (p.a[i].mn_major != p.a[0].mn_major || p.b[i].mn_major != p.b[0].mn_major) {
      set_error("all K segments / groups of one launch must use the same operand majors");
      return kErrUnsupported;
    }
  }
  GemmShape sh;
  sh.m = p.m;
  sh.n = p.n;
  sh.kb0 = ceil_div_i(p.k0, kBlockK);
  sh.kb1 = p.k1 > 0 ? ceil_div_i(p.k1, kBlockK) : 0;
  sh.groups = p.groups;
  sh.a_mn = p.a[0].mn_major;
  sh.b_mn = p.b[0].mn_major;
  sh.tiles_m = ceil_div_i(p.m, 2 * kBlockM);   // 256-row tile pairs
  sh.tiles_n = ceil_div_i(p.n, kBlockN);
  sh.status = p.status;
  sh.tile_counter = p.tile_counter;
  sh.k_splits = 1;
  sh.mma_n = kBlockN;
  auto kern = gemm_tcgen05_pair_kernel<Epi>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) != cudaSuccess)
    return check_last("gemm pair smem attribute");
  static int max_clusters = 0;
  if (max_clusters == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count());
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_clusters = n;
  }
  const int tiles = sh.tiles_m * sh.tiles_n * sh.groups;
  int avail = max_clusters - (p.sm_reserve + 1) / 2;
  if (avail < 1) avail = 1;
  const int pairs = tiles < avail ? tiles : avail;
  if (!p.no_prof) prof_mark(kProfGemmTc, stream);
  kern<<<2 * pairs, kGemmThreads, kPairSmemBytes, stream>>>(maps, sh, epi);
  return check_last("gemm_tcgen05_pair");
}

// MOC_B200_GEMM_PAIR=0 in the environment keeps every launch on the single-CTA kernel (a switch for A/B timing).
static bool pair_kernel_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("MOC_B200_GEMM_PAIR");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <typename T>
static SimtOperand<T> simt_operand(const MatOperand& op) {
  SimtOperand<T> o;
  o.p = static_cast<const T*>(op.ptr);
  o.s_mn = op.mn_major ? 1 : op.ld;
  o.s_k = op.mn_major ? op.ld : 1;
  return o;
}

template <typename T, class Epi>
static int launch_simt(const GemmProblem& p, const Epi& epi, cudaStream_t stream) {
  const dim3 grid(ceil_div_i(p.n, kSimtBN), ceil_div_i(p.m, kSimtBM));
  for (int g = 0; g < p.groups; ++g) {
    SimtOperand<T> a0 = simt_operand<T>(p.a[g]), b0 = simt_operand<T>(p.b[g]);
    SimtOperand<T> a1 = p.k1 > 0 ? simt_operand<T>(p.a[1]) : a0;
    SimtOperand<T> b1 = p.k1 > 0 ? simt_operand<T>(p.b[1]) : b0;
    prof_mark(kProfGemmSimt, stream);
    gemm_simt_kernel<T, Epi><<<grid, kSimtThreads, 0, stream>>>(a0, b0, p.k0, a1, b1, p.k1 > 0 ? p.k1 : 0, p.m, p.n, g,
                                                                epi);
    const int rc = check_last("gemm_simt");
    if (rc != kOk) return rc;
  }
  return kOk;
}

template <class Epi>
static int launch_core_bf16(const GemmProblem& p, const Epi& epi, cudaStream_t stream) {
  if (p.impl == 1) return launch_simt<__nv_bfloat16, Epi>(p, epi, stream);
  if (!p.status) {
    set_error("tcgen05 GEMM needs a device status word");
    return kErrInvalidArg;
  }
  // A pair of CTAs shares each 256-column B tile, which cuts the operand bytes an SM pulls from L2 per flop by a
  // third; with a single 128-row tile in M the second CTA would only multiply padding.
  if (p.k_splits > 1) return launch_tcgen05<Epi>(p, epi, stream);   // split-K lives in the single-CTA kernel
  if (p.impl == 2 || (p.impl == 0 && p.m > kBlockM && pair_kernel_enabled()))
    return launch_tcgen05_pair<Epi>(p, epi, stream);
  return launch_tcgen05<Epi>(p, epi, stream);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
static int dispatch_epilogue(const GemmProblem& p, cudaStream_t stream) {
  const EpiArgs& e = p.epi;
  auto run = [&](auto epi) -> int {
    using E = decltype(epi);
    if constexpr (Num<T>::kIsBf16) return launch_core_bf16<E>(p, epi, stream);
    else return launch_simt<T, E>(p, epi, stream);
  };
  const bool dense_ok = aligned16(e.dense0) && aligned16(e.dense1) && aligned16(e.dense2) && e.ld_dense % 128 == 0;
  switch (e.kind) {
    case kEpiStore: {
      EpiStore<T> epi;
      for (int g = 0; g < kMaxGroups; ++g) {
        const int s = g < p.groups ? g : 0;
        epi.c[g] = static_cast<T*>(e.c[s]);
        epi.ldc[g] = e.ldc[s];
        epi.transposed[g] = e.transposed[s];
        epi.vec_ok[g] = (!e.transposed[s] && aligned16(e.c[s]) &&
                         (e.ldc[s] * static_cast<int64_t>(sizeof(T))) % 16 == 0) ? 1 : 0;
        if (g < p.groups && !e.c[s]) {
          set_error("GEMM output pointer of group %d is null", g);
          return kErrInvalidArg;
        }
      }
      epi.n = p.n;
      return run(epi);
    }
    case kEpiPartialF32: {
      if constexpr (!Num<T>::kIsBf16) {
        set_error("split-K partial results are a bf16 tensor-core path");
        return kErrUnsupported;
      } else {
        if (!e.partial || e.ld_partial % 4 != 0 || !aligned16(e.partial)) {
          set_error("split-K needs a 16-byte aligned partial buffer with a leading dimension that is a multiple of 4");
          return kErrWorkspace;
        }
        EpiPartialF32<T> epi;
        epi.p = e.partial;
        epi.ld = e.ld_partial;
        epi.block_stride = static_cast<int64_t>(p.m) * e.ld_partial;
        epi.n = p.n;
        return launch_tcgen05<EpiPartialF32<T>>(p, epi, stream);
      }
    }
    case kEpiDenseSwiGLU: {
      if (!dense_ok) {
        set_error("dense scratch must be 16-byte aligned with a leading dimension that is a multiple of 128");
        return kErrWorkspace;
      }
      EpiDenseSwiGLU<T> epi;
      epi.g = static_cast<const T*>(e.dense0);
      epi.u_out = static_cast<T*>(e.dense1);
      epi.z_out = static_cast<T*>(e.dense2);
      epi.ld = e.ld_dense;
      return run(epi);
    }
    default:
      set_error("unknown epilogue kind %d", e.kind);
      return kErrInvalidArg;
  }
}

static int launch_gemm_whole(const GemmProblem& p, cudaStream_t stream) {
  if (p.dtype == kBF16) return dispatch_epilogue<__nv_bfloat16>(p, stream);
  if (p.dtype == kF32) return dispatch_epilogue<float>(p, stream);
  set_error("unsupported dtype %d", p.dtype);
  return kErrInvalidArg;
}

// ---- M-tail split ------------------------------------------------------------------------------------
// The CTA-pair kernel works in 256-row tiles on sm_count / 2 clusters with a static schedule, so a launch takes
// ceil(tiles / clusters) rounds. When the last rows of M fill at most half a tile pair and cutting them off saves
// a whole round, they run as 128-row tiles of the single-CTA kernel on a side stream instead, on the SMs whose
// clusters have no tile in the last round (the weight-gradient GEMM of the 1b preset: 528 pair tiles = 8 rounds,
// against 504 = 7 rounds plus 24 single-CTA tiles on the 28 SMs that idle in the 7th).
struct SideLane {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool ok = false;
};
static std::mutex g_side_mutex;
static int64_t g_side_launches = 0;   // guarded by g_side_mutex
int64_t side_launch_count() {
  std::lock_guard<std::mutex> lock(g_side_mutex);
  return g_side_launches;
}

// One side stream and event pair per device, created at the first split launch on that device (a call that
// should not be the first one inside a stream capture).
static SideLane* side_lane() {
  static SideLane lanes[64];
  static bool tried[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!tried[dev]) {
    tried[dev] = true;
    SideLane& l = lanes[dev];
    l.ok = cudaStreamCreateWithFlags(&l.stream, cudaStreamNonBlocking) == cudaSuccess &&
           cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&l.join, cudaEventDisableTiming) == cudaSuccess;
    if (!l.ok) cudaGetLastError();
  }
  return lanes[dev].ok ? &lanes[dev] : nullptr;
}

static bool tail_split_rows(const GemmProblem& p, int* m_main) {
  if (p.dtype != kBF16 || p.impl != 0 || p.epi.kind != kEpiStore || !pair_kernel_enabled() || !p.status ||
      p.sm_reserve > 0)
    return false;
  const int pair_rows = 2 * kBlockM;
  const int tail = p.m % pair_rows;
  if (tail == 0 || tail > kBlockM || p.m < 2 * pair_rows) return false;
  const int clusters = sm_count() / 2;
  const int per_row = ceil_div_i(p.n, kBlockN) * p.groups;
  const int main_tiles = (p.m / pair_rows) * per_row;
  const int rounds_main = ceil_div_i(main_tiles, clusters);
  if (rounds_main >= ceil_div_i(main_tiles + per_row, clusters)) return false;   // no round saved
  if (per_row > 2 * (rounds_main * clusters - main_tiles)) return false;          // tail would not fit the idle SMs
  *m_main = p.m - tail;
  return true;
}

int launch_gemm(const GemmProblem& p, cudaStream_t stream) {
  if (p.m <= 0 || p.n <= 0) return kOk;
  if (p.groups < 1 || p.groups > kGemmMaxGroups || (p.groups > 1 && p.k1 > 0)) {
    set_error("GEMM: groups must be 1..%d and exclude a second K segment", kGemmMaxGroups);
    return kErrInvalidArg;
  }
  if (p.k0 <= 0 || !p.a[0].ptr || !p.b[0].ptr) {
    set_error("GEMM needs K >= 1 and non-null operands");
    return kErrInvalidArg;
  }
  int m_main = 0;
  if (!tail_split_rows(p, &m_main)) return launch_gemm_whole(p, stream);
  // From here on under the lock: the lane's stream and events are created once and shared by all host threads,
  // and the fork / join sequence below must not interleave with another thread's.
  std::lock_guard<std::mutex> lock(g_side_mutex);
  SideLane* lane = side_lane();
  if (!lane) return launch_gemm_whole(p, stream);

  GemmProblem head = p, tail = p;
  head.m = m_main;
  head.impl = 2;
  tail.m = p.m - m_main;
  tail.impl = 3;
  tail.no_prof = 1;
  const int nops = p.k1 > 0 ? 2 : p.groups;
  for (int i = 0; i < nops; ++i) {
    const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(p.a[i].ptr);
    tail.a[i].ptr = a + (p.a[i].mn_major ? static_cast<int64_t>(m_main) : static_cast<int64_t>(m_main) * p.a[i].ld);
  }
  for (int g = 0; g < p.groups; ++g) {
    __nv_bfloat16* c = static_cast<__nv_bfloat16*>(p.epi.c[g]);
    if (c) tail.epi.c[g] = c + (p.epi.transposed[g] ? static_cast<int64_t>(m_main) : static_cast<int64_t>(m_main) * p.epi.ldc[g]);
  }
  if (cudaEventRecord(lane->fork, stream) != cudaSuccess ||
      cudaStreamWaitEvent(lane->stream, lane->fork, 0) != cudaSuccess)
    return check_last("GEMM tail fork");
  int rc = launch_gemm_whole(head, stream);
  const int rc_tail = launch_gemm_whole(tail, lane->stream);
  if (rc_tail == kOk) ++g_side_launches;
  // join even after a failed launch so that the side stream never stays attached to a capture
  if (cudaEventRecord(lane->join, lane->stream) != cudaSuccess ||
      cudaStreamWaitEvent(stream, lane->join, 0) != cudaSuccess)
    return check_last("GEMM tail join");
  return rc != kOk ? rc : rc_tail;
}

}  // namespace moc
