// C ABI of libmoc_b200: argument checks and the launch sequences of the MoC FFN
// forward / backward passes. Declarations and reference citations: include/moc_b200.h.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/moc_b200.h"
#include "common.cuh"
#include "internal.h"

namespace moc {
void profile_begin(cudaEvent_t* events, int capacity);
int profile_end(int* tags_out, int capacity);
}

using namespace moc;

namespace {

constexpr int64_t kStatusBytes = 256;
// The status area holds 64 ints, zeroed at the start of every FFN call: [0] the time-out word of the bounded
// device waits, [16..] one tile counter per GEMM launch of the call (CTA-pair kernel, tiles in arrival order).
constexpr int kTileCounterFirst = 16;
// SMs that the dX GEMM of a backward call leaves free (moc_set_overlap_sm_reserve)
std::atomic<int> g_overlap_sm_reserve{0};

inline size_t esize(int dtype) { return dtype == kBF16 ? 2 : 4; }
inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

bool bad_dtype(int dtype) {
  if (dtype == kBF16 || dtype == kF32) return false;
  set_error("unsupported dtype code %d", dtype);
  return true;
}

int check_dims(int64_t tokens, int64_t d, int64_t d_ffn, int64_t k) {
  if (tokens < 0 || d <= 0 || d_ffn <= 0 || k <= 0 || k > d_ffn) {
    set_error("bad sizes: tokens=%lld d=%lld d_ffn=%lld k=%lld", (long long)tokens, (long long)d, (long long)d_ffn,
              (long long)k);
    return kErrInvalidArg;
  }
  if (d_ffn > 32768) {
    set_error("d_ffn=%lld: channel indices are stored as int16, d_ffn must be <= 32768", (long long)d_ffn);
    return kErrUnsupported;
  }
  if (tokens > (int64_t(1) << 30) || d > (int64_t(1) << 24)) {
    set_error("sizes exceed the 32-bit tile arithmetic of the kernels");
    return kErrUnsupported;
  }
  return kOk;
}

MatOperand operand(const void* p, int64_t ld, int mn_major) {
  MatOperand o;
  o.ptr = p;
  o.ld = ld;
  o.mn_major = mn_major;
  return o;
}

EpiArgs store_epi(void* c, int64_t ldc, int transposed) {
  EpiArgs e = {};
  e.kind = kEpiStore;
  e.c[0] = c;
  e.ldc[0] = ldc;
  e.transposed[0] = transposed;
  return e;
}

GemmProblem problem(int dtype, int* status, int64_t m, int64_t n, int64_t k) {
  GemmProblem p = {};
  p.dtype = dtype;
  p.status = status;
  p.m = (int)m;
  p.n = (int)n;
  p.k0 = (int)k;
  p.groups = 1;
  return p;
}

int record(void* ev, cudaStream_t stream) {
  if (!ev) return kOk;
  if (cudaEventRecord(reinterpret_cast<cudaEvent_t>(ev), stream) != cudaSuccess) return check_last("cudaEventRecord");
  return kOk;
}

__global__ void publish_status_kernel(const int* __restrict__ status, volatile int* host_word) {
  const int w = *status;
  if (w != 0) *host_word = w;
}

}  // namespace

extern "C" {

int moc_b200_abi_version(void) { return MOC_B200_ABI_VERSION; }

const char* moc_last_error(void) { return last_error_text(); }

int64_t moc_ffn_ld(int64_t d_ffn) { return ffn_ld(d_ffn); }
int64_t moc_mask_words(int64_t d_ffn) { return mask_words(d_ffn); }
int64_t moc_select_2of8_k(int64_t d_ffn) { return (d_ffn / 8) * 2 + (d_ffn % 8 < 2 ? d_ffn % 8 : 2); }

int64_t moc_ffn_fwd_workspace_bytes(int dtype, int64_t tokens, int64_t d_ffn) {
  return kStatusBytes + 2 * round_up_i64(tokens * ffn_ld(d_ffn) * (int64_t)esize(dtype), 256);
}
int64_t moc_ffn_fwd_workspace_bytes_select(int dtype, int select, int64_t tokens, int64_t d_ffn) {
  const int dense = select == MOC_SELECT_POST_SILU_ABS ? 3 : 2;
  return kStatusBytes + dense * round_up_i64(tokens * ffn_ld(d_ffn) * (int64_t)esize(dtype), 256);
}
int64_t moc_ffn_bwd_workspace_bytes(int dtype, int64_t tokens, int64_t d_ffn) {
  return kStatusBytes + 3 * round_up_i64(tokens * ffn_ld(d_ffn) * (int64_t)esize(dtype), 256);
}

int moc_transpose(int dtype, const void* in, void* out, int64_t rows, int64_t cols, void* stream) {
  if (bad_dtype(dtype)) return kErrInvalidArg;
  if (!in || !out || rows < 0 || cols < 0) {
    set_error("moc_transpose: null pointer or negative size");
    return kErrInvalidArg;
  }
  return launch_transpose(dtype, in, cols, out, rows, (int)rows, (int)cols, as_stream(stream));
}

int moc_topk_select(int dtype, const void* g, int64_t ldg, int64_t tokens, int64_t d_ffn, int64_t k, int16_t* idx,
                    void* g_sel, uint32_t* bitmap, uint16_t* rank0, void* stream) {
  if (bad_dtype(dtype)) return kErrInvalidArg;
  int rc = check_dims(tokens, 1, d_ffn, k);
  if (rc != kOk) return rc;
  if (!g || !idx || !g_sel || !bitmap || !rank0 || ldg < d_ffn) {
    set_error("moc_topk_select: null pointer or ldg < d_ffn");
    return kErrInvalidArg;
  }
  return launch_topk_select(dtype, const_cast<void*>(g), ldg, (int)tokens, (int)d_ffn, (int)k, nullptr, idx, g_sel,
                            bitmap, rank0, as_stream(stream));
}

int moc_select_2of8(int dtype, const void* g, int64_t ldg, int64_t tokens, int64_t d_ffn, int16_t* idx, void* g_sel,
                    uint32_t* bitmap, uint16_t* rank0, void* stream) {
  if (bad_dtype(dtype)) return kErrInvalidArg;
  int rc = check_dims(tokens, 1, d_ffn, 1);
  if (rc != kOk) return rc;
  if (!g || !idx || !g_sel || !bitmap || !rank0 || ldg < d_ffn) {
    set_error("moc_select_2of8: null pointer or ldg < d_ffn");
    return kErrInvalidArg;
  }
  return launch_select_2of8(dtype, const_cast<void*>(g), ldg, (int)tokens, (int)d_ffn, nullptr, idx, g_sel, bitmap,
                            rank0, as_stream(stream));
}

int moc_gemm(int dtype, int impl, int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, int a_mn,
             const void* b, int64_t ldb, int b_mn, void* c, int64_t ldc, int c_transposed, int* status,
             void* stream) {
  if (bad_dtype(dtype)) return kErrInvalidArg;
  if (m < 0 || n < 0 || k <= 0 || !a || !b || !c || m > (int64_t(1) << 30) || n > (int64_t(1) << 30) ||
      k > (int64_t(1) << 30)) {
    set_error("moc_gemm: bad sizes or null pointer");
    return kErrInvalidArg;
  }
  GemmProblem p = problem(dtype, status, m, n, k);
  p.impl = impl;
  p.a[0] = operand(a, lda, a_mn);
  p.b[0] = operand(b, ldb, b_mn);
  p.epi = store_epi(c, ldc, c_transposed);
  return launch_gemm(p, as_stream(stream));
}

int moc_ffn_fwd(int dtype, int select, int64_t tokens, int64_t d, int64_t d_ffn, int64_t k, const void* x,
                const void* w_gate, const void* w_up, const void* w_down_t, void* y, int16_t* idx, void* g_sel,
                void* u_sel, void* s_sel, void* z_sel, uint32_t* bitmap, uint16_t* rank0, void* workspace,
                int64_t workspace_bytes, void* stream_) {
  if (bad_dtype(dtype)) return kErrInvalidArg;
  int rc = check_dims(tokens, d, d_ffn, k);
  if (rc != kOk) return rc;
  // tensors with a token dimension have no storage when tokens == 0
  if (!w_gate || !w_up || !w_down_t || !workspace ||
      (tokens > 0 && (!x || !y || !idx || !g_sel || !u_sel || !bitmap || !rank0))) {
    set_error("moc_ffn_fwd: null pointer");
    return kErrInvalidArg;
  }
  if (select != MOC_SELECT_TOPK && select != MOC_SELECT_2OF8 && select != MOC_SELECT_POST_SILU_ABS) {
    set_error("moc_ffn_fwd: unknown selection rule %d", select);
    return kErrInvalidArg;
  }
  if (select == MOC_SELECT_2OF8 && k != moc_select_2of8_k(d_ffn)) {
    set_error("moc_ffn_fwd: the 2:8 rule selects k=%lld channels for d_ffn=%lld, got k=%lld",
              (long long)moc_select_2of8_k(d_ffn), (long long)d_ffn, (long long)k);
    return kErrInvalidArg;
  }
  if (workspace_bytes < moc_ffn_fwd_workspace_bytes_select(dtype, select, tokens, d_ffn) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_error("moc_ffn_fwd: workspace too small (%lld < %lld bytes) or not 256-byte aligned",
              (long long)workspace_bytes, (long long)moc_ffn_fwd_workspace_bytes_select(dtype, select, tokens, d_ffn));
    return kErrWorkspace;
  }
  cudaStream_t stream = as_stream(stream_);
  int* status = static_cast<int*>(workspace);
  if (cudaMemsetAsync(status, 0, kStatusBytes, stream) != cudaSuccess) return check_last("cudaMemsetAsync");
  if (tokens == 0) return kOk;
  void* dense = static_cast<uint8_t*>(workspace) + kStatusBytes;
  const int64_t ld = ffn_ld(d_ffn);
  const int words = (int)mask_words(d_ffn);

  // G = X Wg^T and U = X Wu^T (moc/ffn.py:141, :146) in one grouped launch, both rounded to the storage type,
  // rows padded to ld
  void* u_dense = static_cast<uint8_t*>(dense) + round_up_i64(tokens * ld * (int64_t)esize(dtype), 256);
  GemmProblem p = problem(dtype, status, tokens, d_ffn, d);
  p.groups = 2;
  p.a[0] = operand(x, d, 0);
  p.b[0] = operand(w_gate, d, 0);
  p.a[1] = operand(x, d, 0);
  p.b[1] = operand(w_up, d, 0);
  p.epi = EpiArgs{};
  p.epi.kind = kEpiStore;
  p.epi.c[0] = dense;
  p.epi.ldc[0] = ld;
  p.epi.c[1] = u_dense;
  p.epi.ldc[1] = ld;
  p.tile_counter = status + kTileCounterFirst;
  if ((rc = launch_gemm(p, stream)) != kOk) return rc;

  // channel selection on the rounded G (moc/ffn.py:144-147); the same kernel gathers the selected channels of U
  // into the compact saved set and turns the G rows into Z' = mask * round(round(SiLU(G)) * U) in place
  // (moc/ffn.py:156-161, :166-169)
  SelectFuse fuse{u_dense, u_sel, s_sel, z_sel, status};
  if (select == MOC_SELECT_POST_SILU_ABS) {
    // Top-K on |SiLU(G)| (moc/ffn.py:336-339): scores in a third scratch matrix, plain selection on them (the
    // g_sel array receives scores first), then g, u of the chosen channels are gathered from the dense rows and
    // the G rows become Z'
    void* score = static_cast<uint8_t*>(u_dense) + round_up_i64(tokens * ld * (int64_t)esize(dtype), 256);
    if ((rc = launch_abs_silu(dtype, dense, score, tokens * ld, stream)) != kOk ||
        (rc = launch_topk_select(dtype, score, ld, (int)tokens, (int)d_ffn, (int)k, nullptr, idx, g_sel, bitmap, rank0,
                                 stream)) != kOk ||
        (rc = launch_post_gather(dtype, idx, dense, u_dense, g_sel, u_sel, s_sel, z_sel, ld, (int)tokens, (int)k,
                                 stream)) != kOk)
      return rc;
  } else if (select == MOC_SELECT_TOPK)
    rc = launch_topk_select(dtype, dense, ld, (int)tokens, (int)d_ffn, (int)k, &fuse, idx, g_sel, bitmap, rank0,
                            stream);
  else
    rc = launch_select_2of8(dtype, dense, ld, (int)tokens, (int)d_ffn, &fuse, idx, g_sel, bitmap, rank0, stream);
  if (rc != kOk) return rc;

  // Y = Z' Wd^T (moc/ffn.py:163): A = Z' [tokens, F] K-major, B = W_down^T [F, d] N-contiguous
  GemmProblem q = problem(dtype, status, tokens, d, d_ffn);
  q.a[0] = operand(dense, ld, 0);
  q.b[0] = operand(w_down_t, d, 1);
  q.epi = store_epi(y, d, 0);
  q.tile_counter = status + kTileCounterFirst + 1;
  rc = launch_gemm(q, stream);
  prof_mark(kProfEnd, stream);
  return rc;
}

int moc_ffn_bwd(int dtype, int64_t tokens, int64_t d, int64_t d_ffn, int64_t k, const void* grad_y, const void* x,
                const void* w_gate, const void* w_up, const void* w_down_t, const int16_t* idx,
                const void* g_sel, const void* u_sel, const void* s_sel, const void* z_sel,
                void* grad_x, void* grad_w_gate, void* grad_w_up, void* grad_w_down, void* workspace,
                int64_t workspace_bytes, void* ev_down, void* ev_gate, void* ev_up, void* stream_) {
  if (bad_dtype(dtype)) return kErrInvalidArg;
  int rc = check_dims(tokens, d, d_ffn, k);
  if (rc != kOk) return rc;
  if (!w_gate || !w_up || !w_down_t || !grad_w_gate || !grad_w_up || !grad_w_down || !workspace ||
      (tokens > 0 && (!grad_y || !x || !idx || !g_sel || !u_sel || !grad_x))) {
    set_error("moc_ffn_bwd: null pointer");
    return kErrInvalidArg;
  }
  if (workspace_bytes < moc_ffn_bwd_workspace_bytes(dtype, tokens, d_ffn) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_error("moc_ffn_bwd: workspace too small (%lld < %lld bytes) or not 256-byte aligned",
              (long long)workspace_bytes, (long long)moc_ffn_bwd_workspace_bytes(dtype, tokens, d_ffn));
    return kErrWorkspace;
  }
  (void)s_sel;   // s = round(SiLU(g)) is recomputed; the saved copy holds the same bits
  cudaStream_t stream = as_stream(stream_);
  int* status = static_cast<int*>(workspace);
  if (cudaMemsetAsync(status, 0, kStatusBytes, stream) != cudaSuccess) return check_last("cudaMemsetAsync");
  const size_t es = esize(dtype);
  if (tokens == 0) {
    // no tokens: every gradient is zero
    if (cudaMemsetAsync(grad_w_gate, 0, (size_t)d_ffn * d * es, stream) != cudaSuccess ||
        cudaMemsetAsync(grad_w_up, 0, (size_t)d_ffn * d * es, stream) != cudaSuccess ||
        cudaMemsetAsync(grad_w_down, 0, (size_t)d_ffn * d * es, stream) != cudaSuccess)
      return check_last("cudaMemsetAsync");
    if ((rc = record(ev_down, stream)) != kOk || (rc = record(ev_gate, stream)) != kOk ||
        (rc = record(ev_up, stream)) != kOk)
      return rc;
    return kOk;
  }
  const int64_t ld = ffn_ld(d_ffn);
  const int64_t dense_bytes = round_up_i64(tokens * ld * (int64_t)es, 256);
  void* buf_z = static_cast<uint8_t*>(workspace) + kStatusBytes;     // Z'
  void* buf_u = static_cast<uint8_t*>(buf_z) + dense_bytes;          // dZ, then dU'
  void* buf_g = static_cast<uint8_t*>(buf_u) + dense_bytes;          // dG'

  // dZ = dY W_down (moc/ffn.py:206), rounded to the storage type
  GemmProblem z = problem(dtype, status, tokens, d_ffn, d);
  z.a[0] = operand(grad_y, d, 0);
  z.b[0] = operand(w_down_t, d, 0);
  z.epi = store_epi(buf_u, ld, 0);
  z.tile_counter = status + kTileCounterFirst;
  if ((rc = launch_gemm(z, stream)) != kOk) return rc;

  // one pass over the selected channels: gather through the mask, SiLU', zero fill -> dense dG', dU'
  // (moc/ffn.py:209-237), and Z' from the saved or recomputed activations (moc/ffn.py:196-199, :435-442)
  if ((rc = launch_bwd_sparse(dtype, idx, g_sel, u_sel, z_sel, buf_u, buf_g, buf_z, ld, (int)tokens, (int)d_ffn,
                              (int)k, stream)) != kOk)
    return rc;

  // The three weight gradients in one grouped launch, each an [F, d] product over the tokens:
  //   dW_down[d, F] = dY^T Z'  (moc/ffn.py:203)  computed as Z'^T dY and stored transposed,
  //   dW_gate[F, d] = dG'^T X, dW_up[F, d] = dU'^T X  (moc/ffn.py:239-253).
  GemmProblem w = problem(dtype, status, d_ffn, d, tokens);
  w.groups = 3;
  w.a[0] = operand(buf_z, ld, 1);
  w.b[0] = operand(grad_y, d, 1);
  w.a[1] = operand(buf_g, ld, 1);
  w.b[1] = operand(x, d, 1);
  w.a[2] = operand(buf_u, ld, 1);
  w.b[2] = operand(x, d, 1);
  w.epi = EpiArgs{};
  w.epi.kind = kEpiStore;
  w.epi.c[0] = grad_w_down;
  w.epi.ldc[0] = d_ffn;
  w.epi.transposed[0] = 1;
  w.epi.c[1] = grad_w_gate;
  w.epi.ldc[1] = d;
  w.epi.c[2] = grad_w_up;
  w.epi.ldc[2] = d;
  w.tile_counter = status + kTileCounterFirst + 1;
  if ((rc = launch_gemm(w, stream)) != kOk) return rc;
  if ((rc = record(ev_down, stream)) != kOk || (rc = record(ev_gate, stream)) != kOk ||
      (rc = record(ev_up, stream)) != kOk)
    return rc;

  // dX = dG' W_gate + dU' W_up (moc/ffn.py:245-255), one accumulator over two K segments
  GemmProblem gx = problem(dtype, status, tokens, d, d_ffn);
  gx.k1 = (int)d_ffn;
  gx.a[0] = operand(buf_g, ld, 0);
  gx.b[0] = operand(w_gate, d, 1);
  gx.a[1] = operand(buf_u, ld, 0);
  gx.b[1] = operand(w_up, d, 1);
  gx.epi = store_epi(grad_x, d, 0);
  gx.tile_counter = status + kTileCounterFirst + 2;
  gx.sm_reserve = g_overlap_sm_reserve.load(std::memory_order_relaxed);   // room for the gradient all-reduce
  rc = launch_gemm(gx, stream);
  prof_mark(kProfEnd, stream);
  return rc;
}

int moc_dense_ffn_fwd(int dtype, int64_t tokens, int64_t d, int64_t d_ffn, const void* x, const void* w_gate,
                      const void* w_up, const void* w_down_t, void* y, void* g_out, void* u_out, void* workspace,
                      int64_t workspace_bytes, void* stream_) {
  if (bad_dtype(dtype)) return kErrInvalidArg;
  int rc = check_dims(tokens, d, d_ffn, 1);
  if (rc != kOk) return rc;
  if (!w_gate || !w_up || !w_down_t || !workspace || (tokens > 0 && (!x || !y || !g_out || !u_out))) {
    set_error("moc_dense_ffn_fwd: null pointer");
    return kErrInvalidArg;
  }
  if (workspace_bytes < moc_ffn_fwd_workspace_bytes(dtype, tokens, d_ffn) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_error("moc_dense_ffn_fwd: workspace too small or not 256-byte aligned");
    return kErrWorkspace;
  }
  cudaStream_t stream = as_stream(stream_);
  int* status = static_cast<int*>(workspace);
  if (cudaMemsetAsync(status, 0, kStatusBytes, stream) != cudaSuccess) return check_last("cudaMemsetAsync");
  if (tokens == 0) return kOk;
  void* z = static_cast<uint8_t*>(workspace) + kStatusBytes;
  const int64_t ld = ffn_ld(d_ffn);
  // G = X Wg^T, then U = X Wu^T with Z = SiLU(G) * U in the epilogue, then Y = Z Wd^T (moc/ffn.py:120-121)
  GemmProblem p = problem(dtype, status, tokens, d_ffn, d);
  p.a[0] = operand(x, d, 0);
  p.b[0] = operand(w_gate, d, 0);
  p.epi = store_epi(g_out, ld, 0);
  if ((rc = launch_gemm(p, stream)) != kOk) return rc;
  p.b[0] = operand(w_up, d, 0);
  p.epi = EpiArgs{};
  p.epi.kind = kEpiDenseSwiGLU;
  p.epi.dense0 = g_out;
  p.epi.dense1 = u_out;
  p.epi.dense2 = z;
  p.epi.ld_dense = ld;
  if ((rc = launch_gemm(p, stream)) != kOk) return rc;
  GemmProblem q = problem(dtype, status, tokens, d, d_ffn);
  q.a[0] = operand(z, ld, 0);
  q.b[0] = operand(w_down_t, d, 1);
  q.epi = store_epi(y, d, 0);
  q.tile_counter = status + kTileCounterFirst + 1;
  rc = launch_gemm(q, stream);
  prof_mark(kProfEnd, stream);
  return rc;
}

int moc_dense_ffn_bwd(int dtype, int64_t tokens, int64_t d, int64_t d_ffn, const void* grad_y, const void* x,
                      const void* w_gate, const void* w_up, const void* w_down_t, const void* g, const void* u,
                      void* grad_x, void* grad_w_gate, void* grad_w_up, void* grad_w_down, void* workspace,
                      int64_t workspace_bytes, void* stream_) {
  if (bad_dtype(dtype)) return kErrInvalidArg;
  int rc = check_dims(tokens, d, d_ffn, 1);
  if (rc != kOk) return rc;
  if (!w_gate || !w_up || !w_down_t || !grad_w_gate || !grad_w_up || !grad_w_down || !workspace ||
      (tokens > 0 && (!grad_y || !x || !g || !u || !grad_x))) {
    set_error("moc_dense_ffn_bwd: null pointer");
    return kErrInvalidArg;
  }
  if (workspace_bytes < moc_ffn_bwd_workspace_bytes(dtype, tokens, d_ffn) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_error("moc_dense_ffn_bwd: workspace too small or not 256-byte aligned");
    return kErrWorkspace;
  }
  cudaStream_t stream = as_stream(stream_);
  int* status = static_cast<int*>(workspace);
  if (cudaMemsetAsync(status, 0, kStatusBytes, stream) != cudaSuccess) return check_last("cudaMemsetAsync");
  const size_t es = esize(dtype);
  if (tokens == 0) {
    if (cudaMemsetAsync(grad_w_gate, 0, (size_t)d_ffn * d * es, stream) != cudaSuccess ||
        cudaMemsetAsync(grad_w_up, 0, (size_t)d_ffn * d * es, stream) != cudaSuccess ||
        cudaMemsetAsync(grad_w_down, 0, (size_t)d_ffn * d * es, stream) != cudaSuccess)
      return check_last("cudaMemsetAsync");
    return kOk;
  }
  const int64_t ld = ffn_ld(d_ffn);
  const int64_t dense_bytes = round_up_i64(tokens * ld * (int64_t)es, 256);
  void* buf_z = static_cast<uint8_t*>(workspace) + kStatusBytes;
  void* buf_u = static_cast<uint8_t*>(buf_z) + dense_bytes;   // dZ, then dU
  void* buf_g = static_cast<uint8_t*>(buf_u) + dense_bytes;   // dG
  GemmProblem z = problem(dtype, status, tokens, d_ffn, d);
  z.a[0] = operand(grad_y, d, 0);
  z.b[0] = operand(w_down_t, d, 0);
  z.epi = store_epi(buf_u, ld, 0);
  z.tile_counter = status + kTileCounterFirst;
  if ((rc = launch_gemm(z, stream)) != kOk) return rc;
  // (padding columns [d_ffn, ld) of the dense matrices hold unspecified values; no GEMM reads them)
  if ((rc = launch_dense_bwd(dtype, g, u, buf_u, buf_z, buf_g, tokens * ld, stream)) != kOk) return rc;
  GemmProblem w = problem(dtype, status, d_ffn, d, tokens);
  w.groups = 3;
  w.a[0] = operand(buf_z, ld, 1);
  w.b[0] = operand(grad_y, d, 1);
  w.a[1] = operand(buf_g, ld, 1);
  w.b[1] = operand(x, d, 1);
  w.a[2] = operand(buf_u, ld, 1);
  w.b[2] = operand(x, d, 1);
  w.epi = EpiArgs{};
  w.epi.kind = kEpiStore;
  w.epi.c[0] = grad_w_down;
  w.epi.ldc[0] = d_ffn;
  w.epi.transposed[0] = 1;
  w.epi.c[1] = grad_w_gate;
  w.epi.ldc[1] = d;
  w.epi.c[2] = grad_w_up;
  w.epi.ldc[2] = d;
  w.tile_counter = status + kTileCounterFirst + 1;
  if ((rc = launch_gemm(w, stream)) != kOk) return rc;
  GemmProblem gx = problem(dtype, status, tokens, d, d_ffn);
  gx.k1 = (int)d_ffn;
  gx.a[0] = operand(buf_g, ld, 0);
  gx.b[0] = operand(w_gate, d, 1);
  gx.a[1] = operand(buf_u, ld, 0);
  gx.b[1] = operand(w_up, d, 1);
  gx.epi = store_epi(grad_x, d, 0);
  gx.tile_counter = status + kTileCounterFirst + 2;
  gx.sm_reserve = g_overlap_sm_reserve.load(std::memory_order_relaxed);   // room for the gradient all-reduce
  rc = launch_gemm(gx, stream);
  prof_mark(kProfEnd, stream);
  return rc;
}

int64_t moc_decode_workspace_bytes(int64_t batch, int64_t d, int64_t d_ffn) {
  return decode_workspace_bytes(batch, d, d_ffn);
}

int moc_decode_global(int64_t batch, int64_t d, int64_t d_ffn, int64_t k, const void* x, const void* w_gate,
                      const void* w_up, const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes,
                      void* stream) {
  if (!x || !w_gate || !w_up || !w_down_t || !y) {
    set_error("moc_decode_global: null pointer");
    return kErrInvalidArg;
  }
  return decode_global(batch, d, d_ffn, k, 0, x, nullptr, w_gate, w_up, w_down_t, y, workspace, workspace_bytes,
                       as_stream(stream));
}

int moc_decode_after_gate(int64_t batch, int64_t d, int64_t d_ffn, int64_t k, const void* x, const void* gate_scores,
                          const void* w_up, const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes,
                          void* stream) {
  if (!x || !gate_scores || !w_up || !w_down_t || !y) {
    set_error("moc_decode_after_gate: null pointer");
    return kErrInvalidArg;
  }
  return decode_global(batch, d, d_ffn, k, 0, x, gate_scores, nullptr, w_up, w_down_t, y, workspace, workspace_bytes,
                       as_stream(stream));
}

int moc_decode_2of8(int64_t batch, int64_t d, int64_t d_ffn, const void* x, const void* w_gate, const void* w_up,
                    const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!x || !w_gate || !w_up || !w_down_t || !y) {
    set_error("moc_decode_2of8: null pointer");
    return kErrInvalidArg;
  }
  return decode_global(batch, d, d_ffn, moc_select_2of8_k(d_ffn), 1, x, nullptr, w_gate, w_up, w_down_t, y, workspace,
                       workspace_bytes, as_stream(stream));
}

int moc_decode_dense(int64_t batch, int64_t d, int64_t d_ffn, const void* x, const void* w_gate, const void* w_up,
                     const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!x || !w_gate || !w_up || !w_down_t || !y) {
    set_error("moc_decode_dense: null pointer");
    return kErrInvalidArg;
  }
  return decode_dense(batch, d, d_ffn, x, w_gate, w_up, w_down_t, y, workspace, workspace_bytes, as_stream(stream));
}

int moc_decode_selected_up(int64_t batch, int64_t k, int64_t d, int64_t d_ffn, const void* x, const void* g_sel,
                           const int16_t* idx, const void* w_up, void* sparse_z, void* stream) {
  if (batch < 0 || d <= 0 || d % 8 != 0 || d_ffn <= 0 || k <= 0 || k > d_ffn) {
    set_error("moc_decode_selected_up: bad sizes batch=%lld d=%lld d_ffn=%lld k=%lld", (long long)batch, (long long)d,
              (long long)d_ffn, (long long)k);
    return kErrInvalidArg;
  }
  if (batch > 0 && (!x || !g_sel || !idx || !w_up || !sparse_z)) {
    set_error("moc_decode_selected_up: null pointer");
    return kErrInvalidArg;
  }
  return decode_selected_up(batch, k, d, x, g_sel, idx, w_up, sparse_z, as_stream(stream));
}

int moc_decode_selected_down(int64_t batch, int64_t k, int64_t d, int64_t d_ffn, const void* sparse_z,
                             const int16_t* idx, const void* w_down_t, void* y, void* workspace,
                             int64_t workspace_bytes, void* stream) {
  if (!sparse_z || !idx || !w_down_t || !y) {
    set_error("moc_decode_selected_down: null pointer");
    return kErrInvalidArg;
  }
  return decode_selected_down(batch, k, d, d_ffn, sparse_z, idx, w_down_t, y, workspace, workspace_bytes,
                              as_stream(stream));
}

int moc_profile_begin(void** events, int capacity) {
  if (!events || capacity <= 0) {
    set_error("moc_profile_begin: need a host array of cudaEvent_t handles");
    return kErrInvalidArg;
  }
  profile_begin(reinterpret_cast<cudaEvent_t*>(events), capacity);
  return kOk;
}

int moc_profile_end(int* tags_out, int capacity) { return profile_end(tags_out, capacity); }
int64_t moc_side_launch_count(void) { return side_launch_count(); }

int moc_set_overlap_sm_reserve(int sms) {
  if (sms < 0 || sms > 64) {
    set_error("moc_set_overlap_sm_reserve: %d is outside 0..64", sms);
    return kErrInvalidArg;
  }
  g_overlap_sm_reserve.store(sms, std::memory_order_relaxed);
  return kOk;
}

int moc_read_status(const void* workspace, void* stream_) {
  if (!workspace) {
    set_error("moc_read_status: null workspace");
    return kErrInvalidArg;
  }
  int word = 0;
  cudaStream_t stream = as_stream(stream_);
  if (cudaMemcpyAsync(&word, workspace, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return check_last("moc_read_status");
  if (word != 0) {
    set_error("device-side wait timed out: role %d, detail 0x%x", (word >> 24) & 0xFF, word & 0xFFFFFF);
    return kErrDeviceTimeout;
  }
  return kOk;
}

int moc_debug_set_wait_cycles(int64_t cycles) {
  decode_stream_set_wait_cycles(static_cast<long long>(cycles));
  return kOk;
}

int moc_publish_status(const void* workspace, int* host_word, void* stream_) {
  if (!workspace || !host_word) {
    set_error("moc_publish_status: null pointer");
    return kErrInvalidArg;
  }
  publish_status_kernel<<<1, 1, 0, as_stream(stream_)>>>(static_cast<const int*>(workspace), host_word);
  return check_last("moc_publish_status");
}

}  // extern "C"
