// Host-side launch interfaces shared between the translation units of libmoc_b200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace moc {

// ---- GEMM cores (gemm.cu) ---------------------------------------------------------------
// One operand of a product C[M,N] += A[M,K] * B[N,K]^T.
struct MatOperand {
  const void* ptr;
  int64_t ld;     // elements between consecutive rows in memory
  int mn_major;   // 0: memory is [mn][k] (K contiguous); 1: memory is [k][mn] (M/N contiguous)
};

enum EpiKind : int { kEpiStore = 0, kEpiDenseSwiGLU = 2, kEpiPartialF32 = 3 };

constexpr int kGemmMaxGroups = 3;

struct EpiArgs {
  int kind;
  // kEpiStore: one output per group
  void* c[kGemmMaxGroups];
  int64_t ldc[kGemmMaxGroups];
  int transposed[kGemmMaxGroups];
  // kEpiDenseSwiGLU: dense0 = G (in), dense1 = U (out), dense2 = Z (out)
  void* dense0;
  void* dense1;
  void* dense2;
  int64_t ld_dense;
  // kEpiPartialF32: [groups * k_splits][m][ld_partial] floats
  float* partial;
  int64_t ld_partial;
};

// C_g[m, n] = A_g[m, k0] * B_g[n, k0]^T for g < groups, or, with groups == 1 and k1 > 0,
// C = A_0[m, k0] * B_0[n, k0]^T + A_1[m, k1] * B_1[n, k1]^T.
struct GemmProblem {
  int dtype;                 // DType
  int impl;                  // 0: default for the dtype (bf16 -> tcgen05, f32 -> SIMT); 1: force SIMT;
                             // 2 / 3: force the CTA-pair / single-CTA tcgen05 kernel
  int no_prof;               // 1: the launch records no profile event (used for side-stream launches)
  int* tile_counter;         // CTA-pair kernel: zeroed device int -> tiles are handed out in arrival order
                             // (null: round-robin over the clusters)
  int sm_reserve;            // CTA-pair kernel: SMs left free for a kernel that runs beside this launch
  int k_splits;              // > 1 (bf16, kEpiPartialF32 only): K is cut into that many ranges, each tile writes an
                             // fp32 partial block to epi.partial; the caller adds the blocks up
  int m, n;
  int groups;                // 1..3 same-shape problems in one launch
  int k0;
  int k1;                    // K extent of the second segment (0: none)
  MatOperand a[kGemmMaxGroups], b[kGemmMaxGroups];
  EpiArgs epi;
  int* status;               // device status word (may be null for SIMT)
};

int launch_gemm(const GemmProblem& p, cudaStream_t stream);
// GEMM launches put on the side stream so far (tail rows of M, see launch_gemm)
int64_t side_launch_count();

// ---- selection / auxiliary kernels (kernels.cu) ---------------------------------------------
// Optional forward fusion of a selection launch: with `fuse` set the kernel also gathers u = U[t, ch] of every
// selected channel from the dense rows u_dense (same leading dimension as g), writes u_sel (and s_sel =
// round(SiLU(g)), z_sel = round(s * u) when set) and overwrites the gate rows (ldg >= ffn_ld) in place by
// Z' = mask * z.
struct SelectFuse {
  const void* u_dense;
  void* u_sel;
  void* s_sel;   // may be null
  void* z_sel;   // may be null
  int* status;   // device status word for kernels with bounded waits; null: only kernels without waits are used
};
// Persistent shared-memory-staged form of the fused Top-K launch for bf16 rows (select_stream.cu)
bool select_stream_supported(int64_t ldg, int d_ffn, int k, const void* g, const void* u_dense);
int launch_select_stream(void* g, int64_t ldg, int tokens, int d_ffn, int k, const SelectFuse& fuse, int16_t* idx,
                         void* g_sel, uint32_t* bitmap, uint16_t* rank0, int* status, cudaStream_t stream);
int launch_topk_select(int dtype, void* g, int64_t ldg, int tokens, int d_ffn, int k, const SelectFuse* fuse,
                       int16_t* idx, void* g_sel, uint32_t* bitmap, uint16_t* rank0, cudaStream_t stream);
int launch_select_2of8(int dtype, void* g, int64_t ldg, int tokens, int d_ffn, const SelectFuse* fuse, int16_t* idx,
                       void* g_sel, uint32_t* bitmap, uint16_t* rank0, cudaStream_t stream);
// score[i] = |round(SiLU(g[i]))| over `elems` elements (a multiple of 128), the selection key of the post-SiLU mode
int launch_abs_silu(int dtype, const void* g, void* score, int64_t elems, cudaStream_t stream);
// after a selection on another tensor: compact g_sel, u_sel (+ s_sel, z_sel) from the dense rows; the dense gate
// rows become Z'
int launch_post_gather(int dtype, const int16_t* idx, void* g_dense, const void* u_dense, void* g_sel, void* u_sel,
                       void* s_sel, void* z_sel, int64_t ld, int tokens, int k, cudaStream_t stream);
// dZ[tokens, ld] (in) -> dG' (grad_g_out) and dU' (written over dZ in place): gather, SiLU', zero fill. z_dense set:
// also Z'[tokens, ld], the zero-filled scatter of z_sel (or of round(round(SiLU(g)) * u) when z_sel is null)
int launch_bwd_sparse(int dtype, const int16_t* idx, const void* g_sel, const void* u_sel, const void* z_sel,
                      void* dz_to_du, void* grad_g_out, void* z_dense, int64_t ld, int tokens, int d_ffn, int k,
                      cudaStream_t stream);
// dense SwiGLU backward, elementwise over tokens * ld elements (a multiple of 128)
int launch_dense_bwd(int dtype, const void* g, const void* u, void* dz_to_du, void* z_out, void* grad_g_out,
                     int64_t elems, cudaStream_t stream);
// out[cols, rows] <- in[rows, cols]^T
int launch_transpose(int dtype, const void* in, int64_t ld_in, void* out, int64_t ld_out, int rows, int cols,
                     cudaStream_t stream);

// Optional per-kernel timing: while a profile is active (moc_profile_begin), every launcher
// records the next caller-provided event right before its kernel launch, tagged with the
// kernel kind; API entry points add an end marker. Intervals between consecutive events on
// one stream are the kernels' durations.
enum ProfTag : int {
  kProfEnd = 0, kProfGemmTc = 1, kProfGemmSimt = 2, kProfTopk = 3, kProfSel2of8 = 4, kProfExpand = 5,
  kProfTranspose = 6, kProfDecodeGate = 7, kProfDecodeUp = 8, kProfDecodeDown = 9, kProfDecodeFused28 = 10,
  kProfDecodeDense = 11, kProfBwdSparse = 12, kProfDecodeFused = 13,
};
void prof_mark(int tag, cudaStream_t stream);

// ---- decode path (decode.cu), bf16 only ---------------------------------------------------------
int64_t decode_workspace_bytes(int64_t batch, int64_t d, int64_t d_ffn);
// Single persistent launch for batches of up to 8 rows (decode_stream.cu): every CTA streams the W_gate, W_up and
// W_down^T rows of its own channels through a shared-memory ring. rule 0: Top-K, 1: 2-of-8, 2: dense baseline.
// g_scratch: [batch, ld] bf16; hist: [batch, 2048] ints directly behind the 256-byte status area (status word at
// [0], barrier counter at [32]); partial: decode_stream_partial_bytes(batch, d) bytes.
bool decode_stream_supported(int64_t batch, int64_t d, int64_t d_ffn, int rule);
int64_t decode_stream_partial_bytes(int64_t batch, int64_t d);
int launch_decode_stream(int rule, int batch, int d, int d_ffn, int k, const void* x, const void* scores,
                         int64_t ld_scores, const void* w_gate, const void* w_up, const void* w_down_t, void* y,
                         void* g_scratch, int64_t ld, int* hist, int* status_area, float* partial,
                         cudaStream_t stream);
// limit (cycles) of the bounded grid-barrier waits of the persistent decode kernel; <= 0 restores the default
void decode_stream_set_wait_cycles(long long cycles);
// rule 0: global Top-K, 1: 2-of-8. gate_scores != null: use the caller's [batch, d_ffn] scores instead of x * W_gate^T
int decode_selected_up(int64_t batch, int64_t k, int64_t d, const void* x, const void* g_sel, const int16_t* idx,
                       const void* w_up, void* z, cudaStream_t stream);
int decode_global(int64_t batch, int64_t d, int64_t d_ffn, int64_t k, int rule, const void* x, const void* gate_scores,
                  const void* w_gate, const void* w_up, const void* w_down_t, void* y, void* workspace,
                  int64_t workspace_bytes, cudaStream_t stream);
int decode_dense(int64_t batch, int64_t d, int64_t d_ffn, const void* x, const void* w_gate, const void* w_up,
                 const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes, cudaStream_t stream);
int decode_selected_down(int64_t batch, int64_t k, int64_t d, int64_t d_ffn, const void* z, const int16_t* idx,
                         const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes, cudaStream_t stream);

int check_last(const char* what);
const char* last_error_text();
void set_error(const char* fmt, ...);

}  // namespace moc
