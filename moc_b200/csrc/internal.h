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

enum EpiKind : int { kEpiStore = 0, kEpiUpSparse = 1, kEpiBwdSparse = 2, kEpiDenseSwiGLU = 3 };

struct EpiArgs {
  int kind;
  // kEpiStore
  void* c;
  int64_t ldc;
  int transposed;
  // sparse epilogues / dense SwiGLU
  void* dense0;             // up: G -> Z' in place; bwd: dG'; dense: G -> Z
  void* dense1;             // bwd: dU'; dense: U out (or null)
  int64_t ld_dense;
  const uint32_t* bitmap;
  const uint16_t* rank0;
  int words;
  int k_sel;
  void* u_sel;
  void* s_sel;
  void* z_sel;
  const void* g_sel;
};

struct GemmProblem {
  int dtype;                 // DType
  int impl;                  // 0: default for the dtype (bf16 -> tcgen05, f32 -> SIMT); 1: force SIMT
  int m, n;
  int k0;                    // K extent of segment 0
  MatOperand a0, b0;
  int k1;                    // K extent of segment 1 (0: none)
  MatOperand a1, b1;
  EpiArgs epi;
  int* status;               // device status word (may be null for SIMT)
};

int launch_gemm(const GemmProblem& p, cudaStream_t stream);

// ---- selection / auxiliary kernels (kernels.cu) ---------------------------------------------
int launch_topk_select(int dtype, const void* g, int64_t ldg, int tokens, int d_ffn, int k, int16_t* idx,
                       void* g_sel, uint32_t* bitmap, uint16_t* rank0, cudaStream_t stream);
int launch_select_2of8(int dtype, const void* g, int64_t ldg, int tokens, int d_ffn, int16_t* idx, void* g_sel,
                       uint32_t* bitmap, uint16_t* rank0, cudaStream_t stream);
// Z'[tokens, ld] <- zero-filled scatter of the compact z (or of round(round(SiLU(g)) * u) when z_sel is null)
int launch_expand_z(int dtype, const uint32_t* bitmap, const uint16_t* rank0, const void* z_sel, const void* g_sel,
                    const void* u_sel, void* dense, int64_t ld, int tokens, int d_ffn, int k, cudaStream_t stream);
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
  kProfDecodeDense = 11,
};
void prof_mark(int tag, cudaStream_t stream);

int check_last(const char* what);
const char* last_error_text();
void set_error(const char* fmt, ...);

}  // namespace moc
