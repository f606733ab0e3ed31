// Epilogue functors shared by the tcgen05 GEMM core (bf16) and the CUDA-core GEMM core
// (fp32). One thread owns one output row and walks a run of 32-column chunks of it:
//
//   Ctx ctx;                                         per-thread state for the run
//   epi.begin(ctx, group, row, col_first, nchunks);  issue loads needed by the whole run
//   for c in [0, nchunks):  col0 = col_first + 32 * c
//     epi.prefetch(ctx, row, col0, c);               issue global loads of chunk c (the
//                                                    accumulator load is still in flight)
//     epi(ctx, group, row, col0, c, acc);            acc[j] = fp32 accumulator of column col0 + j
//
// with col0 % 32 == 0, row < M, col0 < N, nchunks <= 4, and acc zero for columns >= N.
// `group` is the problem index of a grouped launch (0 otherwise).
//
// Epilogues are kept to dense, branch-free, vectorised work: an epilogue warp is a serial
// instruction stream next to the tensor pipe, and measured on B200 every per-element branch,
// scalar f32->bf16 conversion (XU pipe) or 2-byte store in it shows up one-to-one in the GEMM's
// duration. All index-dependent work (gather / scatter by selected channel) is done by the
// row kernels in kernels.cu.
#pragma once

#include "common.cuh"

namespace moc {

constexpr int kMaxGroups = 3;
constexpr int kEpiMaxChunks = 4;

// ---- 32-element row-chunk load / store ------------------------------------------------
template <typename T> struct Chunk32;

template <> struct Chunk32<__nv_bfloat16> {
  static constexpr int kVecs = 4;   // 16-byte vectors per chunk
  __device__ __forceinline__ static void unpack(const uint4 (&q)[4], float (&v)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t a[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i * 8 + 2 * j] = __uint_as_float(a[j] << 16);
        v[i * 8 + 2 * j + 1] = __uint_as_float(a[j] & 0xFFFF0000u);
      }
    }
  }
  // p must be 16-byte aligned
  __device__ __forceinline__ static void load_raw(const __nv_bfloat16* p, uint4 (&q)[4]) {
    const uint4* s = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = s[i];
  }
  // rounds to nearest even with packed conversions
  __device__ __forceinline__ static void store(__nv_bfloat16* p, const float (&v)[32]) {
    uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t a[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[i * 8 + 2 * j], v[i * 8 + 2 * j + 1]);
        a[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      q[i] = make_uint4(a[0], a[1], a[2], a[3]);
    }
  }
  // values already representable in bf16: pure bit packing, no conversion instruction
  __device__ __forceinline__ static void store_rounded(__nv_bfloat16* p, const float (&v)[32]) {
    uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t a[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        a[j] = (__float_as_uint(v[i * 8 + 2 * j]) >> 16) | (__float_as_uint(v[i * 8 + 2 * j + 1]) & 0xFFFF0000u);
      q[i] = make_uint4(a[0], a[1], a[2], a[3]);
    }
  }
};

template <> struct Chunk32<float> {
  static constexpr int kVecs = 8;
  __device__ __forceinline__ static void unpack(const uint4 (&q)[8], float (&v)[32]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[4 * i] = __uint_as_float(q[i].x);
      v[4 * i + 1] = __uint_as_float(q[i].y);
      v[4 * i + 2] = __uint_as_float(q[i].z);
      v[4 * i + 3] = __uint_as_float(q[i].w);
    }
  }
  __device__ __forceinline__ static void load_raw(const float* p, uint4 (&q)[8]) {
    const uint4* s = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = s[i];
  }
  __device__ __forceinline__ static void store(float* p, const float (&v)[32]) {
    float4* q = reinterpret_cast<float4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  }
  __device__ __forceinline__ static void store_rounded(float* p, const float (&v)[32]) { store(p, v); }
};

// ---- plain store: C[row, col] (or C[col, row] when transposed), one C per group ------------
template <typename T>
struct EpiStore {
  struct Ctx {};
  T* c[kMaxGroups];
  int64_t ldc[kMaxGroups];
  int transposed[kMaxGroups];   // 1: write C[col * ldc + row]
  int vec_ok[kMaxGroups];       // 1: rows of C are 16-byte aligned at every col0 (checked on the host)
  int n;                        // valid columns

  __device__ __forceinline__ void begin(Ctx&, int, int, int, int) const {}
  __device__ __forceinline__ void prefetch(Ctx&, int, int, int) const {}
  __device__ __forceinline__ void operator()(Ctx&, int group, int row, int col0, int, const float (&acc)[32]) const {
    const int ncols = min(32, n - col0);
    T* base = c[group];
    const int64_t ld = ldc[group];
    if (transposed[group]) {
      T* p = base + static_cast<int64_t>(col0) * ld + row;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) p[static_cast<int64_t>(j) * ld] = Num<T>::from_float(acc[j]);
      return;
    }
    T* p = base + static_cast<int64_t>(row) * ld + col0;
    if (vec_ok[group] && ncols == 32) {
      Chunk32<T>::store(p, acc);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) p[j] = Num<T>::from_float(acc[j]);
    }
  }
};

// ---- split-K partial results: fp32 accumulator rows, one [m, ld] block per (group, split) -----------
// A reduction kernel adds the blocks of a group in a fixed order and rounds once (splitk_reduce_kernel).
template <typename T>
struct EpiPartialF32 {
  struct Ctx {};
  float* p;               // [groups * splits][m][ld]
  int64_t ld;             // floats per row, a multiple of 4
  int64_t block_stride;   // m * ld
  int n;

  __device__ __forceinline__ void begin(Ctx&, int, int, int, int) const {}
  __device__ __forceinline__ void prefetch(Ctx&, int, int, int) const {}
  __device__ __forceinline__ void operator()(Ctx&, int group, int row, int col0, int, const float (&acc)[32]) const {
    float* dst = p + group * block_stride + static_cast<int64_t>(row) * ld + col0;
    const int ncols = min(32, n - col0);
    if (ncols == 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) dst[j] = acc[j];
    }
  }
};

// ---- dense SwiGLU forward: acc = U tile, Z = round(round(SiLU(G)) * round(U)) ------------
// (moc/ffn.py:120-121). Reads G, writes U (kept for the backward pass) and Z.
template <typename T>
struct EpiDenseSwiGLU {
  struct Ctx {
    uint4 g[Chunk32<T>::kVecs];
  };
  const T* g;   // [tokens, ld]
  T* u_out;     // [tokens, ld]
  T* z_out;     // [tokens, ld]
  int64_t ld;

  __device__ __forceinline__ void begin(Ctx&, int, int, int, int) const {}
  __device__ __forceinline__ void prefetch(Ctx& ctx, int row, int col0, int) const {
    Chunk32<T>::load_raw(g + static_cast<int64_t>(row) * ld + col0, ctx.g);
  }
  __device__ __forceinline__ void operator()(Ctx& ctx, int, int row, int col0, int, const float (&acc)[32]) const {
    float gv[32], out[32], u[32];
    Chunk32<T>::unpack(ctx.g, gv);
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      u[j] = acc[j];
      u[j + 1] = acc[j + 1];
      Num<T>::round_pair(u[j], u[j + 1]);
      float s0 = gv[j] * sigmoid_act<T>(gv[j]), s1 = gv[j + 1] * sigmoid_act<T>(gv[j + 1]);
      Num<T>::round_pair(s0, s1);
      out[j] = s0 * u[j];
      out[j + 1] = s1 * u[j + 1];
    }
    const int64_t off = static_cast<int64_t>(row) * ld + col0;
    Chunk32<T>::store_rounded(u_out + off, u);
    Chunk32<T>::store(z_out + off, out);
  }
};

}  // namespace moc
