// Epilogue functors shared by the tcgen05 GEMM core (bf16) and the SIMT GEMM core
// (fp32). A functor is called by one thread with one output row and 32 consecutive
// columns [col0, col0 + 32), col0 % 32 == 0, row < M, col0 < N; acc[j] is the fp32
// accumulator of column col0 + j (zero for columns >= N).
//
// The sparse epilogues are where the MoC-specific work is fused into the GEMMs; they
// replace the gather / scatter helper kernels of the reference
// (moc/training/triton_sparse_aux.py:17-182) and never write a full U or dZ to HBM.
#pragma once

#include "common.cuh"

namespace moc {

// ---- 32-element row-chunk load / store ------------------------------------------------
template <typename T> struct Chunk32;

template <> struct Chunk32<__nv_bfloat16> {
  // p must be 16-byte aligned
  __device__ __forceinline__ static void load(const __nv_bfloat16* p, float (&v)[32]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 w = q[i];
      const uint32_t a[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i * 8 + 2 * j] = __uint_as_float(a[j] << 16);
        v[i * 8 + 2 * j + 1] = __uint_as_float(a[j] & 0xFFFF0000u);
      }
    }
  }
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
};

template <> struct Chunk32<float> {
  __device__ __forceinline__ static void load(const float* p, float (&v)[32]) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 w = q[i];
      v[4 * i] = w.x; v[4 * i + 1] = w.y; v[4 * i + 2] = w.z; v[4 * i + 3] = w.w;
    }
  }
  __device__ __forceinline__ static void store(float* p, const float (&v)[32]) {
    float4* q = reinterpret_cast<float4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  }
};

// ---- plain store: C[row, col] (or C[col, row] when transposed) --------------------------
template <typename T>
struct EpiStore {
  T* c;
  int64_t ldc;
  int n;            // valid columns
  int transposed;   // 1: write C[col * ldc + row]
  int vec_ok;       // 1: rows of C are 16-byte aligned at every col0 (checked on the host)

  __device__ __forceinline__ void operator()(int row, int col0, const float (&acc)[32]) const {
    const int ncols = min(32, n - col0);
    if (transposed) {
      T* p = c + static_cast<int64_t>(col0) * ldc + row;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) p[static_cast<int64_t>(j) * ldc] = Num<T>::from_float(acc[j]);
      return;
    }
    T* p = c + static_cast<int64_t>(row) * ldc + col0;
    if (vec_ok && ncols == 32) {
      Chunk32<T>::store(p, acc);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) p[j] = Num<T>::from_float(acc[j]);
    }
  }
};

// ---- forward: up projection -> selected activations -------------------------------------
// acc = U tile. For every selected channel (bit set in the row's bitmap) computes
// u = round(U), s = round(SiLU(g)), z = round(s * u) (moc/ffn.py:156-158), writes them
// to the compact per-token arrays at the channel's rank, and overwrites the dense G
// chunk in place with the zero-filled Z' chunk that the down projection consumes
// (moc/ffn.py:160-163).
template <typename T>
struct EpiUpSparse {
  T* gz;                    // in: G [tokens, ld]; out: Z' [tokens, ld]
  int64_t ld;
  const uint32_t* bitmap;   // [tokens, words]
  const uint16_t* rank0;    // [tokens, words] rank of the first channel of each word
  int words;
  int k;
  T* u_sel;                 // [tokens, k]
  T* s_sel;                 // [tokens, k] or null
  T* z_sel;                 // [tokens, k] or null

  __device__ __forceinline__ void operator()(int row, int col0, const float (&acc)[32]) const {
    const int w = col0 >> 5;
    const uint32_t word = bitmap[static_cast<int64_t>(row) * words + w];
    T* chunk = gz + static_cast<int64_t>(row) * ld + col0;
    float out[32];
    if (word == 0u) {
#pragma unroll
      for (int j = 0; j < 32; ++j) out[j] = 0.0f;
      Chunk32<T>::store(chunk, out);
      return;
    }
    float g[32];
    Chunk32<T>::load(chunk, g);
    const int base = rank0[static_cast<int64_t>(row) * words + w];
    const int64_t crow = static_cast<int64_t>(row) * k;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      out[j] = 0.0f;
      if ((word >> j) & 1u) {
        const int pos = base + __popc(word & ((1u << j) - 1u));
        const float u = Num<T>::round(acc[j]);
        float s, z;
        moc_fwd_point<T>(g[j], u, s, z);
        u_sel[crow + pos] = Num<T>::from_float(u);
        if (s_sel) s_sel[crow + pos] = Num<T>::from_float(s);
        if (z_sel) z_sel[crow + pos] = Num<T>::from_float(z);
        out[j] = z;
      }
    }
    Chunk32<T>::store(chunk, out);
  }
};

// ---- backward: dZ = dY * W_down -> dense zero-filled dG', dU' ---------------------------
// acc = dZ tile. For every selected channel: gz = round(dZ), grad_s = round(u * gz),
// grad_u = round(s * gz), grad_g = round(grad_s * SiLU'(g)) with SiLU' rounded step by
// step as the reference does (moc/ffn.py:219-237, moc/training/triton_sparse_aux.py:376-400).
// With s_sel == null (moc_gcp) s is recomputed from g (moc/ffn.py:435).
template <typename T>
struct EpiBwdSparse {
  T* grad_g;                // [tokens, ld] dense out
  T* grad_u;                // [tokens, ld] dense out
  int64_t ld;
  const uint32_t* bitmap;
  const uint16_t* rank0;
  int words;
  int k;
  const T* g_sel;
  const T* u_sel;
  const T* s_sel;           // null -> recompute

  __device__ __forceinline__ void operator()(int row, int col0, const float (&acc)[32]) const {
    const int w = col0 >> 5;
    const uint32_t word = bitmap[static_cast<int64_t>(row) * words + w];
    T* pg = grad_g + static_cast<int64_t>(row) * ld + col0;
    T* pu = grad_u + static_cast<int64_t>(row) * ld + col0;
    float og[32], ou[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) { og[j] = 0.0f; ou[j] = 0.0f; }
    if (word != 0u) {
      const int base = rank0[static_cast<int64_t>(row) * words + w];
      const int64_t crow = static_cast<int64_t>(row) * k;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if ((word >> j) & 1u) {
          const int pos = base + __popc(word & ((1u << j) - 1u));
          const float g = Num<T>::to_float(g_sel[crow + pos]);
          const float u = Num<T>::to_float(u_sel[crow + pos]);
          const float s = s_sel ? Num<T>::to_float(s_sel[crow + pos]) : Num<T>::round(silu_f32(g));
          const float gz = Num<T>::round(acc[j]);
          moc_bwd_point<T>(g, u, s, gz, og[j], ou[j]);
        }
      }
    }
    Chunk32<T>::store(pg, og);
    Chunk32<T>::store(pu, ou);
  }
};

// ---- dense SwiGLU forward: acc = U tile, Z = round(round(SiLU(G)) * round(U)) ------------
// (moc/ffn.py:120-121). Overwrites G in place with Z and keeps U for the backward pass.
template <typename T>
struct EpiDenseSwiGLU {
  T* gz;       // in: G, out: Z
  T* u_out;    // U (saved for backward) or null
  int64_t ld;

  __device__ __forceinline__ void operator()(int row, int col0, const float (&acc)[32]) const {
    T* chunk = gz + static_cast<int64_t>(row) * ld + col0;
    float g[32], out[32], u[32];
    Chunk32<T>::load(chunk, g);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      u[j] = Num<T>::round(acc[j]);
      float s, z;
      moc_fwd_point<T>(g[j], u[j], s, z);
      out[j] = z;
    }
    if (u_out) Chunk32<T>::store(u_out + static_cast<int64_t>(row) * ld + col0, u);
    Chunk32<T>::store(chunk, out);
  }
};

}  // namespace moc
