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
// The sparse forward epilogue is where the MoC-specific work is fused into the up-projection
// GEMM; it replaces sparse_forward_aux of the reference
// (moc/training/triton_sparse_aux.py:17-49, :197-231) and never writes a full U to HBM.
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
};

template <typename T>
__device__ __forceinline__ void chunk_load(const T* p, float (&v)[32]) {
  uint4 q[Chunk32<T>::kVecs];
  Chunk32<T>::load_raw(p, q);
  Chunk32<T>::unpack(q, v);
}

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

// ---- forward: up projection -> selected activations -------------------------------------
// acc = U tile. The selection kernel has already replaced the dense gate row by
// S' = mask * round(SiLU(G)) (zero outside the selected channels, moc/ffn.py:157), so the
// epilogue is branch-free dense math: u = round(U), z = round(S' * u) (moc/ffn.py:158),
// written over the S' chunk in place as the zero-filled Z' chunk that the down projection
// consumes (moc/ffn.py:160-163). The selected u (and on request s, z) also go to the
// compact per-token arrays at the channel's rank (moc/ffn.py:156, :166-169). Mask words and
// ranks of the whole run are fetched in begin(); the S' chunk is fetched in prefetch(),
// while the accumulator load is in flight.
template <typename T>
struct EpiUpSparse {
  struct Ctx {
    uint32_t word[kEpiMaxChunks];
    uint32_t rank[kEpiMaxChunks];
    uint4 s[Chunk32<T>::kVecs];
  };
  T* sz;                    // in: S' [tokens, ld]; out: Z' [tokens, ld]
  int64_t ld;
  const uint32_t* bitmap;   // [tokens, words], words % 4 == 0
  const uint16_t* rank0;    // [tokens, words] rank of the first channel of each word
  int words;
  int k;
  T* u_sel;                 // [tokens, k]
  T* s_sel;                 // [tokens, k] or null
  T* z_sel;                 // [tokens, k] or null

  __device__ __forceinline__ void begin(Ctx& ctx, int, int row, int col_first, int nchunks) const {
    const int w0 = col_first >> 5;
    const uint32_t* bw = bitmap + static_cast<int64_t>(row) * words + w0;
    const uint16_t* rk = rank0 + static_cast<int64_t>(row) * words + w0;
    if ((w0 & 3) == 0) {   // aligned run of four words: one 16-byte and one 8-byte load
      const uint4 b = *reinterpret_cast<const uint4*>(bw);
      const uint2 r = *reinterpret_cast<const uint2*>(rk);
      ctx.word[0] = b.x; ctx.word[1] = b.y; ctx.word[2] = b.z; ctx.word[3] = b.w;
      ctx.rank[0] = r.x & 0xFFFFu; ctx.rank[1] = r.x >> 16; ctx.rank[2] = r.y & 0xFFFFu; ctx.rank[3] = r.y >> 16;
    } else {
#pragma unroll
      for (int c = 0; c < kEpiMaxChunks; ++c) {
        ctx.word[c] = (c < nchunks) ? bw[c] : 0u;
        ctx.rank[c] = (c < nchunks) ? rk[c] : 0u;
      }
    }
  }
  __device__ __forceinline__ void prefetch(Ctx& ctx, int row, int col0, int c) const {
    if (ctx.word[c] != 0u) Chunk32<T>::load_raw(sz + static_cast<int64_t>(row) * ld + col0, ctx.s);
  }
  __device__ __forceinline__ void operator()(Ctx& ctx, int, int row, int col0, int c, const float (&acc)[32]) const {
    const uint32_t word = ctx.word[c];
    T* chunk = sz + static_cast<int64_t>(row) * ld + col0;
    if (word == 0u) return;   // the S' chunk is all zero already and stays the Z' chunk
    float s[32], out[32];
    Chunk32<T>::unpack(ctx.s, s);
#pragma unroll
    for (int j = 0; j < 32; ++j) out[j] = Num<T>::round(s[j] * Num<T>::round(acc[j]));
    Chunk32<T>::store(chunk, out);
    T* up = u_sel + static_cast<int64_t>(row) * k + ctx.rank[c];
    T* sp = s_sel ? s_sel + static_cast<int64_t>(row) * k + ctx.rank[c] : nullptr;
    T* zp = z_sel ? z_sel + static_cast<int64_t>(row) * k + ctx.rank[c] : nullptr;
    int pos = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if ((word >> j) & 1u) {
        up[pos] = Num<T>::from_float(acc[j]);
        if (sp) sp[pos] = Num<T>::from_float(s[j]);
        if (zp) zp[pos] = Num<T>::from_float(out[j]);
        ++pos;
      }
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
    for (int j = 0; j < 32; ++j) {
      u[j] = Num<T>::round(acc[j]);
      float s;
      moc_fwd_point<T>(gv[j], u[j], s, out[j]);
    }
    Chunk32<T>::store(u_out + static_cast<int64_t>(row) * ld + col0, u);
    Chunk32<T>::store(z_out + static_cast<int64_t>(row) * ld + col0, out);
  }
};

}  // namespace moc
