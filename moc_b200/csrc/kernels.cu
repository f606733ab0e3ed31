// Channel selection and layout kernels of the MoC FFN path (HBM-bound integer/byte work).
//
//   topk_select_kernel : row-wise Top-K over d_ffn pre-SiLU gate values. Replaces
//                        torch.topk (moc/ffn.py:144, :392) and the CUB block sort of the decode
//                        extension (moc/inference/cuda/optimized_global_moc_ext.cu:85-125) by a
//                        radix *select*: one warp per token finds the K-th largest order key
//                        digit by digit (11-bit shared-memory histograms), ties at the threshold
//                        go to the lower channel index, and the selected set is emitted in
//                        ascending channel order together with a bitmap. On request the same
//                        kernel gathers the selected channels of the dense U rows into the compact
//                        saved set and overwrites the gate row by Z' = mask * round(SiLU(G)) * U,
//                        the operand of the down projection (moc/ffn.py:156-163).
//   select_2of8_kernel : structured top-2 of every 8 consecutive channels (moc/ffn.py:68-108).
//   bwd_sparse_kernel  : dense dZ -> zero-filled dense dG', dU' through the selected channels
//                        (moc/ffn.py:219-237, moc/training/triton_sparse_aux.py:363-423), and compact z ->
//                        zero-filled dense Z' (moc/ffn.py:196-199, :435-442) in the same pass.
//   transpose_kernel   : W_down [d, F] <-> W_down^T [F, d] (moc/inference/inference_ffn.py:104-110).
#include <cuda_bf16.h>
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"
#include "internal.h"

namespace moc {

// ------------------------------------------------------------------------------------------
// key traits
// ------------------------------------------------------------------------------------------
template <typename T> struct KeyTraits;
template <> struct KeyTraits<__nv_bfloat16> {
  using Bits = uint16_t;
  static constexpr int kBits = 16;
  __device__ __forceinline__ static uint32_t key(uint32_t b) { return order_key16(static_cast<uint16_t>(b)); }
  __device__ __forceinline__ static float value(Bits b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
  __device__ __forceinline__ static Bits bits(float v) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    return *reinterpret_cast<const Bits*>(&h);
  }
};
template <> struct KeyTraits<float> {
  using Bits = uint32_t;
  static constexpr int kBits = 32;
  __device__ __forceinline__ static uint32_t key(uint32_t b) { return order_key32(b); }
  __device__ __forceinline__ static float value(Bits b) { return __uint_as_float(b); }
  __device__ __forceinline__ static Bits bits(float v) { return __float_as_uint(v); }
};

constexpr int kSelWarpsPerCta = 8;
constexpr int kSelHistWords = 1024;   // 2048 bins of 16 bits, two per word

__device__ __forceinline__ uint32_t hist_count(const uint32_t* hist, int b) {
  return (hist[b >> 1] >> ((b & 1) * 16)) & 0xFFFFu;
}

// Forward fusion of the selection kernels. With u_dense set (rows of ldg elements like g), a kernel
// also gathers u = U[row, ch] of every selected channel, stores it in the compact saved set (with
// s = round(SiLU(g)) and z = round(s * u) on request) and overwrites the row of g in place by
// Z' = selected ? z : 0 over the full padded width 32 * words (moc/ffn.py:156-161).
template <typename T>
struct SelFuseT {
  const T* u_dense;
  T* u_sel;
  T* s_sel;
  T* z_sel;
};

// One selected channel: returns the bits of z for the dense row, writes the compact outputs.
template <typename T>
__device__ __forceinline__ typename KeyTraits<T>::Bits fuse_point(const SelFuseT<T>& f, int64_t dense_off,
                                                                  int64_t compact_off, float gv) {
  const T u = f.u_dense[dense_off];
  float sv, zv;
  moc_fwd_point<T>(gv, Num<T>::to_float(u), sv, zv);
  f.u_sel[compact_off] = u;
  if (f.s_sel) f.s_sel[compact_off] = Num<T>::from_float(sv);
  const T z = Num<T>::from_float(zv);
  if (f.z_sel) f.z_sel[compact_off] = z;
  return *reinterpret_cast<const typename KeyTraits<T>::Bits*>(&z);
}

// One warp per token row; lane l handles the channels l, l + 32, l + 64, ... so that a warp
// ballot over one step is exactly one 32-channel word of the selection bitmap and channel
// order equals (step, lane) order.
template <typename T>
__global__ void __launch_bounds__(kSelWarpsPerCta * 32)
topk_select_kernel(T* __restrict__ g, int64_t ldg, int tokens, int d_ffn, int k, int words, SelFuseT<T> fuse,
                   int16_t* __restrict__ idx, T* __restrict__ g_sel, uint32_t* __restrict__ bitmap,
                   uint16_t* __restrict__ rank0) {
  using KT = KeyTraits<T>;
  using Bits = typename KT::Bits;
  __shared__ uint32_t hist_all[kSelWarpsPerCta][kSelHistWords];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kSelWarpsPerCta + warp;
  if (row >= tokens) return;   // whole warps leave; no block-wide barrier is used below
  uint32_t* hist = hist_all[warp];
  Bits* grow = reinterpret_cast<Bits*>(g) + static_cast<int64_t>(row) * ldg;
  const uint32_t lt_mask = (1u << lane) - 1u;

  // ---- K-th largest key, one digit per pass, most significant first ----
  uint32_t prefix = 0, prefix_mask = 0, k_rem = static_cast<uint32_t>(k);
  int hi_bit = KT::kBits;
#pragma unroll 1
  while (hi_bit > 0) {
    const int nbits = (hi_bit == 32) ? 11 : (hi_bit >= 11 ? 11 : hi_bit);   // 16: 11+5, 32: 11+11+10
    const int shift = hi_bit - nbits;
    const int nbins = 1 << nbits;
    for (int i = lane; i < (nbins >> 1); i += 32) hist[i] = 0u;
    __syncwarp();
#pragma unroll 4
    for (int c = lane; c < d_ffn; c += 32) {
      const uint32_t key = KT::key(grow[c]);
      if ((key & prefix_mask) == prefix) {
        const uint32_t b = (key >> shift) & (nbins - 1);
        atomicAdd(&hist[b >> 1], 1u << ((b & 1u) * 16));
      }
    }
    __syncwarp();
    // lane l owns the bins [lo, lo + per) counted from the top; `above` = keys in higher bins
    const int per = nbins >> 5;   // nbins >= 32
    const int lo = (31 - lane) * per;
    uint32_t local = 0;
    for (int b = 0; b < per; ++b) local += hist_count(hist, lo + b);
    uint32_t inc = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t nb = __shfl_up_sync(0xFFFFFFFFu, inc, o);
      if (lane >= o) inc += nb;
    }
    uint32_t above = inc - local;
    const bool mine = above < k_rem && above + local >= k_rem;
    uint32_t digit = 0, new_k = 0;
    if (mine) {
      for (int b = lo + per - 1; b >= lo; --b) {
        const uint32_t c = hist_count(hist, b);
        if (above + c >= k_rem) {
          digit = static_cast<uint32_t>(b);
          new_k = k_rem - above;
          break;
        }
        above += c;
      }
    }
    const int src = __ffs(__ballot_sync(0xFFFFFFFFu, mine)) - 1;   // exactly one lane
    digit = __shfl_sync(0xFFFFFFFFu, digit, src);
    k_rem = __shfl_sync(0xFFFFFFFFu, new_k, src);
    prefix |= digit << shift;
    prefix_mask |= static_cast<uint32_t>(nbins - 1) << shift;
    hi_bit = shift;
    __syncwarp();
  }
  const uint32_t thr = prefix;        // K-th largest key
  const uint32_t take_eq = k_rem;     // ties admitted, lowest channels first

  // ---- emit: one bitmap word per step ----
  int16_t* idx_row = idx + static_cast<int64_t>(row) * k;
  Bits* gsel_row = reinterpret_cast<Bits*>(g_sel) + static_cast<int64_t>(row) * k;
  uint32_t* bm_row = bitmap + static_cast<int64_t>(row) * words;
  uint16_t* rk_row = rank0 + static_cast<int64_t>(row) * words;
  uint32_t run = 0, eq_seen = 0;
#pragma unroll 2
  for (int w = 0; w < words; ++w) {
    const int c = w * 32 + lane;
    const bool valid = c < d_ffn;
    const Bits raw = valid ? grow[c] : Bits(0);
    const uint32_t key = KT::key(raw);
    const bool is_eq = valid && key == thr;
    const uint32_t eq_ballot = __ballot_sync(0xFFFFFFFFu, is_eq);
    const bool sel = valid && (key > thr || (is_eq && eq_seen + __popc(eq_ballot & lt_mask) < take_eq));
    const uint32_t word = __ballot_sync(0xFFFFFFFFu, sel);
    Bits zbits = Bits(0);
    if (sel) {
      const uint32_t pos = run + __popc(word & lt_mask);
      idx_row[pos] = static_cast<int16_t>(c);
      gsel_row[pos] = raw;
      if (fuse.u_dense)
        zbits = fuse_point<T>(fuse, static_cast<int64_t>(row) * ldg + c, static_cast<int64_t>(row) * k + pos,
                              KT::value(raw));
    }
    if (fuse.u_dense) grow[c] = zbits;
    if (lane == 0) {
      bm_row[w] = word;
      rk_row[w] = static_cast<uint16_t>(run);
    }
    run += __popc(word);
    eq_seen += __popc(eq_ballot);
  }
}

// ------------------------------------------------------------------------------------------
// One CTA per token row, for calls with few rows (decode batches, tiny training batches) where one
// warp per row would leave the GPU idle and make the call as long as one warp's serial pass.
// Thread t owns the contiguous channels [t * chunk, (t + 1) * chunk), so thread order is channel order.
// ------------------------------------------------------------------------------------------
constexpr int kCtaSelThreads = 512;
constexpr int kCtaSelWarps = kCtaSelThreads / 32;
constexpr int kCtaSelBins = 2048;

__device__ __forceinline__ uint32_t cta_exscan(uint32_t v, uint32_t* wsum /*[kCtaSelWarps]*/, uint32_t& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= o) inc += nb;
  }
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  uint32_t woff = 0, tot = 0;
#pragma unroll
  for (int i = 0; i < kCtaSelWarps; ++i) {
    const uint32_t s = wsum[i];
    if (i < warp) woff += s;
    tot += s;
  }
  total = tot;
  __syncthreads();
  return woff + inc - v;
}

template <typename T>
__global__ void __launch_bounds__(kCtaSelThreads)
topk_select_cta_kernel(T* __restrict__ g, int64_t ldg, int d_ffn, int k, int words, SelFuseT<T> fuse,
                       int16_t* __restrict__ idx, T* __restrict__ g_sel, uint32_t* __restrict__ bitmap,
                       uint16_t* __restrict__ rank0) {
  using KT = KeyTraits<T>;
  using Bits = typename KT::Bits;
  extern __shared__ __align__(16) uint8_t cta_sel_smem[];
  uint32_t* hist = reinterpret_cast<uint32_t*>(cta_sel_smem);   // [kCtaSelBins]
  uint32_t* bm = hist + kCtaSelBins;                            // [words]
  Bits* raw = reinterpret_cast<Bits*>(bm + words);              // [d_ffn] raw bit patterns of the row
  __shared__ uint32_t wsum[kCtaSelWarps];
  __shared__ uint32_t found[2];
  const int row = blockIdx.x, tid = threadIdx.x;
  Bits* grow = reinterpret_cast<Bits*>(g) + static_cast<int64_t>(row) * ldg;
  for (int i = tid; i < d_ffn; i += kCtaSelThreads) raw[i] = grow[i];
  for (int w = tid; w < words; w += kCtaSelThreads) bm[w] = 0u;
  __syncthreads();

  // ---- K-th largest key, one digit per pass ----
  uint32_t prefix = 0, prefix_mask = 0, k_rem = static_cast<uint32_t>(k);
  int hi_bit = KT::kBits;
#pragma unroll 1
  while (hi_bit > 0) {
    const int nbits = (hi_bit == 32) ? 11 : (hi_bit >= 11 ? 11 : hi_bit);
    const int shift = hi_bit - nbits;
    const int nbins = 1 << nbits;
    for (int b = tid; b < nbins; b += kCtaSelThreads) hist[b] = 0u;
    __syncthreads();
    for (int i = tid; i < d_ffn; i += kCtaSelThreads) {
      const uint32_t key = KT::key(raw[i]);
      if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & (nbins - 1)], 1u);
    }
    __syncthreads();
    const int per = nbins >= kCtaSelThreads ? nbins / kCtaSelThreads : 1;
    const int lo = (kCtaSelThreads - 1 - tid) * per;   // bins counted from the top
    uint32_t local = 0;
    if (lo < nbins)
      for (int b = 0; b < per; ++b) local += hist[lo + b];
    uint32_t total = 0;
    uint32_t above = cta_exscan(local, wsum, total);
    if (lo < nbins && above < k_rem && above + local >= k_rem) {
      for (int b = lo + per - 1; b >= lo; --b) {
        const uint32_t c = hist[b];
        if (above + c >= k_rem) {
          found[0] = static_cast<uint32_t>(b);
          found[1] = k_rem - above;
          break;
        }
        above += c;
      }
    }
    __syncthreads();
    prefix |= found[0] << shift;
    prefix_mask |= static_cast<uint32_t>(nbins - 1) << shift;
    k_rem = found[1];
    hi_bit = shift;
  }
  const uint32_t thr = prefix, take_eq = k_rem;

  // ---- emit ----
  const int chunk = (d_ffn + kCtaSelThreads - 1) / kCtaSelThreads;
  const int begin = min(tid * chunk, d_ffn), end = min(begin + chunk, d_ffn);
  uint32_t n_gt = 0, n_eq = 0;
  for (int i = begin; i < end; ++i) {
    const uint32_t key = KT::key(raw[i]);
    n_gt += (key > thr) ? 1u : 0u;
    n_eq += (key == thr) ? 1u : 0u;
  }
  uint32_t total = 0;
  const uint32_t ex = cta_exscan(n_gt | (n_eq << 16), wsum, total);
  uint32_t eq_seen = ex >> 16;
  uint32_t pos = (ex & 0xFFFFu) + min(eq_seen, take_eq);
  int16_t* idx_row = idx + static_cast<int64_t>(row) * k;
  Bits* gsel_row = reinterpret_cast<Bits*>(g_sel) + static_cast<int64_t>(row) * k;
  for (int i = begin; i < end; ++i) {
    const Bits r = raw[i];
    const uint32_t key = KT::key(r);
    bool sel = key > thr;
    if (key == thr) {
      sel = eq_seen < take_eq;
      ++eq_seen;
    }
    Bits zbits = Bits(0);
    if (sel) {
      idx_row[pos] = static_cast<int16_t>(i);
      gsel_row[pos] = r;
      if (fuse.u_dense)
        zbits = fuse_point<T>(fuse, static_cast<int64_t>(row) * ldg + i, static_cast<int64_t>(row) * k + pos,
                              KT::value(r));
      ++pos;
      atomicOr(&bm[i >> 5], 1u << (i & 31));
    }
    if (fuse.u_dense) grow[i] = zbits;
  }
  if (fuse.u_dense)
    for (int i = d_ffn + tid; i < words * 32; i += kCtaSelThreads) grow[i] = Bits(0);
  __syncthreads();
  const int wchunk = (words + kCtaSelThreads - 1) / kCtaSelThreads;
  const int wb = min(tid * wchunk, words), we = min(wb + wchunk, words);
  uint32_t pc = 0;
  for (int w = wb; w < we; ++w) pc += __popc(bm[w]);
  uint32_t tot2 = 0;
  uint32_t run = cta_exscan(pc, wsum, tot2);
  for (int w = wb; w < we; ++w) {
    const uint32_t m = bm[w];
    bitmap[static_cast<int64_t>(row) * words + w] = m;
    rank0[static_cast<int64_t>(row) * words + w] = static_cast<uint16_t>(run);
    run += __popc(m);
  }
}

// ------------------------------------------------------------------------------------------
// bf16 fast path of the Top-K selection: one warp per token, 16-byte loads of 8 channels per
// lane (vector v = slot * 32 + lane), packed 16-bit order keys. Needs 16-byte aligned rows padded
// to 32 * words elements.
// ------------------------------------------------------------------------------------------
constexpr int kVecSelWarps = 4;
constexpr int kVecSelBins = 2048;
constexpr int kVecSelHistWords = kVecSelBins / 2;   // 16-bit counters, two per word (a row has < 65536 channels)

__device__ __forceinline__ uint32_t keys2_from_bits(uint32_t x) {   // two bf16 patterns -> two order keys
  const uint32_t m = (x >> 15) & 0x00010001u;
  return x ^ 0x80008000u ^ (m * 0x7FFFu);
}
__device__ __forceinline__ uint32_t bits_from_key16(uint32_t key) {
  return (key & 0x8000u) ? (key ^ 0x8000u) : (key ^ 0xFFFFu);
}
__device__ __forceinline__ uint32_t warp_exscan(uint32_t v, uint32_t& total) {
  const int lane = threadIdx.x & 31;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= o) inc += nb;
  }
  total = __shfl_sync(0xFFFFFFFFu, inc, 31);
  return inc - v;
}

// Order keys of vector v of a padded row (8 channels, two per word); channels >= d_ffn get key 0,
// which is below every real key.
__device__ __forceinline__ void load_keys8(const uint4* grow4, int v, int nvec, int d_ffn, uint32_t (&a)[4]) {
  uint4 q = make_uint4(0u, 0u, 0u, 0u);
  if (v < nvec) q = grow4[v];
  a[0] = keys2_from_bits(q.x);
  a[1] = keys2_from_bits(q.y);
  a[2] = keys2_from_bits(q.z);
  a[3] = keys2_from_bits(q.w);
  const int nval = d_ffn - 8 * v;
  if (nval < 8) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (2 * j >= nval) a[j] = 0u;
      else if (2 * j + 1 >= nval) a[j] &= 0xFFFFu;
    }
  }
}

// The row is re-read for each of the three passes (two histogram passes, one emit pass); with
// a few warps per SM it stays in L1, so HBM sees it once. Loops are kept rolled: the kernel is
// issue-bound and a fully unrolled body thrashes the instruction cache.
__global__ void __launch_bounds__(kVecSelWarps * 32)
topk_select_bf16_vec_kernel(uint16_t* __restrict__ g, int64_t ldg, int tokens, int d_ffn, int k, int words,
                            SelFuseT<__nv_bfloat16> fuse, int16_t* __restrict__ idx, uint16_t* __restrict__ g_sel,
                            uint32_t* __restrict__ bitmap, uint16_t* __restrict__ rank0) {
  __shared__ uint32_t hist_all[kVecSelWarps][kVecSelHistWords];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kVecSelWarps + warp;
  if (row >= tokens) return;   // whole warps leave; only warp-level synchronisation below
  uint32_t* hist = hist_all[warp];
  uint16_t* grow = g + static_cast<int64_t>(row) * ldg;
  uint4* grow4 = reinterpret_cast<uint4*>(grow);
  const int nvec = words * 4;                       // 16-byte vectors in the padded row
  const int nslots = (nvec + 31) >> 5;              // vector v = slot * 32 + lane

  // ---- digit 1: the upper 11 key bits ----
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist);
    for (int i = lane; i < kVecSelHistWords / 4; i += 32) h4[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  __syncwarp();
#pragma unroll 2
  for (int i = 0; i < nslots; ++i) {
    const int v = i * 32 + lane;
    uint32_t a[4];
    load_keys8(grow4, v, nvec, d_ffn, a);
    if (v * 8 < d_ffn) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t b0 = (a[j] & 0xFFFFu) >> 5, b1 = a[j] >> 21;
        atomicAdd(&hist[b0 >> 1], (b0 & 1u) ? 0x10000u : 1u);
        atomicAdd(&hist[b1 >> 1], (b1 & 1u) ? 0x10000u : 1u);
      }
    }
  }
  __syncwarp();
  uint32_t k_rem = static_cast<uint32_t>(k);
  uint32_t digit1, digit2;
  {
    // lane l sums the 64 bins [lo, lo + 64) counted from the top = 32 words (rotated start: no bank conflicts)
    const int lo = (31 - lane) * 64;
    uint32_t local = 0;
#pragma unroll 8
    for (int j = 0; j < 32; ++j) {
      const uint32_t w = hist[(lo >> 1) + ((j + lane) & 31)];
      local += (w & 0xFFFFu) + (w >> 16);
    }
    uint32_t total;
    const uint32_t above = warp_exscan(local, total);
    const bool mine = above < k_rem && above + local >= k_rem;
    const int src = __ffs(__ballot_sync(0xFFFFFFFFu, mine)) - 1;
    const uint32_t above_src = __shfl_sync(0xFFFFFFFFu, above, src);
    const int top = (31 - src) * 64 + 63;            // highest bin of the owning range
    const uint32_t cw = hist[(top - 2 * lane) >> 1];              // bins top-2l (odd, upper half) and top-2l-1
    const uint32_t c0 = cw >> 16, c1 = cw & 0xFFFFu;
    const uint32_t ex = warp_exscan(c0 + c1, total) + above_src;
    const bool hit = ex < k_rem && ex + c0 + c1 >= k_rem;
    uint32_t d = 0, nk = 0;
    if (hit) {
      if (ex + c0 >= k_rem) { d = top - 2 * lane; nk = k_rem - ex; }
      else { d = top - 2 * lane - 1; nk = k_rem - ex - c0; }
    }
    const int src2 = __ffs(__ballot_sync(0xFFFFFFFFu, hit)) - 1;
    digit1 = __shfl_sync(0xFFFFFFFFu, d, src2);
    k_rem = __shfl_sync(0xFFFFFFFFu, nk, src2);
  }
  __syncwarp();

  // ---- digit 2: the lower 5 key bits of the keys that share digit 1 ----
  hist[lane] = 0u;
  __syncwarp();
#pragma unroll 2
  for (int i = 0; i < nslots; ++i) {
    uint32_t a[4];
    load_keys8(grow4, i * 32 + lane, nvec, d_ffn, a);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t lo16 = a[j] & 0xFFFFu, hi16 = a[j] >> 16;
      if ((lo16 >> 5) == digit1) atomicAdd(&hist[lo16 & 31u], 1u);
      if ((hi16 >> 5) == digit1) atomicAdd(&hist[hi16 & 31u], 1u);
    }
  }
  __syncwarp();
  {
    const uint32_t c = hist[31 - lane];
    uint32_t total;
    const uint32_t ex = warp_exscan(c, total);
    const bool hit = ex < k_rem && ex + c >= k_rem;
    const int src = __ffs(__ballot_sync(0xFFFFFFFFu, hit)) - 1;
    digit2 = 31 - src;
    k_rem = k_rem - __shfl_sync(0xFFFFFFFFu, ex, src);
  }
  const uint32_t thr = (digit1 << 5) | digit2;   // K-th largest key
  const uint32_t take_eq = k_rem;                // ties admitted, lowest channels first

  // ---- emit ----
  int16_t* idx_row = idx + static_cast<int64_t>(row) * k;
  uint16_t* gsel_row = g_sel + static_cast<int64_t>(row) * k;
  uint32_t* bm_row = bitmap + static_cast<int64_t>(row) * words;
  uint16_t* rk_row = rank0 + static_cast<int64_t>(row) * words;
  // fused forward: the U row is read with the same coalesced vectors as the gate row and the selected values
  // go to u_sel beside idx and g_sel, so that the compact pass below needs no scattered reads
  const uint4* urow4 = reinterpret_cast<const uint4*>(fuse.u_dense + static_cast<int64_t>(row) * ldg);
  uint16_t* usel_row = reinterpret_cast<uint16_t*>(fuse.u_sel) + static_cast<int64_t>(row) * k;
  uint32_t run = 0, eq_seen = 0;
#pragma unroll 1
  for (int i = 0; i < nslots; ++i) {
    const int v = i * 32 + lane;
    uint32_t a[4];
    load_keys8(grow4, v, nvec, d_ffn, a);
    uint4 uv = make_uint4(0u, 0u, 0u, 0u);
    if (fuse.u_dense && v < nvec) uv = urow4[v];
    const uint32_t ua[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t gtm = 0, eqm = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t lo16 = a[j] & 0xFFFFu, hi16 = a[j] >> 16;
      gtm |= (lo16 > thr ? 1u : 0u) << (2 * j);
      gtm |= (hi16 > thr ? 1u : 0u) << (2 * j + 1);
      eqm |= (lo16 == thr ? 1u : 0u) << (2 * j);
      eqm |= (hi16 == thr ? 1u : 0u) << (2 * j + 1);
    }
    uint32_t tot_eq, tot_sel;
    const uint32_t ex_eq = warp_exscan(__popc(eqm), tot_eq);
    const int allowed = static_cast<int>(take_eq) - static_cast<int>(eq_seen + ex_eq);
    uint32_t sel_eq = allowed > 0 ? eqm : 0u;
    while (static_cast<int>(__popc(sel_eq)) > allowed && sel_eq) sel_eq &= ~(0x80000000u >> __clz(sel_eq));
    const uint32_t selm = gtm | sel_eq;
    const uint32_t ex_sel = warp_exscan(__popc(selm), tot_sel);
    uint32_t b = selm << (8 * (lane & 3));
    b |= __shfl_xor_sync(0xFFFFFFFFu, b, 1);
    b |= __shfl_xor_sync(0xFFFFFFFFu, b, 2);
    const int widx = i * 8 + (lane >> 2);
    if ((lane & 3) == 0 && widx < words) {
      bm_row[widx] = b;
      rk_row[widx] = static_cast<uint16_t>(run + ex_sel);
    }
    uint32_t pos = run + ex_sel;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if ((selm >> j) & 1u) {
        const uint32_t key16 = (a[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
        idx_row[pos] = static_cast<int16_t>(8 * v + j);
        gsel_row[pos] = static_cast<uint16_t>(bits_from_key16(key16));
        if (fuse.u_dense) usel_row[pos] = static_cast<uint16_t>((ua[j >> 1] >> (16 * (j & 1))) & 0xFFFFu);
        ++pos;
      }
    }
    if (fuse.u_dense && v < nvec) grow4[v] = make_uint4(0u, 0u, 0u, 0u);   // selected channels: filled in below
    run += tot_sel;
    eq_seen += tot_eq;
  }

  // ---- Z' and the saved u (s, z) of the selected channels, computed in compact space (full lanes) ----
  if (fuse.u_dense) {
    __syncwarp();   // orders the zero fill and the compact outputs above before the accesses below
    uint16_t* ssel_row = fuse.s_sel ? reinterpret_cast<uint16_t*>(fuse.s_sel) + static_cast<int64_t>(row) * k : nullptr;
    uint16_t* zsel_row = fuse.z_sel ? reinterpret_cast<uint16_t*>(fuse.z_sel) + static_cast<int64_t>(row) * k : nullptr;
#pragma unroll 4
    for (int p = lane; p < k; p += 32) {
      const int ch = idx_row[p];
      const float gv = __uint_as_float(static_cast<uint32_t>(gsel_row[p]) << 16);
      const float uf = __uint_as_float(static_cast<uint32_t>(usel_row[p]) << 16);
      float sv, zv;
      moc_fwd_point<__nv_bfloat16>(gv, uf, sv, zv);
      const uint16_t zb = static_cast<uint16_t>(__float_as_uint(zv) >> 16);   // zv is already a bf16 value
      grow[ch] = zb;
      if (ssel_row) ssel_row[p] = static_cast<uint16_t>(__float_as_uint(sv) >> 16);
      if (zsel_row) zsel_row[p] = zb;
    }
  }
}

// bf16 fast path of the 2:8 rule: one warp per token row, and one 16-byte vector = one group of 8 channels
// per lane and step, so the gate row, the dense U row and the Z' row move as coalesced vectors and the compact
// outputs of a group land at the fixed position 2 * group. Needs rows padded to the mask width and 16-byte
// aligned; same outputs as select_2of8_kernel.
constexpr int kVec28Warps = 4;

__global__ void __launch_bounds__(kVec28Warps * 32)
select_2of8_bf16_vec_kernel(uint16_t* __restrict__ g, int64_t ldg, int tokens, int d_ffn, int k_eff, int words,
                            SelFuseT<__nv_bfloat16> fuse, int16_t* __restrict__ idx, uint16_t* __restrict__ g_sel,
                            uint32_t* __restrict__ bitmap, uint16_t* __restrict__ rank0) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kVec28Warps + warp;
  if (row >= tokens) return;
  uint4* grow4 = reinterpret_cast<uint4*>(g + static_cast<int64_t>(row) * ldg);
  const uint4* urow4 = reinterpret_cast<const uint4*>(fuse.u_dense + static_cast<int64_t>(row) * ldg);
  const int64_t crow = static_cast<int64_t>(row) * k_eff;
  int16_t* idx_row = idx + crow;
  uint16_t* gsel_row = g_sel + crow;
  uint16_t* usel_row = reinterpret_cast<uint16_t*>(fuse.u_sel) + crow;
  uint16_t* ssel_row = fuse.s_sel ? reinterpret_cast<uint16_t*>(fuse.s_sel) + crow : nullptr;
  uint16_t* zsel_row = fuse.z_sel ? reinterpret_cast<uint16_t*>(fuse.z_sel) + crow : nullptr;
  uint32_t* bm_row = bitmap + static_cast<int64_t>(row) * words;
  uint16_t* rk_row = rank0 + static_cast<int64_t>(row) * words;
  const int nvec = words * 4;
  const int nslots = (nvec + 31) >> 5;
  // even k_eff and 4-byte aligned arrays: every group's pair of compact entries starts on a 4-byte boundary
  const bool pair_stores = (k_eff & 1) == 0 &&
                           ((reinterpret_cast<uintptr_t>(idx) | reinterpret_cast<uintptr_t>(g_sel) |
                             reinterpret_cast<uintptr_t>(fuse.u_sel) | reinterpret_cast<uintptr_t>(fuse.s_sel) |
                             reinterpret_cast<uintptr_t>(fuse.z_sel)) & 3u) == 0;
  // the vectors of the next step are requested before the current ones are worked on
  uint4 q_next = make_uint4(0u, 0u, 0u, 0u), uq_next = make_uint4(0u, 0u, 0u, 0u);
  if (lane < nvec) {
    q_next = grow4[lane];
    if (fuse.u_dense) uq_next = urow4[lane];
  }
#pragma unroll 1
  for (int i = 0; i < nslots; ++i) {
    const int v = i * 32 + lane;
    uint4 q = q_next, uq = uq_next;
    if (v + 32 < nvec) {
      q_next = grow4[v + 32];
      if (fuse.u_dense) uq_next = urow4[v + 32];
    }
    const int nv = min(8, max(0, d_ffn - 8 * v));
    const uint32_t gw[4] = {q.x, q.y, q.z, q.w}, uw[4] = {uq.x, uq.y, uq.z, uq.w};
    uint32_t bits[8], key[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      bits[j] = (gw[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
      key[j] = j < nv ? order_key16(static_cast<uint16_t>(bits[j])) : 0u;
    }
    int b1 = 0;
#pragma unroll
    for (int j = 1; j < 8; ++j)
      if (j < nv && key[j] > key[b1]) b1 = j;     // first maximum: the lower channel wins ties
    int b2 = -1;
    uint32_t k2 = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool cand = j < nv && j != b1 && (b2 < 0 || key[j] > k2);
      if (cand) {
        b2 = j;
        k2 = key[j];
      }
    }
    const int lo = (b2 >= 0 && b2 < b1) ? b2 : b1;
    const int hi = (b2 >= 0 && b2 < b1) ? b1 : b2;
    uint32_t g_lo = 0, g_hi = 0, u_lo = 0, u_hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {   // constant-index register reads only
      const uint32_t ub = (uw[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
      if (j == lo) { g_lo = bits[j]; u_lo = ub; }
      if (j == hi) { g_hi = bits[j]; u_hi = ub; }
    }
    uint32_t m8 = 0;
    if (nv > 0) {
      const int pos = 2 * v;
      m8 = 1u << lo;
      if (hi >= 0) m8 |= 1u << hi;
      if (hi >= 0 && pair_stores) {   // both entries of the group in one 4-byte store
        *reinterpret_cast<uint32_t*>(idx_row + pos) = static_cast<uint32_t>(8 * v + lo) | (static_cast<uint32_t>(8 * v + hi) << 16);
        *reinterpret_cast<uint32_t*>(gsel_row + pos) = g_lo | (g_hi << 16);
      } else {
        idx_row[pos] = static_cast<int16_t>(8 * v + lo);
        gsel_row[pos] = static_cast<uint16_t>(g_lo);
        if (hi >= 0) {
          idx_row[pos + 1] = static_cast<int16_t>(8 * v + hi);
          gsel_row[pos + 1] = static_cast<uint16_t>(g_hi);
        }
      }
      if (fuse.u_dense) {
        float s0, z0, s1 = 0.0f, z1 = 0.0f;
        moc_fwd_point<__nv_bfloat16>(__uint_as_float(g_lo << 16), __uint_as_float(u_lo << 16), s0, z0);
        if (hi >= 0) moc_fwd_point<__nv_bfloat16>(__uint_as_float(g_hi << 16), __uint_as_float(u_hi << 16), s1, z1);
        const uint32_t zb0 = __float_as_uint(z0) >> 16, zb1 = __float_as_uint(z1) >> 16;   // already bf16 values
        const uint32_t sb0 = __float_as_uint(s0) >> 16, sb1 = __float_as_uint(s1) >> 16;
        if (hi >= 0 && pair_stores) {
          *reinterpret_cast<uint32_t*>(usel_row + pos) = u_lo | (u_hi << 16);
          if (ssel_row) *reinterpret_cast<uint32_t*>(ssel_row + pos) = sb0 | (sb1 << 16);
          if (zsel_row) *reinterpret_cast<uint32_t*>(zsel_row + pos) = zb0 | (zb1 << 16);
        } else {
          usel_row[pos] = static_cast<uint16_t>(u_lo);
          if (ssel_row) ssel_row[pos] = static_cast<uint16_t>(sb0);
          if (zsel_row) zsel_row[pos] = static_cast<uint16_t>(zb0);
          if (hi >= 0) {
            usel_row[pos + 1] = static_cast<uint16_t>(u_hi);
            if (ssel_row) ssel_row[pos + 1] = static_cast<uint16_t>(sb1);
            if (zsel_row) zsel_row[pos + 1] = static_cast<uint16_t>(zb1);
          }
        }
        uint32_t zw[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t zj = (j == lo) ? zb0 : ((j == hi) ? zb1 : 0u);
          zw[j >> 1] |= zj << (16 * (j & 1));
        }
        q = make_uint4(zw[0], zw[1], zw[2], zw[3]);
      }
    } else if (fuse.u_dense) {
      q = make_uint4(0u, 0u, 0u, 0u);
    }
    if (fuse.u_dense && v < nvec) grow4[v] = q;    // Z' over the whole padded row
    uint32_t b = m8 << (8 * (lane & 3));
    b |= __shfl_xor_sync(0xFFFFFFFFu, b, 1);
    b |= __shfl_xor_sync(0xFFFFFFFFu, b, 2);
    const int widx = i * 8 + (lane >> 2);
    if ((lane & 3) == 0 && widx < words) {
      bm_row[widx] = b;
      rk_row[widx] = static_cast<uint16_t>(min(widx * 8, k_eff));
    }
  }
}

// One thread per (token, 32-channel word) = 4 groups of 8. Lower channel index wins ties
// (moc/inference/triton_fused_ffn_kernels.py:103-114). fuse: as in topk_select_kernel.
template <typename T>
__global__ void select_2of8_kernel(T* __restrict__ g, int64_t ldg, int tokens, int d_ffn, int k_eff, int words,
                                   SelFuseT<T> fuse, int16_t* __restrict__ idx, T* __restrict__ g_sel,
                                   uint32_t* __restrict__ bitmap, uint16_t* __restrict__ rank0) {
  using KT = KeyTraits<T>;
  using Bits = typename KT::Bits;
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<int64_t>(tokens) * words) return;
  const int row = static_cast<int>(gid / words);
  const int w = static_cast<int>(gid % words);
  Bits* grow = reinterpret_cast<Bits*>(g) + static_cast<int64_t>(row) * ldg;
  int16_t* idx_row = idx + static_cast<int64_t>(row) * k_eff;
  Bits* gsel_row = reinterpret_cast<Bits*>(g_sel) + static_cast<int64_t>(row) * k_eff;
  uint32_t mask = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int c0 = w * 32 + q * 8;
    const int nv = min(8, d_ffn - c0);
    Bits raw[8];
    uint32_t key[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      raw[j] = (j < nv) ? grow[c0 + j] : Bits(0);
      key[j] = KT::key(raw[j]);
    }
    int lo = -1, hi = -1;
    if (nv > 0) {
      int b1 = 0;
#pragma unroll
      for (int j = 1; j < 8; ++j)
        if (j < nv && key[j] > key[b1]) b1 = j;
      int b2 = -1;
      if (nv >= 2) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nv && j != b1 && (b2 < 0 || key[j] > key[b2])) b2 = j;
      }
      lo = (b2 >= 0 && b2 < b1) ? b2 : b1;
      hi = (b2 >= 0 && b2 < b1) ? b1 : b2;
      const int pos = (c0 >> 3) * 2;
#pragma unroll
      for (int j = 0; j < 8; ++j) {   // constant-index register reads only
        if (j == lo) {
          idx_row[pos] = static_cast<int16_t>(c0 + j);
          gsel_row[pos] = raw[j];
        }
        if (j == hi) {
          idx_row[pos + 1] = static_cast<int16_t>(c0 + j);
          gsel_row[pos + 1] = raw[j];
        }
      }
      mask |= 1u << (q * 8 + lo);
      if (hi >= 0) mask |= 1u << (q * 8 + hi);
    }
    if (fuse.u_dense) {
      const int pos = (c0 >> 3) * 2;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        Bits zbits = Bits(0);
        if (j == lo || j == hi)
          zbits = fuse_point<T>(fuse, static_cast<int64_t>(row) * ldg + c0 + j,
                                static_cast<int64_t>(row) * k_eff + pos + (j == hi ? 1 : 0), KT::value(raw[j]));
        grow[c0 + j] = zbits;
      }
    }
  }
  bitmap[gid] = mask;
  rank0[gid] = static_cast<uint16_t>(min(w * 8, k_eff));
}

// The dense <-> compact kernels below run one CTA per token and work in COMPACT space: every
// thread handles selected channels only (full lanes for the SiLU math), scatters its results
// into a zeroed shared-memory image of the dense row, and the CTA then writes the row out
// with 16-byte coalesced stores.
constexpr int kRowThreads = 256;

template <typename T>
__device__ __forceinline__ void row_zero(T* row, int ld) {
  uint4* r4 = reinterpret_cast<uint4*>(row);
  const int nvec = ld * static_cast<int>(sizeof(T)) / 16;
  for (int v = threadIdx.x; v < nvec; v += kRowThreads) r4[v] = make_uint4(0, 0, 0, 0);
}
template <typename T>
__device__ __forceinline__ void row_store(const T* row, T* dst, int ld) {
  const uint4* r4 = reinterpret_cast<const uint4*>(row);
  uint4* d4 = reinterpret_cast<uint4*>(dst);
  const int nvec = ld * static_cast<int>(sizeof(T)) / 16;
  for (int v = threadIdx.x; v < nvec; v += kRowThreads) d4[v] = r4[v];
}

// Post-SiLU selection (moc/ffn.py:313-369): the score that Top-K runs on is |SiLU(g)|, rounded to the storage
// type like the reference's F.silu(g).abs(). SiLU is evaluated with expf and a true division here (the other
// kernels use the fast forms) so that the scores equal PyTorch's wherever its own exp agrees to the last bit.
template <typename T>
__global__ void __launch_bounds__(256)
abs_silu_kernel(const T* __restrict__ g, T* __restrict__ score, int64_t nvec) {
  constexpr int E = 16 / sizeof(T);
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const uint4 q = reinterpret_cast<const uint4*>(g)[i];
  const T* in = reinterpret_cast<const T*>(&q);
  T out[E];
#pragma unroll
  for (int j = 0; j < E; ++j) {
    const float gv = Num<T>::to_float(in[j]);
    const float sv = Num<T>::round(gv / (1.0f + expf(-gv)));
    out[j] = Num<T>::from_float(fabsf(sv));
  }
  reinterpret_cast<uint4*>(score)[i] = *reinterpret_cast<const uint4*>(out);
}

// After a selection that ran on another tensor than the gate: gather g and u of the selected channels from
// the dense rows, store the compact saved set and replace the dense gate row by Z' (one CTA per token, compact
// space, shared-memory row image as in bwd_sparse_kernel).
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
post_gather_kernel(const int16_t* __restrict__ idx, T* __restrict__ g_dense, const T* __restrict__ u_dense,
                   T* __restrict__ g_sel, T* __restrict__ u_sel, T* __restrict__ s_sel, T* __restrict__ z_sel,
                   int64_t ld, int k) {
  extern __shared__ __align__(16) uint8_t row_smem[];
  T* zrow = reinterpret_cast<T*>(row_smem);
  const int row = blockIdx.x;
  const int64_t crow = static_cast<int64_t>(row) * k;
  T* grow = g_dense + static_cast<int64_t>(row) * ld;
  const T* urow = u_dense + static_cast<int64_t>(row) * ld;
  row_zero(zrow, static_cast<int>(ld));
  __syncthreads();
  for (int p = threadIdx.x; p < k; p += kRowThreads) {
    const int ch = idx[crow + p];
    const T gv = grow[ch], uv = urow[ch];
    float s, z;
    moc_fwd_point<T>(Num<T>::to_float(gv), Num<T>::to_float(uv), s, z);
    g_sel[crow + p] = gv;
    u_sel[crow + p] = uv;
    if (s_sel) s_sel[crow + p] = Num<T>::from_float(s);
    const T zt = Num<T>::from_float(z);
    if (z_sel) z_sel[crow + p] = zt;
    zrow[ch] = zt;
  }
  __syncthreads();   // every gather from the gate row is done before the row is overwritten
  row_store(zrow, grow, static_cast<int>(ld));
}

// dZ (dense, rounded GEMM output) -> dG', dU' (dense, zero outside the selected channels).
// dU' overwrites dZ in place, dG' goes to its own buffer. With z_dense set the same pass also rebuilds the
// zero-filled Z' rows (from z_sel, or from g and u) that the weight-gradient GEMM of the down projection reads.
// gz = dZ, grad_s = round(u * gz), grad_u = round(s * gz), grad_g = round(grad_s * SiLU'(g)), with
// s = round(SiLU(g)) recomputed from g (identical to the saved s of the reference, moc/ffn.py:157).
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
bwd_sparse_kernel(const int16_t* __restrict__ idx, const T* __restrict__ g_sel, const T* __restrict__ u_sel,
                  const T* __restrict__ z_sel, T* __restrict__ dz_du, T* __restrict__ grad_g, T* __restrict__ z_dense,
                  int64_t ld, int k) {
  extern __shared__ __align__(16) uint8_t row_smem[];
  T* grow = reinterpret_cast<T*>(row_smem);
  T* urow = grow + ld;
  T* zrow = urow + ld;   // only when z_dense is set
  const int row = blockIdx.x;
  const int64_t crow = static_cast<int64_t>(row) * k;
  T* dzrow = dz_du + static_cast<int64_t>(row) * ld;
  row_zero(grow, static_cast<int>((z_dense ? 3 : 2) * ld));
  __syncthreads();
  for (int p = threadIdx.x; p < k; p += kRowThreads) {
    const int ch = idx[crow + p];
    const float gv = Num<T>::to_float(g_sel[crow + p]), uv = Num<T>::to_float(u_sel[crow + p]);
    float gg, gu;
    moc_bwd_point<T>(gv, uv, Num<T>::to_float(dzrow[ch]), gg, gu);
    grow[ch] = Num<T>::from_float(gg);
    urow[ch] = Num<T>::from_float(gu);
    if (z_dense) {
      if (z_sel) {
        zrow[ch] = z_sel[crow + p];
      } else {
        float sv, zv;
        moc_fwd_point<T>(gv, uv, sv, zv);
        zrow[ch] = Num<T>::from_float(zv);
      }
    }
  }
  __syncthreads();   // all gathers from dZ are done before the row is overwritten
  row_store(grow, grad_g + static_cast<int64_t>(row) * ld, static_cast<int>(ld));
  row_store(urow, dzrow, static_cast<int>(ld));
  if (z_dense) row_store(zrow, z_dense + static_cast<int64_t>(row) * ld, static_cast<int>(ld));
}

// Dense SwiGLU backward, elementwise part (autograd of moc/ffn.py:120-121 with stored-dtype tensors):
// s = round(SiLU(g)), z = round(s * u); grad_u = round(dz * s), grad_s = round(dz * u),
// grad_g = round(grad_s * SiLU'(g)) with SiLU' evaluated in fp32 in one step (PyTorch's silu_backward).
// dz is overwritten by grad_u in place; z and grad_g go to their own buffers. One thread per 16 bytes.
template <typename T>
__global__ void __launch_bounds__(256)
dense_bwd_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ dz_du, T* __restrict__ z_out,
                 T* __restrict__ grad_g, int64_t nvec) {
  constexpr int E = 16 / sizeof(T);
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  __align__(16) T gv[E], uv[E], dv[E], zo[E], go[E], uo[E];
  *reinterpret_cast<uint4*>(gv) = reinterpret_cast<const uint4*>(g)[i];
  *reinterpret_cast<uint4*>(uv) = reinterpret_cast<const uint4*>(u)[i];
  *reinterpret_cast<uint4*>(dv) = reinterpret_cast<const uint4*>(dz_du)[i];
#pragma unroll
  for (int j = 0; j < E; ++j) {
    const float gf = Num<T>::to_float(gv[j]), uf = Num<T>::to_float(uv[j]), dz = Num<T>::to_float(dv[j]);
    const float sig = sigmoid_act<T>(gf);
    const float s = Num<T>::round(gf * sig);
    zo[j] = Num<T>::from_float(s * uf);
    uo[j] = Num<T>::from_float(dz * s);
    const float gs = Num<T>::round(dz * uf);
    go[j] = Num<T>::from_float(gs * (sig * (1.0f + gf * (1.0f - sig))));
  }
  reinterpret_cast<uint4*>(z_out)[i] = *reinterpret_cast<const uint4*>(zo);
  reinterpret_cast<uint4*>(grad_g)[i] = *reinterpret_cast<const uint4*>(go);
  reinterpret_cast<uint4*>(dz_du)[i] = *reinterpret_cast<const uint4*>(uo);
}

template <typename T>
__global__ void transpose_kernel(const T* __restrict__ in, int64_t ld_in, T* __restrict__ out, int64_t ld_out,
                                 int rows, int cols) {
  __shared__ T tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[i][threadIdx.x] = in[static_cast<int64_t>(r) * ld_in + c];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < rows && c < cols) out[static_cast<int64_t>(c) * ld_out + r] = tile[threadIdx.x][i];
  }
}

// ------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------
template <typename T>
static SelFuseT<T> typed_fuse(const SelectFuse* f) {
  SelFuseT<T> t;
  t.u_dense = f ? static_cast<const T*>(f->u_dense) : nullptr;
  t.u_sel = f ? static_cast<T*>(f->u_sel) : nullptr;
  t.s_sel = f ? static_cast<T*>(f->s_sel) : nullptr;
  t.z_sel = f ? static_cast<T*>(f->z_sel) : nullptr;
  return t;
}

static int check_fuse(const SelectFuse* fuse, int64_t ldg, int words) {
  if (!fuse) return kOk;
  if (!fuse->u_dense || !fuse->u_sel) {
    set_error("select: the fused forward needs the dense U rows and the u_sel output");
    return kErrInvalidArg;
  }
  if (ldg < static_cast<int64_t>(words) * 32) {
    set_error("select: in-place Z' output needs ldg >= %d", words * 32);
    return kErrInvalidArg;
  }
  return kOk;
}

int launch_topk_select(int dtype, void* g, int64_t ldg, int tokens, int d_ffn, int k, const SelectFuse* fuse,
                       int16_t* idx, void* g_sel, uint32_t* bitmap, uint16_t* rank0, cudaStream_t stream) {
  if (tokens == 0) return kOk;
  const int words = static_cast<int>(mask_words(d_ffn));
  const int frc = check_fuse(fuse, ldg, words);
  if (frc != kOk) return frc;
  prof_mark(kProfTopk, stream);
  // bf16 rows with the forward fusion: the persistent shared-memory-staged kernel (any number of rows)
  if (dtype == kBF16 && fuse && fuse->status && select_stream_supported(ldg, d_ffn, k, g, fuse->u_dense))
    return launch_select_stream(g, ldg, tokens, d_ffn, k, *fuse, idx, g_sel, bitmap, rank0, fuse->status, stream);
  if (tokens <= 1024) {   // few rows: one CTA per row
    const size_t esz = dtype == kBF16 ? 2 : 4;
    const size_t smem = sizeof(uint32_t) * (kCtaSelBins + words) + esz * d_ffn;
    if (dtype == kBF16) {
      auto kern = topk_select_cta_kernel<__nv_bfloat16>;
      if (smem > 48 * 1024 &&
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
        return check_last("topk_select smem attribute");
      kern<<<tokens, kCtaSelThreads, smem, stream>>>(static_cast<__nv_bfloat16*>(g), ldg, d_ffn, k, words,
                                                     typed_fuse<__nv_bfloat16>(fuse), idx,
                                                     static_cast<__nv_bfloat16*>(g_sel), bitmap, rank0);
    } else {
      auto kern = topk_select_cta_kernel<float>;
      if (smem > 48 * 1024 &&
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
        return check_last("topk_select smem attribute");
      kern<<<tokens, kCtaSelThreads, smem, stream>>>(static_cast<float*>(g), ldg, d_ffn, k, words,
                                                     typed_fuse<float>(fuse), idx, static_cast<float*>(g_sel), bitmap,
                                                     rank0);
    }
    return check_last("topk_select");
  }
  // bf16 fast path: needs aligned rows padded to the mask width
  if (dtype == kBF16 && ldg >= static_cast<int64_t>(words) * 32 && ldg % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(g) & 15u) == 0) {
    const unsigned vblocks = static_cast<unsigned>((tokens + kVecSelWarps - 1) / kVecSelWarps);
    uint16_t* gp = static_cast<uint16_t*>(g);
    uint16_t* gs = static_cast<uint16_t*>(g_sel);
    topk_select_bf16_vec_kernel<<<vblocks, kVecSelWarps * 32, 0, stream>>>(
        gp, ldg, tokens, d_ffn, k, words, typed_fuse<__nv_bfloat16>(fuse), idx, gs, bitmap, rank0);
    return check_last("topk_select");
  }
  const unsigned blocks = static_cast<unsigned>((tokens + kSelWarpsPerCta - 1) / kSelWarpsPerCta);
  if (dtype == kBF16)
    topk_select_kernel<__nv_bfloat16><<<blocks, kSelWarpsPerCta * 32, 0, stream>>>(
        static_cast<__nv_bfloat16*>(g), ldg, tokens, d_ffn, k, words, typed_fuse<__nv_bfloat16>(fuse), idx,
        static_cast<__nv_bfloat16*>(g_sel), bitmap, rank0);
  else
    topk_select_kernel<float><<<blocks, kSelWarpsPerCta * 32, 0, stream>>>(
        static_cast<float*>(g), ldg, tokens, d_ffn, k, words, typed_fuse<float>(fuse), idx, static_cast<float*>(g_sel),
        bitmap, rank0);
  return check_last("topk_select");
}

int launch_select_2of8(int dtype, void* g, int64_t ldg, int tokens, int d_ffn, const SelectFuse* fuse, int16_t* idx,
                       void* g_sel, uint32_t* bitmap, uint16_t* rank0, cudaStream_t stream) {
  if (tokens == 0) return kOk;
  const int words = static_cast<int>(mask_words(d_ffn));
  const int frc = check_fuse(fuse, ldg, words);
  if (frc != kOk) return frc;
  const int k_eff = (d_ffn / 8) * 2 + min(2, d_ffn % 8);
  const int64_t total = static_cast<int64_t>(tokens) * words;
  const int threads = 128;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  prof_mark(kProfSel2of8, stream);
  // one warp per row pays off once there are enough rows to fill the GPU; decode batches keep one thread per word
  if (dtype == kBF16 && tokens >= 512 && ldg >= static_cast<int64_t>(words) * 32 && ldg % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(g) & 15u) == 0 &&
      (!fuse || (reinterpret_cast<uintptr_t>(fuse->u_dense) & 15u) == 0)) {
    const unsigned vblocks = static_cast<unsigned>((tokens + kVec28Warps - 1) / kVec28Warps);
    select_2of8_bf16_vec_kernel<<<vblocks, kVec28Warps * 32, 0, stream>>>(
        static_cast<uint16_t*>(g), ldg, tokens, d_ffn, k_eff, words, typed_fuse<__nv_bfloat16>(fuse), idx,
        static_cast<uint16_t*>(g_sel), bitmap, rank0);
    return check_last("select_2of8");
  }
  if (dtype == kBF16)
    select_2of8_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
        static_cast<__nv_bfloat16*>(g), ldg, tokens, d_ffn, k_eff, words, typed_fuse<__nv_bfloat16>(fuse), idx,
        static_cast<__nv_bfloat16*>(g_sel), bitmap, rank0);
  else
    select_2of8_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<float*>(g), ldg, tokens, d_ffn, k_eff, words,
                                                              typed_fuse<float>(fuse), idx, static_cast<float*>(g_sel),
                                                              bitmap, rank0);
  return check_last("select_2of8");
}

template <typename T, class Kern>
static int row_smem_setup(Kern kern, size_t smem, const char* what) {
  if (smem > 220 * 1024) {
    set_error("%s: d_ffn too large for the %zu-byte row image in shared memory", what, smem);
    return kErrUnsupported;
  }
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return check_last(what);
  return kOk;
}

int launch_abs_silu(int dtype, const void* g, void* score, int64_t elems, cudaStream_t stream) {
  if (elems == 0) return kOk;
  const int64_t nvec = elems * (dtype == kBF16 ? 2 : 4) / 16;
  const unsigned blocks = static_cast<unsigned>((nvec + 255) / 256);
  prof_mark(kProfExpand, stream);
  if (dtype == kBF16)
    abs_silu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(g),
                                                              static_cast<__nv_bfloat16*>(score), nvec);
  else
    abs_silu_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(g), static_cast<float*>(score), nvec);
  return check_last("abs_silu");
}

int launch_post_gather(int dtype, const int16_t* idx, void* g_dense, const void* u_dense, void* g_sel, void* u_sel,
                       void* s_sel, void* z_sel, int64_t ld, int tokens, int k, cudaStream_t stream) {
  if (tokens == 0) return kOk;
  int rc;
  prof_mark(kProfExpand, stream);
  if (dtype == kBF16) {
    const size_t smem = static_cast<size_t>(ld) * 2;
    auto kern = post_gather_kernel<__nv_bfloat16>;
    if ((rc = row_smem_setup<__nv_bfloat16>(kern, smem, "post_gather")) != kOk) return rc;
    kern<<<tokens, kRowThreads, smem, stream>>>(idx, static_cast<__nv_bfloat16*>(g_dense),
                                                static_cast<const __nv_bfloat16*>(u_dense),
                                                static_cast<__nv_bfloat16*>(g_sel), static_cast<__nv_bfloat16*>(u_sel),
                                                static_cast<__nv_bfloat16*>(s_sel), static_cast<__nv_bfloat16*>(z_sel), ld,
                                                k);
  } else {
    const size_t smem = static_cast<size_t>(ld) * 4;
    auto kern = post_gather_kernel<float>;
    if ((rc = row_smem_setup<float>(kern, smem, "post_gather")) != kOk) return rc;
    kern<<<tokens, kRowThreads, smem, stream>>>(idx, static_cast<float*>(g_dense), static_cast<const float*>(u_dense),
                                                static_cast<float*>(g_sel), static_cast<float*>(u_sel),
                                                static_cast<float*>(s_sel), static_cast<float*>(z_sel), ld, k);
  }
  return check_last("post_gather");
}

int launch_bwd_sparse(int dtype, const int16_t* idx, const void* g_sel, const void* u_sel, const void* z_sel,
                      void* dz_to_du, void* grad_g_out, void* z_dense, int64_t ld, int tokens, int d_ffn, int k,
                      cudaStream_t stream) {
  (void)d_ffn;
  if (tokens == 0) return kOk;
  int rc;
  const size_t rows = z_dense ? 3 : 2;
  if (dtype == kBF16) {
    using T = __nv_bfloat16;
    const size_t smem = rows * ld * sizeof(T);
    if ((rc = row_smem_setup<T>(bwd_sparse_kernel<T>, smem, "bwd_sparse")) != kOk) return rc;
    prof_mark(kProfBwdSparse, stream);
    bwd_sparse_kernel<T><<<tokens, kRowThreads, smem, stream>>>(
        idx, static_cast<const T*>(g_sel), static_cast<const T*>(u_sel), static_cast<const T*>(z_sel),
        static_cast<T*>(dz_to_du), static_cast<T*>(grad_g_out), static_cast<T*>(z_dense), ld, k);
  } else {
    using T = float;
    const size_t smem = rows * ld * sizeof(T);
    if ((rc = row_smem_setup<T>(bwd_sparse_kernel<T>, smem, "bwd_sparse")) != kOk) return rc;
    prof_mark(kProfBwdSparse, stream);
    bwd_sparse_kernel<T><<<tokens, kRowThreads, smem, stream>>>(
        idx, static_cast<const T*>(g_sel), static_cast<const T*>(u_sel), static_cast<const T*>(z_sel),
        static_cast<T*>(dz_to_du), static_cast<T*>(grad_g_out), static_cast<T*>(z_dense), ld, k);
  }
  return check_last("bwd_sparse");
}

int launch_dense_bwd(int dtype, const void* g, const void* u, void* dz_to_du, void* z_out, void* grad_g_out,
                     int64_t elems, cudaStream_t stream) {
  if (elems == 0) return kOk;
  prof_mark(kProfBwdSparse, stream);
  if (dtype == kBF16) {
    const int64_t nvec = elems / 8;
    dense_bwd_kernel<__nv_bfloat16><<<static_cast<unsigned>((nvec + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(u),
        static_cast<__nv_bfloat16*>(dz_to_du), static_cast<__nv_bfloat16*>(z_out),
        static_cast<__nv_bfloat16*>(grad_g_out), nvec);
  } else {
    const int64_t nvec = elems / 4;
    dense_bwd_kernel<float><<<static_cast<unsigned>((nvec + 255) / 256), 256, 0, stream>>>(
        static_cast<const float*>(g), static_cast<const float*>(u), static_cast<float*>(dz_to_du),
        static_cast<float*>(z_out), static_cast<float*>(grad_g_out), nvec);
  }
  return check_last("dense_bwd");
}

int launch_transpose(int dtype, const void* in, int64_t ld_in, void* out, int64_t ld_out, int rows, int cols,
                     cudaStream_t stream) {
  if (rows == 0 || cols == 0) return kOk;
  const dim3 block(32, 8);
  const dim3 grid((cols + 31) / 32, (rows + 31) / 32);
  prof_mark(kProfTranspose, stream);
  if (dtype == kBF16)
    transpose_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16*>(in), ld_in,
                                                                static_cast<__nv_bfloat16*>(out), ld_out, rows, cols);
  else
    transpose_kernel<float><<<grid, block, 0, stream>>>(static_cast<const float*>(in), ld_in,
                                                        static_cast<float*>(out), ld_out, rows, cols);
  return check_last("transpose");
}

}  // namespace moc
