// Channel selection and layout kernels of the MoC FFN path (HBM-bound integer/byte work).
//
//   topk_select_kernel : row-wise Top-K over d_ffn pre-SiLU gate values. Replaces
//                        torch.topk (moc/ffn.py:144, :392) and the CUB block sort of the decode
//                        extension (moc/inference/cuda/optimized_global_moc_ext.cu:85-125) by a
//                        radix *select*: the K-th largest order key is found bit by bit, ties
//                        at the threshold go to the lower channel index, and the selected set
//                        is emitted in ascending channel order together with a bitmap.
//   select_2of8_kernel : structured top-2 of every 8 consecutive channels (moc/ffn.py:68-108).
//   expand_z_kernel    : compact z -> zero-filled dense Z' (moc/ffn.py:196-199, :435-442).
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
  __device__ __forceinline__ static uint32_t key(Bits b) { return order_key16(b); }
  __device__ __forceinline__ static Bits unkey(uint32_t k) {
    return static_cast<Bits>((k & 0x8000u) ? (k ^ 0x8000u) : (k ^ 0xFFFFu));
  }
};
template <> struct KeyTraits<float> {
  using Bits = uint32_t;
  static constexpr int kBits = 32;
  __device__ __forceinline__ static uint32_t key(Bits b) { return order_key32(b); }
  __device__ __forceinline__ static Bits unkey(uint32_t k) { return (k & 0x80000000u) ? (k ^ 0x80000000u) : ~k; }
};

constexpr int kSelThreads = 256;
constexpr int kSelWarps = kSelThreads / 32;

__device__ __forceinline__ uint32_t block_sum(uint32_t v, uint32_t* red /*[2][kSelWarps]*/, int iter) {
  const uint32_t w = __reduce_add_sync(0xFFFFFFFFu, v);
  uint32_t* buf = red + (iter & 1) * kSelWarps;
  if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = w;
  __syncthreads();
  uint32_t tot = 0;
#pragma unroll
  for (int i = 0; i < kSelWarps; ++i) tot += buf[i];
  return tot;
}

__device__ __forceinline__ uint32_t block_exscan(uint32_t v, uint32_t* wsum /*[kSelWarps]*/, uint32_t& total) {
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
  for (int i = 0; i < kSelWarps; ++i) {
    const uint32_t s = wsum[i];
    if (i < warp) woff += s;
    tot += s;
  }
  total = tot;
  __syncthreads();
  return woff + inc - v;
}

// One CTA per token row. Thread t owns the contiguous channels [t*chunk, (t+1)*chunk), so
// walking the threads in order walks the channels in order. REG > 0: the thread keeps its
// keys in REG registers (chunk <= REG); REG == 0: keys stay in shared memory.
template <typename T, int REG>
__global__ void __launch_bounds__(kSelThreads)
topk_select_kernel(const T* __restrict__ g, int64_t ldg, int d_ffn, int k, int words, int16_t* __restrict__ idx,
                   T* __restrict__ g_sel, uint32_t* __restrict__ bitmap, uint16_t* __restrict__ rank0) {
  using KT = KeyTraits<T>;
  using Bits = typename KT::Bits;
  extern __shared__ __align__(16) uint8_t sel_smem[];
  uint32_t* bm = reinterpret_cast<uint32_t*>(sel_smem);                    // [words]
  Bits* keys = reinterpret_cast<Bits*>(sel_smem + sizeof(uint32_t) * words);   // [d_ffn] order keys
  __shared__ uint32_t red[2 * kSelWarps];
  __shared__ uint32_t wsum[kSelWarps];

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const Bits* grow = reinterpret_cast<const Bits*>(g) + static_cast<int64_t>(row) * ldg;

  for (int i = tid; i < d_ffn; i += kSelThreads) keys[i] = static_cast<Bits>(KT::key(grow[i]));
  for (int w = tid; w < words; w += kSelThreads) bm[w] = 0u;
  __syncthreads();

  const int chunk = (d_ffn + kSelThreads - 1) / kSelThreads;
  const int begin = min(tid * chunk, d_ffn);
  const int end = min(begin + chunk, d_ffn);
  const int mine = end - begin;

  uint32_t kr[REG > 0 ? REG : 1];
  if (REG > 0) {
#pragma unroll
    for (int i = 0; i < REG; ++i) kr[i] = (i < mine) ? static_cast<uint32_t>(keys[begin + i]) : 0u;
  }

  // K-th largest key, most significant bit first: the largest t with count(key >= t) >= k.
  uint32_t thr = 0;
#pragma unroll 1
  for (int bit = KT::kBits - 1; bit >= 0; --bit) {
    const uint32_t cand = thr | (1u << bit);
    uint32_t cnt = 0;
    if (REG > 0) {
#pragma unroll
      for (int i = 0; i < REG; ++i) cnt += (kr[i] >= cand) ? 1u : 0u;   // padding keys are 0 < cand
    } else {
      for (int i = begin; i < end; ++i) cnt += (static_cast<uint32_t>(keys[i]) >= cand) ? 1u : 0u;
    }
    if (block_sum(cnt, red, bit) >= static_cast<uint32_t>(k)) thr = cand;
  }

  // counts above / equal to the threshold in front of this thread's chunk
  uint32_t n_gt = 0, n_eq = 0;
  if (REG > 0) {
#pragma unroll
    for (int i = 0; i < REG; ++i) {
      if (i < mine) {
        n_gt += (kr[i] > thr) ? 1u : 0u;
        n_eq += (kr[i] == thr) ? 1u : 0u;
      }
    }
  } else {
    for (int i = begin; i < end; ++i) {
      const uint32_t key = keys[i];
      n_gt += (key > thr) ? 1u : 0u;
      n_eq += (key == thr) ? 1u : 0u;
    }
  }
  uint32_t total = 0;
  const uint32_t ex = block_exscan(n_gt | (n_eq << 16), wsum, total);
  const uint32_t gt_before = ex & 0xFFFFu, eq_before = ex >> 16;
  const uint32_t take_eq = static_cast<uint32_t>(k) - (total & 0xFFFFu);   // ties admitted, lowest channels first
  uint32_t eq_seen = eq_before;
  uint32_t pos = gt_before + min(eq_before, take_eq);

  int16_t* idx_row = idx + static_cast<int64_t>(row) * k;
  Bits* gsel_row = reinterpret_cast<Bits*>(g_sel) + static_cast<int64_t>(row) * k;
  int cur_w = -1;
  uint32_t cur_m = 0;
  auto visit = [&](int ch, uint32_t key) {
    bool sel = key > thr;
    if (key == thr) {
      sel = eq_seen < take_eq;
      ++eq_seen;
    }
    if (sel) {
      idx_row[pos] = static_cast<int16_t>(ch);
      gsel_row[pos] = KT::unkey(key);
      ++pos;
      const int w = ch >> 5;
      if (w != cur_w) {
        if (cur_m) atomicOr(&bm[cur_w], cur_m);
        cur_w = w;
        cur_m = 0;
      }
      cur_m |= 1u << (ch & 31);
    }
  };
  if (REG > 0) {
#pragma unroll
    for (int i = 0; i < REG; ++i)
      if (i < mine) visit(begin + i, kr[i]);
  } else {
    for (int i = begin; i < end; ++i) visit(i, keys[i]);
  }
  if (cur_m) atomicOr(&bm[cur_w], cur_m);
  __syncthreads();

  // bitmap words and the rank of each word's first channel
  const int wchunk = (words + kSelThreads - 1) / kSelThreads;
  const int wb = min(tid * wchunk, words), we = min(wb + wchunk, words);
  uint32_t pc = 0;
  for (int w = wb; w < we; ++w) pc += __popc(bm[w]);
  uint32_t tot2 = 0;
  uint32_t run = block_exscan(pc, wsum, tot2);
  uint32_t* bm_row = bitmap + static_cast<int64_t>(row) * words;
  uint16_t* rk_row = rank0 + static_cast<int64_t>(row) * words;
  for (int w = wb; w < we; ++w) {
    const uint32_t m = bm[w];
    bm_row[w] = m;
    rk_row[w] = static_cast<uint16_t>(run);
    run += __popc(m);
  }
}

// One thread per (token, 32-channel word) = 4 groups of 8. Lower channel index wins ties
// (moc/inference/triton_fused_ffn_kernels.py:103-114).
template <typename T>
__global__ void select_2of8_kernel(const T* __restrict__ g, int64_t ldg, int tokens, int d_ffn, int k_eff, int words,
                                   int16_t* __restrict__ idx, T* __restrict__ g_sel, uint32_t* __restrict__ bitmap,
                                   uint16_t* __restrict__ rank0) {
  using KT = KeyTraits<T>;
  using Bits = typename KT::Bits;
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<int64_t>(tokens) * words) return;
  const int row = static_cast<int>(gid / words);
  const int w = static_cast<int>(gid % words);
  const Bits* grow = reinterpret_cast<const Bits*>(g) + static_cast<int64_t>(row) * ldg;
  int16_t* idx_row = idx + static_cast<int64_t>(row) * k_eff;
  Bits* gsel_row = reinterpret_cast<Bits*>(g_sel) + static_cast<int64_t>(row) * k_eff;
  uint32_t mask = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int c0 = w * 32 + q * 8;
    const int nv = min(8, d_ffn - c0);
    if (nv <= 0) break;
    uint32_t key[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) key[j] = (j < nv) ? KT::key(grow[c0 + j]) : 0u;
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
    const int pos = (c0 >> 3) * 2;
    const int lo = (b2 >= 0 && b2 < b1) ? b2 : b1;
    const int hi = (b2 >= 0 && b2 < b1) ? b1 : b2;
    idx_row[pos] = static_cast<int16_t>(c0 + lo);
    gsel_row[pos] = KT::unkey(key[lo]);
    mask |= 1u << (q * 8 + lo);
    if (hi >= 0) {
      idx_row[pos + 1] = static_cast<int16_t>(c0 + hi);
      gsel_row[pos + 1] = KT::unkey(key[hi]);
      mask |= 1u << (q * 8 + hi);
    }
  }
  bitmap[gid] = mask;
  rank0[gid] = static_cast<uint16_t>(min(w * 8, k_eff));
}

// One thread per (token, word): writes 32 dense values.
template <typename T>
__global__ void expand_z_kernel(const uint32_t* __restrict__ bitmap, const uint16_t* __restrict__ rank0,
                                const T* __restrict__ z_sel, const T* __restrict__ g_sel, const T* __restrict__ u_sel,
                                T* __restrict__ dense, int64_t ld, int tokens, int words, int k) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<int64_t>(tokens) * words) return;
  const int row = static_cast<int>(gid / words);
  const int w = static_cast<int>(gid % words);
  const uint32_t word = bitmap[gid];
  const int base = rank0[gid];
  const int64_t crow = static_cast<int64_t>(row) * k;
  T* out = dense + static_cast<int64_t>(row) * ld + w * 32;
  __align__(16) T vals[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float z = 0.0f;
    if ((word >> j) & 1u) {
      const int pos = base + __popc(word & ((1u << j) - 1u));
      if (z_sel) {
        z = Num<T>::to_float(z_sel[crow + pos]);
      } else {
        float s;
        moc_fwd_point<T>(Num<T>::to_float(g_sel[crow + pos]), Num<T>::to_float(u_sel[crow + pos]), s, z);
      }
    }
    vals[j] = Num<T>::from_float(z);
  }
  uint4* o4 = reinterpret_cast<uint4*>(out);
  const uint4* v4 = reinterpret_cast<const uint4*>(vals);
#pragma unroll
  for (int i = 0; i < static_cast<int>(32 * sizeof(T) / 16); ++i) o4[i] = v4[i];
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
static int topk_select_t(const void* g, int64_t ldg, int tokens, int d_ffn, int k, int16_t* idx, void* g_sel,
                         uint32_t* bitmap, uint16_t* rank0, cudaStream_t stream) {
  using Bits = typename KeyTraits<T>::Bits;
  const int words = static_cast<int>(mask_words(d_ffn));
  const size_t smem = sizeof(uint32_t) * words + sizeof(Bits) * d_ffn;
  const int chunk = (d_ffn + kSelThreads - 1) / kSelThreads;
  const T* gp = static_cast<const T*>(g);
  T* gs = static_cast<T*>(g_sel);
#define MOC_SEL_LAUNCH(REG)                                                                                      \
  do {                                                                                                           \
    auto kern = topk_select_kernel<T, REG>;                                                                      \
    if (smem > 48 * 1024) {                                                                                      \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=     \
          cudaSuccess)                                                                                           \
        return check_last("topk_select smem attribute");                                                         \
    }                                                                                                            \
    prof_mark(kProfTopk, stream);                                                                                \
    kern<<<tokens, kSelThreads, smem, stream>>>(gp, ldg, d_ffn, k, words, idx, gs, bitmap, rank0);               \
  } while (0)
  if (chunk <= 8) MOC_SEL_LAUNCH(8);
  else if (chunk <= 16) MOC_SEL_LAUNCH(16);
  else if (chunk <= 24) MOC_SEL_LAUNCH(24);
  else if (chunk <= 32) MOC_SEL_LAUNCH(32);
  else MOC_SEL_LAUNCH(0);
#undef MOC_SEL_LAUNCH
  return check_last("topk_select");
}

int launch_topk_select(int dtype, const void* g, int64_t ldg, int tokens, int d_ffn, int k, int16_t* idx,
                       void* g_sel, uint32_t* bitmap, uint16_t* rank0, cudaStream_t stream) {
  if (tokens == 0) return kOk;
  if (dtype == kBF16)
    return topk_select_t<__nv_bfloat16>(g, ldg, tokens, d_ffn, k, idx, g_sel, bitmap, rank0, stream);
  return topk_select_t<float>(g, ldg, tokens, d_ffn, k, idx, g_sel, bitmap, rank0, stream);
}

int launch_select_2of8(int dtype, const void* g, int64_t ldg, int tokens, int d_ffn, int16_t* idx, void* g_sel,
                       uint32_t* bitmap, uint16_t* rank0, cudaStream_t stream) {
  if (tokens == 0) return kOk;
  const int words = static_cast<int>(mask_words(d_ffn));
  const int k_eff = (d_ffn / 8) * 2 + min(2, d_ffn % 8);
  const int64_t total = static_cast<int64_t>(tokens) * words;
  const int threads = 128;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  prof_mark(kProfSel2of8, stream);
  if (dtype == kBF16)
    select_2of8_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(g), ldg, tokens, d_ffn, k_eff, words, idx,
        static_cast<__nv_bfloat16*>(g_sel), bitmap, rank0);
  else
    select_2of8_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<const float*>(g), ldg, tokens, d_ffn,
                                                              k_eff, words, idx, static_cast<float*>(g_sel), bitmap,
                                                              rank0);
  return check_last("select_2of8");
}

int launch_expand_z(int dtype, const uint32_t* bitmap, const uint16_t* rank0, const void* z_sel, const void* g_sel,
                    const void* u_sel, void* dense, int64_t ld, int tokens, int d_ffn, int k, cudaStream_t stream) {
  if (tokens == 0) return kOk;
  const int words = static_cast<int>(mask_words(d_ffn));
  const int64_t total = static_cast<int64_t>(tokens) * words;
  const int threads = 128;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  prof_mark(kProfExpand, stream);
  if (dtype == kBF16)
    expand_z_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
        bitmap, rank0, static_cast<const __nv_bfloat16*>(z_sel), static_cast<const __nv_bfloat16*>(g_sel),
        static_cast<const __nv_bfloat16*>(u_sel), static_cast<__nv_bfloat16*>(dense), ld, tokens, words, k);
  else
    expand_z_kernel<float><<<blocks, threads, 0, stream>>>(bitmap, rank0, static_cast<const float*>(z_sel),
                                                           static_cast<const float*>(g_sel),
                                                           static_cast<const float*>(u_sel),
                                                           static_cast<float*>(dense), ld, tokens, words, k);
  return check_last("expand_z");
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
