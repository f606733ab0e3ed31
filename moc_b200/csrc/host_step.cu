// Kernels for the non-FFN part of one static-cache decode step of the LLaMA-style host model (bf16): the step is a
// chain of tiny operations that the reference leaves to PyTorch (benchmarks/inference/benchmark_decode.py:312-362,
// DecoderModel.forward_step_static, with the blocks of moc/model.py:19-88). Around a 22 us decode FFN those ~45
// framework kernels per layer dominate the time of a token; here they are three launches per layer:
//
//   host_rmsnorm_kernel     h = h + delta (optional), y = RMSNorm(h) * w                      (moc/model.py:19-27)
//   host_rope_cache_kernel  rotary embedding of q and k at position pos, k and v into the caches (moc/model.py:37-43,
//                           benchmark_decode.py:337-346)
//   host_attn_step_kernel   one query row against the cached keys and values of positions <= pos (benchmark_decode.py:
//                           347-356)
//
// Rounding follows the chain of bf16 PyTorch ops where that is well defined (every elementwise product and sum is
// rounded to bf16, the norm statistics are fp32); attention accumulates in fp32 like the library kernels PyTorch uses.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moc_b200.h"
#include "common.cuh"
#include "internal.h"

namespace moc {

using hbf = __nv_bfloat16;

__device__ __forceinline__ float hs_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float hs_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hs_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t hs_pack(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// One CTA per row; d % 8 == 0. delta != null: h <- round(h + delta) first (the residual update of the block).
constexpr int kNormThreads = 256;
__global__ void __launch_bounds__(kNormThreads)
host_rmsnorm_kernel(hbf* __restrict__ h, const hbf* __restrict__ delta, const hbf* __restrict__ w, hbf* __restrict__ y,
                    int d, float eps) {
  __shared__ float red[kNormThreads / 32];
  const int row = blockIdx.x, tid = threadIdx.x;
  uint4* hr = reinterpret_cast<uint4*>(h + static_cast<int64_t>(row) * d);
  const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + static_cast<int64_t>(row) * d) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<int64_t>(row) * d);
  const int nvec = d >> 3;
  float ss = 0.0f;
  for (int v = tid; v < nvec; v += kNormThreads) {
    uint4 q = hr[v];
    uint32_t a[4] = {q.x, q.y, q.z, q.w};
    if (dr) {
      const uint4 e = dr[v];
      const uint32_t b[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) a[j] = hs_pack(hs_lo(a[j]) + hs_lo(b[j]), hs_hi(a[j]) + hs_hi(b[j]));
      hr[v] = make_uint4(a[0], a[1], a[2], a[3]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += hs_lo(a[j]) * hs_lo(a[j]) + hs_hi(a[j]) * hs_hi(a[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) tot += red[i];
  const float inv = rsqrtf(tot / static_cast<float>(d) + eps);
  for (int v = tid; v < nvec; v += kNormThreads) {
    const uint4 q = hr[v];          // own earlier writes (same thread, same vector)
    const uint4 g = wr[v];
    const uint32_t a[4] = {q.x, q.y, q.z, q.w}, ww[4] = {g.x, g.y, g.z, g.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = hs_pack(hs_round(hs_lo(a[j]) * inv) * hs_lo(ww[j]), hs_round(hs_hi(a[j]) * inv) * hs_hi(ww[j]));
    yr[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// qkv: [batch, 3, heads, hd] (the output row of the fused projection); cos, sin: [positions, hd / 2] bf16;
// caches: [batch, heads, t_max, hd]; q_out: [batch, heads, hd]. One CTA per (batch row, head), hd / 2 threads.
__global__ void host_rope_cache_kernel(const hbf* __restrict__ qkv, const hbf* __restrict__ cos_t,
                                       const hbf* __restrict__ sin_t, const int64_t* __restrict__ pos_p,
                                       hbf* __restrict__ q_out, hbf* __restrict__ cache_k, hbf* __restrict__ cache_v,
                                       int heads, int hd, int t_max) {
  const int b = blockIdx.x / heads, hh = blockIdx.x - b * heads, i = threadIdx.x;
  const int64_t pos = *pos_p;
  if (pos < 0 || pos >= t_max) return;
  const int half = hd >> 1;
  const float c = __bfloat162float(cos_t[pos * half + i]), s = __bfloat162float(sin_t[pos * half + i]);
  const int64_t row = static_cast<int64_t>(b) * 3 * heads * hd;
  const uint32_t* q2 = reinterpret_cast<const uint32_t*>(qkv + row + static_cast<int64_t>(hh) * hd);
  const uint32_t* k2 = reinterpret_cast<const uint32_t*>(qkv + row + static_cast<int64_t>(heads + hh) * hd);
  const uint32_t* v2 = reinterpret_cast<const uint32_t*>(qkv + row + static_cast<int64_t>(2 * heads + hh) * hd);
  const int64_t slot = ((static_cast<int64_t>(b) * heads + hh) * t_max + pos) * hd;
  const uint32_t qw = q2[i], kw = k2[i];
  // (even, odd) -> (even * cos - odd * sin, even * sin + odd * cos), every product and sum rounded to bf16
  const float qe = hs_lo(qw), qo = hs_hi(qw), ke = hs_lo(kw), ko = hs_hi(kw);
  reinterpret_cast<uint32_t*>(q_out + (static_cast<int64_t>(b) * heads + hh) * hd)[i] =
      hs_pack(hs_round(qe * c) - hs_round(qo * s), hs_round(qe * s) + hs_round(qo * c));
  reinterpret_cast<uint32_t*>(cache_k + slot)[i] =
      hs_pack(hs_round(ke * c) - hs_round(ko * s), hs_round(ke * s) + hs_round(ko * c));
  reinterpret_cast<uint32_t*>(cache_v + slot)[i] = v2[i];
}

// One CTA per (batch row, head): scores of positions 0..pos in shared memory (fp32), softmax, weighted sum of the
// values. hd in {8, 16, 32, 64, 128} (it divides the block size), t_max * 4 bytes of dynamic shared memory.
constexpr int kAttnThreads = 128;
__global__ void __launch_bounds__(kAttnThreads)
host_attn_step_kernel(const hbf* __restrict__ q, const hbf* __restrict__ cache_k, const hbf* __restrict__ cache_v,
                      const int64_t* __restrict__ pos_p, hbf* __restrict__ y, int heads, int hd, int t_max, float scale) {
  extern __shared__ float sc[];
  __shared__ float red[kAttnThreads / 32];
  __shared__ float qs[128];
  __shared__ float part[kAttnThreads];     // [groups][hd]
  const int b = blockIdx.x / heads, hh = blockIdx.x - b * heads, tid = threadIdx.x;
  int64_t pos = *pos_p;
  if (pos < 0) return;
  if (pos >= t_max) pos = t_max - 1;
  const int n = static_cast<int>(pos) + 1;
  const int64_t base = (static_cast<int64_t>(b) * heads + hh) * t_max * hd;
  if (tid < hd) qs[tid] = __bfloat162float(q[(static_cast<int64_t>(b) * heads + hh) * hd + tid]);
  __syncthreads();
  const int nv = hd >> 3;
  float mx = -INFINITY;
  for (int p = tid; p < n; p += kAttnThreads) {
    const uint4* kr = reinterpret_cast<const uint4*>(cache_k + base + static_cast<int64_t>(p) * hd);
    float acc = 0.0f;
    for (int v = 0; v < nv; ++v) {
      const uint4 k4 = kr[v];
      const uint32_t w[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) acc += qs[8 * v + 2 * j] * hs_lo(w[j]) + qs[8 * v + 2 * j + 1] * hs_hi(w[j]);
    }
    acc *= scale;
    sc[p] = acc;
    mx = fmaxf(mx, acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < kAttnThreads / 32; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = 0.0f;
  for (int p = tid; p < n; p += kAttnThreads) {
    const float e = __expf(sc[p] - mx);
    sc[p] = e;
    sum += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  if ((tid & 31) == 0) red[tid >> 5] = sum;
  __syncthreads();
  sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kAttnThreads / 32; ++i) sum += red[i];
  // weighted values: thread (g, j) adds the positions p = g, g + groups, ... of column j
  const int groups = kAttnThreads / hd;          // hd divides the block size
  const int g = tid / hd, j = tid - g * hd;
  {
    float acc = 0.0f;
    const hbf* vr = cache_v + base + j;
    for (int p = g; p < n; p += groups) acc += sc[p] * __bfloat162float(vr[static_cast<int64_t>(p) * hd]);
    part[tid] = acc;
  }
  __syncthreads();
  if (tid < hd) {
    float o = 0.0f;
    for (int gg = 0; gg < groups; ++gg) o += part[gg * hd + tid];
    y[(static_cast<int64_t>(b) * heads + hh) * hd + tid] = __float2bfloat16_rn(o / sum);
  }
}

}  // namespace moc

using namespace moc;

extern "C" {

int moc_host_rmsnorm(int64_t rows, int64_t d, void* h, const void* delta, const void* weight, void* y, float eps,
                     void* stream) {
  if (rows < 0 || d <= 0 || d % 8 != 0 || !h || !weight || !y) {
    set_error("moc_host_rmsnorm: bad sizes (d %% 8 == 0 required) or null pointer");
    return kErrInvalidArg;
  }
  if (rows == 0) return kOk;
  host_rmsnorm_kernel<<<static_cast<unsigned>(rows), kNormThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<hbf*>(h), static_cast<const hbf*>(delta), static_cast<const hbf*>(weight), static_cast<hbf*>(y),
      static_cast<int>(d), eps);
  return check_last("moc_host_rmsnorm");
}

int moc_host_rope_cache(int64_t batch, int64_t heads, int64_t head_dim, int64_t t_max, const void* qkv,
                        const void* cos_table, const void* sin_table, const int64_t* pos, void* q_out, void* cache_k,
                        void* cache_v, void* stream) {
  if (batch < 0 || heads <= 0 || head_dim <= 0 || head_dim % 2 != 0 || head_dim > 2048 || t_max <= 0 || !qkv ||
      !cos_table || !sin_table || !pos || !q_out || !cache_k || !cache_v) {
    set_error("moc_host_rope_cache: bad sizes or null pointer");
    return kErrInvalidArg;
  }
  if (batch == 0) return kOk;
  host_rope_cache_kernel<<<static_cast<unsigned>(batch * heads), static_cast<unsigned>(head_dim / 2), 0,
                           reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const hbf*>(qkv), static_cast<const hbf*>(cos_table), static_cast<const hbf*>(sin_table), pos,
      static_cast<hbf*>(q_out), static_cast<hbf*>(cache_k), static_cast<hbf*>(cache_v), static_cast<int>(heads),
      static_cast<int>(head_dim), static_cast<int>(t_max));
  return check_last("moc_host_rope_cache");
}

int moc_host_attn_step(int64_t batch, int64_t heads, int64_t head_dim, int64_t t_max, const void* q, const void* cache_k,
                       const void* cache_v, const int64_t* pos, void* y, void* stream) {
  if (batch < 0 || heads <= 0 || head_dim < 8 || head_dim > kAttnThreads || kAttnThreads % head_dim != 0 ||
      head_dim % 8 != 0 || t_max <= 0 || t_max > 11000 || !q || !cache_k || !cache_v || !pos || !y) {
    set_error("moc_host_attn_step: head_dim must be 8, 16, 32, 64 or 128, t_max <= 11000, no null pointers");
    return kErrInvalidArg;
  }
  if (batch == 0) return kOk;
  const size_t smem = static_cast<size_t>(t_max) * 4;
  host_attn_step_kernel<<<static_cast<unsigned>(batch * heads), kAttnThreads, smem,
                          reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const hbf*>(q), static_cast<const hbf*>(cache_k), static_cast<const hbf*>(cache_v), pos,
      static_cast<hbf*>(y), static_cast<int>(heads), static_cast<int>(head_dim), static_cast<int>(t_max),
      rsqrtf(static_cast<float>(head_dim)));
  return check_last("moc_host_attn_step");
}

}  // extern "C"
