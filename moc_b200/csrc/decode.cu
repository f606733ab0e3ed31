// Decode-time MoC FFN kernels (bf16, batches of a few token rows): bandwidth-bound streaming and
// gathering of weight rows with 128-bit coalesced loads and fp32 accumulation.
//
//   decode_gemv_kernel     : out[b, f] = x[b, :] . W[f, :] for every row f of W (the gate projection,
//                            nn.Linear in moc/inference/inference_ffn.py:188, or gate and up
//                            together for the dense baseline, inference_ffn.py:164-167)
//   decode_sel_up_kernel   : z[b, k] = SiLU(g[b, k]) * (x[b, :] . W_up[idx[b, k], :]) - one warp per selected
//                            channel (selected_up_silu_*_kernel,
//                            moc/inference/cuda/optimized_global_moc_ext.cu:127-245)
//   decode_z_from_u_kernel : same from a dense U row, used when the batch selects more rows than W_up has
//   decode_down_kernel     : partial[s, b, :] = sum over a slice of k of z[b, k] * W_down^T[idx[b, k], :]
//                            (selected_down_*_tile_kernel, optimized_global_moc_ext.cu:247-372; split-K as
//                            in moc/inference/triton_fused_ffn_kernels.py:315-370 but without atomics)
//   decode_reduce_kernel   : y[b, :] = round(sum over s of partial[s, b, :]), fixed summation order
//   skinny_consume_kernel  : batches of 16 rows and more: the three projections run as skinny split-K products on
//                            the tcgen05 core (one 128-row tile and K range per SM, each weight matrix streamed
//                            once); this kernel reduces the up (and gate) partial blocks, applies SiLU, the product
//                            and the selection bitmap and writes the dense zero-filled Z' that the down product reads
//
// Rounding points follow the dense masking reference (inference_ffn.py:169-180) with bf16 tensors:
// gate scores, U, s = SiLU(g), z = s * u and y are each rounded to bf16 once.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "common.cuh"
#include "internal.h"

namespace moc {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ void unpack8(const uint4& q, float (&v)[8]) {
  const uint32_t a[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(a[j] << 16);
    v[2 * j + 1] = __uint_as_float(a[j] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ float bf16_round(float v) { return Num<bf16>::round(v); }
__device__ __forceinline__ float bf16_load(const bf16* p) { return __bfloat162float(*p); }

constexpr int kGemvWarps = 8;
constexpr int kGemvRowsPerWarp = 2;
constexpr int kGemvRowsPerCta = kGemvWarps * kGemvRowsPerWarp;

// BT batch rows of x (a tile of the batch) stay in shared memory; every warp streams two weight rows
// at a time and reuses each x vector for both. FUSED: rows of W_gate and W_up are streamed together and
// out = round(round(SiLU(round(g))) * round(u)) (dense SwiGLU); otherwise out = round(x . W[f]).
template <int BT, bool FUSED>
__global__ void __launch_bounds__(kGemvWarps * 32)
decode_gemv_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ w2,
                   bf16* __restrict__ out, int64_t ld_out, int batch, int d, int rows) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  uint4* xs = reinterpret_cast<uint4*>(gemv_smem);   // [BT][d / 8]; unused for BT <= 2 (x read through L1)
  const int nvec = d >> 3;
  const int b0 = blockIdx.y * BT;
  if (BT > 2) {
    for (int i = threadIdx.x; i < BT * nvec; i += blockDim.x) {
      const int b = i / nvec, v = i - b * nvec;
      xs[i] = (b0 + b < batch) ? reinterpret_cast<const uint4*>(x + static_cast<int64_t>(b0 + b) * d)[v]
                               : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = blockIdx.x * kGemvRowsPerCta + warp * kGemvRowsPerWarp;
  if (f0 >= rows) return;
  const int f1 = min(f0 + 1, rows - 1);   // a clamped duplicate row when the count is odd
  const uint4* wr0 = reinterpret_cast<const uint4*>(w + static_cast<int64_t>(f0) * d);
  const uint4* wr1 = reinterpret_cast<const uint4*>(w + static_cast<int64_t>(f1) * d);
  const uint4* ur0 = FUSED ? reinterpret_cast<const uint4*>(w2 + static_cast<int64_t>(f0) * d) : nullptr;
  const uint4* ur1 = FUSED ? reinterpret_cast<const uint4*>(w2 + static_cast<int64_t>(f1) * d) : nullptr;
  float acc0[BT], acc1[BT], uac0[FUSED ? BT : 1], uac1[FUSED ? BT : 1];
#pragma unroll
  for (int b = 0; b < BT; ++b) {
    acc0[b] = 0.0f;
    acc1[b] = 0.0f;
    if (FUSED) {
      uac0[b] = 0.0f;
      uac1[b] = 0.0f;
    }
  }
#pragma unroll(FUSED ? 4 : 8)
  for (int v = lane; v < nvec; v += 32) {
    float a0[8], a1[8], c0[8], c1[8];
    unpack8(wr0[v], a0);
    unpack8(wr1[v], a1);
    if (FUSED) {
      unpack8(ur0[v], c0);
      unpack8(ur1[v], c1);
    }
#pragma unroll
    for (int b = 0; b < BT; ++b) {
      float xv[8];
      if (BT > 2) {
        unpack8(xs[b * nvec + v], xv);
      } else {   // no staging and no barrier in front of the weight stream
        const int bb = min(b0 + b, batch - 1);
        unpack8(__ldg(reinterpret_cast<const uint4*>(x + static_cast<int64_t>(bb) * d) + v), xv);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc0[b] = fmaf(xv[j], a0[j], acc0[b]);
        acc1[b] = fmaf(xv[j], a1[j], acc1[b]);
        if (FUSED) {
          uac0[b] = fmaf(xv[j], c0[j], uac0[b]);
          uac1[b] = fmaf(xv[j], c1[j], uac1[b]);
        }
      }
    }
  }
#pragma unroll
  for (int b = 0; b < BT; ++b) {
    float r0 = warp_sum(acc0[b]), r1 = warp_sum(acc1[b]);
    if (FUSED) {
      const float u0 = bf16_round(warp_sum(uac0[b])), u1 = bf16_round(warp_sum(uac1[b]));
      r0 = silu_round<bf16>(bf16_round(r0)) * u0;
      r1 = silu_round<bf16>(bf16_round(r1)) * u1;
    }
    if (lane == 0 && b0 + b < batch) {
      bf16* o = out + static_cast<int64_t>(b0 + b) * ld_out;
      o[f0] = __float2bfloat16_rn(r0);
      if (f0 + 1 < rows) o[f0 + 1] = __float2bfloat16_rn(r1);
    }
  }
}

// One warp per (b, k): z = round(round(SiLU(g)) * round(x[b] . W_up[idx[b, k]])).
__global__ void __launch_bounds__(256)
decode_sel_up_kernel(const bf16* __restrict__ x, const bf16* __restrict__ g_sel, const int16_t* __restrict__ idx,
                     const bf16* __restrict__ w_up, bf16* __restrict__ z, int batch, int d, int k) {
  const int64_t wid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<int64_t>(batch) * k) return;
  const int b = static_cast<int>(wid / k);
  const int row = idx[wid];
  const uint4* wr = reinterpret_cast<const uint4*>(w_up + static_cast<int64_t>(row) * d);
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(b) * d);
  const int nvec = d >> 3;
  float acc = 0.0f;
#pragma unroll 4
  for (int v = lane; v < nvec; v += 32) {
    float a[8], xv[8];
    unpack8(wr[v], a);
    unpack8(xr[v], xv);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc = fmaf(xv[j], a[j], acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const float s = silu_round<bf16>(bf16_load(g_sel + wid));
    z[wid] = __float2bfloat16_rn(s * bf16_round(acc));
  }
}

// z[b, k] = round(round(SiLU(g[b, k])) * U[b, idx[b, k]]) from a dense (already rounded) U.
__global__ void decode_z_from_u_kernel(const bf16* __restrict__ u, int64_t ld_u, const bf16* __restrict__ g_sel,
                                       const int16_t* __restrict__ idx, bf16* __restrict__ z, int batch, int k) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(batch) * k) return;
  const int b = static_cast<int>(i / k);
  const float s = silu_round<bf16>(bf16_load(g_sel + i));
  z[i] = __float2bfloat16_rn(s * bf16_load(u + static_cast<int64_t>(b) * ld_u + idx[i]));
}

// Consumers of the split-K partial blocks of a skinny product (element [i][b] of block s at (s * rows + i) * ldp
// + b, i = weight row, b = batch row). Both read the blocks along b (coalesced), turn 32 x 32 tiles in shared
// memory and write bf16 rows out[b, i] along i (coalesced).
//   MODE 0: out[b, i] = round(sum_s P[s][i][b])                                   (gate scores, y)
//   MODE 1: Z'[b, f] = mask ? round(round(SiLU(g)) * round(sum_s U[s][f][b])) : 0 for f < ld (zero beyond d_ffn);
//           g from bf16 score rows, or round(sum_s G[s][f][b]) for the dense baseline; bitmap null: every channel.
template <int MODE>
__global__ void __launch_bounds__(256)
skinny_consume_kernel(const float* __restrict__ p0, const float* __restrict__ p1, int splits, int rows, int batch,
                      int64_t ldp, bf16* __restrict__ out, int64_t ld_out, int out_cols, const bf16* __restrict__ g_rows,
                      int64_t ld_g, const uint32_t* __restrict__ bitmap, int words) {
  __shared__ float tile0[32][33];
  __shared__ float tile1[MODE == 1 ? 32 : 1][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  const int i0 = blockIdx.x * 32, b0 = blockIdx.y * 32;
  const int64_t block = static_cast<int64_t>(rows) * ldp;
  {
    // the four rows of a thread are loaded together for every split: independent loads, one round trip per split
    float v0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, v1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const int b = b0 + tx;
    for (int sidx = 0; sidx < splits; ++sidx) {
      float t0[4], t1[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = i0 + ty + 8 * k;
        const bool ok = i < rows && b < batch;
        const int64_t at = sidx * block + static_cast<int64_t>(ok ? i : 0) * ldp + (ok ? b : 0);
        t0[k] = ok ? __ldcs(p0 + at) : 0.0f;
        t1[k] = (MODE == 1 && p1 && ok) ? __ldcs(p1 + at) : 0.0f;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v0[k] += t0[k];
        v1[k] += t1[k];
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      tile0[ty + 8 * k][tx] = v0[k];
      if (MODE == 1) tile1[ty + 8 * k][tx] = v1[k];
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 32; k += 8) {
    const int b = b0 + ty + k, i = i0 + tx;
    if (b >= batch || i >= out_cols) continue;
    float r = 0.0f;
    if (MODE == 0) {
      r = tile0[tx][ty + k];
    } else if (i < rows && (!bitmap || ((bitmap[static_cast<int64_t>(b) * words + (i >> 5)] >> (i & 31)) & 1u))) {
      const float u = bf16_round(tile0[tx][ty + k]);
      const float g = p1 ? bf16_round(tile1[tx][ty + k]) : bf16_load(g_rows + static_cast<int64_t>(b) * ld_g + i);
      r = silu_round<bf16>(g) * u;
    }
    out[static_cast<int64_t>(b) * ld_out + i] = __float2bfloat16_rn(r);
  }
}

template <int MODE>
static int launch_skinny_consume(const float* p0, const float* p1, int splits, int rows, int batch, bf16* out,
                                 int64_t ld_out, int out_cols, const bf16* g_rows, int64_t ld_g,
                                 const uint32_t* bitmap, int words, cudaStream_t stream) {
  const dim3 grid(ceil_div_i(out_cols, 32), ceil_div_i(batch, 32));
  skinny_consume_kernel<MODE><<<grid, 256, 0, stream>>>(p0, p1, splits, rows, batch, round_up_i64(batch, 4), out, ld_out,
                                                       out_cols, g_rows, ld_g, bitmap, words);
  return check_last("skinny_consume");
}

constexpr int kDownMaxRows = 256;

// grid = (splits, d / (THREADS * 8), batch). Each thread owns 8 output columns and walks the rows of
// its k-slice with independent 16-byte loads (unrolled: many loads in flight per thread).
// idx == null: rows are k0, k0 + 1, ... (dense down projection through W_down^T).
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
decode_down_kernel(const bf16* __restrict__ z, const int16_t* __restrict__ idx, const bf16* __restrict__ w_down_t,
                   float* __restrict__ partial, int batch, int k, int d, int rows_per_split) {
  __shared__ int rows[kDownMaxRows];
  __shared__ float zs[kDownMaxRows];
  const int b = blockIdx.z, s = blockIdx.x;
  const int k0 = s * rows_per_split;
  const int n = min(rows_per_split, k - k0);
  for (int i = threadIdx.x; i < n; i += THREADS) {
    rows[i] = idx ? static_cast<int>(idx[static_cast<int64_t>(b) * k + k0 + i]) : k0 + i;
    zs[i] = bf16_load(z + static_cast<int64_t>(b) * k + k0 + i);
  }
  __syncthreads();
  const int col = (blockIdx.y * THREADS + threadIdx.x) * 8;
  if (col >= d) return;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll 8
  for (int i = 0; i < n; ++i) {
    const uint4 q = *reinterpret_cast<const uint4*>(w_down_t + static_cast<int64_t>(rows[i]) * d + col);
    float wv[8];
    unpack8(q, wv);
    const float zv = zs[i];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = fmaf(zv, wv[j], acc[j]);
  }
  float4* out = reinterpret_cast<float4*>(partial + (static_cast<int64_t>(s) * batch + b) * d + col);
  out[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  out[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// y[b, c..c+4) = round(sum_s partial[s, b, c..c+4)). 16 threads share one output vector: thread j sums the
// splits j, j + 16, ... and the 16 sums are added in a fixed tree, so the result does not depend on timing.
constexpr int kReduceLanes = 16;
__global__ void __launch_bounds__(256)
decode_reduce_kernel(const float* __restrict__ partial, bf16* __restrict__ y, int batch, int d, int splits) {
  __shared__ float4 part[256];
  const int64_t n4 = static_cast<int64_t>(batch) * d / 4;
  const int j = threadIdx.x & (kReduceLanes - 1);
  const int64_t i = static_cast<int64_t>(blockIdx.x) * (256 / kReduceLanes) + (threadIdx.x / kReduceLanes);
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (i < n4) {
#pragma unroll 4
    for (int s = j; s < splits; s += kReduceLanes) {
      const float4 p = reinterpret_cast<const float4*>(partial)[static_cast<int64_t>(s) * n4 + i];
      acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
  }
  part[threadIdx.x] = acc;
  __syncthreads();
#pragma unroll
  for (int o = kReduceLanes / 2; o > 0; o >>= 1) {
    if (j < o) {
      const float4 q = part[threadIdx.x + o];
      acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
      part[threadIdx.x] = acc;
    }
    __syncthreads();
  }
  if (j == 0 && i < n4) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
    reinterpret_cast<uint2*>(y)[i] = o;
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
struct DownPlan {
  int threads;          // 128 or 256
  int dchunks;
  int rows_per_split;
  int splits;
};

static int device_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

static DownPlan plan_down(int batch, int d, int k) {
  DownPlan p;
  p.threads = (batch <= 2 && d <= 4096) ? 128 : 256;
  p.dchunks = ceil_div_i(d, p.threads * 8);
  const int target = device_sms() * 3 / 2;
  int splits = ceil_div_i(target, batch * p.dchunks);
  if (splits < 1) splits = 1;
  int rps = ceil_div_i(k, splits);
  if (rps < 8) rps = 8;
  if (rps > kDownMaxRows) rps = kDownMaxRows;
  p.rows_per_split = rps;
  p.splits = ceil_div_i(k, rps);
  return p;
}

struct DecodeWs {
  int* status;
  bf16* gate;        // [batch, ld]
  bf16* u;           // [batch, ld]
  int16_t* idx;      // [batch, d_ffn]
  bf16* g_sel;       // [batch, d_ffn]
  bf16* z;           // [batch, d_ffn]
  uint32_t* bitmap;  // [batch, words]
  uint16_t* rank0;   // [batch, words]
  float* partial;    // [splits, batch, d]
  int64_t partial_set_bytes;   // bytes of one split-K partial set of a skinny product (0: batch too small for them)
  int* hist;         // single-launch path: [min(batch, 8), 2048] key histograms
  int64_t bytes;
};

// measured at the 1b shape: the skinny tensor-core products win from 16 rows for the MoC paths (56 against 59 us at
// 8 rows) and from 8 rows for the dense baseline (47 against 68 us)
constexpr int kDecodeGemmMinBatch = 16;
constexpr int kDenseGemmMinBatch = 8;
// from this many rows on (beyond the persistent launch): grouped full-K gate + up launch, fused selection, split-K down
constexpr int kWideMinBatch = 9;

// fp32 bytes of the split-K partial blocks of one skinny product over `rows` weight rows: splits * tiles of 128
// rows <= SM count while the tiles fit the SMs, one block of round_up(rows, 128) rows (splits = 1) beyond that
static int64_t splitk_partial_bytes(int64_t batch, int64_t rows) {
  const int64_t by_sms = (static_cast<int64_t>(device_sms()) + 2) * 128;
  const int64_t by_rows = round_up_i64(rows, 128);
  return (by_sms > by_rows ? by_sms : by_rows) * round_up_i64(batch, 4) * 4;
}

static int64_t partial_bound(int64_t batch, int64_t d, int64_t d_ffn) {
  // plan_down: splits <= target / (batch * dchunks) + 2, or ceil(k / kDownMaxRows) when the slice cap binds
  const int64_t by_target = static_cast<int64_t>(device_sms()) * 3 / 2 + 2 * batch + 8;
  const int64_t by_cap = batch * ((d_ffn + kDownMaxRows - 1) / kDownMaxRows + 1);
  const int64_t gather = (by_target > by_cap ? by_target : by_cap) * d * 4;
  // batches that go through the split-K GEMMs keep two partial sets (gate and up of the dense baseline)
  const int64_t skinny =
      batch >= kDenseGemmMinBatch ? 2 * round_up_i64(splitk_partial_bytes(batch, d_ffn > d ? d_ffn : d), 256) : 0;
  // the single persistent launch keeps one fp32 partial output per CTA
  const bool stream = decode_stream_supported(batch, d, d_ffn, 0) || decode_stream_supported(batch, d, d_ffn, 1) ||
                      decode_stream_supported(batch, d, d_ffn, 2);
  const int64_t persistent = stream ? decode_stream_partial_bytes(batch, d) : 0;
  const int64_t m = gather > skinny ? gather : skinny;
  return m > persistent ? m : persistent;
}

static DecodeWs carve(void* base, int64_t batch, int64_t d, int64_t d_ffn) {
  DecodeWs w;
  const int64_t ld = ffn_ld(d_ffn), words = mask_words(d_ffn);
  uint8_t* p = static_cast<uint8_t*>(base);
  auto take = [&](int64_t nbytes) {
    uint8_t* r = p;
    p += round_up_i64(nbytes, 256);
    return r;
  };
  w.status = reinterpret_cast<int*>(take(256));
  // directly behind the status area: one memset clears both before a single-launch call
  w.hist = reinterpret_cast<int*>(take((batch < 8 ? batch : 8) * 2048 * 4));
  w.gate = reinterpret_cast<bf16*>(take(batch * ld * 2));
  w.u = reinterpret_cast<bf16*>(take(batch * ld * 2));
  w.idx = reinterpret_cast<int16_t*>(take(batch * d_ffn * 2));
  w.g_sel = reinterpret_cast<bf16*>(take(batch * d_ffn * 2));
  w.z = reinterpret_cast<bf16*>(take(batch * d_ffn * 2));
  w.bitmap = reinterpret_cast<uint32_t*>(take(batch * words * 4));
  w.rank0 = reinterpret_cast<uint16_t*>(take(batch * words * 2));
  w.partial = reinterpret_cast<float*>(take(partial_bound(batch, d, d_ffn)));
  w.partial_set_bytes =
      batch >= kDenseGemmMinBatch ? round_up_i64(splitk_partial_bytes(batch, d_ffn > d ? d_ffn : d), 256) : 0;
  w.bytes = p - static_cast<uint8_t*>(base);
  return w;
}

int64_t decode_workspace_bytes(int64_t batch, int64_t d, int64_t d_ffn) {
  return carve(nullptr, batch, d, d_ffn).bytes;
}

template <bool FUSED>
static int launch_gemv(const bf16* x, const bf16* w, const bf16* w2, bf16* out, int64_t ld_out, int batch, int d,
                       int rows, cudaStream_t stream) {
  const int bt = batch >= 8 ? 8 : (batch >= 4 ? 4 : (batch >= 2 ? 2 : 1));
  const dim3 grid(ceil_div_i(rows, kGemvRowsPerCta), ceil_div_i(batch, bt));
  const size_t smem = static_cast<size_t>(bt) * d * 2;
  prof_mark(kProfDecodeGate, stream);
#define MOC_GEMV(BT)                                                                                              \
  do {                                                                                                            \
    auto kern = decode_gemv_kernel<BT, FUSED>;                                                                    \
    if (smem > 48 * 1024 &&                                                                                       \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=        \
            cudaSuccess)                                                                                          \
      return check_last("decode_gemv smem attribute");                                                            \
    kern<<<grid, kGemvWarps * 32, smem, stream>>>(x, w, w2, out, ld_out, batch, d, rows);                         \
  } while (0)
  if (bt == 8) MOC_GEMV(8);
  else if (bt == 4) MOC_GEMV(4);
  else if (bt == 2) MOC_GEMV(2);
  else MOC_GEMV(1);
#undef MOC_GEMV
  return check_last("decode_gemv");
}

// Skinny product on the tensor cores for batches of 16 rows and more: P[s][i][b] = partial sums over the s-th range
// of K of A[i, :] . Bt[b, :], with A the weight matrix ([rows, K] K-major, or [K, rows] when a_mn) and Bt the
// [batch, K] activations. The single-CTA tcgen05 kernel runs rows / 128 tiles x `splits` K ranges so that about
// one tile per SM streams the weights once; the caller reduces the partial blocks (launch_splitk_reduce or a
// consumer kernel). ldp = round_up(batch, 4) floats per partial row.
static int skinny_splits(int rows, int k) {
  const int tiles = ceil_div_i(rows, 128);
  const int kb = ceil_div_i(k, 64);
  int splits = device_sms() / tiles;
  if (splits < 1) splits = 1;
  if (splits > kb) splits = kb;
  while (splits > 1 && ceil_div_i(kb, splits) * (splits - 1) >= kb) --splits;   // every range gets a k-block
  return splits;
}

static int skinny_gemm(const bf16* a, int64_t lda, int a_mn, const bf16* bt, int64_t ldb, int rows, int batch, int k,
                       float* partial, int64_t partial_bytes, int* splits_out, int* status, cudaStream_t stream) {
  GemmProblem p = {};
  p.dtype = kBF16;
  p.status = status;
  p.m = rows;
  p.n = batch;
  p.k0 = k;
  p.groups = 1;
  p.k_splits = skinny_splits(rows, k);
  p.a[0].ptr = a;
  p.a[0].ld = lda;
  p.a[0].mn_major = a_mn;
  p.b[0].ptr = bt;
  p.b[0].ld = ldb;
  p.b[0].mn_major = 0;
  p.epi.kind = kEpiPartialF32;
  p.epi.partial = partial;
  p.epi.ld_partial = round_up_i64(batch, 4);
  *splits_out = p.k_splits;
  if (static_cast<int64_t>(p.k_splits) * round_up_i64(rows, 128) * p.epi.ld_partial * 4 > partial_bytes) {
    set_error("decode: split-K partial blocks (%d x %d rows) exceed their workspace region", p.k_splits, rows);
    return kErrWorkspace;
  }
  return launch_gemm(p, stream);
}

// out[b, f] = round(x[b, :] . W[f, :]) for every row of W: CUDA-core GEMV for small batches, split-K tensor-core
// product plus reduction for batches of 16 rows and more.
static int project_rows(const bf16* x, const bf16* w, bf16* out, int64_t ld_out, int batch, int d, int rows,
                        int* status, float* partial, int64_t partial_bytes, cudaStream_t stream) {
  if (batch < kDecodeGemmMinBatch) return launch_gemv<false>(x, w, nullptr, out, ld_out, batch, d, rows, stream);
  int splits = 1;
  int rc = skinny_gemm(w, d, 0, x, d, rows, batch, d, partial, partial_bytes, &splits, status, stream);
  if (rc != kOk) return rc;
  return launch_skinny_consume<0>(partial, nullptr, splits, rows, batch, out, ld_out, rows, nullptr, 0, nullptr, 0, stream);
}

// y[b, :] = round(sum over f of Z'[b, f] * W_down^T[f, :]) from dense zero-filled Z' rows (leading dimension ld)
static int down_dense(const bf16* z_dense, int64_t ld, const bf16* w_down_t, bf16* y, int batch, int d, int d_ffn,
                      int* status, float* partial, int64_t partial_bytes, cudaStream_t stream) {
  int splits = 1;
  prof_mark(kProfDecodeDown, stream);
  int rc = skinny_gemm(w_down_t, d, 1, z_dense, ld, d, batch, d_ffn, partial, partial_bytes, &splits, status, stream);
  if (rc != kOk) return rc;
  return launch_skinny_consume<0>(partial, nullptr, splits, d, batch, y, d, d, nullptr, 0, nullptr, 0, stream);
}

// z = round(round(SiLU(g)) * u) over n8 vectors of 8 elements (dense baseline for more than 8 rows)
__global__ void __launch_bounds__(256)
decode_swiglu_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, uint4* __restrict__ z, int64_t n8) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float gv[8], uv[8];
  unpack8(g[i], gv);
  unpack8(u[i], uv);
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float s0, z0, s1, z1;
    moc_fwd_point<bf16>(gv[2 * j], uv[2 * j], s0, z0);
    moc_fwd_point<bf16>(gv[2 * j + 1], uv[2 * j + 1], s1, z1);
    o[j] = (__float_as_uint(z0) >> 16) | (__float_as_uint(z1) & 0xFFFF0000u);   // both already bf16 values
  }
  z[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// G[b, f] = round(x[b] . W_gate[f]) and U[b, f] = round(x[b] . W_up[f]) for every channel, as ONE grouped launch of
// the single-CTA tcgen05 kernel with the weights as the M operand (128-row tiles, full K, MMA N = batch rounded up
// to 16) and a transposed store: each weight matrix is streamed once, no split-K partial blocks. Either weight may
// be null (that product is skipped).
static int gate_up_rows(const bf16* x, const bf16* w_gate, const bf16* w_up, bf16* g_out, bf16* u_out, int64_t ld,
                        int batch, int d, int d_ffn, int* status, cudaStream_t stream) {
  GemmProblem p = {};
  p.dtype = kBF16;
  p.impl = 3;
  p.status = status;
  p.m = d_ffn;
  p.n = batch;
  p.k0 = d;
  p.epi.kind = kEpiStore;
  int g = 0;
  const bf16* w[2] = {w_gate, w_up};
  bf16* out[2] = {g_out, u_out};
  for (int i = 0; i < 2; ++i) {
    if (!w[i]) continue;
    p.a[g].ptr = w[i];
    p.a[g].ld = d;
    p.a[g].mn_major = 0;
    p.b[g].ptr = x;
    p.b[g].ld = d;
    p.b[g].mn_major = 0;
    p.epi.c[g] = out[i];
    p.epi.ldc[g] = ld;
    p.epi.transposed[g] = 1;
    ++g;
  }
  if (g == 0) return kOk;
  p.groups = g;
  prof_mark(kProfDecodeGate, stream);
  return launch_gemm(p, stream);
}

static int launch_down(const bf16* z, const int16_t* idx, const bf16* w_down_t, bf16* y, float* partial, int batch,
                       int k, int d, cudaStream_t stream) {
  const DownPlan p = plan_down(batch, d, k);
  const dim3 grid(p.splits, p.dchunks, batch);
  prof_mark(kProfDecodeDown, stream);
  if (p.threads == 128)
    decode_down_kernel<128><<<grid, 128, 0, stream>>>(z, idx, w_down_t, partial, batch, k, d, p.rows_per_split);
  else
    decode_down_kernel<256><<<grid, 256, 0, stream>>>(z, idx, w_down_t, partial, batch, k, d, p.rows_per_split);
  int rc = check_last("decode_down");
  if (rc != kOk) return rc;
  const int64_t n4 = static_cast<int64_t>(batch) * d / 4;
  const int64_t per_cta = 256 / kReduceLanes;
  decode_reduce_kernel<<<static_cast<unsigned>((n4 + per_cta - 1) / per_cta), 256, 0, stream>>>(partial, y, batch, d,
                                                                                            p.splits);
  return check_last("decode_reduce");
}

// after the channel set is known: z for the selected channels, then the gathered down projection
static int selected_tail(const DecodeWs& w, const bf16* x, const bf16* scores, int64_t ld_scores, const bf16* w_up,
                         const bf16* w_down_t, bf16* y, int batch, int d, int d_ffn, int k, cudaStream_t stream) {
  int rc;
  const int64_t total = static_cast<int64_t>(batch) * k;
  if (total > d_ffn && batch >= kDecodeGemmMinBatch) {
    // Larger batches select (nearly) every row of W_up and W_down between them: three skinny tensor-core
    // products that stream each weight matrix once, with the mask applied to a dense zero-filled Z'.
    const int64_t ld = ffn_ld(d_ffn);
    int splits = 1;
    float* up_partial = w.partial;
    prof_mark(kProfDecodeUp, stream);
    if ((rc = skinny_gemm(w_up, d, 0, x, d, d_ffn, batch, d, up_partial, w.partial_set_bytes, &splits, w.status,
                          stream)) != kOk)
      return rc;
    if ((rc = launch_skinny_consume<1>(up_partial, nullptr, splits, d_ffn, batch, w.u, ld, static_cast<int>(ld), scores,
                                       ld_scores, w.bitmap, static_cast<int>(mask_words(d_ffn)), stream)) != kOk)
      return rc;
    return down_dense(w.u, ld, w_down_t, y, batch, d, d_ffn, w.status, w.partial, w.partial_set_bytes, stream);
  }
  if (total > d_ffn) {
    // the batch selects more rows than W_up has: one dense pass over W_up, then pick
    if ((rc = project_rows(x, w_up, w.u, ffn_ld(d_ffn), batch, d, d_ffn, w.status, w.partial, w.partial_set_bytes,
                           stream)) != kOk)
      return rc;
    prof_mark(kProfDecodeUp, stream);
    decode_z_from_u_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(w.u, ffn_ld(d_ffn), w.g_sel,
                                                                                         w.idx, w.z, batch, k);
  } else {
    prof_mark(kProfDecodeUp, stream);
    decode_sel_up_kernel<<<static_cast<unsigned>((total * 32 + 255) / 256), 256, 0, stream>>>(x, w.g_sel, w.idx, w_up,
                                                                                              w.z, batch, d, k);
  }
  if ((rc = check_last("decode_up")) != kOk) return rc;
  return launch_down(w.z, w.idx, w_down_t, y, w.partial, batch, k, d, stream);
}

static int check_decode_args(const char* who, int64_t batch, int64_t d, int64_t d_ffn, int64_t k, const void* ws,
                             int64_t ws_bytes) {
  if (batch < 0 || d <= 0 || d_ffn <= 0 || k <= 0 || k > d_ffn) {
    set_error("%s: bad sizes batch=%lld d=%lld d_ffn=%lld k=%lld", who, (long long)batch, (long long)d,
              (long long)d_ffn, (long long)k);
    return kErrInvalidArg;
  }
  if (d % 8 != 0 || d_ffn > 32768 || batch > 65535) {
    set_error("%s: needs d %% 8 == 0, d_ffn <= 32768 and batch <= 65535", who);
    return kErrUnsupported;
  }
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0 || ws_bytes < decode_workspace_bytes(batch, d, d_ffn)) {
    set_error("%s: workspace missing, not 256-byte aligned or smaller than %lld bytes", who,
              (long long)decode_workspace_bytes(batch, d, d_ffn));
    return kErrWorkspace;
  }
  return kOk;
}

// MOC_B200_DECODE_STREAM=0 in the environment keeps small batches off the persistent streaming launch (a switch for
// A/B timing against the older paths).
static bool stream_decode_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("MOC_B200_DECODE_STREAM");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}
// bulk copies read whole weight rows: the matrices must start on 16-byte boundaries (rows are d * 2 bytes, d % 256 == 0)
static bool aligned16(const void* a, const void* b, const void* c) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) == 0;
}

int decode_global(int64_t batch, int64_t d, int64_t d_ffn, int64_t k, int rule, const void* x, const void* gate_scores,
                  const void* w_gate, const void* w_up, const void* w_down_t, void* y, void* workspace,
                  int64_t workspace_bytes, cudaStream_t stream) {
  int rc = check_decode_args("moc_decode", batch, d, d_ffn, k, workspace, workspace_bytes);
  if (rc != kOk) return rc;
  if (batch == 0) return kOk;
  const DecodeWs w = carve(workspace, batch, d, d_ffn);
  if (stream_decode_enabled() && decode_stream_supported(batch, d, d_ffn, rule) &&
      aligned16(gate_scores ? w_up : w_gate, w_up, w_down_t) && (reinterpret_cast<uintptr_t>(x) & 3u) == 0) {
    // up to 8 rows: the whole FFN in one persistent launch that streams every weight row once
    rc = launch_decode_stream(rule, (int)batch, (int)d, (int)d_ffn, (int)k, x, gate_scores, d_ffn, w_gate, w_up,
                              w_down_t, y, w.gate, ffn_ld(d_ffn), w.hist, w.status, w.partial, stream);
    prof_mark(kProfEnd, stream);
    return rc;
  }
  if (cudaMemsetAsync(w.status, 0, 256, stream) != cudaSuccess) return check_last("cudaMemsetAsync");
  const bf16* xb = static_cast<const bf16*>(x);
  if (batch >= kWideMinBatch && aligned16(w_up, w_down_t, x) && (gate_scores || aligned16(w_gate, w_gate, w_gate))) {
    // More than 8 rows: between them the rows select (nearly) every channel, so all three weight matrices are
    // streamed once. Four launches: gate and up projections of every channel in one grouped tensor-core launch,
    // the fused selection of the training forward (the score rows become the zero-filled Z' rows in place), the
    // down projection as a split-K product over Z', and its fixed-order reduction.
    const int64_t ld = ffn_ld(d_ffn);
    if (gate_scores &&
        cudaMemcpy2DAsync(w.gate, ld * 2, gate_scores, d_ffn * 2, d_ffn * 2, batch, cudaMemcpyDeviceToDevice, stream) !=
            cudaSuccess)
      return check_last("decode: copy of the caller's gate scores");
    if ((rc = gate_up_rows(xb, gate_scores ? nullptr : static_cast<const bf16*>(w_gate), static_cast<const bf16*>(w_up),
                           w.gate, w.u, ld, (int)batch, (int)d, (int)d_ffn, w.status, stream)) != kOk)
      return rc;
    SelectFuse fuse{w.u, w.z, nullptr, nullptr, w.status};   // u_sel lands in the z buffer; it is not used further
    if (rule == 0)
      rc = launch_topk_select(kBF16, w.gate, ld, (int)batch, (int)d_ffn, (int)k, &fuse, w.idx, w.g_sel, w.bitmap, w.rank0,
                              stream);
    else
      rc = launch_select_2of8(kBF16, w.gate, ld, (int)batch, (int)d_ffn, &fuse, w.idx, w.g_sel, w.bitmap, w.rank0, stream);
    if (rc != kOk) return rc;
    rc = down_dense(w.gate, ld, static_cast<const bf16*>(w_down_t), static_cast<bf16*>(y), (int)batch, (int)d,
                    (int)d_ffn, w.status, w.partial, w.partial_set_bytes, stream);
    prof_mark(kProfEnd, stream);
    return rc;
  }
  void* scores = w.gate;
  int64_t ld_scores = ffn_ld(d_ffn);
  if (gate_scores) {   // scores computed by the caller: contiguous [batch, d_ffn]
    scores = const_cast<void*>(gate_scores);
    ld_scores = d_ffn;
  } else if ((rc = project_rows(xb, static_cast<const bf16*>(w_gate), w.gate, ld_scores, (int)batch, (int)d,
                                (int)d_ffn, w.status, w.partial, w.partial_set_bytes, stream)) != kOk) {
    return rc;
  }
  if (rule == 0)
    rc = launch_topk_select(kBF16, scores, ld_scores, (int)batch, (int)d_ffn, (int)k, nullptr, w.idx, w.g_sel, w.bitmap,
                            w.rank0, stream);
  else
    rc = launch_select_2of8(kBF16, scores, ld_scores, (int)batch, (int)d_ffn, nullptr, w.idx, w.g_sel, w.bitmap, w.rank0,
                            stream);
  if (rc != kOk) return rc;
  rc = selected_tail(w, xb, static_cast<const bf16*>(scores), ld_scores, static_cast<const bf16*>(w_up),
                     static_cast<const bf16*>(w_down_t), static_cast<bf16*>(y), (int)batch, (int)d, (int)d_ffn, (int)k,
                     stream);
  prof_mark(kProfEnd, stream);
  return rc;
}

int decode_dense(int64_t batch, int64_t d, int64_t d_ffn, const void* x, const void* w_gate, const void* w_up,
                 const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes, cudaStream_t stream) {
  int rc = check_decode_args("moc_decode_dense", batch, d, d_ffn, d_ffn, workspace, workspace_bytes);
  if (rc != kOk) return rc;
  if (batch == 0) return kOk;
  const DecodeWs w = carve(workspace, batch, d, d_ffn);
  if (stream_decode_enabled() && decode_stream_supported(batch, d, d_ffn, 2) && aligned16(w_gate, w_up, w_down_t) &&
      (reinterpret_cast<uintptr_t>(x) & 3u) == 0) {
    rc = launch_decode_stream(2, (int)batch, (int)d, (int)d_ffn, (int)d_ffn, x, nullptr, 0, w_gate, w_up, w_down_t, y,
                              w.gate, ffn_ld(d_ffn), w.hist, w.status, w.partial, stream);
    prof_mark(kProfEnd, stream);
    return rc;
  }
  if (cudaMemsetAsync(w.status, 0, 256, stream) != cudaSuccess) return check_last("cudaMemsetAsync");
  if (batch >= kWideMinBatch && aligned16(w_gate, w_up, w_down_t) && aligned16(x, x, x)) {
    // gate and up of every channel in one grouped launch, SwiGLU elementwise, split-K down projection
    const int64_t ld = ffn_ld(d_ffn);
    if ((rc = gate_up_rows(static_cast<const bf16*>(x), static_cast<const bf16*>(w_gate), static_cast<const bf16*>(w_up),
                           w.gate, w.u, ld, (int)batch, (int)d, (int)d_ffn, w.status, stream)) != kOk)
      return rc;
    const int64_t n8 = batch * ld / 8;
    prof_mark(kProfDecodeDense, stream);
    decode_swiglu_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(w.gate), reinterpret_cast<const uint4*>(w.u), reinterpret_cast<uint4*>(w.gate), n8);
    if ((rc = check_last("decode_swiglu")) != kOk) return rc;
    rc = down_dense(w.gate, ld, static_cast<const bf16*>(w_down_t), static_cast<bf16*>(y), (int)batch, (int)d,
                    (int)d_ffn, w.status, w.partial, w.partial_set_bytes, stream);
    prof_mark(kProfEnd, stream);
    return rc;
  }
  if (batch >= kDenseGemmMinBatch) {
    // three skinny tensor-core products; SwiGLU is applied while the gate and up partial blocks are reduced
    const int64_t ld = ffn_ld(d_ffn);
    const bf16* xb = static_cast<const bf16*>(x);
    float* g_partial = w.partial;
    float* u_partial = w.partial + w.partial_set_bytes / 4;
    int splits = 1, splits_u = 1;
    prof_mark(kProfDecodeDense, stream);
    if ((rc = skinny_gemm(static_cast<const bf16*>(w_gate), d, 0, xb, d, (int)d_ffn, (int)batch, (int)d, g_partial,
                          w.partial_set_bytes, &splits, w.status, stream)) != kOk ||
        (rc = skinny_gemm(static_cast<const bf16*>(w_up), d, 0, xb, d, (int)d_ffn, (int)batch, (int)d, u_partial,
                          w.partial_set_bytes, &splits_u, w.status, stream)) != kOk)
      return rc;
    if ((rc = launch_skinny_consume<1>(u_partial, g_partial, splits, (int)d_ffn, (int)batch, w.u, ld, static_cast<int>(ld),
                                       nullptr, 0, nullptr, 0, stream)) != kOk)
      return rc;
    rc = down_dense(w.u, ld, static_cast<const bf16*>(w_down_t), static_cast<bf16*>(y), (int)batch, (int)d, (int)d_ffn,
                    w.status, w.partial, w.partial_set_bytes, stream);
    prof_mark(kProfEnd, stream);
    return rc;
  }
  // z[b, f] = SiLU(g) * u for every channel, stored with row stride d_ffn so that it reads as a compact z
  if ((rc = launch_gemv<true>(static_cast<const bf16*>(x), static_cast<const bf16*>(w_gate),
                                     static_cast<const bf16*>(w_up), w.z, d_ffn, (int)batch, (int)d, (int)d_ffn,
                                     stream)) != kOk) {
    return rc;
  }
  rc = launch_down(w.z, nullptr, static_cast<const bf16*>(w_down_t), static_cast<bf16*>(y), w.partial, (int)batch,
                   (int)d_ffn, (int)d, stream);
  prof_mark(kProfEnd, stream);
  return rc;
}

int decode_selected_up(int64_t batch, int64_t k, int64_t d, const void* x, const void* g_sel, const int16_t* idx,
                       const void* w_up, void* z, cudaStream_t stream) {
  const int64_t total = batch * k;
  if (total == 0) return kOk;
  prof_mark(kProfDecodeUp, stream);
  decode_sel_up_kernel<<<static_cast<unsigned>((total * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(g_sel), idx, static_cast<const bf16*>(w_up),
      static_cast<bf16*>(z), (int)batch, (int)d, (int)k);
  return check_last("decode_selected_up");
}

int decode_selected_down(int64_t batch, int64_t k, int64_t d, int64_t d_ffn, const void* z, const int16_t* idx,
                         const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes, cudaStream_t stream) {
  int rc = check_decode_args("moc_decode_selected_down", batch, d, d_ffn, k, workspace, workspace_bytes);
  if (rc != kOk) return rc;
  if (batch == 0) return kOk;
  const DecodeWs w = carve(workspace, batch, d, d_ffn);
  return launch_down(static_cast<const bf16*>(z), idx, static_cast<const bf16*>(w_down_t), static_cast<bf16*>(y),
                     w.partial, (int)batch, (int)k, (int)d, stream);
}

}  // namespace moc
