// Decode-time MoC FFN for batches of up to 8 token rows as ONE cooperative kernel launch.
//
// The multi-kernel decode path (decode.cu) spends most of its time between kernels: at batch 1 it moves
// 31 MB, 5 us of HBM time, in five dependent launches. Here every CTA owns a contiguous slice of the d_ffn
// channels and the whole FFN runs in one grid with two grid-wide barriers:
//
//   A  gate scores of the own channels (stream the own W_gate rows once, x in shared memory), rounded to
//      bf16, kept in shared memory and published to global memory together with a global 2048-bin
//      histogram of the upper 11 bits of their order keys                       (inference_ffn.py:188)
//   -- grid barrier (Top-K rule only; the 2:8 rule is local to groups of 8 channels) --
//   B  every CTA finds the K-th largest key redundantly: threshold bin from the global histogram, the
//      lower 5 key bits from one pass over the published scores, ties at the threshold admitted in
//      ascending channel order (optimized_global_moc_ext.cu:85-125 replaced by a radix select)
//   C  u = x . W_up[ch] for the own selected channels, z = round(round(SiLU(g)) * round(u)), published as a
//      compact (channel, z per row) segment per CTA               (optimized_global_moc_ext.cu:127-245)
//   -- grid barrier --
//   D  every CTA concatenates all segments in shared memory (ascending channels) and owns 16 output
//      columns: y[b, cols] = sum over the listed channels of z[b, ch] * W_down^T[ch, cols], 32-byte row
//      segments gathered with 16-byte loads, four in flight per thread, fixed summation order (no float
//      atomics, no partial buffers)                               (optimized_global_moc_ext.cu:247-372)
//
// The grid barriers are generation-free counters in the caller's scratch, zeroed by a memset node before
// the launch; every wait is bounded, a time-out sets the status word and makes all CTAs return.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace moc {

using bf16 = __nv_bfloat16;

constexpr int kFusedThreads = 512;
constexpr int kFusedWarps = kFusedThreads / 32;
constexpr int kFusedBins = 2048;
constexpr int kFusedColsPerCta = 16;
constexpr long long kGridWaitCycles = 400000000LL;   // about 0.2 s

struct FusedArgs {
  const bf16* x;          // [batch, d]
  const bf16* scores;     // caller's gate scores [batch, ld_scores], or null: computed from w_gate
  const bf16* w_gate;     // [d_ffn, d]
  const bf16* w_up;       // [d_ffn, d]
  const bf16* w_down_t;   // [d_ffn, d]
  bf16* y;                // [batch, d]
  bf16* g;                // scratch [batch, ld]: gate scores when computed here
  uint16_t* seg;          // scratch: one compact (channel, z per row) segment per CTA, see phase C
  int* hist;              // scratch [batch, 2048], zeroed before the launch
  unsigned* sync;         // scratch: [0] barrier counter (zeroed before the launch)
  int* status;            // device status word
  int64_t ld_scores, ld;
  int batch, d, d_ffn, k, rule, cpc;
};

__device__ __forceinline__ void unpack8f(const uint4& q, float (&v)[8]) {
  const uint32_t a[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(a[j] << 16);
    v[2 * j + 1] = __uint_as_float(a[j] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ uint16_t bf16_bits(float v) {
  const bf16 h = __float2bfloat16_rn(v);
  return *reinterpret_cast<const uint16_t*>(&h);
}
__device__ __forceinline__ float bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

// All CTAs of the cooperative grid arrive; returns false (in every thread of the CTA) when the wait ran out.
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, int* status) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    __threadfence();
    atomicAdd(counter, 1u);
    const long long t0 = clock64();
    while (true) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
      if (v >= target) break;
      if (clock64() - t0 > kGridWaitCycles) {
        atomicCAS(status, 0, (kDevTimeoutProducer << 24) | 0x00D00000 | static_cast<int>(target & 0xFFFF));
        ok = 0;
        break;
      }
      __nanosleep(20);
    }
    __threadfence();
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

#ifdef MOC_FUSED_TIMING
__device__ unsigned long long g_fused_t[8 * 512];
#define FUSED_STAMP(i)                                                         \
  do {                                                                         \
    if (threadIdx.x == 0) {                                                    \
      unsigned long long t_;                                                   \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                   \
      g_fused_t[blockIdx.x * 8 + (i)] = t_;                                    \
    }                                                                          \
  } while (0)
#else
#define FUSED_STAMP(i)
#endif

// Shared-memory plan (dynamic part): a staging area that is reused phase by phase - the own W_gate slice
// (A), the published score rows (B), the selected W_up rows (C), all segments (D) - followed, for A-C, by the
// x rows, the own scores, the selection flags and the entry positions. Everything is staged with bulk async
// copies (cp.async.bulk, no multicast) on single-use mbarriers, so a CTA has its whole slice in flight at
// once instead of one round trip per row and warp.
constexpr int kFusedRowsPerRound = kFusedWarps;   // A: one barrier per 16 rows, one row per warp and round
constexpr int kFusedMaxRounds = 8;
constexpr uint32_t kBulkChunk = 32768;

struct FusedSmem {
  uint32_t stage_bytes;   // staging area
  uint32_t off_x, off_g, off_sel, off_pos, total;
};

__host__ __device__ inline FusedSmem fused_smem_plan(int bp, int batch, int d, int d_ffn, int cpc, int grid) {
  FusedSmem p;
  const uint32_t slice = static_cast<uint32_t>(cpc) * d * 2;
  const uint32_t rowpad = (static_cast<uint32_t>(d_ffn) + 15u) / 8u * 8u;
  const uint32_t rows = static_cast<uint32_t>(batch) * rowpad * 2;
  uint32_t st = slice > rows ? slice : rows;
  st = (st + 127u) & ~127u;
  p.stage_bytes = st;
  p.off_x = st;
  p.off_g = p.off_x + static_cast<uint32_t>(bp) * d * 2;
  p.off_sel = p.off_g + static_cast<uint32_t>(bp) * cpc * 2;
  p.off_pos = (p.off_sel + static_cast<uint32_t>(bp) * cpc + 1u) & ~1u;
  const uint32_t ac = p.off_pos + static_cast<uint32_t>(cpc) * 2 + 16;
  const uint32_t segs = (static_cast<uint32_t>(grid) * (1 + cpc * (1 + batch)) * 2 + 15u) & ~15u;
  p.total = ac > segs ? ac : segs;
  return p;
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(ptx::smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(ptx::smem_u32(bar))
               : "memory");
}
// contiguous copy of any 16-byte multiple, in chunks; the caller has already announced the bytes on `bar`
__device__ __forceinline__ void bulk_g2s_chunked(uint8_t* dst, const uint8_t* src, uint32_t bytes, uint64_t* bar) {
  for (uint32_t o = 0; o < bytes; o += kBulkChunk) bulk_g2s(dst + o, src + o, min(kBulkChunk, bytes - o), bar);
}

template <int B>
__global__ void __launch_bounds__(kFusedThreads, 1) decode_fused_kernel(const FusedArgs a) {
  extern __shared__ __align__(128) uint8_t fsm[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int batch = a.batch, d = a.d, F = a.d_ffn, cpc = a.cpc;
  const FusedSmem sp = fused_smem_plan(B, batch, d, F, cpc, gridDim.x);
  uint8_t* stage = fsm;
  bf16* xs = reinterpret_cast<bf16*>(fsm + sp.off_x);               // [B][d]
  uint16_t* g_own = reinterpret_cast<uint16_t*>(fsm + sp.off_g);    // [B][cpc] bf16 bits
  uint8_t* sel = fsm + sp.off_sel;                                  // [B][cpc]
  uint16_t* s_pos = reinterpret_cast<uint16_t*>(fsm + sp.off_pos);  // [cpc] entry index of a channel, 0xFFFF: none
  __shared__ uint64_t s_bar_a[kFusedMaxRounds];   // A: W_gate rows, one per round
  __shared__ uint64_t s_bar_x, s_bar_s, s_bar_u, s_bar_d;   // x rows; score rows; W_up rows; segments
  __shared__ int s_abort;
  __shared__ uint32_t s_wsum[B][kFusedWarps];
  __shared__ uint32_t s_hist2[B][32];
  __shared__ uint32_t s_thr[B], s_take[B], s_eqb[B], s_d1[B], s_krem[B];
  __shared__ uint32_t s_nsel;
  __shared__ uint32_t s_off[kFusedThreads + 1];
  __shared__ float s_red[kFusedWarps][2][B][8];

  const int ch0 = blockIdx.x * cpc;
  const int ncl = max(0, min(cpc, F - ch0));
  const int nvec = d >> 3;
  const uint32_t row_bytes = static_cast<uint32_t>(d) * 2;
  unsigned barrier_no = 0;
  volatile int* abort_flag = &s_abort;
#define FUSED_WAIT(bar)                                                                      \
  do {                                                                                       \
    const bool ok_ = ptx::mbar_wait((bar), 0u, abort_flag);                                  \
    if (!ok_) {                                                                              \
      *abort_flag = 1;                                                                       \
      atomicCAS(a.status, 0, (kDevTimeoutEpilogue << 24) | 0x00D00000 | (__LINE__ & 0xFFFF)); \
    }                                                                                        \
  } while (0)

  FUSED_STAMP(0);
  // ---------------- A: x and the own W_gate slice to shared memory, own gate scores, histogram ----------------
  if (tid == 0) {
    for (int r = 0; r < kFusedMaxRounds; ++r) ptx::mbar_init(&s_bar_a[r], 1);
    ptx::mbar_init(&s_bar_x, 1);
    ptx::mbar_init(&s_bar_s, 1);
    ptx::mbar_init(&s_bar_u, 1);
    ptx::mbar_init(&s_bar_d, 1);
    s_abort = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
    const uint32_t xbytes = static_cast<uint32_t>(batch) * row_bytes;
    ptx::mbar_arrive_expect_tx(&s_bar_x, xbytes);
    bulk_g2s_chunked(reinterpret_cast<uint8_t*>(xs), reinterpret_cast<const uint8_t*>(a.x), xbytes, &s_bar_x);
    if (!a.scores) {
      for (int l0 = 0, r = 0; l0 < ncl; l0 += kFusedRowsPerRound, ++r) {
        const int n = min(kFusedRowsPerRound, ncl - l0);
        ptx::mbar_arrive_expect_tx(&s_bar_a[r], static_cast<uint32_t>(n) * row_bytes);
        for (int i = 0; i < n; ++i)
          bulk_g2s(stage + static_cast<size_t>(l0 + i) * row_bytes, a.w_gate + static_cast<int64_t>(ch0 + l0 + i) * d,
                   row_bytes, &s_bar_a[r]);
      }
    }
  }
  __syncthreads();   // barriers initialised
  FUSED_WAIT(&s_bar_x);
  if (a.scores) {
    for (int i = tid; i < batch * ncl; i += kFusedThreads) {
      const int b = i / ncl, lc = i - b * ncl;
      const bf16 v = a.scores[static_cast<int64_t>(b) * a.ld_scores + ch0 + lc];
      const uint16_t bits = *reinterpret_cast<const uint16_t*>(&v);
      g_own[b * cpc + lc] = bits;
      if (a.rule == 0) atomicAdd(&a.hist[b * kFusedBins + (order_key16(bits) >> 5)], 1);
    }
  } else {
    for (int lc = warp, r = 0; lc < ncl; lc += kFusedWarps, ++r) {
      FUSED_WAIT(&s_bar_a[r]);
      const uint4* wrow = reinterpret_cast<const uint4*>(stage + static_cast<size_t>(lc) * row_bytes);
      float acc[B];
#pragma unroll
      for (int b = 0; b < B; ++b) acc[b] = 0.0f;
      for (int v = lane; v < nvec; v += 32) {
        float w[8];
        unpack8f(wrow[v], w);
#pragma unroll
        for (int b = 0; b < B; ++b) {
          if (b < batch) {
            float xv[8];
            unpack8f(reinterpret_cast<const uint4*>(xs + static_cast<size_t>(b) * d)[v], xv);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[b] = fmaf(w[j], xv[j], acc[b]);
          }
        }
      }
#pragma unroll
      for (int b = 0; b < B; ++b) {
        if (b < batch) {
          const float s = warp_sum_f(acc[b]);
          if (lane == 0) {
            const uint16_t bits = bf16_bits(s);
            g_own[b * cpc + lc] = bits;
            reinterpret_cast<uint16_t*>(a.g)[static_cast<int64_t>(b) * a.ld + ch0 + lc] = bits;
            if (a.rule == 0) atomicAdd(&a.hist[b * kFusedBins + (order_key16(bits) >> 5)], 1);
          }
        }
      }
    }
  }

  // ---------------- B: selection ----------------
  FUSED_STAMP(1);
  if (a.rule == 0) {
    if (!grid_barrier(a.sync, ++barrier_no * gridDim.x, a.status)) return;
    FUSED_STAMP(2);
    // score rows of the whole batch into the staging area (the W_gate slice is no longer needed)
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(a.scores ? a.scores : a.g);
    const int64_t lds = a.scores ? a.ld_scores : a.ld;
    const uint32_t rowpad = (static_cast<uint32_t>(F) + 15u) / 8u * 8u;
    uint16_t* srow = reinterpret_cast<uint16_t*>(stage);   // [batch][rowpad]
    const bool bulk_rows = !a.scores;                      // own rows start on 256-byte boundaries
    if (bulk_rows) {
      if (tid == 0) {
        ptx::fence_proxy_async_smem();
        const uint32_t rb = (static_cast<uint32_t>(F) * 2 + 15u) & ~15u;
        ptx::mbar_arrive_expect_tx(&s_bar_s, rb * batch);
        for (int b = 0; b < batch; ++b)
          bulk_g2s(srow + static_cast<size_t>(b) * rowpad, sc + static_cast<int64_t>(b) * lds, rb, &s_bar_s);
      }
    } else {
      for (int b = 0; b < batch; ++b)
        for (int i = tid; i < F; i += kFusedThreads) srow[b * rowpad + i] = __ldcg(sc + static_cast<int64_t>(b) * lds + i);
    }
    // threshold bin of every row from the global histogram: thread t owns 4 bins counted from the top
    const int base = kFusedBins - 4 * (tid + 1);
    uint32_t c[B][4], inc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      int4 c4 = make_int4(0, 0, 0, 0);
      if (b < batch) c4 = __ldcg(reinterpret_cast<const int4*>(a.hist + b * kFusedBins + base));
      c[b][0] = c4.x; c[b][1] = c4.y; c[b][2] = c4.z; c[b][3] = c4.w;
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
      uint32_t v = c[b][0] + c[b][1] + c[b][2] + c[b][3];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t nb = __shfl_up_sync(0xFFFFFFFFu, v, o);
        if (lane >= o) v += nb;
      }
      inc[b] = v;
      if (lane == 31) s_wsum[b][warp] = v;
    }
    for (int i = tid; i < B * 32; i += kFusedThreads) (&s_hist2[0][0])[i] = 0u;
    __syncthreads();
    const uint32_t kk = static_cast<uint32_t>(a.k);
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (b < batch) {
        uint32_t woff = 0;
#pragma unroll
        for (int i = 0; i < kFusedWarps; ++i)
          if (i < warp) woff += s_wsum[b][i];
        const uint32_t local = c[b][0] + c[b][1] + c[b][2] + c[b][3];
        uint32_t above = woff + inc[b] - local;
        if (above < kk && above + local >= kk) {
#pragma unroll
          for (int j = 3; j >= 0; --j) {
            if (above + c[b][j] >= kk) {
              s_d1[b] = static_cast<uint32_t>(base + j);
              s_krem[b] = kk - above;
              break;
            }
            above += c[b][j];
          }
        }
      }
    }
    if (bulk_rows) FUSED_WAIT(&s_bar_s);
    __syncthreads();
    // lower 5 key bits among the keys of the threshold bin
    for (int i = tid; i < F; i += kFusedThreads) {
#pragma unroll
      for (int b = 0; b < B; ++b) {
        if (b < batch) {
          const uint32_t key = order_key16(srow[b * rowpad + i]);
          if ((key >> 5) == s_d1[b]) atomicAdd(&s_hist2[b][key & 31u], 1u);
        }
      }
    }
    __syncthreads();
    if (warp < batch) {
      const int b = warp;
      const uint32_t cc = s_hist2[b][31 - lane];
      uint32_t v = cc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t nb = __shfl_up_sync(0xFFFFFFFFu, v, o);
        if (lane >= o) v += nb;
      }
      const uint32_t ex = v - cc, krem = s_krem[b];
      if (ex < krem && ex + cc >= krem) {
        s_thr[b] = (s_d1[b] << 5) | static_cast<uint32_t>(31 - lane);
        s_take[b] = krem - ex;      // ties admitted, lowest channels first
      }
      if (lane == 0) s_eqb[b] = 0u;
    }
    __syncthreads();
    // ties at the threshold key below the own slice
    {
      const int lim = min(ch0, F);
#pragma unroll
      for (int b = 0; b < B; ++b) {
        if (b < batch) {
          const uint32_t thr = s_thr[b];
          uint32_t cnt = 0;
          for (int i = tid; i < lim; i += kFusedThreads) cnt += (order_key16(srow[b * rowpad + i]) == thr) ? 1u : 0u;
          cnt = __reduce_add_sync(0xFFFFFFFFu, cnt);
          if (lane == 0 && cnt) atomicAdd(&s_eqb[b], cnt);
        }
      }
    }
    __syncthreads();
    if (tid < batch) {
      const int b = tid;
      const uint32_t thr = s_thr[b], take = s_take[b];
      uint32_t seen = s_eqb[b];
      for (int lc = 0; lc < ncl; ++lc) {
        const uint32_t key = order_key16(g_own[b * cpc + lc]);
        bool s = key > thr;
        if (key == thr) {
          s = seen < take;
          ++seen;
        }
        sel[b * cpc + lc] = s ? 1 : 0;
      }
    }
  } else {
    // top-2 of every 8 channels, lower channel wins ties; slices start on multiples of 8
    __syncthreads();
    const int groups = (ncl + 7) >> 3;
    for (int i = tid; i < batch * groups; i += kFusedThreads) {
      const int b = i / groups, gi = i - b * groups;
      const int c0 = gi * 8, nv = min(8, ncl - c0);
      uint32_t key[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) key[j] = j < nv ? order_key16(g_own[b * cpc + c0 + j]) : 0u;
      int b1 = 0;
#pragma unroll
      for (int j = 1; j < 8; ++j)
        if (j < nv && key[j] > key[b1]) b1 = j;
      int b2 = -1;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nv && j != b1 && (b2 < 0 || key[j] > key[b2])) b2 = j;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nv) sel[b * cpc + c0 + j] = (j == b1 || j == b2) ? 1 : 0;
    }
  }
  __syncthreads();

  FUSED_STAMP(3);
  // ---------------- C: z of the own selected channels -> compact segment of this CTA ----------------
  // Segment layout (16-bit words): [0] number of entries, then per entry the channel and z of every batch row,
  // in ascending channel order. Only channels that some row selected get an entry. The selected W_up rows are
  // staged at their entry positions.
  const int ewords = 1 + batch;
  const int segw = 1 + cpc * ewords;
  uint16_t* seg = a.seg + static_cast<int64_t>(blockIdx.x) * segw;
  if (warp == 0) {
    uint32_t run = 0;
    for (int l0 = 0; l0 < ncl; l0 += 32) {
      const int lc = l0 + lane;
      bool any = false;
      if (lc < ncl)
        for (int b2 = 0; b2 < batch; ++b2) any = any || sel[b2 * cpc + lc] != 0;
      const uint32_t m = __ballot_sync(0xFFFFFFFFu, any);
      if (lc < ncl) s_pos[lc] = any ? static_cast<uint16_t>(run + __popc(m & ((1u << lane) - 1u))) : uint16_t(0xFFFF);
      run += __popc(m);
    }
    __syncwarp();
    if (lane == 0) {
      seg[0] = static_cast<uint16_t>(run);
      s_nsel = run;
      if (run) {
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive_expect_tx(&s_bar_u, run * row_bytes);
        for (int lc = 0; lc < ncl; ++lc) {
          const uint32_t pos = s_pos[lc];
          if (pos != 0xFFFFu)
            bulk_g2s(stage + static_cast<size_t>(pos) * row_bytes, a.w_up + static_cast<int64_t>(ch0 + lc) * d, row_bytes,
                     &s_bar_u);
        }
      }
    }
  }
  __syncthreads();
  if (s_nsel) FUSED_WAIT(&s_bar_u);
  for (int lc = warp; lc < ncl; lc += kFusedWarps) {
    const uint32_t pos = s_pos[lc];
    if (pos == 0xFFFFu) continue;
    uint32_t mask = 0;
#pragma unroll
    for (int b = 0; b < B; ++b)
      if (b < batch && sel[b * cpc + lc]) mask |= 1u << b;
    const uint4* wrow = reinterpret_cast<const uint4*>(stage + static_cast<size_t>(pos) * row_bytes);
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.0f;
    for (int v = lane; v < nvec; v += 32) {
      float w[8];
      unpack8f(wrow[v], w);
#pragma unroll
      for (int b = 0; b < B; ++b) {
        if ((mask >> b) & 1u) {
          float xv[8];
          unpack8f(reinterpret_cast<const uint4*>(xs + static_cast<size_t>(b) * d)[v], xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[b] = fmaf(w[j], xv[j], acc[b]);
        }
      }
    }
    uint16_t* entry = seg + 1 + pos * ewords;
    if (lane == 0) entry[0] = static_cast<uint16_t>(ch0 + lc);
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (b < batch) {
        uint16_t zb = 0;
        if ((mask >> b) & 1u) {
          const float u = Num<bf16>::round(warp_sum_f(acc[b]));
          float sv, zv;
          moc_fwd_point<bf16>(bits_to_float(g_own[b * cpc + lc]), u, sv, zv);
          zb = bf16_bits(zv);
        }
        if (lane == 0) entry[1 + b] = zb;
      }
    }
  }
  FUSED_STAMP(4);
  if (!grid_barrier(a.sync, ++barrier_no * gridDim.x, a.status)) return;
  FUSED_STAMP(5);

  // ---------------- D: gathered down projection, 16 output columns per CTA ----------------
  // all segments into shared memory (they are contiguous in global memory), entry e of the concatenation is
  // found through the prefix sums of the segment counts
  const uint16_t* raw = reinterpret_cast<const uint16_t*>(fsm);
  if (tid == 0) {
    ptx::fence_proxy_async_smem();
    const uint32_t bytes = (static_cast<uint32_t>(gridDim.x) * segw * 2 + 15u) & ~15u;
    ptx::mbar_arrive_expect_tx(&s_bar_d, bytes);
    bulk_g2s_chunked(fsm, reinterpret_cast<const uint8_t*>(a.seg), bytes, &s_bar_d);
  }
  FUSED_WAIT(&s_bar_d);
  if (__syncthreads_or(s_abort)) return;
  uint32_t n_total;
  {
    const uint32_t cnt = tid < static_cast<int>(gridDim.x) ? raw[static_cast<size_t>(tid) * segw] : 0u;
    uint32_t v = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t nb = __shfl_up_sync(0xFFFFFFFFu, v, o);
      if (lane >= o) v += nb;
    }
    if (lane == 31) s_wsum[0][warp] = v;
    __syncthreads();
    uint32_t woff = 0, tot = 0;
#pragma unroll
    for (int i = 0; i < kFusedWarps; ++i) {
      const uint32_t s = s_wsum[0][i];
      if (i < warp) woff += s;
      tot += s;
    }
    n_total = tot;
    s_off[tid] = woff + v - cnt;
    if (tid == kFusedThreads - 1) s_off[kFusedThreads] = tot;
    __syncthreads();
  }
  FUSED_STAMP(6);
  const int r = tid >> 1, h = tid & 1;            // 256 entry lanes x 2 column halves of 8
  const int nslices = d / kFusedColsPerCta;
  constexpr int kLanes = kFusedThreads / 2;
  const int nseg = gridDim.x;
  for (int slice = blockIdx.x; slice < nslices; slice += gridDim.x) {
    float acc[B][8];
#pragma unroll
    for (int b = 0; b < B; ++b)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[b][j] = 0.0f;
    const bf16* wcol = a.w_down_t + slice * kFusedColsPerCta + h * 8;
    for (uint32_t e0 = r; e0 < n_total; e0 += 4 * kLanes) {
      uint4 wv[4];
      const uint16_t* ent[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {   // four independent 16-byte gathers in flight per thread
        const uint32_t e = e0 + u * kLanes;
        wv[u] = make_uint4(0u, 0u, 0u, 0u);
        ent[u] = raw;
        if (e < n_total) {
          int lo = 0, hi = nseg;       // last segment whose offset is <= e
          while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_off[mid] <= e) lo = mid; else hi = mid;
          }
          ent[u] = raw + static_cast<size_t>(lo) * segw + 1 + (e - s_off[lo]) * ewords;
          wv[u] = __ldg(reinterpret_cast<const uint4*>(wcol + static_cast<int64_t>(ent[u][0]) * d));
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t e = e0 + u * kLanes;
        if (e < n_total) {
          float w[8];
          unpack8f(wv[u], w);
#pragma unroll
          for (int b = 0; b < B; ++b) {
            if (b < batch) {
              const float zf = bits_to_float(ent[u][1 + b]);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[b][j] = fmaf(zf, w[j], acc[b][j]);
            }
          }
        }
      }
    }
    // fixed-order reduction over the 256 entry lanes: 16 per warp by shuffles, then over the warps
#pragma unroll
    for (int b = 0; b < B; ++b)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v = acc[b][j];
#pragma unroll
        for (int o = 2; o < 32; o <<= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        acc[b][j] = v;
      }
    if (lane < 2) {
#pragma unroll
      for (int b = 0; b < B; ++b)
#pragma unroll
        for (int j = 0; j < 8; ++j) s_red[warp][lane][b][j] = acc[b][j];
    }
    __syncthreads();
    if (tid < batch * 16) {
      const int b = tid >> 4, c = tid & 15;
      float s = 0.0f;
#pragma unroll
      for (int w = 0; w < kFusedWarps; ++w) s += s_red[w][c >> 3][b][c & 7];
      a.y[static_cast<int64_t>(b) * d + slice * kFusedColsPerCta + c] = __float2bfloat16_rn(s);
    }
    __syncthreads();
  }
  FUSED_STAMP(7);
#undef FUSED_WAIT
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static int fused_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

static int fused_cpc(int d_ffn, int rule) {
  int cpc = ceil_div_i(d_ffn, fused_sms());
  if (rule != 0) cpc = (cpc + 7) / 8 * 8;
  return cpc;
}

static size_t fused_smem_bytes(int bp, int batch, int d, int d_ffn, int cpc) {
  return fused_smem_plan(bp, batch, d, d_ffn, cpc, fused_sms()).total;
}

// 16-bit words of the segment area: one count and up to cpc entries of (1 + batch) words per CTA
int64_t decode_fused_seg_words(int64_t batch, int64_t d_ffn) {
  const int64_t cpc = (ceil_div_i(static_cast<int>(d_ffn), fused_sms()) + 7) / 8 * 8;
  return static_cast<int64_t>(fused_sms()) * (1 + cpc * (1 + batch)) + 8;   // + 8: bulk copies round up to 16 bytes
}

bool decode_fused_supported(int64_t batch, int64_t d, int64_t d_ffn) {
  if (batch < 1 || batch > 8 || d % 16 != 0 || d_ffn < 32 || d_ffn > 32768 || fused_sms() > kFusedThreads) return false;
  const int bp = batch > 4 ? 8 : (batch > 2 ? 4 : (batch > 1 ? 2 : 1));
  const int cpc = (ceil_div_i((int)d_ffn, fused_sms()) + 7) / 8 * 8;
  if (cpc > kFusedRowsPerRound * kFusedMaxRounds) return false;
  return fused_smem_bytes(bp, (int)batch, (int)d, (int)d_ffn, cpc) <= 200 * 1024;
}

int64_t decode_fused_hist_bytes(int64_t batch) { return batch * kFusedBins * 4; }

int launch_decode_fused(int rule, int batch, int d, int d_ffn, int k, const void* x, const void* scores,
                        int64_t ld_scores, const void* w_gate, const void* w_up, const void* w_down_t, void* y,
                        void* g_scratch, void* seg_scratch, int64_t ld, int* hist, int* status_area,
                        cudaStream_t stream) {
  FusedArgs a;
  a.x = static_cast<const bf16*>(x);
  a.scores = static_cast<const bf16*>(scores);
  a.w_gate = static_cast<const bf16*>(w_gate);
  a.w_up = static_cast<const bf16*>(w_up);
  a.w_down_t = static_cast<const bf16*>(w_down_t);
  a.y = static_cast<bf16*>(y);
  a.g = static_cast<bf16*>(g_scratch);
  a.seg = static_cast<uint16_t*>(seg_scratch);
  a.hist = hist;
  a.status = status_area;
  a.sync = reinterpret_cast<unsigned*>(status_area + 32);
  a.ld_scores = ld_scores;
  a.ld = ld;
  a.batch = batch;
  a.d = d;
  a.d_ffn = d_ffn;
  a.k = k;
  a.rule = rule;
  a.cpc = fused_cpc(d_ffn, rule);
  // status word, barrier counter and (Top-K rule) the histograms, which lie directly behind the status area,
  // start from zero on every call: one memset
  if (reinterpret_cast<uint8_t*>(hist) != reinterpret_cast<uint8_t*>(status_area) + 256) {
    set_error("decode_fused: the histograms must follow the status area");
    return kErrInvalidArg;
  }
  const size_t clear = 256 + (rule == 0 ? static_cast<size_t>(decode_fused_hist_bytes(batch)) : 0);
  if (cudaMemsetAsync(status_area, 0, clear, stream) != cudaSuccess) return check_last("cudaMemsetAsync");
  const int bp = batch > 4 ? 8 : (batch > 2 ? 4 : (batch > 1 ? 2 : 1));
  const size_t smem = fused_smem_bytes(bp, batch, d, d_ffn, a.cpc);
  void (*kern)(const FusedArgs) = bp == 8   ? decode_fused_kernel<8>
                                  : bp == 4 ? decode_fused_kernel<4>
                                  : bp == 2 ? decode_fused_kernel<2>
                                            : decode_fused_kernel<1>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return check_last("decode_fused smem attribute");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(fused_sms());
  cfg.blockDim = dim3(kFusedThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeCooperative;   // all CTAs resident at once: the grid barriers need it
  attr.val.cooperative = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  prof_mark(kProfDecodeFused, stream);
  if (cudaLaunchKernelEx(&cfg, kern, a) != cudaSuccess) return check_last("decode_fused launch");
  return check_last("decode_fused");
}

}  // namespace moc

#ifdef MOC_FUSED_TIMING
extern "C" int moc_debug_fused_times(unsigned long long* out_host) {
  return cudaMemcpyFromSymbol(out_host, moc::g_fused_t, sizeof(unsigned long long) * 8 * 512) == cudaSuccess ? 0 : -1;
}
#endif
