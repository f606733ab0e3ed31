// Decode-time MoC FFN for batches of up to 8 token rows as ONE cooperative, persistent kernel launch that
// streams every weight byte exactly once through a shared-memory ring of bulk asynchronous copies.
//
// Work split: CTA c (one per SM) owns the contiguous slice of channels [c * cpc, (c + 1) * cpc) of d_ffn for
// ALL three projections, so the only data that crosses CTAs are the gate scores (selection is global) and the
// partial output vectors:
//
//   A  gate scores of the own channels: the own W_gate rows arrive 16 rows at a time in the ring
//      (cp.async.bulk, 4 KB rows, no multicast); the 16 consumer warps split the hidden dimension, keep their
//      slice of x as mma B-fragments in registers for the whole kernel and run m16n8k16 warp MMAs (weight rows
//      = M, batch rows padded to 8 = N); the per-warp partial sums are added in a fixed order in shared memory,
//      rounded to bf16, published, and their order keys enter a global 2048-bin histogram
//                                                                        (inference_ffn.py:188)
//   -- grid barrier (Top-K rule only; the 2:8 rule is local to groups of 8 channels) --
//   B  every CTA derives the K-th largest key redundantly: threshold bin from the global histogram, the
//      lower 5 key bits and the ties from the published score rows (staged in the idle ring)
//                                    (optimized_global_moc_ext.cu:85-125 replaced by a radix select)
//   C  the W_up rows AND the W_down^T rows of the own selected channels are requested together (their
//      addresses are known at the same moment, so the two gathers cost one DRAM round trip, not two);
//      u = x . W_up[ch] by the same warp MMAs, z = round(round(SiLU(g)) * round(u))
//                                                                   (optimized_global_moc_ext.cu:127-245)
//   D  partial y of the own channels: cols = M (each warp owns d / 16 output columns), own channels = K,
//      batch = N, A-fragments read transposed (ldmatrix.trans) from the staged W_down^T rows; fp32 partial
//      vectors go to the workspace                                  (optimized_global_moc_ext.cu:247-372)
//   -- grid barrier --
//   E  y = fixed-order sum of the partial vectors of all CTAs, rounded to bf16 (no float atomics)
//
// The dense baseline (inference_ffn.py:164-167) is the same kernel without B: gate, up and down rows of the
// own channels stream back to back through the ring and nothing but the final reduction waits for another CTA.
// A producer warp owns the ring (3 stages x 16 rows, full / empty mbarriers); every wait in the kernel is
// bounded: a time-out sets the status word and all roles leave.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>

#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace moc {

using bf16 = __nv_bfloat16;

constexpr int kSWarps = 16;                       // consumer warps
constexpr int kSConsumers = kSWarps * 32;         // 512
constexpr int kSThreads = kSConsumers + 32;       // + one producer warp
constexpr int kSStages = 3;
constexpr int kSTile = 16;                        // weight rows per ring stage = M of one MMA
constexpr int kSMaxTiles = 3;                     // own channels <= 48
constexpr int kSMaxCh = kSMaxTiles * kSTile;
constexpr int kSBins = 2048;
constexpr int kSMaxKSteps = 8;                    // 16-deep k steps per warp: d <= 16 * 16 * 8 = 2048
constexpr int kSMaxMTiles = 8;                    // 16-column tiles per warp in phase D
constexpr int kSNB = 8;                           // batch rows per launch = N of one MMA
constexpr int kSZPitch = 56;                      // bf16 elements per row of z (bank-conflict-free fragment loads)
constexpr int kSCandMax = 768;                    // candidate list entries per row at 8 rows (more with fewer rows)
constexpr long long kStreamWaitCycles = 400000000LL;   // about 0.2 s

// limit of the grid-barrier waits, in cycles; a test lowers it to watch a wait run out (moc_debug_set_wait_cycles)
static std::atomic<long long> g_stream_wait_cycles{kStreamWaitCycles};

struct StreamArgs {
  const bf16* x;          // [batch, d]
  const bf16* scores;     // caller's gate scores [batch, ld_scores], or null: computed from w_gate
  const bf16* w_gate;     // [d_ffn, d]
  const bf16* w_up;       // [d_ffn, d]
  const bf16* w_down_t;   // [d_ffn, d]
  bf16* y;                // [batch, d]
  bf16* g;                // scratch [batch, ld]: published gate scores
  float* partial;         // scratch [grid, batch, d]
  int* hist;              // scratch [batch, 2048], zeroed before the launch
  unsigned* sync;         // scratch: barrier counter, zeroed before the launch
  int* status;            // device status word
  int64_t ld_scores, ld;
  long long wait_cycles;
  int batch, d, d_ffn, k, rule, cpc;   // rule 0: Top-K, 1: 2-of-8, 2: dense (every channel)
};

struct StreamShared {
  uint64_t full[kSStages], empty[kSStages], bar_rows, bar_ent, bar_thr;
  int abort, ok;
  uint32_t n_ent;
  uint16_t g_own[kSNB][kSMaxCh];       // bf16 bits of the own gate scores
  uint8_t sel[kSNB][kSMaxCh];          // row b selects own channel lc
  uint8_t ent[kSMaxCh];                // own channels that some row selected, ascending
  uint16_t zs[kSNB][kSZPitch];         // z of entry e for row b (0: not selected)
  uint32_t wsum[kSNB][kSWarps];
  uint32_t hist2[kSNB][32];
  uint32_t thr[kSNB], take[kSNB], eqb[kSNB], d1[kSNB], krem[kSNB];
  uint32_t ncand[kSNB];                // threshold-bin keys found in row b (candidate list length)
  uint32_t overflow;                   // some row has more candidates than the list holds
};

__device__ __forceinline__ uint16_t stream_bf16_bits(float v) {
  const bf16 h = __float2bfloat16_rn(v);
  return *reinterpret_cast<const uint16_t*>(&h);
}
__device__ __forceinline__ float stream_bits_to_float(uint16_t b) {
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}
// barrier over the 512 consumer threads (the producer warp never joins it)
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

__device__ __forceinline__ bool stream_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                 long long limit) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x1F) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > limit) return false;
    }
  }
}

// All CTAs of the cooperative grid arrive; false (in every consumer thread of the CTA) when the wait ran out.
__device__ __forceinline__ bool stream_grid_barrier(unsigned* counter, unsigned target, int* status, long long limit,
                                                    StreamShared& sh) {
  consumer_sync();
  if (threadIdx.x == 0) {
    int ok = 1;
    // arrival: a reduction with release semantics (no return value to wait for); it also publishes what the other
    // threads of the CTA wrote before the barrier above
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(counter), "r"(1u) : "memory");
    const long long t0 = clock64();
    while (true) {
      // the clock is checked before each poll, so a limit of one cycle gives up at once whatever the other CTAs do
      if (clock64() - t0 >= limit) {
        atomicCAS(status, 0, (kDevTimeoutProducer << 24) | 0x00E00000 | static_cast<int>(target & 0xFFFF));
        ok = 0;
        break;
      }
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
      if (v >= target) break;
    }
    sh.ok = ok;
    if (!ok) sh.abort = 1;
  }
  consumer_sync();
  return sh.ok != 0;
}

__host__ __device__ inline uint32_t stream_pitch(int d) { return static_cast<uint32_t>(d) * 2u + 16u; }
__host__ __device__ inline uint32_t stream_rowpad(int d_ffn) { return (static_cast<uint32_t>(d_ffn) + 15u) / 8u * 8u; }
// dynamic shared memory: the ring, reused during selection for the score rows and (Top-K rule) the histogram
// rows of the batch; then the reduction buffer
__host__ __device__ inline uint32_t stream_rows_bytes(int batch, int d_ffn) {
  return (static_cast<uint32_t>(batch) * stream_rowpad(d_ffn) * 2u + 127u) & ~127u;
}
__host__ __device__ inline uint32_t stream_stage_bytes(int batch, int d, int d_ffn) {
  const uint32_t ring = kSStages * kSTile * stream_pitch(d);
  const uint32_t sel = stream_rows_bytes(batch, d_ffn) + static_cast<uint32_t>(batch) * kSBins * 4u;
  return ((ring > sel ? ring : sel) + 127u) & ~127u;
}
// reduction buffer: two tile buffers [16 warps][16 rows][8] for the row phases; the candidate lists of the
// selection and the stage of phase E reuse it
constexpr uint32_t kSTileRedFloats = kSWarps * kSTile * kSNB;
constexpr uint32_t kSRedBytes = kSNB * kSCandMax * 4;
static_assert(kSRedBytes >= 2 * kSTileRedFloats * 4, "reduction buffer holds two tile buffers");

__device__ __forceinline__ uint32_t stream_exscan(uint32_t v, int lane) {
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= o) inc += nb;
  }
  return inc - v;
}

// Clears the status area and (Top-K rule) the histograms of a call. The persistent kernel is launched as its
// programmatic dependent: it starts streaming weights at once and waits for this grid (griddepcontrol.wait)
// only before it first touches the workspace.
__global__ void __launch_bounds__(256) decode_stream_clear_kernel(int4* __restrict__ area, int n16) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // This kernel is itself launched as a programmatic dependent of whatever kernel precedes it in the stream: when
  // that is the persistent kernel of the previous decode call (which lets its dependents be scheduled as soon as it
  // starts), the launch latency of this call hides behind that call. The previous call may use the same workspace,
  // so nothing is touched before it has completed.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x)
    area[i] = make_int4(0, 0, 0, 0);
}

__global__ void __launch_bounds__(kSThreads, 1) decode_stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(128) uint8_t ssm[];
  __shared__ StreamShared sh;
  // the clear kernel of a following decode call may be scheduled now (it waits for this grid to complete)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int batch = a.batch, d = a.d, F = a.d_ffn, cpc = a.cpc, rule = a.rule;
  const uint32_t pitch = stream_pitch(d);
  const uint32_t row_bytes = static_cast<uint32_t>(d) * 2u;
  uint8_t* ring = ssm;
  float* red = reinterpret_cast<float*>(ssm + stream_stage_bytes(batch, d, F));
  const int ch0 = blockIdx.x * cpc;
  const int ncl = max(0, min(cpc, F - ch0));
  const int nt_own = (ncl + kSTile - 1) / kSTile;
  const long long barrier_limit = a.wait_cycles;   // grid barriers (a test may shorten it)
  // Copy-completion and ring waits keep the fixed limit: a CTA never leaves while a bulk copy into its shared
  // memory may still be in flight (when a grid barrier gives up, every copy issued so far has been consumed).
  const long long limit = kStreamWaitCycles;
  volatile int* abort_flag = &sh.abort;

  if (tid == 0) {
    for (int s = 0; s < kSStages; ++s) {
      ptx::mbar_init(&sh.full[s], 1);
      ptx::mbar_init(&sh.empty[s], kSWarps);
    }
    ptx::mbar_init(&sh.bar_rows, 1);
    ptx::mbar_init(&sh.bar_ent, 1);
    ptx::mbar_init(&sh.bar_thr, 1);
    sh.abort = 0;
    sh.ok = 1;
    sh.n_ent = 0;
    sh.overflow = 0u;
    for (int b = 0; b < kSNB; ++b) sh.ncand[b] = 0u;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  for (int i = tid; i < kSNB * kSZPitch; i += kSThreads) (&sh.zs[0][0])[i] = 0;
  __syncthreads();

  // ------------------------------------------------------------------------------------------------------
  // producer warp: the ring. Job order = consumption order: [gate (and up, dense)] tiles, then up tiles and
  // down tiles of the entries. It touches the workspace only to report a time-out.
  // ------------------------------------------------------------------------------------------------------
  if (warp == kSWarps) {
    uint32_t job = 0;
    bool alive = true;
    // one tile: lane i copies row `src` into slot i of the stage
    auto put_tile = [&](int nrows, const bf16* src) {
      if (!alive) return;
      const uint32_t s = job % kSStages, u = job / kSStages;
      if (u > 0 && !stream_mbar_wait(&sh.empty[s], (u - 1) & 1u, abort_flag, limit)) {
        if (lane == 0) {
          sh.abort = 1;
          atomicCAS(a.status, 0, (kDevTimeoutProducer << 24) | 0x00E10000 | static_cast<int>(job & 0xFFFF));
        }
        alive = false;
        return;
      }
      if (lane == 0) ptx::mbar_arrive_expect_tx(&sh.full[s], static_cast<uint32_t>(nrows) * row_bytes);
      __syncwarp();
      if (lane < nrows) ptx::bulk_load(ring + (s * kSTile + lane) * pitch, src, row_bytes, &sh.full[s]);
      ++job;
    };
    const int n_first = rule == 2 ? 3 * nt_own : (a.scores ? 0 : nt_own);
#pragma unroll 1
    for (int j = 0; j < n_first; ++j) {
      // dense: gate 0, up 0, gate 1, up 1, ..., then the down tiles; otherwise the gate tiles
      const int t = rule == 2 ? (j < 2 * nt_own ? (j >> 1) : j - 2 * nt_own) : j;
      const bf16* w = rule == 2 ? (j < 2 * nt_own ? ((j & 1) ? a.w_up : a.w_gate) : a.w_down_t) : a.w_gate;
      const int nrows = min(kSTile, ncl - t * kSTile);
      put_tile(nrows, w + static_cast<int64_t>(ch0 + t * kSTile + (lane < nrows ? lane : 0)) * d);
    }
    if (rule == 2) return;
    if (rule == 0) {
      // Top-K rule: as soon as the threshold BIN of every row is known, the own channels whose key lies in a
      // higher bin are certainly selected. Their W_up and W_down^T rows are requested into L2 now, while the
      // consumers still resolve the exact threshold and the ties (a few microseconds), so that the copies issued
      // after the selection find them there. Channels inside the threshold bin (a few percent) are left alone.
      if (stream_mbar_wait(&sh.bar_thr, 0u, abort_flag, 8 * limit)) {
        for (int lc = lane; lc < ncl; lc += 32) {
          bool certain = false;
          for (int b = 0; b < batch; ++b) certain = certain || (order_key16(sh.g_own[b][lc]) >> 5) > sh.d1[b];
          if (certain) {
            ptx::bulk_prefetch_l2(a.w_up + static_cast<int64_t>(ch0 + lc) * d, row_bytes);
            ptx::bulk_prefetch_l2(a.w_down_t + static_cast<int64_t>(ch0 + lc) * d, row_bytes);
          }
        }
      }
    }
    // the entry list of this CTA (written by the consumers after selection)
    if (!stream_mbar_wait(&sh.bar_ent, 0u, abort_flag, 8 * limit)) {
      if (lane == 0) {
        sh.abort = 1;
        atomicCAS(a.status, 0, (kDevTimeoutProducer << 24) | 0x00E40000);
      }
      return;
    }
    const int n_ent = static_cast<int>(sh.n_ent);
    const int nt_ent = (n_ent + kSTile - 1) / kSTile;
#pragma unroll 1
    for (int j = 0; j < 2 * nt_ent; ++j) {
      const int t = j < nt_ent ? j : j - nt_ent;
      const bf16* w = j < nt_ent ? a.w_up : a.w_down_t;
      const int nrows = min(kSTile, n_ent - t * kSTile);
      const int lc = sh.ent[t * kSTile + (lane < nrows ? lane : 0)];
      put_tile(nrows, w + static_cast<int64_t>(ch0 + lc) * d);
    }
    return;
  }

  // ------------------------------------------------------------------------------------------------------
  // consumer warps
  // ------------------------------------------------------------------------------------------------------
  const int g8 = lane >> 2, t4 = lane & 3;
  const int ksteps = d >> 8;                 // 16-deep k steps of this warp's slice of the hidden dimension
  const int kbase = warp * (d >> 4);
  // x as B-fragments (column n = batch row g8, k = 2 * t4 + {0, 1} and + 8), zero beyond the batch
  uint32_t xf[2 * kSMaxKSteps];
#pragma unroll
  for (int s = 0; s < kSMaxKSteps; ++s) {
    xf[2 * s] = 0u;
    xf[2 * s + 1] = 0u;
    if (s < ksteps && g8 < batch) {
      const uint32_t* xr = reinterpret_cast<const uint32_t*>(a.x + static_cast<int64_t>(g8) * d + kbase + 16 * s);
      xf[2 * s] = __ldg(xr + t4);
      xf[2 * s + 1] = __ldg(xr + 4 + t4);
    }
  }
  // from here on the workspace is used: the grid that cleared it must be complete
  asm volatile("griddepcontrol.wait;" ::: "memory");

  uint32_t job = 0;
  auto wait_full = [&](uint32_t j) {
    if (!stream_mbar_wait(&sh.full[j % kSStages], (j / kSStages) & 1u, abort_flag, limit)) {
      sh.abort = 1;
      atomicCAS(a.status, 0, (kDevTimeoutEpilogue << 24) | 0x00E20000 | static_cast<int>(j & 0xFFFF));
    }
  };
  auto release = [&](uint32_t j) {
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(&sh.empty[j % kSStages]);
  };
  const uint32_t a_row = static_cast<uint32_t>((lane & 7) + ((lane >> 3) & 1) * 8);
  const uint32_t a_kc = static_cast<uint32_t>((lane >> 4) * 8);
  const int my_r = tid >> 3, my_b = tid & 7;   // reduction role of threads 0..127: (row of the tile, batch row)

  // ---------------- row phases: gate scores (A), selection (B), u and z of the entries (C) ----------------
  // One rolled loop over the row tiles of this CTA: [gate tiles | gate, up pairs (dense)], the selection, then
  // the up tiles of the entries. Per tile: this warp's slice of the hidden dimension by warp MMAs (tile rows
  // = M, K contiguous), the 16 per-warp partial sums meet in a double-buffered shared-memory tile and are
  // added in a fixed order.
  unsigned barrier_no = 0;
  const int n_a = rule == 2 ? 2 * nt_own : (a.scores ? 0 : nt_own);
  int n_rows_jobs = n_a;            // grows by the up tiles once the entries are known
  if (rule != 2 && a.scores) {
    for (int i = tid; i < batch * ncl; i += kSConsumers) {
      const int b = i / ncl, lc = i - b * ncl;
      const bf16 v = a.scores[static_cast<int64_t>(b) * a.ld_scores + ch0 + lc];
      const uint16_t bits = *reinterpret_cast<const uint16_t*>(&v);
      sh.g_own[b][lc] = bits;
      if (rule == 0) atomicAdd(&a.hist[b * kSBins + (order_key16(bits) >> 5)], 1);
    }
  }
#pragma unroll 1
  for (int j = 0;; ++j) {
    if (j == n_a && rule != 2) {
      // ---------------- B: selection ----------------
      if (rule == 0) {
        if (!stream_grid_barrier(a.sync, ++barrier_no * gridDim.x, a.status, barrier_limit, sh)) return;
        // score rows and histogram rows of the whole batch into the idle ring
        const uint16_t* sc = reinterpret_cast<const uint16_t*>(a.scores ? a.scores : a.g);
        const int64_t lds = a.scores ? a.ld_scores : a.ld;
        const uint32_t rowpad = stream_rowpad(F);
        uint16_t* srow = reinterpret_cast<uint16_t*>(ring);                                   // [batch][rowpad]
        const uint32_t* hrow = reinterpret_cast<const uint32_t*>(ring + stream_rows_bytes(batch, F));   // [batch][2048]
        const bool bulk_rows = !a.scores;                     // own rows start on 256-byte boundaries
        if (tid == 0) {
          asm volatile("fence.proxy.async;" ::: "memory");
          const uint32_t rb = (static_cast<uint32_t>(F) * 2u + 15u) & ~15u;
          ptx::mbar_arrive_expect_tx(&sh.bar_rows, (bulk_rows ? rb * batch : 0u) + static_cast<uint32_t>(batch) * kSBins * 4u);
          for (int b = 0; b < batch; ++b)
            ptx::bulk_load(ring + stream_rows_bytes(batch, F) + b * (kSBins * 4), a.hist + b * kSBins, kSBins * 4u, &sh.bar_rows);
          if (bulk_rows)
            for (int b = 0; b < batch; ++b)
              ptx::bulk_load(srow + static_cast<size_t>(b) * rowpad, sc + static_cast<int64_t>(b) * lds, rb, &sh.bar_rows);
        }
        if (!bulk_rows) {
#pragma unroll 1
          for (int i = tid; i < batch * F; i += kSConsumers) {
            const int b = i / F, c = i - b * F;
            srow[b * rowpad + c] = __ldcg(sc + static_cast<int64_t>(b) * lds + c);
          }
        }
        if (tid < kSNB * 32) (&sh.hist2[0][0])[tid] = 0u;
        if (!stream_mbar_wait(&sh.bar_rows, 0u, abort_flag, limit)) {
          sh.abort = 1;
          atomicCAS(a.status, 0, (kDevTimeoutEpilogue << 24) | 0x00E30000);
        }
        consumer_sync();
        // threshold bin of row b (warp b): the K-th largest key lies in bin d1, krem-th from the top inside it
        if (warp < batch) {
          const uint32_t* h = hrow + warp * kSBins;
          const uint32_t kk = static_cast<uint32_t>(a.k);
          const int lo = (31 - lane) * 64;           // lane l sums the 64 bins [lo, lo + 64), counted from the top
          uint32_t local = 0;
#pragma unroll 4
          for (int i = 0; i < 64; ++i) local += h[lo + ((i + lane) & 63)];
          const uint32_t above = stream_exscan(local, lane);
          const int src = __ffs(__ballot_sync(0xFFFFFFFFu, above < kk && above + local >= kk)) - 1;
          const uint32_t above_src = __shfl_sync(0xFFFFFFFFu, above, src & 31);
          const int top = (31 - (src & 31)) * 64 + 63;
          const uint32_t c0 = h[top - 2 * lane], c1 = h[top - 2 * lane - 1];
          const uint32_t ex = stream_exscan(c0 + c1, lane) + above_src;
          if (ex < kk && ex + c0 + c1 >= kk) {
            const bool first = ex + c0 >= kk;
            sh.d1[warp] = static_cast<uint32_t>(first ? top - 2 * lane : top - 2 * lane - 1);
            sh.krem[warp] = first ? kk - ex : kk - ex - c0;
          }
          __syncwarp();
          // the padding channels [F, rowpad) of the staged row get a pattern outside the threshold bin
          const uint32_t klo = sh.d1[warp] << 5;
          const uint32_t pat = (klo >= 0x8000u ? (klo ^ 0x8000u) : (klo ^ 0xFFFFu)) & 0xFFE0u;
          if (F + lane < static_cast<int>(rowpad)) srow[warp * rowpad + F + lane] = static_cast<uint16_t>(~pat);
        }
        consumer_sync();
        if (tid == 0) ptx::mbar_arrive(&sh.bar_thr);   // the producer warp may prefetch the certain rows
        // One vectorised pass over the score rows collects the keys of each row's threshold bin (a few percent
        // of a row) as (channel, lower 5 key bits) candidates in one flat list per row; the rest works on these
        // short lists. The 16 warps split the rows (16 / batch' warps per row); a warp places the hits of its 32
        // vectors with one scan and one atomic per step.
        uint32_t* cand = reinterpret_cast<uint32_t*>(red);   // [batch'][cap]
        const int bp = batch > 4 ? 8 : (batch > 2 ? 4 : (batch > 1 ? 2 : 1));
        const int wpr = kSWarps / bp;
        const uint32_t cap = (kSRedBytes / 4u) / static_cast<uint32_t>(bp);
        const int cb = warp / wpr, csub = warp - cb * wpr;
        if (cb < batch) {
          const int nvec = static_cast<int>(rowpad >> 3);
          // The keys of bin d1 share their upper 11 bits, and so do their raw bf16 patterns (key = bits ^ 0x8000
          // for positive values, ~bits for negative ones): a channel is a candidate iff (bits & 0xFFE0) == pat.
          // Two channels are tested per 32-bit word: t = (word & 0xFFE0FFE0) ^ pat2 has a zero half exactly for a
          // candidate, found by the has-zero identity (t - 0x00010001) & ~t & 0x80008000 (exact here: the halves of
          // t are multiples of 32, so a borrow out of a zero low half cannot fake a zero in the high half).
          const uint32_t klo = sh.d1[cb] << 5;
          const bool positive = klo >= 0x8000u;
          const uint32_t pat = (positive ? (klo ^ 0x8000u) : (klo ^ 0xFFFFu)) & 0xFFE0u;
          const uint32_t pat2 = pat * 0x00010001u;
          const uint32_t raw_lo = pat;                     // lowest raw pattern of the bin (low 5 bits clear)
          const uint16_t* rowp = srow + cb * rowpad;
          uint32_t* list = cand + cb * cap;
          // A lane tests 4 vectors (32 channels) per step into one 32-bit hit mask and keeps the masks of up to
          // kSteps steps in registers, so the warp pays one scan and one atomic per round. Bit p of a mask:
          // half = p >> 4 (odd channel of a word), vector u = ((p >> 3) & 1) * 2 + (p & 1), word j = (p & 7) >> 1.
          constexpr int kVecs = 4, kSteps = 6;
          const int stride = wpr * 32 * kVecs;
#pragma unroll 1
          for (int r0 = csub * 32 * kVecs; r0 < nvec; r0 += stride * kSteps) {
            uint32_t hits[kSteps];
            uint32_t c = 0;
#pragma unroll
            for (int st = 0; st < kSteps; ++st) {
              hits[st] = 0u;
              const int v0 = r0 + st * stride;
              if (v0 < nvec) {
#pragma unroll
                for (int u = 0; u < kVecs; ++u) {
                  const int v = v0 + u * 32 + lane;
                  uint4 q = make_uint4(~pat2, ~pat2, ~pat2, ~pat2);   // never a candidate
                  if (v < nvec) q = *reinterpret_cast<const uint4*>(rowp + v * 8);
                  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                  uint32_t m = 0;
#pragma unroll
                  for (int jw = 0; jw < 4; ++jw) {
                    const uint32_t t = (w[jw] & 0xFFE0FFE0u) ^ pat2;
                    m |= ((((t - 0x00010001u) & ~t) & 0x80008000u) >> 15) << (2 * jw);
                  }
                  hits[st] |= m << ((u >> 1) * 8 + (u & 1));
                }
                c += __popc(hits[st]);
              }
            }
            const uint32_t ex = stream_exscan(c, lane);
            const uint32_t total = __shfl_sync(0xFFFFFFFFu, ex + c, 31);
            if (total) {
              uint32_t base = 0;
              if (lane == 0) base = atomicAdd(&sh.ncand[cb], total);
              uint32_t pos = __shfl_sync(0xFFFFFFFFu, base, 0) + ex;
#pragma unroll
              for (int st = 0; st < kSteps; ++st) {
                uint32_t h = hits[st];
                while (h) {
                  const int p2 = __ffs(h) - 1;
                  h &= h - 1u;
                  const int u = ((p2 >> 3) & 1) * 2 + (p2 & 1);
                  const int ch = (r0 + st * stride + u * 32 + lane) * 8 + ((p2 & 7) >> 1) * 2 + (p2 >> 4);
                  const uint32_t off = static_cast<uint32_t>(rowp[ch]) - raw_lo;      // 0..31
                  if (pos < cap) list[pos] = (static_cast<uint32_t>(ch) << 5) | (positive ? off : 31u - off);
                  ++pos;
                }
              }
            }
          }
        }
        consumer_sync();
        if (tid < batch && sh.ncand[tid] > cap) sh.overflow = 1u;
        consumer_sync();
        if (!sh.overflow) {
          if (csub == 0 && cb < batch) {
            const int b = cb;
            const uint32_t n = sh.ncand[b];
            const uint32_t* list = cand + b * cap;
            // lower 5 key bits of the candidates -> 32-bin histogram -> the K-th largest key and the ties to admit
#pragma unroll 2
            for (uint32_t i = lane; i < n; i += 32) atomicAdd(&sh.hist2[b][list[i] & 31u], 1u);
            __syncwarp();
            const uint32_t cc = sh.hist2[b][31 - lane];
            const uint32_t ex = stream_exscan(cc, lane), krem = sh.krem[b];
            const uint32_t src = static_cast<uint32_t>(__ffs(__ballot_sync(0xFFFFFFFFu, ex < krem && ex + cc >= krem)) - 1) & 31u;
            const uint32_t lowk = 31u - src;
            const uint32_t take = __shfl_sync(0xFFFFFFFFu, krem - ex, src);   // ties admitted, lowest channels first
            uint32_t cnt = 0;                                                // ties below the own slice
#pragma unroll 2
            for (uint32_t i = lane; i < n; i += 32) {
              const uint32_t e = list[i];
              cnt += ((e & 31u) == lowk && static_cast<int>(e >> 5) < ch0) ? 1u : 0u;
            }
            cnt = __reduce_add_sync(0xFFFFFFFFu, cnt);
            if (lane == 0) {
              sh.thr[b] = (sh.d1[b] << 5) | lowk;
              sh.take[b] = take;
              sh.eqb[b] = cnt;
            }
          }
        } else {
          // a threshold bin too crowded for the lists (many equal scores): full passes over the rows instead
#pragma unroll 1
          for (int i = tid; i < batch * F; i += kSConsumers) {
            const int b = i / F;
            const uint32_t key = order_key16(srow[b * rowpad + (i - b * F)]);
            if ((key >> 5) == sh.d1[b]) atomicAdd(&sh.hist2[b][key & 31u], 1u);
          }
          consumer_sync();
          if (warp < batch) {
            const int b = warp;
            const uint32_t cc = sh.hist2[b][31 - lane];
            const uint32_t ex = stream_exscan(cc, lane), krem = sh.krem[b];
            if (ex < krem && ex + cc >= krem) {
              sh.thr[b] = (sh.d1[b] << 5) | static_cast<uint32_t>(31 - lane);
              sh.take[b] = krem - ex;
            }
            if (lane == 0) sh.eqb[b] = 0u;
          }
          consumer_sync();
          const int lim = min(ch0, F);
#pragma unroll 1
          for (int b = 0; b < batch; ++b) {
            const uint32_t thr = sh.thr[b];
            uint32_t cnt = 0;
            for (int i = tid; i < lim; i += kSConsumers) cnt += (order_key16(srow[b * rowpad + i]) == thr) ? 1u : 0u;
            cnt = __reduce_add_sync(0xFFFFFFFFu, cnt);
            if (lane == 0 && cnt) atomicAdd(&sh.eqb[b], cnt);
          }
        }
        consumer_sync();
#pragma unroll 1
        for (int i = tid; i < batch * ncl; i += kSConsumers) {
          const int b = i / ncl, lc = i - b * ncl;
          const uint32_t thr = sh.thr[b];
          const uint32_t key = order_key16(sh.g_own[b][lc]);
          bool s = key > thr;
          if (key == thr) {
            uint32_t seen = sh.eqb[b];
            for (int c = 0; c < lc; ++c) seen += (order_key16(sh.g_own[b][c]) == thr) ? 1u : 0u;
            s = seen < sh.take[b];
          }
          sh.sel[b][lc] = s ? 1 : 0;
        }
      } else {
        // top-2 of every 8 channels, lower channel wins ties; slices start on multiples of 8
        consumer_sync();
        const int groups = (ncl + 7) >> 3;
#pragma unroll 1
        for (int i = tid; i < batch * groups; i += kSConsumers) {
          const int b = i / groups, c0 = (i - b * groups) * 8, nv = min(8, ncl - c0);
          int b1 = 0, b2 = -1;
          uint32_t k1 = order_key16(sh.g_own[b][c0]), k2 = 0;
#pragma unroll 1
          for (int e = 1; e < nv; ++e) {       // first and second maximum, the lower channel wins ties
            const uint32_t key = order_key16(sh.g_own[b][c0 + e]);
            if (key > k1) { b2 = b1; k2 = k1; b1 = e; k1 = key; }
            else if (b2 < 0 || key > k2) { b2 = e; k2 = key; }
          }
#pragma unroll 1
          for (int e = 0; e < nv; ++e) sh.sel[b][c0 + e] = (e == b1 || e == b2) ? 1 : 0;
        }
      }
      consumer_sync();
      // entries: own channels that some row selected, ascending
      if (warp == 0) {
        uint32_t run = 0;
#pragma unroll 1
        for (int l0 = 0; l0 < ncl; l0 += 32) {
          const int lc = l0 + lane;
          bool any = false;
          if (lc < ncl)
            for (int b = 0; b < batch; ++b) any = any || sh.sel[b][lc] != 0;
          const uint32_t m = __ballot_sync(0xFFFFFFFFu, any);
          if (any) sh.ent[run + __popc(m & ((1u << lane) - 1u))] = static_cast<uint8_t>(lc);
          run += __popc(m);
        }
        if (lane == 0) sh.n_ent = run;
      }
      consumer_sync();
      if (tid == 0) ptx::mbar_arrive(&sh.bar_ent);   // the producer may fetch the rows of the entries
      n_rows_jobs = n_a + (static_cast<int>(sh.n_ent) + kSTile - 1) / kSTile;
    }
    if (j >= n_rows_jobs) break;

    // ---- one row tile ----
    const int kind = rule == 2 ? (j & 1) + 1 : (j < n_a ? 0 : 3);   // 0 gate, 1 dense gate, 2 dense up, 3 up of entries
    const int t = rule == 2 ? (j >> 1) : (j < n_a ? j : j - n_a);
    wait_full(job);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    {
      const uint32_t addr = ptx::smem_u32(ring + (job % kSStages) * kSTile * pitch) + a_row * pitch + (kbase + a_kc) * 2u;
#pragma unroll
      for (int s = 0; s < kSMaxKSteps; ++s) {
        if (s < ksteps) {
          uint32_t r0, r1, r2, r3;
          ptx::ldmatrix_x4(addr + s * 32, r0, r1, r2, r3);
          ptx::mma_m16n8k16_bf16(acc, r0, r1, r2, r3, xf[2 * s], xf[2 * s + 1]);
        }
      }
    }
    release(job);
    ++job;
    float* rt = red + (j & 1) * kSTileRedFloats;     // [16 warps][16 rows][8]
    {
      float* r = rt + ((warp * kSTile + g8) * kSNB + 2 * t4);
      *reinterpret_cast<float2*>(r) = make_float2(acc[0], acc[1]);
      *reinterpret_cast<float2*>(r + 8 * kSNB) = make_float2(acc[2], acc[3]);
    }
    consumer_sync();
    if (tid < kSTile * kSNB && my_b < batch) {
      const int row = t * kSTile + my_r;       // own channel (gate, dense) or entry (up of entries)
      float sum = 0.0f;
#pragma unroll
      for (int w = 0; w < kSWarps; ++w) sum += rt[w * kSTile * kSNB + tid];
      if (kind <= 1) {
        if (row < ncl) {
          const uint16_t bits = stream_bf16_bits(sum);
          sh.g_own[my_b][row] = bits;
          if (kind == 0) {
            reinterpret_cast<uint16_t*>(a.g)[static_cast<int64_t>(my_b) * a.ld + ch0 + row] = bits;
            if (rule == 0) atomicAdd(&a.hist[my_b * kSBins + (order_key16(bits) >> 5)], 1);
          }
        }
      } else {
        const int n_lim = kind == 2 ? ncl : static_cast<int>(sh.n_ent);
        if (row < n_lim) {
          const int lc = kind == 2 ? row : sh.ent[row];
          uint16_t zb = 0;
          if (kind == 2 || sh.sel[my_b][lc]) {
            float sv, zv;
            moc_fwd_point<bf16>(stream_bits_to_float(sh.g_own[my_b][lc]), Num<bf16>::round(sum), sv, zv);
            zb = stream_bf16_bits(zv);
          }
          sh.zs[my_b][row] = zb;
        }
      }
    }
  }
  if (rule == 2 && tid == 0) sh.n_ent = static_cast<uint32_t>(ncl);
  consumer_sync();

  // ---------------- D: partial y of the own entries ----------------
  const int n_ent = static_cast<int>(sh.n_ent);
  const int nt_ent = (n_ent + kSTile - 1) / kSTile;
  const int mtiles = d >> 8;                  // 16-column tiles of this warp's d / 16 output columns
  const int mbase = warp * (d >> 4);
  float acc_d[kSMaxMTiles][4];
#pragma unroll
  for (int mt = 0; mt < kSMaxMTiles; ++mt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc_d[mt][e] = 0.0f;
  const uint32_t d_krow = static_cast<uint32_t>((lane & 7) + ((lane >> 4) & 1) * 8);
  const uint32_t d_mcol = static_cast<uint32_t>(((lane >> 3) & 1) * 8);
#pragma unroll 1
  for (int t = 0; t < nt_ent; ++t) {
    wait_full(job);
    // entries of this stage beyond the list hold stale rows: their A columns are masked to zero
    const int nvalid = n_ent - t * kSTile;
    const uint32_t m_lo = ((2 * t4 < nvalid) ? 0x0000FFFFu : 0u) | ((2 * t4 + 1 < nvalid) ? 0xFFFF0000u : 0u);
    const uint32_t m_hi = ((2 * t4 + 8 < nvalid) ? 0x0000FFFFu : 0u) | ((2 * t4 + 9 < nvalid) ? 0xFFFF0000u : 0u);
    const uint32_t zb0 = *reinterpret_cast<const uint32_t*>(&sh.zs[g8][t * kSTile + 2 * t4]);
    const uint32_t zb1 = *reinterpret_cast<const uint32_t*>(&sh.zs[g8][t * kSTile + 8 + 2 * t4]);
    const uint32_t addr = ptx::smem_u32(ring + (job % kSStages) * kSTile * pitch) + d_krow * pitch + (mbase + d_mcol) * 2u;
#pragma unroll
    for (int mt = 0; mt < kSMaxMTiles; ++mt) {
      if (mt < mtiles) {
        uint32_t r0, r1, r2, r3;
        ptx::ldmatrix_x4_trans(addr + mt * 32, r0, r1, r2, r3);
        ptx::mma_m16n8k16_bf16(acc_d[mt], r0 & m_lo, r1 & m_lo, r2 & m_hi, r3 & m_hi, zb0, zb1);
      }
    }
    release(job);
    ++job;
  }
  {
    float* pb = a.partial + static_cast<int64_t>(blockIdx.x) * batch * d;
    const int b0 = 2 * t4;
#pragma unroll
    for (int mt = 0; mt < kSMaxMTiles; ++mt) {
      if (mt < mtiles) {
        const int col = mbase + mt * 16 + g8;
        if (b0 < batch) {
          __stcg(pb + static_cast<int64_t>(b0) * d + col, acc_d[mt][0]);
          __stcg(pb + static_cast<int64_t>(b0) * d + col + 8, acc_d[mt][2]);
        }
        if (b0 + 1 < batch) {
          __stcg(pb + static_cast<int64_t>(b0 + 1) * d + col, acc_d[mt][1]);
          __stcg(pb + static_cast<int64_t>(b0 + 1) * d + col + 8, acc_d[mt][3]);
        }
      }
    }
  }
  if (!stream_grid_barrier(a.sync, ++barrier_no * gridDim.x, a.status, barrier_limit, sh)) return;

  // ---------------- E: y = sum of the partial vectors, fixed order ----------------
  // Each CTA owns a run of 8-output groups. Warps and lane quarters split the partial vectors (64 ways) and
  // four groups are loaded at a time, so a lane has about ten independent loads in flight; the 64 sums meet
  // by shuffles and a small shared-memory stage and are added in a fixed order.
  {
    const int ngroups = batch * d / 8;
    const int grid = gridDim.x;
    const int gpc = (ngroups + grid - 1) / grid;
    const int g_first = blockIdx.x * gpc;
    const int64_t stride = static_cast<int64_t>(batch) * d;
    const int o8 = lane & 7, cj = (lane >> 3) + 4 * warp;
    float* stage2 = red;   // [gpc][16 warps][8]
    constexpr int kGroupsAtOnce = 8;
    constexpr int kCtaSteps = 3;   // partial vectors per lane: grid <= 3 * 64 (checked on the host)
#pragma unroll 1
    for (int g0 = 0; g0 < gpc; g0 += kGroupsAtOnce) {
      float v[kCtaSteps][kGroupsAtOnce];
#pragma unroll
      for (int cs = 0; cs < kCtaSteps; ++cs) {
        const int c = cj + cs * 4 * kSWarps;
#pragma unroll
        for (int u = 0; u < kGroupsAtOnce; ++u) {
          const int gi = g_first + g0 + u;
          v[cs][u] = (c < grid && g0 + u < gpc && gi < ngroups)
                         ? __ldcg(a.partial + c * stride + static_cast<int64_t>(gi) * 8 + o8) : 0.0f;
        }
      }
#pragma unroll
      for (int u = 0; u < kGroupsAtOnce; ++u) {
        float t = (v[0][u] + v[1][u]) + v[2][u];
        t += __shfl_xor_sync(0xFFFFFFFFu, t, 8);
        t += __shfl_xor_sync(0xFFFFFFFFu, t, 16);
        if (lane < 8 && g0 + u < gpc) stage2[((g0 + u) * kSWarps + warp) * 8 + lane] = t;
      }
    }
    consumer_sync();
#pragma unroll 1
    for (int i = tid; i < gpc * 8; i += kSConsumers) {
      const int gl = i >> 3, gi = g_first + gl;
      if (gi < ngroups) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kSWarps; ++w) v += stage2[(gl * kSWarps + w) * 8 + (i & 7)];
        a.y[static_cast<int64_t>(gi) * 8 + (i & 7)] = __float2bfloat16_rn(v);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static int stream_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}
static int stream_max_smem() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (n <= 0) n = 48 * 1024;
  }
  return n;
}
static int stream_cpc(int d_ffn, int rule) {
  int cpc = ceil_div_i(d_ffn, stream_sms());
  if (rule == 1) cpc = (cpc + 7) / 8 * 8;
  return cpc;
}

bool decode_stream_supported(int64_t batch, int64_t d, int64_t d_ffn, int rule) {
  if (batch < 1 || batch > kSNB || d < 256 || d % 256 != 0 || d > 16 * 16 * kSMaxKSteps || d_ffn < 1 || d_ffn > 32768)
    return false;
  if (stream_cpc(static_cast<int>(d_ffn), rule) > kSMaxCh || stream_sms() > 3 * 4 * kSWarps) return false;
  // phase E stages (groups per CTA) x 16 x 8 floats in the reduction buffer
  if ((batch * d / 8 + stream_sms() - 1) / stream_sms() * kSWarps * 8 * 4 > static_cast<int64_t>(kSRedBytes)) return false;
  const size_t smem = stream_stage_bytes((int)batch, (int)d, (int)d_ffn) + kSRedBytes + sizeof(StreamShared) + 256;
  return smem <= static_cast<size_t>(stream_max_smem());
}

int64_t decode_stream_partial_bytes(int64_t batch, int64_t d) {
  return static_cast<int64_t>(stream_sms()) * batch * d * 4;
}

void decode_stream_set_wait_cycles(long long cycles) {
  g_stream_wait_cycles.store(cycles > 0 ? cycles : kStreamWaitCycles, std::memory_order_relaxed);
}

int launch_decode_stream(int rule, int batch, int d, int d_ffn, int k, const void* x, const void* scores,
                         int64_t ld_scores, const void* w_gate, const void* w_up, const void* w_down_t, void* y,
                         void* g_scratch, int64_t ld, int* hist, int* status_area, float* partial,
                         cudaStream_t stream) {
  StreamArgs a;
  a.x = static_cast<const bf16*>(x);
  a.scores = static_cast<const bf16*>(scores);
  a.w_gate = static_cast<const bf16*>(w_gate);
  a.w_up = static_cast<const bf16*>(w_up);
  a.w_down_t = static_cast<const bf16*>(w_down_t);
  a.y = static_cast<bf16*>(y);
  a.g = static_cast<bf16*>(g_scratch);
  a.partial = partial;
  a.hist = hist;
  a.status = status_area;
  a.sync = reinterpret_cast<unsigned*>(status_area + 32);
  a.ld_scores = ld_scores;
  a.ld = ld;
  a.wait_cycles = g_stream_wait_cycles.load(std::memory_order_relaxed);
  a.batch = batch;
  a.d = d;
  a.d_ffn = d_ffn;
  a.k = k;
  a.rule = rule;
  a.cpc = stream_cpc(d_ffn, rule);
  // Status word, barrier counter and (Top-K rule) the histograms, which lie directly behind the status area,
  // start from zero on every call. A small kernel clears them (a memset node in front of a kernel node costs a
  // CUDA graph about 3 us more than a kernel node) and the persistent kernel is its programmatic dependent: it
  // may start while the clear kernel runs and waits for it only before its first workspace access.
  if (reinterpret_cast<uint8_t*>(hist) != reinterpret_cast<uint8_t*>(status_area) + 256) {
    set_error("decode_stream: the histograms must follow the status area");
    return kErrInvalidArg;
  }
  const size_t clear = 256 + (rule == 0 ? static_cast<size_t>(batch) * kSBins * 4 : 0);
  const int n16 = static_cast<int>(clear / 16);
  static std::atomic<int> clear_pdl{-1};   // 1: the clear kernel is launched as a programmatic dependent
  int cmode = clear_pdl.load(std::memory_order_relaxed);
  if (cmode < 0) {
    const char* e = getenv("MOC_B200_DECODE_PDL");
    cmode = (e && e[0] == '0') ? 0 : 1;
    clear_pdl.store(cmode, std::memory_order_relaxed);
  }
  {
    cudaLaunchConfig_t ccfg = {};
    ccfg.gridDim = dim3(rule == 0 ? 8 : 1);
    ccfg.blockDim = dim3(256);
    ccfg.stream = stream;
    cudaLaunchAttribute cattr[1];
    cattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    cattr[0].val.programmaticStreamSerializationAllowed = 1;
    ccfg.attrs = cattr;
    ccfg.numAttrs = cmode ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&ccfg, decode_stream_clear_kernel, reinterpret_cast<int4*>(status_area), n16);
    if (err != cudaSuccess && cmode) {
      cudaGetLastError();
      clear_pdl.store(0, std::memory_order_relaxed);
      ccfg.numAttrs = 0;
      err = cudaLaunchKernelEx(&ccfg, decode_stream_clear_kernel, reinterpret_cast<int4*>(status_area), n16);
    }
    if (err != cudaSuccess) {
      set_error("decode_stream clear launch: %s", cudaGetErrorString(err));
      return kErrCuda;
    }
  }
  int rc = check_last("decode_stream clear");
  if (rc != kOk) return rc;
  const size_t smem = stream_stage_bytes(batch, d, d_ffn) + kSRedBytes;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(decode_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem)) != cudaSuccess)
    return check_last("decode_stream smem attribute");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(stream_sms());
  cfg.blockDim = dim3(kSThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // Launch modes, settled by the first launch outside a stream capture: 2 = cooperative + programmatic
  // dependent, 1 = programmatic dependent alone (if the driver refuses the combination; one CTA per SM with the
  // grid = SM count is co-resident on an otherwise idle device, and every grid-barrier wait is bounded),
  // 0 = cooperative alone (MOC_B200_DECODE_PDL=0, or while a capture is running before the mode is settled).
  static std::atomic<int> launch_mode{-1};
  int mode = launch_mode.load(std::memory_order_relaxed);
  bool settle = false;
  if (mode < 0) {
    const char* e = getenv("MOC_B200_DECODE_PDL");
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(stream, &cap);
    if (e && e[0] == '0') {
      mode = 0;
      launch_mode.store(0, std::memory_order_relaxed);
    } else if (cap != cudaStreamCaptureStatusNone) {
      mode = 0;
    } else {
      mode = 2;
      settle = true;
    }
  }
  prof_mark(kProfDecodeFused, stream);
  while (true) {
    cudaLaunchAttribute attrs[2];
    int na = 0;
    if (mode == 0 || mode == 2) {
      attrs[na].id = cudaLaunchAttributeCooperative;   // all CTAs resident at once: the grid barriers need it
      attrs[na].val.cooperative = 1;
      ++na;
    }
    if (mode >= 1) {
      attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attrs[na].val.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, decode_stream_kernel, a);
    if (err == cudaSuccess) break;
    cudaGetLastError();   // a refused launch configuration is not sticky
    if (settle && mode > 0) {
      --mode;             // 2 -> 1 -> 0
      continue;
    }
    set_error("decode_stream launch: %s", cudaGetErrorString(err));
    return kErrCuda;
  }
  if (settle) launch_mode.store(mode, std::memory_order_relaxed);
  return check_last("decode_stream");
}

}  // namespace moc
