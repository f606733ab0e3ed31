// Row-wise Top-K with the forward fusion of the MoC FFN (moc/ffn.py:141-161,
// moc/training/triton_sparse_aux.py:17-49) as a persistent, shared-memory-staged kernel for bf16 rows.
//
// One CTA works on one token row at a time. A producer warp moves rows with bulk asynchronous copies: the gate
// row and the dense U row of row i + 2 are in flight into one buffer pair while the six compute warps work on
// row i in the other, and the finished row leaves the same way (the gate buffer, rewritten in place to
// Z' = mask * round(round(SiLU(g)) * u), as one bulk store; the compact idx / g_sel / u_sel arrays are written by
// coalesced stores from compact space). Each row is read from HBM once and every pass below runs on shared memory:
//
//   1  2048-bin histogram of the upper 11 bits of the RAW bf16 patterns (no key transform per element: the
//      order key is a per-bin bijection of the raw pattern, so the scan walks the bins in key order instead)
//   2  a block scan over the bins in key order finds the bin of the K-th largest key
//   3  the keys of that bin (a few percent of the row, found by a two-per-word pattern test) enter a 32-bin
//      histogram of their lower 5 bits -> K-th largest key and the number of ties to admit. Pass 1 already does
//      this for the threshold bin of the CTA's previous row; rows of a batch are alike, so the extra pass
//      over the row is rarely needed
//   4  thread t owns the 32-channel word t of the row: selection mask by compares, one block scan over
//      (count greater, count equal) gives the output position and the ties admitted before the word (lower
//      channel wins, as optimized_global_moc_ext.cu:85-125); bitmap and rank words; the selected (channel, g, u)
//      go to the compact stage in ascending channel order
//   5  SiLU and the product in compact space with full lanes; z scattered into the zeroed row
//
// Channels beyond d_ffn in the padded row are given the smallest key, so they behave like extra channels that
// can never be selected (K <= d_ffn). Every wait is bounded; a time-out sets the status word, and all roles
// leave the row loop together.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace moc {

constexpr int kRsWarps = 6;                        // compute warps
constexpr int kRsCompute = kRsWarps * 32;          // 192: one mask word per thread and chunk
constexpr int kRsThreads = kRsCompute + 32;        // + the producer warp
constexpr int kRsBins = 2048;
constexpr int kRsMaxCtasPerSm = 4;

struct RowSelArgs {
  uint16_t* g;             // [tokens, ldg] gate rows in, Z' rows out
  const uint16_t* u;       // [tokens, ldg] dense U rows
  int16_t* idx;            // [tokens, k]
  uint16_t* g_sel;         // [tokens, k]
  uint16_t* u_sel;         // [tokens, k]
  uint16_t* s_sel;         // [tokens, k] or null
  uint16_t* z_sel;         // [tokens, k] or null
  uint32_t* bitmap;        // [tokens, words]
  uint16_t* rank0;         // [tokens, words]
  int* status;
  int64_t ldg;
  int tokens, d_ffn, k, words;
  int kpad;                // k rounded up to 8
  int stage_in_hist;       // the compact stage (6 * kpad bytes) fits the first-level histogram's storage
};

struct RowSelShared {
  uint32_t hist[kRsBins];
  uint32_t hist2[32];
  uint64_t full[2];
  uint32_t wtot[2][8];     // warp totals of the block scan of pass 4, double-buffered over chunks
  uint32_t stot[8];        // warp totals of the block scan of pass 2
  uint32_t has_top;        // the row holds +inf or a positive NaN
  uint32_t bin_pos;        // position of the threshold bin in key order, counted from the top
  uint32_t k_rem;          // rank of the K-th key inside that bin, counted from the top
  int abort;
};

__device__ __forceinline__ void rs_compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kRsCompute) : "memory"); }
__device__ __forceinline__ void rs_all_sync() { asm volatile("bar.sync 2, %0;" ::"n"(kRsThreads) : "memory"); }

__device__ __forceinline__ uint32_t rs_incl_scan(uint32_t v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xFFFFFFFFu, v, o);
    if (lane >= o) v += nb;
  }
  return v;
}

// bits 0..15 -> even positions, bits 16..31 -> odd positions (outer perfect shuffle)
__device__ __forceinline__ uint32_t rs_interleave16(uint32_t x) {
  uint32_t t = (x ^ (x >> 8)) & 0x0000FF00u;
  x = x ^ t ^ (t << 8);
  t = (x ^ (x >> 4)) & 0x00F000F0u;
  x = x ^ t ^ (t << 4);
  t = (x ^ (x >> 2)) & 0x0C0C0C0Cu;
  x = x ^ t ^ (t << 2);
  t = (x ^ (x >> 1)) & 0x22222222u;
  x = x ^ t ^ (t << 1);
  return x;
}

// raw bin (upper 11 bits of the bf16 pattern) at position i of the key order, counted from the largest key:
// positive patterns first, downwards, then the negative ones upwards
__device__ __forceinline__ uint32_t rs_raw_bin(uint32_t i) { return i < 1024u ? 1023u - i : i; }

__global__ void __launch_bounds__(kRsThreads, kRsMaxCtasPerSm) select_stream_kernel(const RowSelArgs a) {
  extern __shared__ __align__(128) uint8_t rs_dyn[];
  __shared__ __align__(16) RowSelShared sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t row_bytes = static_cast<uint32_t>(a.words) * 64u;
  // dynamic shared memory: [buffer][g row | u row], then the compact stage (channel | g, u) of the current row
  uint8_t* rows = rs_dyn;
  uint8_t* stages = rs_dyn + 4u * row_bytes;
  const int grid = gridDim.x;
  volatile int* abort_flag = &sh.abort;

  if (tid == 0) {
    ptx::mbar_init(&sh.full[0], 1);
    ptx::mbar_init(&sh.full[1], 1);
    sh.abort = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  __syncthreads();

  if (warp == kRsWarps) {
    // ------------------------------ producer warp ------------------------------
    auto fetch = [&](int row, int b) {
      ptx::mbar_arrive_expect_tx(&sh.full[b], 2u * row_bytes);
      ptx::bulk_load(rows + (2 * b) * row_bytes, a.g + static_cast<int64_t>(row) * a.ldg, row_bytes, &sh.full[b]);
      ptx::bulk_load(rows + (2 * b + 1) * row_bytes, a.u + static_cast<int64_t>(row) * a.ldg, row_bytes, &sh.full[b]);
    };
    if (lane == 0) {
      if (static_cast<int>(blockIdx.x) < a.tokens) fetch(blockIdx.x, 0);
      if (static_cast<int>(blockIdx.x) + grid < a.tokens) fetch(blockIdx.x + grid, 1);
    }
#pragma unroll 1
    for (int i = 0;; ++i) {
      const int row = blockIdx.x + i * grid;
      if (row >= a.tokens) break;
      const int b = i & 1;
      rs_all_sync();                      // the compute warps are done with row i
      if (sh.abort != 0) break;
      if (lane == 0) {
        ptx::bulk_store(a.g + static_cast<int64_t>(row) * a.ldg, rows + (2 * b) * row_bytes, row_bytes);
        ptx::bulk_commit_group();
        const int next = row + 2 * grid;
        if (next < a.tokens) {
          ptx::bulk_wait_group_read0();   // the stores have read buffer b: it may be refilled
          fetch(next, b);
        }
      }
      __syncwarp();
    }
    if (lane == 0) ptx::bulk_wait_group0();
    return;
  }

  // ------------------------------ compute warps ------------------------------
  const int nvec = a.words * 4;
  const int k = a.k;
  const uint32_t kk = static_cast<uint32_t>(k);
  // Threshold bin of the previous row of this CTA (raw bin; none yet: a pattern no bin has). Rows of one batch are
  // alike, so pass 1 also counts the lower 5 bits of the keys of that bin; when the guess holds, pass 3 is skipped.
  uint32_t guess_bin = 0xFFFFFFFFu;
  // compact stage of the current row: over the first-level histogram (not needed once pass 2 is done) when it
  // fits there, else behind the row buffers
  uint8_t* stage = a.stage_in_hist ? reinterpret_cast<uint8_t*>(sh.hist) : stages;
  uint32_t* st_ig = reinterpret_cast<uint32_t*>(stage);                          // [kpad] channel | g bits << 16
  uint16_t* st_u = reinterpret_cast<uint16_t*>(stage + 4u * a.kpad);             // [kpad]
#pragma unroll 1
  for (int i = 0;; ++i) {
    const int row = blockIdx.x + i * grid;
    if (row >= a.tokens) break;
    const int b = i & 1;
    uint16_t* grow = reinterpret_cast<uint16_t*>(rows + (2 * b) * row_bytes);
    const uint16_t* urow = reinterpret_cast<const uint16_t*>(rows + (2 * b + 1) * row_bytes);

    // clear the histograms while the row may still be landing
    {
      uint4* h4 = reinterpret_cast<uint4*>(sh.hist);
      for (int j = tid; j < kRsBins / 4; j += kRsCompute) h4[j] = make_uint4(0u, 0u, 0u, 0u);
      if (tid < 32) sh.hist2[tid] = 0u;
    }
    if (!ptx::mbar_wait(&sh.full[b], (i >> 1) & 1u, abort_flag)) {
      sh.abort = 1;
      atomicCAS(a.status, 0, (kDevTimeoutEpilogue << 24) | 0x00D00000 | (i & 0xFFFF));
    }
    // padding channels: the smallest key (raw pattern 0xFFFF)
    for (int c = a.d_ffn + tid; c < a.words * 32; c += kRsCompute) grow[c] = 0xFFFFu;
    rs_compute_sync();
    if (sh.abort != 0) {
      rs_all_sync();   // releases the producer warp, which leaves as well
      break;
    }

    // ---- 1: histogram of the upper 11 raw bits (+ the lower 5 bits of the keys of the guessed bin) ----
    {
      // no guess: a pattern with odd halves, which no masked word can equal
      const uint32_t gpat2 = guess_bin < 2048u ? (guess_bin << 5) * 0x00010001u : 0x00010001u;
      const bool gpos = guess_bin < 1024u;
      const uint4* g4 = reinterpret_cast<const uint4*>(grow);
#pragma unroll 2
      for (int v = tid; v < nvec; v += kRsCompute) {
        const uint4 q = g4[v];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          atomicAdd(&sh.hist[(w[j] >> 5) & 0x7FFu], 1u);
          atomicAdd(&sh.hist[w[j] >> 21], 1u);
          // a half of t is zero exactly for a pattern of the bin; the halves are multiples of 32, so the
          // has-zero identity is exact (no borrow can fake a zero in the upper half)
          const uint32_t t = (w[j] & 0xFFE0FFE0u) ^ gpat2;
          const uint32_t hit = ((t - 0x00010001u) & ~t) & 0x80008000u;
          if (hit) {
            if (hit & 0x8000u) atomicAdd(&sh.hist2[gpos ? (w[j] & 31u) : 31u - (w[j] & 31u)], 1u);
            if (hit & 0x80000000u)
              atomicAdd(&sh.hist2[gpos ? ((w[j] >> 16) & 31u) : 31u - ((w[j] >> 16) & 31u)], 1u);
          }
        }
      }
    }
    rs_compute_sync();

    // ---- 2: the bin that holds the K-th largest key: block scan over the bins in key order, 11 per thread ----
    {
      constexpr int kPer = (kRsBins + kRsCompute - 1) / kRsCompute;   // 11
      const uint32_t p0 = static_cast<uint32_t>(tid) * kPer;
      uint32_t c[kPer];
      uint32_t local = 0;
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        c[j] = p0 + j < kRsBins ? sh.hist[rs_raw_bin(p0 + j)] : 0u;
        local += c[j];
      }
      // positions 0..3 are the raw bins of +inf and the positive NaNs
      if (tid == 0) sh.has_top = c[0] | c[1] | c[2] | c[3];
      const uint32_t incl = rs_incl_scan(local, lane);
      if (lane == 31) sh.stot[warp] = incl;
      rs_compute_sync();
      uint32_t above = incl - local;
#pragma unroll
      for (int w = 0; w < kRsWarps; ++w)
        if (w < warp) above += sh.stot[w];
      if (above < kk && above + local >= kk) {     // exactly one thread
        uint32_t ex = above;
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          if (ex < kk && ex + c[j] >= kk) {
            sh.bin_pos = p0 + j;
            sh.k_rem = kk - ex;
          }
          ex += c[j];
        }
      }
    }
    rs_compute_sync();

    // ---- 3: lower 5 bits of the keys of the threshold bin, unless pass 1 counted them already ----
    const uint32_t bin_pos = sh.bin_pos;
    const uint32_t raw_bin = rs_raw_bin(bin_pos);
    const bool positive = bin_pos < 1024u;
    if (raw_bin != guess_bin) {
      if (tid < 32) sh.hist2[tid] = 0u;
      rs_compute_sync();
      const uint32_t pat2 = (raw_bin << 5) * 0x00010001u;
      const uint4* g4 = reinterpret_cast<const uint4*>(grow);
#pragma unroll 2
      for (int v = tid; v < nvec; v += kRsCompute) {
        const uint4 q = g4[v];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t t = (w[j] & 0xFFE0FFE0u) ^ pat2;
          const uint32_t hit = ((t - 0x00010001u) & ~t) & 0x80008000u;
          if (hit) {
            if (hit & 0x8000u) atomicAdd(&sh.hist2[positive ? (w[j] & 31u) : 31u - (w[j] & 31u)], 1u);
            if (hit & 0x80000000u)
              atomicAdd(&sh.hist2[positive ? ((w[j] >> 16) & 31u) : 31u - ((w[j] >> 16) & 31u)], 1u);
          }
        }
      }
      rs_compute_sync();
    }
    guess_bin = raw_bin;
    uint32_t raw_thr, take_eq;
    {
      // every warp derives the threshold redundantly: lane l holds the count of the (31 - l)-th low-bit value
      const uint32_t c = sh.hist2[31 - lane];
      const uint32_t incl = rs_incl_scan(c, lane);
      const uint32_t ex = incl - c, krem = sh.k_rem;
      const int src = __ffs(__ballot_sync(0xFFFFFFFFu, ex < krem && incl >= krem)) - 1;
      const uint32_t low = 31u - static_cast<uint32_t>(src);
      take_eq = krem - __shfl_sync(0xFFFFFFFFu, ex, src);
      raw_thr = (raw_bin << 5) | (positive ? low : 31u - low);
    }

    // ---- 4: masks, positions, compact stage ----
    uint32_t base_gt = 0, base_eq = 0;
    uint32_t* bm_row = a.bitmap + static_cast<int64_t>(row) * a.words;
    uint16_t* rk_row = a.rank0 + static_cast<int64_t>(row) * a.words;
    const uint32_t thr_key = order_key16(static_cast<uint16_t>(raw_thr));
    // Packed bf16 compares order the row like the keys do when the threshold is a positive normal number and the
    // row holds neither +inf nor a positive NaN (a NaN compares false but has the largest key; -0 equals +0 but
    // has a smaller key): every negative pattern then lies below the threshold under both orders.
    const bool packed_cmp = positive && raw_thr >= 0x0080u && sh.has_top == 0u;
    const uint32_t thr_pair = raw_thr * 0x00010001u;
    const __nv_bfloat162 thr2 = *reinterpret_cast<const __nv_bfloat162*>(&thr_pair);
    int chunk = 0;
#pragma unroll 1
    for (int w0 = 0; w0 < a.words; w0 += kRsCompute, ++chunk) {
      const int wd = w0 + tid;
      uint32_t gtm = 0, eqm = 0;
      if (wd < a.words) {
        const uint4* g4 = reinterpret_cast<const uint4*>(grow) + 4 * wd;
#pragma unroll
        for (int v0 = 0; v0 < 4; ++v0) {
          const int v = (v0 + (tid >> 1)) & 3;   // rotated start: the 64-byte stride of the words meets no bank twice
          const uint4 q = g4[v];
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
          if (packed_cmp) {
            // two channels per compare instruction; flags in split order: even channels in bits 0..15, odd
            // channels in bits 16..31 (pair 4 v + j -> bits 4 v + j and 16 + 4 v + j)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
              const uint32_t sel = 0x00010001u << (4 * v + j);
              gtm |= __hgt2_mask(h, thr2) & sel;
              eqm |= __hge2_mask(h, thr2) & sel;     // greater or equal; reduced to equal below
            }
          } else {
            uint32_t gt8 = 0, eq8 = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t m = (w[j] >> 15) & 0x00010001u;
              const uint32_t kx = w[j] ^ 0x80008000u ^ (m * 0x7FFFu);     // two order keys
              const uint32_t lo = kx & 0xFFFFu, hi = kx >> 16;
              gt8 |= (lo > thr_key ? 1u : 0u) << (2 * j);
              gt8 |= (hi > thr_key ? 1u : 0u) << (2 * j + 1);
              eq8 |= (lo == thr_key ? 1u : 0u) << (2 * j);
              eq8 |= (hi == thr_key ? 1u : 0u) << (2 * j + 1);
            }
            gtm |= gt8 << (8 * v);
            eqm |= eq8 << (8 * v);
          }
        }
        if (packed_cmp) {
          eqm &= ~gtm;
          gtm = rs_interleave16(gtm);
          if (eqm) eqm = rs_interleave16(eqm);
        }
      }
      // block scan over (greater, equal) counts, packed 16 + 16 bits
      const uint32_t mine = static_cast<uint32_t>(__popc(gtm)) | (static_cast<uint32_t>(__popc(eqm)) << 16);
      const uint32_t incl = rs_incl_scan(mine, lane);
      if (lane == 31) sh.wtot[chunk & 1][warp] = incl;
      rs_compute_sync();
      uint32_t before = incl - mine, total = 0;
#pragma unroll
      for (int w = 0; w < kRsWarps; ++w) {
        const uint32_t t = sh.wtot[chunk & 1][w];
        if (w < warp) before += t;
        total += t;
      }
      const uint32_t gt_before = base_gt + (before & 0xFFFFu);
      const uint32_t eq_before = base_eq + (before >> 16);
      base_gt += total & 0xFFFFu;
      base_eq += total >> 16;
      // ties: the lowest channels first, take_eq in the whole row
      const int allowed = static_cast<int>(take_eq) - static_cast<int>(min(eq_before, take_eq));
      uint32_t sel_eq = allowed > 0 ? eqm : 0u;
      while (sel_eq && __popc(sel_eq) > allowed) sel_eq &= ~(0x80000000u >> __clz(sel_eq));
      const uint32_t selm = gtm | sel_eq;
      uint32_t pos = gt_before + min(eq_before, take_eq);
      if (wd < a.words) {
        bm_row[wd] = selm;
        rk_row[wd] = static_cast<uint16_t>(pos);
        uint32_t m = selm;
        while (m) {
          const int j = __ffs(m) - 1;
          m &= m - 1u;
          const uint32_t ch = static_cast<uint32_t>(wd * 32 + j);
          st_ig[pos] = ch | (static_cast<uint32_t>(grow[ch]) << 16);
          st_u[pos] = urow[ch];
          ++pos;
        }
        // the row becomes Z': zero now, the selected channels are filled in below
        uint4* z4 = reinterpret_cast<uint4*>(grow) + 4 * wd;
#pragma unroll
        for (int v0 = 0; v0 < 4; ++v0) z4[(v0 + (tid >> 1)) & 3] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    rs_compute_sync();

    // ---- 5: s = round(SiLU(g)), z = round(s * u) in compact space; z into the row; the compact outputs ----
    {
      const int64_t off = static_cast<int64_t>(row) * k;
#pragma unroll 2
      for (int p = tid; p < k; p += kRsCompute) {
        const uint32_t ig = st_ig[p];
        const uint32_t ch = ig & 0xFFFFu, gb = ig >> 16, ub = st_u[p];
        float sv, zv;
        moc_fwd_point<__nv_bfloat16>(__uint_as_float(gb << 16), __uint_as_float(ub << 16), sv, zv);
        const uint16_t zb = static_cast<uint16_t>(__float_as_uint(zv) >> 16);   // zv is already a bf16 value
        grow[ch] = zb;
        a.idx[off + p] = static_cast<int16_t>(ch);
        a.g_sel[off + p] = static_cast<uint16_t>(gb);
        a.u_sel[off + p] = static_cast<uint16_t>(ub);
        if (a.s_sel) a.s_sel[off + p] = static_cast<uint16_t>(__float_as_uint(sv) >> 16);
        if (a.z_sel) a.z_sel[off + p] = zb;
      }
    }
    ptx::fence_proxy_async_smem();   // the bulk store reads what these threads wrote
    rs_all_sync();                   // hands row i to the producer warp
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static size_t rs_dynamic_smem(int words, int k) {
  const size_t kpad = static_cast<size_t>((k + 7) / 8 * 8);
  return 4 * static_cast<size_t>(words) * 64 + (6 * kpad <= kRsBins * 4 ? 0 : 6 * kpad);
}

static void rs_device_limits(int& sms, int& smem_sm, int& smem_block) {
  static int s_sms = 0, s_sm = 0, s_block = 0;
  if (s_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&s_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    cudaDeviceGetAttribute(&s_block, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaDeviceGetAttribute(&s_sms, cudaDevAttrMultiProcessorCount, dev);
    if (s_sms <= 0) s_sms = 148;
  }
  sms = s_sms;
  smem_sm = s_sm;
  smem_block = s_block;
}

bool select_stream_supported(int64_t ldg, int d_ffn, int k, const void* g, const void* u_dense) {
  const int words = static_cast<int>(mask_words(d_ffn));
  if (ldg < static_cast<int64_t>(words) * 32 || ldg % 8 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(g) & 15u) != 0 || (reinterpret_cast<uintptr_t>(u_dense) & 15u) != 0) return false;
  int sms, smem_sm, smem_block;
  rs_device_limits(sms, smem_sm, smem_block);
  return rs_dynamic_smem(words, k) + sizeof(RowSelShared) + 1024 <= static_cast<size_t>(smem_block);
}

int launch_select_stream(void* g, int64_t ldg, int tokens, int d_ffn, int k, const SelectFuse& fuse, int16_t* idx,
                         void* g_sel, uint32_t* bitmap, uint16_t* rank0, int* status, cudaStream_t stream) {
  RowSelArgs a;
  a.g = static_cast<uint16_t*>(g);
  a.u = static_cast<const uint16_t*>(fuse.u_dense);
  a.idx = idx;
  a.g_sel = static_cast<uint16_t*>(g_sel);
  a.u_sel = static_cast<uint16_t*>(fuse.u_sel);
  a.s_sel = static_cast<uint16_t*>(fuse.s_sel);
  a.z_sel = static_cast<uint16_t*>(fuse.z_sel);
  a.bitmap = bitmap;
  a.rank0 = rank0;
  a.status = status;
  a.ldg = ldg;
  a.tokens = tokens;
  a.d_ffn = d_ffn;
  a.k = k;
  a.words = static_cast<int>(mask_words(d_ffn));
  a.kpad = (k + 7) / 8 * 8;
  a.stage_in_hist = 6 * a.kpad <= kRsBins * 4 ? 1 : 0;
  int sms, smem_sm, smem_block;
  rs_device_limits(sms, smem_sm, smem_block);
  const size_t dyn = rs_dynamic_smem(a.words, k);
  // CTAs that fit one SM (each also pays its static shared memory and 1 KB of system reserve)
  int per_sm = static_cast<int>(static_cast<size_t>(smem_sm) / (dyn + sizeof(RowSelShared) + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > kRsMaxCtasPerSm ? kRsMaxCtasPerSm : per_sm);
  if (cudaFuncSetAttribute(select_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dyn)) !=
      cudaSuccess)
    return check_last("select_stream smem attribute");
  int grid = sms * per_sm;
  if (grid > tokens) grid = tokens;
  select_stream_kernel<<<grid, kRsThreads, dyn, stream>>>(a);
  return check_last("select_stream");
}

}  // namespace moc
