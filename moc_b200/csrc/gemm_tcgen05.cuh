// bf16 GEMM core for sm_100a: C[M,N] = A[M,K] * B[N,K]^T, fp32 accumulation in tensor memory,
// fused epilogue functor.
//
//   * persistent: one CTA per SM walks output tiles of 128 x 256;
//   * warp 0 = TMA producer (4-stage ring of 128-byte-swizzled A/B tiles, BLOCK_K = 64),
//     warp 1 = tcgen05.mma issuer (one elected thread; also owns the TMEM allocation),
//     warps 2-17 = epilogue: four warps per 32-lane TMEM quadrant, each taking one 64-column
//     slice of the tile; a fused epilogue is a serial chain of dependent instructions per
//     warp, so its latency is hidden by warps, not by instruction-level parallelism;
//   * two 256-column TMEM accumulators, so the epilogue of tile i overlaps the MMAs of
//     tile i + 1;
//   * both operands may be K-major (K contiguous in memory) or MN-major (M/N contiguous),
//     which covers X*W^T, dY*W and the dW = act^T * X products without any transposed copy;
//   * two K segments may accumulate two products into the same tile
//     (dX = dG'*W_gate + dU'*W_up, moc/ffn.py:245-255) before the epilogue runs;
//   * up to three same-shape problems may share one launch ("groups": the three dW products
//     of the backward pass), which removes most of the wave-quantisation tail;
//   * every mbarrier wait is bounded: on a time-out the kernel records a code in the
//     status word, all roles leave their loops, TMEM is released and the kernel returns.
//
// These GEMMs stand in for the cuBLAS calls of the reference path (moc/ffn.py:141, :146,
// :163, :203-206, :239-254).
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "epilogues.cuh"
#include "ptx.cuh"

namespace moc {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;    // 64 bf16 = one 128-byte swizzle span
constexpr int kUmmaK = 16;
constexpr int kStages = 4;          // ring depth with full-width (48 KiB) stages
constexpr int kMaxStages = 8;       // ring depth with the narrow B tiles of products with few columns
constexpr int kTileABytes = kBlockM * kBlockK * 2;   // 16 KiB
constexpr int kTileBBytes = kBlockN * kBlockK * 2;   // 32 KiB
constexpr int kStageBytes = kTileABytes + kTileBBytes;
constexpr int kMnBoxBytes = 64 * kBlockK * 2;        // one MN-major TMA box: 64 (mn) x 64 (k)
constexpr int kTmemCols = 512;
constexpr int kEpiWarps = 16;
constexpr int kEpiParts = kEpiWarps / 4;              // column slices of a tile, one per warp of a quadrant
constexpr int kEpiPartCols = kBlockN / kEpiParts;
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;
constexpr int kGemmSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

// Operand descriptors of one launch: (a[i], b[i]) is K segment i of a two-segment product, or
// problem i of a grouped launch.
struct GemmMaps {
  CUtensorMap a[kMaxGroups];
  CUtensorMap b[kMaxGroups];
};

struct GemmShape {
  int m, n;          // extents of C (of every group)
  int kb0, kb1;      // number of 64-wide k-blocks in segment 0 / 1 (kb1 == 0: single product)
  int groups;        // >= 1; groups > 1 requires kb1 == 0
  int a_mn, b_mn;    // 1 = operand is MN-major in memory
  int tiles_m, tiles_n;
  int* status;       // device status word
  int* tile_counter; // pair kernel only: zeroed device int; tiles are handed out in arrival order (null: round-robin)
  int k_splits;      // single-CTA kernel only: > 1 splits the k-blocks of segment 0 over that many tiles; the
                     // epilogue then sees group * k_splits + split as its group index (one partial result each)
  int mma_n;         // single-CTA kernel only: N of the MMA instruction and rows of the B tile in shared memory;
                     // kBlockN, or N rounded up to 16 for products with few columns (K-major B), whose MMAs would
                     // otherwise spend most of their time on columns that do not exist
};

// Which problem, which K range and which output block a tile index stands for.
struct TileWork {
  int group, egroup, t, kb_begin, kb_end;
};
__device__ __forceinline__ TileWork decode_tile(const GemmShape& sh, int tile, int tiles_per_group, int kb_total) {
  TileWork w;
  const int gs = tile / tiles_per_group;
  w.t = tile - gs * tiles_per_group;
  if (sh.k_splits > 1) {
    w.group = gs / sh.k_splits;
    const int split = gs - w.group * sh.k_splits;
    const int per = (sh.kb0 + sh.k_splits - 1) / sh.k_splits;
    w.kb_begin = split * per;
    w.kb_end = min(sh.kb0, w.kb_begin + per);
  } else {
    w.group = gs;
    w.kb_begin = 0;
    w.kb_end = kb_total;
  }
  w.egroup = gs;
  return w;
}

template <class Epi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ GemmMaps maps, const GemmShape sh, const Epi epi) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;                     // [stages] TMA -> MMA
  uint64_t* empty_bar = bars + kMaxStages;       // [stages] MMA -> TMA
  uint64_t* tfull_bar = bars + 2 * kMaxStages;   // [2] MMA -> epilogue
  static_assert((2 * kMaxStages + 4) * 8 + 8 <= 256, "barrier area overflow");
  // a stage = the A tile + a B tile of mma_n rows; narrow B tiles leave room for a deeper ring, which a tile that
  // streams its operand once from HBM needs to keep enough bytes in flight
  const uint32_t stage_bytes = kTileABytes + static_cast<uint32_t>(sh.mma_n) * kBlockK * 2;
  const int stages = min(kMaxStages, static_cast<int>((kStages * kStageBytes) / stage_bytes));
  uint64_t* tempty_bar = tfull_bar + 2;       // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_group = sh.tiles_m * sh.tiles_n;
  const int num_tiles = tiles_per_group * sh.groups * (sh.k_splits > 1 ? sh.k_splits : 1);
  const int kb_total = sh.kb0 + sh.kb1;

  if (threadIdx.x == 0) {
    const int nmaps = sh.kb1 > 0 ? 2 : sh.groups;
    for (int i = 0; i < nmaps; ++i) {
      ptx::prefetch_tensormap(&maps.a[i]);
      ptx::prefetch_tensormap(&maps.b[i]);
    }
#pragma unroll
    for (int s = 0; s < kMaxStages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    ptx::mbar_init(&tfull_bar[0], 1);
    ptx::mbar_init(&tfull_bar[1], 1);
    ptx::mbar_init(&tempty_bar[0], 32 * kEpiWarps);
    ptx::mbar_init(&tempty_bar[1], 32 * kEpiWarps);
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_alloc_permit();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0, ph = 0;
      int s = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileWork tw = decode_tile(sh, tile, tiles_per_group, kb_total);
        const int group = tw.group;
        const int t = tw.t;
        const int m0 = (t / sh.tiles_n) * kBlockM;
        const int n0 = (t % sh.tiles_n) * kBlockN;
        for (int kb = tw.kb_begin; kb < tw.kb_end; ++kb, ++it, s = (s + 1 == stages ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
          if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(sh.status, 0, (kDevTimeoutProducer << 24) | (it & 0xFFFFFF));
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(&full_bar[s], stage_bytes);
          const bool seg1 = kb >= sh.kb0;
          const int kk = (seg1 ? kb - sh.kb0 : kb) * kBlockK;
          const int mi = seg1 ? 1 : group;
          const CUtensorMap* ta = &maps.a[mi];
          const CUtensorMap* tb = &maps.b[mi];
          uint8_t* sa = smem + s * stage_bytes;
          uint8_t* sb = sa + kTileABytes;
          if (!sh.a_mn) {
            ptx::tma_load_2d(sa, ta, &full_bar[s], kk, m0);
          } else {
#pragma unroll
            for (int i = 0; i < kBlockM / 64; ++i)
              ptx::tma_load_2d(sa + i * kMnBoxBytes, ta, &full_bar[s], m0 + 64 * i, kk);
          }
          if (!sh.b_mn) {
            ptx::tma_load_2d(sb, tb, &full_bar[s], kk, n0);
          } else {
#pragma unroll
            for (int i = 0; i < kBlockN / 64; ++i)
              ptx::tma_load_2d(sb + i * kMnBoxBytes, tb, &full_bar[s], n0 + 64 * i, kk);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc = ptx::make_idesc_bf16(kBlockM, sh.mma_n, sh.a_mn, sh.b_mn);
      // K-major tile: rows of 128 bytes, 8-row groups 1024 bytes apart; a k-step of 16
      // elements advances the start address by 32 bytes inside the swizzle span.
      // MN-major tile: boxes of 64 (mn) x 64 (k); 8-k groups 1024 bytes apart (SBO),
      // 64-wide mn groups one box (8192 bytes) apart (LBO); a k-step advances by 16 rows.
      const uint32_t a_lbo = sh.a_mn ? kMnBoxBytes : 0, a_step = sh.a_mn ? kUmmaK * 128 : kUmmaK * 2;
      const uint32_t b_lbo = sh.b_mn ? kMnBoxBytes : 0, b_step = sh.b_mn ? kUmmaK * 128 : kUmmaK * 2;
      uint32_t it = 0, tcount = 0, ph = 0;
      int s = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const uint32_t acc = tcount & 1u;
        const uint32_t aph = (tcount >> 1) & 1u;
        if (!ptx::mbar_wait(&tempty_bar[acc], aph ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(sh.status, 0, (kDevTimeoutMma << 24) | 0x800000 | (tcount & 0x7FFFFF));
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBlockN;
        const TileWork tw = decode_tile(sh, tile, tiles_per_group, kb_total);
        for (int kb = tw.kb_begin; kb < tw.kb_end; ++kb, ++it, s = (s + 1 == stages ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
          if (!ptx::mbar_wait(&full_bar[s], ph, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(sh.status, 0, (kDevTimeoutMma << 24) | (it & 0x7FFFFF));
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_base = ptx::smem_u32(smem + s * stage_bytes);
          const uint32_t b_base = a_base + kTileABytes;
#pragma unroll
          for (int ks = 0; ks < kBlockK / kUmmaK; ++ks) {
            const uint64_t da = ptx::make_smem_desc_sw128(a_base + ks * a_step, a_lbo, 1024);
            const uint64_t db = ptx::make_smem_desc_sw128(b_base + ks * b_step, b_lbo, 1024);
            ptx::umma_bf16_ss(d_tmem, da, db, idesc, (kb != tw.kb_begin || ks != 0) ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[s]);   // frees the smem stage once these MMAs have read it
        }
        if (ok) ptx::umma_commit(&tfull_bar[acc]);   // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;              // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    const int part = (warp - 2) >> 2;       // which column slice of the tile
    constexpr int kChunks = kEpiPartCols / 32;
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      const uint32_t acc = tcount & 1u;
      const uint32_t aph = (tcount >> 1) & 1u;
      const TileWork tw = decode_tile(sh, tile, tiles_per_group, kb_total);
      const int group = tw.egroup;
      const int t = tw.t;
      const int m0 = (t / sh.tiles_n) * kBlockM;
      const int col_first = (t % sh.tiles_n) * kBlockN + part * kEpiPartCols;
      const int row = m0 + quad * 32 + lane;
      const int nchunks = min(kChunks, (sh.n - col_first + 31) / 32);   // <= 0: nothing to do
      const bool active = row < sh.m && nchunks > 0;
      typename Epi::Ctx ctx;
      if (active) epi.begin(ctx, group, row, col_first, nchunks);       // overlaps the wait below
      if (!ptx::mbar_wait(&tfull_bar[acc], aph, abort_flag)) {
        *abort_flag = 1;
        atomicCAS(sh.status, 0, (kDevTimeoutEpilogue << 24) | (tcount & 0xFFFFFF));
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kBlockN +
                             part * kEpiPartCols;
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        if (c < nchunks) {   // warp-uniform
          const int col0 = col_first + c * 32;
          uint32_t r[32];
          ptx::tmem_ld_32x32b_x32(t_row + c * 32, r);
          if (active) epi.prefetch(ctx, row, col0, c);
          ptx::tmem_ld_wait();
          if (active) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            epi(ctx, group, row, col0, c, v);
          }
        }
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&tempty_bar[acc]);
    }
  }

  // ------------------------------ tear-down ------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    // give copies that may still be in flight time to land before shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(200);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace moc
