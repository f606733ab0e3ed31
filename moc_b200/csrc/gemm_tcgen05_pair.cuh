// CTA-pair variant of the bf16 GEMM core: two CTAs of a cluster (cta_group::2) compute one 256 x 256
// output tile. Each CTA loads its own 128 rows of A and its own 128-row half of the B tile (32 KB per
// k-block instead of the 48 KB of the single-CTA 128 x 256 tile), the leader CTA issues
// tcgen05.mma.cta_group::2 for both, and each CTA's epilogue warps drain the 128 accumulator rows that
// live in its own tensor memory. The single-CTA core is bound by the rate at which one SM can pull
// operand tiles from L2 (ncu: tensor pipe 75 % active, 88 B/clk/SM needed at full rate); sharing the
// B tile between two SMs removes a third of that traffic. No multicast load is used: every CTA
// fetches its own tiles, only the barrier that its loads complete on lives in the leader CTA.
//
// Same contract, operand majors, K segments, groups and epilogue functors as gemm_tcgen05_kernel.
// Synchronisation between the two CTAs:
//   full[s]    (leader)      <- TMA bytes of both CTAs (+ the leader producer's expect_tx)
//   empty[s]   (both)        <- tcgen05.commit multicast by the leader's MMA thread
//   tfull[a]   (both)        <- tcgen05.commit multicast after the last k-block of a tile
//   tempty[a]  (leader)      <- one arrive per epilogue warp of both CTAs (remote for the peer)
//   sfull[q]   (both)        <- the leader's producer thread after it wrote tile index q of the tile queue
//   sempty[q]  (leader)      <- every consumer of a queue slot: MMA thread, peer producer, all epilogue warps
// Tile queue: the leader's producer thread decides the next tile of the pair - round-robin over the clusters, or,
// when the launch passes a zeroed device counter, by atomicAdd in arrival order, so that clusters that start
// late or lose their SMs to another kernel (a collective on a side stream) simply take fewer tiles - and
// publishes it to a small ring in the shared memory of both CTAs. The fetch of tile i+1 is issued before the
// loads of tile i, so its latency is hidden. A tile index >= num_tiles ends every role.
// Every wait is bounded; an abort is recorded in the status word and makes all roles of the CTA leave.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "epilogues.cuh"
#include "gemm_tcgen05.cuh"
#include "ptx.cuh"

namespace moc {

constexpr int kPairStages = 6;
constexpr int kPairTileABytes = kBlockM * kBlockK * 2;          // 128 rows of A: 16 KiB
constexpr int kPairTileBBytes = (kBlockN / 2) * kBlockK * 2;    // 128 of the 256 rows of B: 16 KiB
constexpr int kPairStageBytes = kPairTileABytes + kPairTileBBytes;
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256;
constexpr int kSchedDepth = 4;   // producer runs at most one tile ahead of the MMAs, the epilogue at most two behind
constexpr uint32_t kSchedConsumers = 2 * kEpiWarps + 2;   // epilogue warps of both CTAs, MMA thread, peer producer

template <class Epi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ GemmMaps maps, const GemmShape sh, const Epi epi) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  uint64_t* full_bar = bars;                      // [kPairStages] used in the leader CTA only
  uint64_t* empty_bar = bars + kPairStages;       // [kPairStages]
  uint64_t* tfull_bar = bars + 2 * kPairStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2] used in the leader CTA only
  uint64_t* sfull_bar = tempty_bar + 2;           // [kSchedDepth]
  uint64_t* sempty_bar = sfull_bar + kSchedDepth; // [kSchedDepth] used in the leader CTA only
  uint32_t* sched_tile = reinterpret_cast<uint32_t*>(sempty_bar + kSchedDepth);   // [kSchedDepth]
  uint32_t* tmem_slot = sched_tile + kSchedDepth;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * kPairStages + 4 + 2 * kSchedDepth) * 8 + kSchedDepth * 4 + 8 <= 256, "barrier area overflow");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();   // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  // sh.tiles_m counts 256-row tile pairs here
  const int tiles_per_group = sh.tiles_m * sh.tiles_n;
  const int num_tiles = tiles_per_group * sh.groups;
  const int kb_total = sh.kb0 + sh.kb1;

  if (threadIdx.x == 0) {
    const int nmaps = sh.kb1 > 0 ? 2 : sh.groups;
    for (int i = 0; i < nmaps; ++i) {
      ptx::prefetch_tensormap(&maps.a[i]);
      ptx::prefetch_tensormap(&maps.b[i]);
    }
#pragma unroll
    for (int s = 0; s < kPairStages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    ptx::mbar_init(&tfull_bar[0], 1);
    ptx::mbar_init(&tfull_bar[1], 1);
    ptx::mbar_init(&tempty_bar[0], 2 * kEpiWarps);
    ptx::mbar_init(&tempty_bar[1], 2 * kEpiWarps);
#pragma unroll
    for (int q = 0; q < kSchedDepth; ++q) {
      ptx::mbar_init(&sfull_bar[q], 1);
      ptx::mbar_init(&sempty_bar[q], kSchedConsumers);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_alloc_permit_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync();          // barriers of both CTAs are initialised before any remote arrive
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs); the leader's also feeds the tile queue ------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      uint32_t cur = 0;
      if (rank == 0)
        cur = sh.tile_counter ? static_cast<uint32_t>(atomicAdd(sh.tile_counter, 1)) : static_cast<uint32_t>(pair);
      for (uint32_t qi = 0; ok; ++qi) {
        const int q = qi % kSchedDepth;
        const uint32_t qph = (qi / kSchedDepth) & 1u;
        uint32_t nxt = 0;
        if (rank == 0) {
          // next tile first: the atomic's round trip overlaps the loads of the current tile
          if (cur < static_cast<uint32_t>(num_tiles))
            nxt = sh.tile_counter ? static_cast<uint32_t>(atomicAdd(sh.tile_counter, 1)) : cur + num_pairs;
          else
            nxt = cur;
          if (!ptx::mbar_wait_cluster(&sempty_bar[q], qph ^ 1u, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(sh.status, 0, (kDevTimeoutProducer << 24) | 0x800000 | (qi & 0x7FFFFF));
            break;
          }
          sched_tile[q] = cur;
          ptx::st_shared_cluster_u32(ptx::map_to_cta(ptx::smem_u32(&sched_tile[q]), 1), cur);
          ptx::mbar_arrive(&sfull_bar[q]);
          ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&sfull_bar[q]), 1));
        } else {
          if (!ptx::mbar_wait_cluster(&sfull_bar[q], qph, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(sh.status, 0, (kDevTimeoutProducer << 24) | 0x400000 | (qi & 0x3FFFFF));
            break;
          }
          cur = sched_tile[q];
          ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&sempty_bar[q]), 0));
        }
        if (cur >= static_cast<uint32_t>(num_tiles)) break;
        const int tile = static_cast<int>(cur);
        const int group = tile / tiles_per_group;
        const int t = tile - group * tiles_per_group;
        const int m0 = (t / sh.tiles_n) * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;
        const int n0 = (t % sh.tiles_n) * kBlockN + static_cast<int>(rank) * (kBlockN / 2);
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1u;
          if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(sh.status, 0, (kDevTimeoutProducer << 24) | (it & 0x3FFFFF));
            ok = false;
            break;
          }
          if (rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * kPairStageBytes);   // bytes of both CTAs
          const uint32_t full_leader = ptx::map_to_cta(ptx::smem_u32(&full_bar[s]), 0);
          const bool seg1 = kb >= sh.kb0;
          const int kk = (seg1 ? kb - sh.kb0 : kb) * kBlockK;
          const int mi = seg1 ? 1 : group;
          const CUtensorMap* ta = &maps.a[mi];
          const CUtensorMap* tb = &maps.b[mi];
          uint8_t* sa = smem + s * kPairStageBytes;
          uint8_t* sb = sa + kPairTileABytes;
          if (!sh.a_mn) {
            ptx::tma_load_2d_pair(sa, ta, full_leader, kk, m0);
          } else {
#pragma unroll
            for (int i = 0; i < kBlockM / 64; ++i)
              ptx::tma_load_2d_pair(sa + i * kMnBoxBytes, ta, full_leader, m0 + 64 * i, kk);
          }
          if (!sh.b_mn) {
            ptx::tma_load_2d_pair(sb, tb, full_leader, kk, n0);
          } else {
#pragma unroll
            for (int i = 0; i < kBlockN / 2 / 64; ++i)
              ptx::tma_load_2d_pair(sb + i * kMnBoxBytes, tb, full_leader, n0 + 64 * i, kk);
          }
        }
        cur = nxt;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = ptx::make_idesc_bf16(2 * kBlockM, kBlockN, sh.a_mn, sh.b_mn);
      const uint32_t a_lbo = sh.a_mn ? kMnBoxBytes : 0, a_step = sh.a_mn ? kUmmaK * 128 : kUmmaK * 2;
      const uint32_t b_lbo = sh.b_mn ? kMnBoxBytes : 0, b_step = sh.b_mn ? kUmmaK * 128 : kUmmaK * 2;
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (; ok; ++tcount) {
        {
          const int q = tcount % kSchedDepth;
          if (!ptx::mbar_wait(&sfull_bar[q], (tcount / kSchedDepth) & 1u, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(sh.status, 0, (kDevTimeoutMma << 24) | 0xC00000 | (tcount & 0x3FFFFF));
            break;
          }
          const uint32_t tile = sched_tile[q];
          ptx::mbar_arrive(&sempty_bar[q]);
          if (tile >= static_cast<uint32_t>(num_tiles)) break;
        }
        const uint32_t acc = tcount & 1u;
        const uint32_t aph = (tcount >> 1) & 1u;
        if (!ptx::mbar_wait_cluster(&tempty_bar[acc], aph ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(sh.status, 0, (kDevTimeoutMma << 24) | 0x800000 | (tcount & 0x7FFFFF));
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBlockN;
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1u;
          if (!ptx::mbar_wait(&full_bar[s], ph, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(sh.status, 0, (kDevTimeoutMma << 24) | (it & 0x7FFFFF));
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_base = ptx::smem_u32(smem + s * kPairStageBytes);
          const uint32_t b_base = a_base + kPairTileABytes;
#pragma unroll
          for (int ks = 0; ks < kBlockK / kUmmaK; ++ks) {
            const uint64_t da = ptx::make_smem_desc_sw128(a_base + ks * a_step, a_lbo, 1024);
            const uint64_t db = ptx::make_smem_desc_sw128(b_base + ks * b_step, b_lbo, 1024);
            ptx::umma_bf16_ss_pair(d_tmem, da, db, idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          ptx::umma_commit_pair(&empty_bar[s], 3);   // both CTAs may refill this stage
        }
        if (ok) ptx::umma_commit_pair(&tfull_bar[acc], 3);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (both CTAs, own 128 rows) ------------------------------
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;
    constexpr int kChunks = kEpiPartCols / 32;
    const uint32_t tempty_leader0 = ptx::map_to_cta(ptx::smem_u32(&tempty_bar[0]), 0);
    const uint32_t tempty_leader1 = ptx::map_to_cta(ptx::smem_u32(&tempty_bar[1]), 0);
    const uint32_t sempty_leader = ptx::map_to_cta(ptx::smem_u32(&sempty_bar[0]), 0);
    for (uint32_t tcount = 0;; ++tcount) {
      const int q = tcount % kSchedDepth;
      if (!ptx::mbar_wait_cluster(&sfull_bar[q], (tcount / kSchedDepth) & 1u, abort_flag)) {
        *abort_flag = 1;
        atomicCAS(sh.status, 0, (kDevTimeoutEpilogue << 24) | 0x800000 | (tcount & 0x7FFFFF));
        break;
      }
      const int tile = static_cast<int>(sched_tile[q]);
      __syncwarp();   // every lane has read the slot before it is handed back
      if (lane == 0) ptx::mbar_arrive_cluster(sempty_leader + q * 8);
      if (tile >= num_tiles) break;
      const uint32_t acc = tcount & 1u;
      const uint32_t aph = (tcount >> 1) & 1u;
      const int group = tile / tiles_per_group;
      const int t = tile - group * tiles_per_group;
      const int m0 = (t / sh.tiles_n) * (2 * kBlockM) + static_cast<int>(rank) * kBlockM;
      const int col_first = (t % sh.tiles_n) * kBlockN + part * kEpiPartCols;
      const int row = m0 + quad * 32 + lane;
      const int nchunks = min(kChunks, (sh.n - col_first + 31) / 32);
      const bool active = row < sh.m && nchunks > 0;
      typename Epi::Ctx ctx;
      if (active) epi.begin(ctx, group, row, col_first, nchunks);
      if (!ptx::mbar_wait(&tfull_bar[acc], aph, abort_flag)) {
        *abort_flag = 1;
        atomicCAS(sh.status, 0, (kDevTimeoutEpilogue << 24) | (tcount & 0x7FFFFF));
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kBlockN +
                             part * kEpiPartCols;
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        if (c < nchunks) {
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
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(acc ? tempty_leader1 : tempty_leader0);
    }
  }

  // ------------------------------ tear-down ------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(200);
    __syncthreads();
  }
  ptx::cluster_sync();   // the peer may still read this CTA's tiles or signal its barriers until here
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace moc
