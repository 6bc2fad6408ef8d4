// fp16 GEMM for sm_100a, 2-CTA variant: a pair of CTAs on neighbouring SMs (a cluster of 2) computes
// one 256x256 output tile with `tcgen05.mma.cta_group::2`.  Each CTA loads its own 128 rows of A and
// its own 128-row half of the W^T tile, so per SM the operand traffic into shared memory drops from
// 48 KB to 32 KB per k-block compared with the 1-CTA kernel (gemm_sm100.cu) -- without any TMA
// multicast: every CTA issues plain per-CTA loads.  Same interface, epilogues and bounded waits.
//
// Roles per CTA (6 warps): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only) + TMEM owner,
// warps 2-5 epilogue for this CTA's 128 rows.
// Barriers: `full[s]` lives in the leader (cluster rank 0); both CTAs' TMA loads signal it.
// `empty[s]` and `tmem_full[a]` exist in both CTAs and are signalled together by the leader's
// tcgen05.commit; `tmem_empty[a]` lives in the leader and collects 4 + 4 epilogue-warp arrivals.
#include <cstdlib>

#include "gemm_epilogue.cuh"

LIGER_REGISTER_WAIT_BUDGET()

namespace liger {

constexpr int kBM2 = 256;  // rows per cluster tile (128 per CTA)
constexpr int kBN2 = 256;

template <int STAGES>
struct Gemm2Cfg {
  static constexpr int kABytes = 128 * BK * 2;   // this CTA's A rows
  static constexpr int kBBytes = 128 * BK * 2;   // this CTA's half of the W^T tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiBytesPerWarp = 32 * 128 * 2;
  static constexpr int kEpiBytes = 4 * kEpiBytesPerWarp;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = STAGES * kStageBytes + kEpiBytes + kBarrierBytes + 1024;
  static constexpr int kTmemCols = 512;  // two 256-column accumulators
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t num_clusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// per-CTA load of a 2-CTA MMA operand: the data goes to this CTA's shared memory, the completion
// (transaction bytes) to the leader CTA's barrier
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t leader_bar, int x, int y,
                                                 uint64_t hint) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      :
      : "r"(smem_u32(smem_dst)), "l"(tmap), "r"(leader_bar), "r"(x), "r"(y), "l"(hint)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once all MMAs issued
// so far have completed (the commit is not a load; no operand data is multicast anywhere)
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 0x3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(both)
               : "memory");
}

// EPI: the epilogue kind, a template parameter so that each kind gets its own register allocation.
template <int STAGES, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmParams p) {
  using Cfg = Gemm2Cfg<STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* epi_stage = smem + STAGES * Cfg::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + Cfg::kEpiBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);   // the leader's arrive.expect_tx; bytes come from both CTAs' loads
      mbar_init(&empty_bar[s], 1);  // one commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);  // 4 epilogue warps of each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int first_tile = (int)cluster_id_x();
  const int tile_step = (int)num_clusters_x();

  if (warp == 0) {
    // ===== TMA producer (both CTAs) =====
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      const uint64_t hint_a = !p.use_hints ? kL2EvictNormal : p.stationary == 0 ? kL2EvictLast : kL2EvictFirst;
      const uint64_t hint_b = !p.use_hints ? kL2EvictNormal : p.stationary == 0 ? kL2EvictFirst : kL2EvictLast;
      for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
        int tm, tn;
        tile_coords(p, t, tm, tn);
        const int m0 = tm * kBM2 + (int)cta_rank * 128;
        const int n0 = p.n_begin + tn * kBN2 + (int)cta_rank * 128;
        if (!wait_rows_ready(p, m0, 128, abort_flag)) { ok = false; break; }
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          const uint32_t leader_full = smem_u32(&full_bar[stage]) & 0xFEFFFFFFu;  // same offset in cluster rank 0
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
          tma_load_2d_pair(sa, &tmap_a, leader_full, kb * BK, m0, hint_a);
          tma_load_2d_pair(sa + Cfg::kABytes, &tmap_b, leader_full, kb * BK, n0, hint_b);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer (leader CTA only) =====
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kBM2, kBN2);
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_step, ++it) {
        const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
        if (!mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN2;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t da = make_sw128_kmajor_desc(sa);
          const uint64_t db = make_sw128_kmajor_desc(sa + Cfg::kABytes);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)
            umma_f16_pair(d_tmem, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb | k4) != 0 ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(&tmem_full[acc]);
      }
    }
  } else {
    // ===== epilogue (both CTAs): this CTA's 128 rows of the tile =====
    const int quad = warp & 3;
    const uint32_t leader_tmem_empty0 = map_to_cta(smem_u32(&tmem_empty[0]), 0);
    uint32_t it = 0;
    for (int t = first_tile; t < num_tiles; t += tile_step, ++it) {
      const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
      int tm, tn;
      tile_coords(p, t, tm, tn);
      const int m0 = tm * kBM2 + (int)cta_rank * 128;
      const int n0 = p.n_begin + tn * kBN2;
      const BiasRef bias8 = epilogue_bias8(p, n0, lane);  // in flight while the MMAs finish
      if (!mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      epilogue_warp_pipelined<EPI>(p, tmem_base + acc * kBN2 + ((uint32_t)(quad * 32) << 16),
                                   epi_stage + (warp - 2) * Cfg::kEpiBytesPerWarp, bias8, m0 + quad * 32, n0, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tmem_empty0 + acc * 8u);
    }
  }

  // ===== teardown: nobody leaves while the partner may still touch its shared memory or barriers =====
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) report_failure(p.status, LIGER_DEV_TIMEOUT, 0x110u, blockIdx.x, 0);
}

// ---- wide variant: one 256x512 tile per CTA pair -----------------------------------------------------
// Both TMEM accumulators of a CTA belong to the same tile (column halves [0,256) and [256,512)), so
// every A tile fetched into shared memory feeds twice as many MMAs: 48 KB of operands per k-block
// and CTA for 128x512 outputs instead of 32 KB for 128x256, i.e. 25 % less L2 and shared-memory
// traffic and less than half the DRAM traffic per FLOP.  The price: a tile owns all of TMEM, so its
// epilogue cannot hide behind the next tile's MMAs.  It is kept short instead -- eight epilogue warps
// (four per column half, working at the same time) running the pipelined epilogue -- and the variant
// is used for long K only, where the tile's MMA time dwarfs it.  Warps: 0 TMA producer, 1 MMA issuer
// and TMEM owner, 2-5 epilogue of half 0, 6-9 epilogue of half 1.
constexpr int kWideThreads = 320;
template <int STAGES>
struct Gemm2WideCfg {
  static constexpr int kABytes = 128 * BK * 2;
  static constexpr int kBHalfBytes = 128 * BK * 2;  // this CTA's 128 rows of one column half
  static constexpr int kStageBytes = kABytes + 2 * kBHalfBytes;
  static constexpr int kEpiBytesPerWarp = 32 * 64 * 2;
  static constexpr int kEpiBytes = 8 * kEpiBytesPerWarp;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = STAGES * kStageBytes + kEpiBytes + kBarrierBytes + 1024;
  static constexpr int kTmemCols = 512;
};
constexpr int kBNW = 512;

// The it-th tile of a CTA pair: a whole 256x512 tile (halves = 2) or, in a split tail, one 256x256
// half of one (halves = 1; it uses operand slot and accumulator 0).  n0 is the tile's first
// accumulator column.  All warps of both CTAs evaluate this identically.
struct WideTile {
  int tm, n0, halves;
};
__device__ __forceinline__ bool wide_tile(const GemmParams& p, int cluster, int nclusters, int it, WideTile& w) {
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int t = cluster + it * nclusters;
  int tn;
  if (t < p.tail_start || !p.tail_split) {
    if (t >= num_tiles) return false;
    tile_coords(p, t, w.tm, tn);
    w.n0 = p.n_begin + tn * kBNW;
    w.halves = 2;
    return true;
  }
  const int r = t - p.tail_start;  // tail_start is a multiple of nclusters: r == cluster in the tail wave
  if (r >= 2 * (num_tiles - p.tail_start)) return false;
  tile_coords(p, p.tail_start + (r >> 1), w.tm, tn);
  w.n0 = p.n_begin + tn * kBNW + (r & 1) * 256;
  w.halves = 1;
  return true;
}

// One instantiation per epilogue kind: inlining all of them behind a run-time switch costs the
// register allocator its footing (heavy spills); separately each fits without.
template <int STAGES, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kWideThreads, 1)
gemm_tcgen05_2cta_wide_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                              const GemmParams p) {
  using Cfg = Gemm2WideCfg<STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* epi_stage = smem + STAGES * Cfg::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + Cfg::kEpiBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;   // [2]: one per column half
  uint64_t* tmem_empty = tmem_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);  // 4 epilogue warps of this half x 2 CTAs
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int cluster = (int)cluster_id_x();
  const int nclusters = (int)num_clusters_x();
  WideTile w;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int it = 0; ok && wide_tile(p, cluster, nclusters, it, w); ++it) {
        const int m0 = w.tm * kBM2 + (int)cta_rank * 128;
        const int n0 = w.n0 + (int)cta_rank * 128;
        const uint32_t tx = 2u * (uint32_t)(Cfg::kABytes + w.halves * Cfg::kBHalfBytes);
        if (!wait_rows_ready(p, m0, 128, abort_flag)) { ok = false; break; }
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          const uint32_t leader_full = smem_u32(&full_bar[stage]) & 0xFEFFFFFFu;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], tx);
          tma_load_2d_pair(sa, &tmap_a, leader_full, kb * BK, m0, kL2EvictNormal);
          tma_load_2d_pair(sa + Cfg::kABytes, &tmap_b, leader_full, kb * BK, n0, kL2EvictNormal);
          if (w.halves == 2)
            tma_load_2d_pair(sa + Cfg::kABytes + Cfg::kBHalfBytes, &tmap_b, leader_full, kb * BK, n0 + 256, kL2EvictNormal);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kBM2, 256);
      uint32_t stage = 0, phase = 0;
      uint32_t uses[2] = {0, 0};  // tiles that have used accumulator h so far
      bool ok = true;
      for (int it = 0; ok && wide_tile(p, cluster, nclusters, it, w); ++it) {
        for (int kb = 0; kb < p.kblocks && ok; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t da = make_sw128_kmajor_desc(sa);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (h >= w.halves) break;
            if (kb == 0) {  // the previous tile's epilogue must have drained this half
              if (!mbar_wait_bounded(&tmem_empty[h], (uses[h] & 1u) ^ 1u, abort_flag)) { ok = false; break; }
              tc_fence_after();
            }
            const uint64_t db = make_sw128_kmajor_desc(sa + Cfg::kABytes + h * Cfg::kBHalfBytes);
#pragma unroll
            for (int k4 = 0; k4 < BK / 16; ++k4)
              umma_f16_pair(tmem_base + h * 256, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc,
                            (kb | k4) != 0 ? 1u : 0u);
          }
          if (!ok) break;
          umma_commit_pair(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          for (int h = 0; h < w.halves; ++h) {
            umma_commit_pair(&tmem_full[h]);
            ++uses[h];
          }
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int h = (warp - 2) >> 2;  // the column half this warp drains
    const uint32_t leader_tmem_empty = map_to_cta(smem_u32(&tmem_empty[h]), 0);
    uint8_t* stage_tile = epi_stage + (warp - 2) * Cfg::kEpiBytesPerWarp;
    uint32_t uses = 0;
    for (int it = 0; wide_tile(p, cluster, nclusters, it, w); ++it) {
      if (h >= w.halves) continue;
      const int m0 = w.tm * kBM2 + (int)cta_rank * 128;
      const int n0 = w.n0 + h * 256;
      const BiasRef bias8 = epilogue_bias8(p, n0, lane);  // in flight while the MMAs finish
      if (!mbar_wait_bounded(&tmem_full[h], uses & 1u, abort_flag)) break;
      ++uses;
      tc_fence_after();
      epilogue_warp_pipelined<EPI>(p, tmem_base + h * 256 + ((uint32_t)(quad * 32) << 16), stage_tile, bias8,
                                   m0 + quad * 32, n0, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tmem_empty);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) report_failure(p.status, LIGER_DEV_TIMEOUT, 0x120u, blockIdx.x, 0);
}

constexpr int kStages2 = 6;
constexpr int kStagesWide = 4;

// (choose_tile_order / choose_arrival_order: gemm_epilogue.cuh)

// Launches the 2-CTA kernel.  Returns LIGER_ERR_UNSUPPORTED (without touching the error text) when
// this shape is better served by the 1-CTA kernel.
template <int EPI>
static int launch_wide_instance(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const GemmParams& p, int clusters,
                                cudaStream_t stream) {
  using Cfg = Gemm2WideCfg<kStagesWide>;
  // per launch: the attribute is per device, and a process may drive several
  LIGER_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_2cta_wide_kernel<kStagesWide, EPI>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  gemm_tcgen05_2cta_wide_kernel<kStagesWide, EPI><<<2 * clusters, kWideThreads, Cfg::kSmemBytes, stream>>>(tm_a, tm_b, p);
  return check_launch("gemm_tcgen05_2cta_wide_kernel");
}

static int launch_gemm_2cta_wide(const liger_gemm_args& a, const GemmParams& p0, int max_clusters, cudaStream_t stream) {
  GemmParams p = p0;
  p.tiles_m = (a.m + kBM2 - 1) / kBM2;
  p.tiles_n = (a.n_end - a.n_begin + kBNW - 1) / kBNW;
  p.kblocks = (a.k + BK - 1) / BK;
  choose_tile_order(p, a, kBM2, kBNW);
  choose_arrival_order(p, kBM2);
  const int tiles = p.tiles_m * p.tiles_n;
  // last wave: when at most half of the CTA pairs would get a tile, split those tiles into halves
  p.tail_start = tiles >= max_clusters ? tiles / max_clusters * max_clusters : tiles;
  p.tail_split = tiles > p.tail_start && 2 * (tiles - p.tail_start) <= max_clusters ? 1 : 0;
  const int clusters = tiles < max_clusters ? tiles : max_clusters;
  CUtensorMap tm_a, tm_b;
  int rc;
  if ((rc = make_tmap_2d_f16(&tm_a, a.a, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, 128)) != LIGER_OK) return rc;
  if ((rc = make_tmap_2d_f16(&tm_b, a.wt, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldw, BK, 128)) != LIGER_OK) return rc;
  switch (p.epilogue) {
    case LIGER_EPI_GELU: return launch_wide_instance<LIGER_EPI_GELU>(tm_a, tm_b, p, clusters, stream);
    case LIGER_EPI_GEGLU: return launch_wide_instance<LIGER_EPI_GEGLU>(tm_a, tm_b, p, clusters, stream);
    case LIGER_EPI_QKV_SPLIT: return launch_wide_instance<LIGER_EPI_QKV_SPLIT>(tm_a, tm_b, p, clusters, stream);
    case LIGER_EPI_RESIDUAL: return launch_wide_instance<LIGER_EPI_RESIDUAL>(tm_a, tm_b, p, clusters, stream);
    case LIGER_EPI_SCATTER: return launch_wide_instance<LIGER_EPI_SCATTER>(tm_a, tm_b, p, clusters, stream);
    default: return launch_wide_instance<LIGER_EPI_STORE>(tm_a, tm_b, p, clusters, stream);
  }
}

template <int EPI>
static int launch_pair_instance(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const GemmParams& p, int clusters,
                                cudaStream_t stream) {
  using Cfg = Gemm2Cfg<kStages2>;
  LIGER_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel<kStages2, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg::kSmemBytes));
  gemm_tcgen05_2cta_kernel<kStages2, EPI><<<2 * clusters, kGemmThreads, Cfg::kSmemBytes, stream>>>(tm_a, tm_b, p);
  return check_launch("gemm_tcgen05_2cta_kernel");
}

int launch_gemm_2cta(const liger_gemm_args& a, const GemmParams& p0, int sm_count, cudaStream_t stream) {
  using Cfg = Gemm2Cfg<kStages2>;
  GemmParams p = p0;
  p.tiles_m = (a.m + kBM2 - 1) / kBM2;
  p.tiles_n = (a.n_end - a.n_begin + kBN2 - 1) / kBN2;
  p.kblocks = (a.k + BK - 1) / BK;
  choose_tile_order(p, a, kBM2, kBN2);
  choose_arrival_order(p, kBM2);
  const int tiles = p.tiles_m * p.tiles_n;
  static int max_clusters = -1;
  if (max_clusters < 0) {
    LIGER_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel<kStages2, LIGER_EPI_STORE>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count / 2 * 2);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_2cta_kernel<kStages2, LIGER_EPI_STORE>, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = 0;
    }
    max_clusters = n;
  }
  if (max_clusters < 1) return LIGER_ERR_UNSUPPORTED;
  {
    // 256x512 tiles for long K when they still fill the machine at least as evenly as 256x256 ones:
    // compare waves x tile width (LIGER_GEMM_WIDE = 0 / 1 forces the choice)
    static int wide_env = -2;
    if (wide_env == -2) { const char* e = getenv("LIGER_GEMM_WIDE"); wide_env = e ? atoi(e) : -1; }
    // cost in 256x256-tile waves: full wide waves count 2, a split tail (at most half of the CTA pairs busy) 1
    const long tiles_w = (long)p.tiles_m * ((a.n_end - a.n_begin + kBNW - 1) / kBNW);
    const long full_w = tiles_w / max_clusters, rem_w = tiles_w - full_w * max_clusters;
    const long cost_w = 2 * full_w + (rem_w == 0 ? 0 : 2 * rem_w <= max_clusters ? 1 : 2);
    const long waves_n = ((long)tiles + max_clusters - 1) / max_clusters;
    const bool geom_ok = a.k >= 8192 && tiles_w >= max_clusters && cost_w <= waves_n + (waves_n + 9) / 10;
    if (!p0.no_wide && (wide_env == 1 || (wide_env < 0 && geom_ok))) return launch_gemm_2cta_wide(a, p0, max_clusters, stream);
  }
  const int clusters = tiles < max_clusters ? tiles : max_clusters;
  CUtensorMap tm_a, tm_b;
  int rc;
  if ((rc = make_tmap_2d_f16(&tm_a, a.a, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, 128)) != LIGER_OK) return rc;
  if ((rc = make_tmap_2d_f16(&tm_b, a.wt, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldw, BK, 128)) != LIGER_OK) return rc;
  switch (p.epilogue) {
    case LIGER_EPI_GELU: return launch_pair_instance<LIGER_EPI_GELU>(tm_a, tm_b, p, clusters, stream);
    case LIGER_EPI_GEGLU: return launch_pair_instance<LIGER_EPI_GEGLU>(tm_a, tm_b, p, clusters, stream);
    case LIGER_EPI_QKV_SPLIT: return launch_pair_instance<LIGER_EPI_QKV_SPLIT>(tm_a, tm_b, p, clusters, stream);
    case LIGER_EPI_RESIDUAL: return launch_pair_instance<LIGER_EPI_RESIDUAL>(tm_a, tm_b, p, clusters, stream);
    case LIGER_EPI_SCATTER: return launch_pair_instance<LIGER_EPI_SCATTER>(tm_a, tm_b, p, clusters, stream);
    default: return launch_pair_instance<LIGER_EPI_STORE>(tm_a, tm_b, p, clusters, stream);
  }
}

int gemm_2cta_max_clusters_hint(int sm_count) { return sm_count / 2; }

}  // namespace liger
