// fp16 GEMM for a handful of rows (M <= 32: a decode step), sm_100a.
//
// With so few rows the contraction is a stream of the weight matrix: every byte of W^T is used once,
// and the kernel is as fast as it keeps HBM busy.  The big-tile kernels (gemm_sm100*.cu) cannot do
// that here: a 128-row accumulator tile holds 32 useful rows, and with one 32-column tile per CTA
// each pipeline step moves only 4 KB of weights.  This kernel swaps the operand roles instead:
//
//   * the 128-row "A" operand of tcgen05.mma is a block of 128 output FEATURES (128 rows of W^T,
//     K-major, fetched by TMA with 128-byte swizzle): 16 KB of weights per 64-deep k-block;
//   * the "B" operand (N = 32) is the activation block X[0:32, k-block] (rows past M are zero-filled
//     by TMA), 4 KB, re-read from L2 by every CTA;
//   * the accumulator D[feature][token] is 128 lanes x 32 fp32 columns of TMEM;
//   * K is split so that even a weight shard with few feature blocks keeps every SM streaming.  Two
//     kernels do that, and the launch picks the one its cost estimate prefers:
//       - gemm_smallm_kernel: K split over the CTAs of a thread-block cluster (1..8); the partial
//         accumulators are summed through distributed shared memory, rank r of the cluster finishing
//         the tokens t = r, r + S, ...  Lowest fixed cost: best when one wave of clusters fills the GPU.
//       - gemm_smallm_streamk_kernel: the k-blocks of all tiles dealt out evenly over one CTA per SM;
//         partial tiles go through an L2-resident workspace and the last CTA to arrive at a tile
//         sums them.  No wave quantisation: best for a long K with few tiles (12288 x 32768: 96 tiles).
//     Both sum in a fixed order (deterministic) and apply bias / activation / layout to rows of 128
//     contiguous features (16-byte stores).
//
// Roles per CTA (6 warps): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 drain the
// accumulator and run the reduction + epilogue.  Every mbarrier wait is bounded; a cluster CTA that
// gives up still arrives at both cluster barriers, so its partners never wait for it without limit,
// and a stream-K CTA never waits for another CTA at all.
#include <algorithm>
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "gemm_epilogue.cuh"

LIGER_REGISTER_WAIT_BUDGET()

namespace liger {

constexpr int kSmFeat = 128;     // features per tile (MMA M)
constexpr int kSmTok = 32;       // tokens per tile (MMA N)
constexpr int kSmStages = 8;
constexpr int kSmWBytes = kSmFeat * BK * 2;   // 16 KB
constexpr int kSmXBytes = kSmTok * BK * 2;    // 4 KB
constexpr int kSmStageBytes = kSmWBytes + kSmXBytes;
constexpr int kSmPartialBytes = kSmTok * kSmFeat * 4;  // fp32 [token][feature]
constexpr int kSmBarrierBytes = 256;
constexpr int kSmSmemBytes = kSmStages * kSmStageBytes + kSmPartialBytes + kSmBarrierBytes + 1024;
constexpr int kSmMaxSplits = 8;

__device__ __forceinline__ uint32_t sm_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t sm_cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t sm_cluster_id() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void sm_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t sm_map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 sm_ld_cluster_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}

// Finishing one 128-feature tile for the tokens t_first, t_first + t_step, ... < p.m: 128 threads (tid 0..127), each
// with up to four items = (token, group of 8 output features), one 16-byte store per item.  The bias and residual
// vectors of a thread's items do not depend on the accumulation, so they are fetched (smallm_prefetch) while the
// weights are still streaming; smallm_finish_tile then only adds the sums: `sum8(t, fa, v)` adds the fp32 sums of
// features fa .. fa + 7 of token t into v.  The four items are unrolled so that their loads overlap.
constexpr int kSmItems = kSmTok * 16 / 128;  // items per thread at most (32 tokens x 16 groups over 128 threads)

struct SmallmPrefetch {
  uint4 bias[kSmItems], bias2[kSmItems], res[kSmItems];
};

struct SmallmItem {
  int t, g, fa, n;
  bool on;
};

__device__ __forceinline__ SmallmItem smallm_item(const GemmParams& p, int f0, int tid, int t_first, int t_step, int u) {
  const bool geglu = p.epilogue == LIGER_EPI_GEGLU;
  const int groups = geglu ? 8 : 16;  // 8-feature output groups per token
  const int my_tokens = (p.m - t_first + t_step - 1) / t_step;
  const int item = tid + u * 128;
  SmallmItem it;
  it.t = t_first + t_step * (item / groups);
  it.g = item % groups;
  // features of this item inside the tile: plain kinds 8g..8g+7; GeGLU: gates 64b+8q.., values 64b+32+8q..
  it.fa = geglu ? (it.g >> 2) * 64 + (it.g & 3) * 8 : it.g * 8;
  it.n = f0 + it.fa;  // accumulator column (row of W^T)
  it.on = item < my_tokens * groups && it.n >= p.n_begin && it.n < p.n_end;
  return it;
}

__device__ __forceinline__ void smallm_prefetch(const GemmParams& p, int f0, int tid, int t_first, int t_step, SmallmPrefetch& pf) {
#pragma unroll
  for (int u = 0; u < kSmItems; ++u) {
    const SmallmItem it = smallm_item(p, f0, tid, t_first, t_step, u);
    pf.bias[u] = pf.bias2[u] = pf.res[u] = make_uint4(0, 0, 0, 0);
    if (!it.on) continue;
    if (p.bias != nullptr) {
      pf.bias[u] = __ldg(reinterpret_cast<const uint4*>(p.bias + it.n));
      if (p.epilogue == LIGER_EPI_GEGLU) pf.bias2[u] = __ldg(reinterpret_cast<const uint4*>(p.bias + it.n + 32));
    }
    // plain load: the residual may be the very tensor this launch writes (each element by the thread that read it)
    if (p.epilogue == LIGER_EPI_RESIDUAL) pf.res[u] = __ldcg(reinterpret_cast<const uint4*>(p.residual + (size_t)it.t * p.ldr + it.n));
  }
}

template <typename Sum8>
__device__ __forceinline__ void smallm_finish_tile(const GemmParams& p, int f0, int tid, int t_first, int t_step,
                                                   const SmallmPrefetch& pf, Sum8 sum8) {
  const bool geglu = p.epilogue == LIGER_EPI_GEGLU;
#pragma unroll
  for (int u = 0; u < kSmItems; ++u) {
    const SmallmItem it = smallm_item(p, f0, tid, t_first, t_step, u);
    if (!it.on) continue;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    sum8(it.t, it.fa, a);
    if (geglu) sum8(it.t, it.fa + 32, v);
    float b[8];
    unpack8(pf.bias[u], b);  // zeros without a bias
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] += b[i];
    int out_col = it.n;
    if (geglu) {
      unpack8(pf.bias2[u], b);
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = gelu_tanh(a[i]) * (v[i] + b[i]);
      out_col = (f0 >> 1) + (it.g >> 2) * 32 + (it.g & 3) * 8;
    } else if (p.epilogue == LIGER_EPI_GELU) {
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = gelu_tanh(a[i]);
    } else if (p.epilogue == LIGER_EPI_RESIDUAL) {
      unpack8(pf.res[u], b);
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] += b[i];
    }
    uint4 o;
    o.x = pack_half2(a[0], a[1]); o.y = pack_half2(a[2], a[3]); o.z = pack_half2(a[4], a[5]); o.w = pack_half2(a[6], a[7]);
    *reinterpret_cast<uint4*>(epilogue_dst(p, it.t, out_col)) = o;
  }
}

__device__ __forceinline__ void add8(float (&v)[8], const float4& x0, const float4& x1) {
  v[0] += x0.x; v[1] += x0.y; v[2] += x0.z; v[3] += x0.w; v[4] += x1.x; v[5] += x1.y; v[6] += x1.z; v[7] += x1.w;
}

// Cluster dimensions are given at launch (1..8 CTAs along x).
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* partial = reinterpret_cast<float*>(smem + kSmStages * kSmStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kSmStages * kSmStageBytes + kSmPartialBytes);
  uint64_t* empty_bar = full_bar + kSmStages;
  uint64_t* tmem_full = empty_bar + kSmStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int splits = (int)sm_cluster_nctarank();
  const int split = (int)sm_cluster_ctarank();
  const int tile = (int)sm_cluster_id();
  const int f0 = p.n_begin + tile * kSmFeat;  // first feature (row of W^T) of this tile
  // this CTA's share of the k-blocks: [kb0, kb1)
  const int kb0 = (int)(((long)p.kblocks * split) / splits);
  const int kb1 = (int)(((long)p.kblocks * (split + 1)) / splits);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSmStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kSmTok);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  SmallmPrefetch pf;  // drain warps only

  if (warp == 0) {
    // ===== TMA producer: weights stream through once (evict first), the activations stay in L2 =====
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) break;
        uint8_t* sw = smem + stage * kSmStageBytes;
        mbar_arrive_expect_tx(&full_bar[stage], kSmStageBytes);
        tma_load_2d_hint(sw, &tmap_w, &full_bar[stage], kb * BK, f0, kL2EvictFirst);
        tma_load_2d_hint(sw + kSmWBytes, &tmap_x, &full_bar[stage], kb * BK, 0, kL2EvictLast);
        if (++stage == kSmStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer: D[feature][token] += W^T tile (M = 128) x X tile^T (N = 32) =====
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kSmFeat, kSmTok);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sw = smem_u32(smem + stage * kSmStageBytes);
        const uint64_t dw = make_sw128_kmajor_desc(sw);
        const uint64_t dx = make_sw128_kmajor_desc(sw + kSmWBytes);
#pragma unroll
        for (int k4 = 0; k4 < BK / 16; ++k4)
          umma_f16(tmem_base, dw + (uint64_t)(k4 * 2), dx + (uint64_t)(k4 * 2), idesc, (kb > kb0 || k4 != 0) ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        if (++stage == kSmStages) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(tmem_full);
    }
  } else {
    // ===== drain: lane = feature, column = token -> partial[token][feature] (fp32) =====
    const int quad = warp & 3;
    const int f = quad * 32 + lane;
    smallm_prefetch(p, f0, threadIdx.x - 64, split, splits, pf);  // bias / residual of this thread's items, meanwhile
    bool have = kb1 > kb0;
    if (have) have = mbar_wait_bounded(tmem_full, 0u, abort_flag);
    if (have) {
      tc_fence_after();
      uint32_t r[32];
      tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16), r);
      tmem_ld_wait_regs(r);
#pragma unroll
      for (int t = 0; t < kSmTok; ++t) partial[t * kSmFeat + f] = __uint_as_float(r[t]);
    } else {
      // an empty k-range (more splits than k-blocks) or a wait that gave up: contribute zeros
#pragma unroll
      for (int t = 0; t < kSmTok; ++t) partial[t * kSmFeat + f] = 0.0f;
    }
    tc_fence_before();
  }

  // every CTA's partial is complete and visible to the whole cluster
  __syncthreads();
  sm_cluster_sync();

  if (warp >= 2 && *abort_flag == 0) {
    // ===== reduction over the cluster + epilogue: this CTA finishes tokens split, split + S, ... =====
    const uint32_t partial_local = smem_u32(partial);
    smallm_finish_tile(p, f0, threadIdx.x - 64, split, splits, pf, [&](int t, int fa, float (&v)[8]) {
      for (int s = 0; s < splits; ++s) {  // fixed order: the result does not depend on timing
        const uint32_t base = sm_map_to_cta(partial_local, (uint32_t)s) + (uint32_t)((t * kSmFeat + fa) * 4);
        add8(v, sm_ld_cluster_f4(base), sm_ld_cluster_f4(base + 16));
      }
    });
  }

  // nobody leaves while a partner may still read its shared memory
  tc_fence_before();
  __syncthreads();
  sm_cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, kSmTok);
  }
  if (threadIdx.x == 0 && *abort_flag) report_failure(p.status, LIGER_DEV_TIMEOUT, 0x130u, blockIdx.x, 0);
}

// ---- the same contraction with the k-blocks of ALL tiles dealt out evenly (no clusters) ---------------------------
//
// The (tile, k-block) pairs of the whole weight, tile-major, form one line of tiles x kblocks units; CTA c takes the
// units [c * per, (c + 1) * per).  Every SM streams the same number of bytes whatever the tile count -- 96 feature
// tiles keep 148 SMs as busy as 296 would -- and there is no second wave.  A CTA's range crosses tile boundaries: a
// segment that covers a tile's whole K finishes it directly; a partial segment (at most the first and the last of a
// CTA) is written as an fp32 tile to a workspace slot, and the CTA that arrives last at the tile's counter adds the
// slots in CTA order (deterministic) and finishes the tile.  Nobody waits for another CTA.  The accumulator is
// double-buffered in TMEM, so the weights keep streaming while a segment drains.
constexpr int kSkMaxTiles = 4096;                      // arrival counters per set
constexpr int kSkSlotFloats = kSmTok * kSmFeat;        // one fp32 partial tile

struct StreamK {
  int per;                       // units (k-blocks) per CTA
  int cta_begin;                 // this launch's first CTA in the partition of the whole weight
  int tile_begin, tile_end;      // feature tiles this launch computes (absolute)
  float* ws;                     // [2 x CTAs of the partition][32 tokens][128 features]
  unsigned int* counters;        // arrivals per tile, all zero when the launch starts
  unsigned int* counters_next;   // the other set, zeroed here for the next launch on this workspace
};

__device__ __forceinline__ void drain_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_smallm_streamk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                           const GemmParams p, const StreamK sk) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* partial = reinterpret_cast<float*>(smem + kSmStages * kSmStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kSmStages * kSmStageBytes + kSmPartialBytes);
  uint64_t* empty_bar = full_bar + kSmStages;
  uint64_t* tmem_full = empty_bar + kSmStages;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;          // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* last_flag = tmem_slot + 2;
  volatile uint32_t* drain_abort = tmem_slot + 3;  // written by the drain warps only, before their barrier

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kblocks = p.kblocks;
  const int c = sk.cta_begin + (int)blockIdx.x;
  const int u_begin = max(c * sk.per, sk.tile_begin * kblocks);
  const int u_end = min((c + 1) * sk.per, sk.tile_end * kblocks);

  // the counters of the next launch on this workspace (nobody is using that set now)
  for (int i = (int)blockIdx.x * kGemmThreads + (int)threadIdx.x; i < kSkMaxTiles; i += (int)gridDim.x * kGemmThreads)
    sk.counters_next[i] = 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSmStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);  // one arrival per drain warp
    }
    *abort_flag = 0;
    *last_flag = 0;
    *drain_abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * kSmTok);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ===== TMA producer: one uninterrupted stream over all segments =====
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int u = u_begin; u < u_end; ++u) {
        const int tile = u / kblocks, kb = u - tile * kblocks;
        if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) break;
        uint8_t* sw = smem + stage * kSmStageBytes;
        mbar_arrive_expect_tx(&full_bar[stage], kSmStageBytes);
        tma_load_2d_hint(sw, &tmap_w, &full_bar[stage], kb * BK, tile * kSmFeat, kL2EvictFirst);
        tma_load_2d_hint(sw + kSmWBytes, &tmap_x, &full_bar[stage], kb * BK, 0, kL2EvictLast);
        if (++stage == kSmStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer: segment s accumulates in TMEM buffer s & 1 =====
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kSmFeat, kSmTok);
      uint32_t stage = 0, phase = 0;
      int seg = 0;
      bool ok = true;
      for (int u = u_begin; u < u_end && ok; ++seg) {
        const int tile = u / kblocks, kb_lo = u - tile * kblocks;
        const int kb_hi = min(kblocks, kb_lo + (u_end - u));
        const int buf = seg & 1;
        if (!mbar_wait_bounded(&tmem_empty[buf], (uint32_t)(((seg >> 1) & 1) ^ 1), abort_flag)) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(buf * kSmTok);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + stage * kSmStageBytes);
          const uint64_t dw = make_sw128_kmajor_desc(sw);
          const uint64_t dx = make_sw128_kmajor_desc(sw + kSmWBytes);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)
            umma_f16(acc, dw + (uint64_t)(k4 * 2), dx + (uint64_t)(k4 * 2), idesc, (kb > kb_lo || k4 != 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kSmStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tmem_full[buf]);
        u += kb_hi - kb_lo;
      }
    }
  } else {
    // ===== drain warps: lane = feature, column = token; finish whole tiles, hand partial ones over =====
    const int quad = warp & 3;
    const int f = quad * 32 + lane;
    const int tid = threadIdx.x - 64;  // 0..127
    int seg = 0;
    for (int u = u_begin; u < u_end; ++seg) {
      const int tile = u / kblocks, kb_lo = u - tile * kblocks;
      const int kb_hi = min(kblocks, kb_lo + (u_end - u));
      const int buf = seg & 1;
      const int f0 = tile * kSmFeat;
      SmallmPrefetch pf;
      smallm_prefetch(p, f0, tid, 0, 1, pf);  // bias / residual of this thread's items, while the segment streams
      if (!mbar_wait_bounded(&tmem_full[buf], (uint32_t)((seg >> 1) & 1), abort_flag)) *drain_abort = 1u;
      drain_bar_sync();
      if (*drain_abort) break;  // the same answer in all 128 threads: only written before the barrier
      tc_fence_after();
      uint32_t r[32];
      tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * kSmTok), r);
      tmem_ld_wait_regs(r);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);  // the issuer may overwrite this buffer
      if (kb_lo == 0 && kb_hi == kblocks) {
        // the tile's whole K: transpose through shared memory and finish it
#pragma unroll
        for (int t = 0; t < kSmTok; ++t) partial[t * kSmFeat + f] = __uint_as_float(r[t]);
        drain_bar_sync();
        smallm_finish_tile(p, f0, tid, 0, 1, pf, [&](int t, int fa, float (&v)[8]) {
          const float4* src = reinterpret_cast<const float4*>(partial + t * kSmFeat + fa);
          add8(v, src[0], src[1]);
        });
        drain_bar_sync();
      } else {
        // part of the tile's K: publish the partial tile, count the arrival; the last one sums and finishes
        const int first_tile = (c * sk.per) / kblocks;
        float* dst = sk.ws + (size_t)(2 * c + (tile != first_tile ? 1 : 0)) * kSkSlotFloats;
#pragma unroll
        for (int t = 0; t < kSmTok; ++t) __stcg(dst + t * kSmFeat + f, __uint_as_float(r[t]));
        drain_bar_sync();
        const int c_first = (tile * kblocks) / sk.per;
        const int c_last = ((tile + 1) * kblocks - 1) / sk.per;
        if (tid == 0) {
          __threadfence();  // one fence after the barrier covers all 128 threads' stores (fences are cumulative)
          const unsigned int old = atomicAdd(&sk.counters[tile], 1u);
          __threadfence();  // the other CTAs' slots, seen through the counter, before this CTA reads them
          *last_flag = (old == (unsigned int)(c_last - c_first)) ? 1u : 0u;
        }
        drain_bar_sync();
        if (*last_flag) {
          smallm_finish_tile(p, f0, tid, 0, 1, pf, [&](int t, int fa, float (&v)[8]) {
            for (int c0 = c_first; c0 <= c_last; c0 += 4) {  // fixed order: the result does not depend on timing
              float4 x[4][2];
#pragma unroll
              for (int j = 0; j < 4; ++j) {                  // all loads of the group first, then the sums
                const int cc = c0 + j;
                if (cc <= c_last) {
                  const int ft = (cc * sk.per) / kblocks;
                  const float4* src = reinterpret_cast<const float4*>(
                      sk.ws + (size_t)(2 * cc + (tile != ft ? 1 : 0)) * kSkSlotFloats + t * kSmFeat + fa);
                  x[j][0] = __ldcg(src);
                  x[j][1] = __ldcg(src + 1);
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (c0 + j <= c_last) add8(v, x[j][0], x[j][1]);
            }
          });
        }
        drain_bar_sync();  // last_flag is rewritten by the next partial segment
      }
      u += kb_hi - kb_lo;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 2 * kSmTok);
  }
  if (threadIdx.x == 0 && *abort_flag) report_failure(p.status, LIGER_DEV_TIMEOUT, 0x131u, blockIdx.x, 0);
}

// How many clusters of `splits` CTAs the device runs at once (cached per device and cluster size).
static int smallm_max_clusters(int device, int sm_count, int splits) {
  static int cache[64][kSmMaxSplits + 1];
  if (device < 0 || device >= 64) return sm_count / splits;
  if (cache[device][splits] > 0) return cache[device][splits];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(sm_count / splits * splits));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kSmSmemBytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = (unsigned)splits; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_smallm_kernel, &cfg) != cudaSuccess || n < 1) {
    cudaGetLastError();
    n = sm_count / splits > 0 ? sm_count / splits : 1;
  }
  // A cluster must fit inside one GPC.  Measured on B200 (148 SMs, 8 GPCs of at least 18 usable SMs) the launch
  // places floor(18 / splits) clusters per GPC -- e.g. 32 clusters of 4, not the 37 that 148 / 4 suggests -- and a
  // launch with more clusters than that runs a second wave; the occupancy query alone is too optimistic.
  if (splits >= 3) {
    const int per_gpc = (sm_count / 8) / splits;
    if (per_gpc >= 1 && 8 * per_gpc < n) n = 8 * per_gpc;
  }
  cache[device][splits] = n;
  return n;
}

// LIGER_GEMM_SMALLM: 0 keeps small-M launches on the big-tile kernels, 2 on the cluster kernel, 3 on the stream-K
// kernel; 1 or unset: whichever the cost estimate below prefers.  Read at every launch (a test may change it).
static int smallm_mode() {
  const char* e = getenv("LIGER_GEMM_SMALLM");
  return e ? atoi(e) : 1;
}

// Partial tiles and arrival counters of the stream-K kernel, one set per (device, stream): launches on one stream
// follow one another, launches on different streams may overlap and must not share slots.  Allocated on first use.
struct StreamKWorkspace {
  float* ws = nullptr;
  unsigned int* counters = nullptr;  // [2][kSkMaxTiles]
  int ctas = 0;
  int flip = 0;
};
static std::mutex g_sk_mu;
static std::map<std::pair<int, cudaStream_t>, StreamKWorkspace> g_sk_ws;

static int streamk_workspace(int device, cudaStream_t stream, int ctas, StreamKWorkspace** out) {
  std::lock_guard<std::mutex> lk(g_sk_mu);
  StreamKWorkspace& w = g_sk_ws[std::make_pair(device, stream)];
  if (w.ctas < ctas) {
    if (w.ws) cudaFree(w.ws);
    w.ws = nullptr;
    w.ctas = 0;
    LIGER_CUDA_TRY(cudaMalloc(&w.ws, (size_t)2 * ctas * kSkSlotFloats * sizeof(float)));
    w.ctas = ctas;
  }
  if (w.counters == nullptr) {
    LIGER_CUDA_TRY(cudaMalloc(&w.counters, (size_t)2 * kSkMaxTiles * sizeof(unsigned int)));
    LIGER_CUDA_TRY(cudaMemset(w.counters, 0, (size_t)2 * kSkMaxTiles * sizeof(unsigned int)));
  }
  *out = &w;
  return LIGER_OK;
}

// Units per CTA of the stream-K partition.  A function of the whole weight (tiles_full, kblocks) and the SM count
// only, so that a decomposed launch [n_begin, n_end) runs the very CTAs -- same k-ranges, same summation order --
// that the whole launch would.  `partial` tells whether any tile is split between CTAs.
static int streamk_units_per_cta(int tiles_full, int kblocks, int sm_count, bool* partial) {
  const int total = tiles_full * kblocks;
  int per = (total + sm_count - 1) / sm_count;
  // whole tiles per CTA when dealing out k-blocks would save less than a partial-tile hand-over costs
  const int waves = (tiles_full + sm_count - 1) / sm_count;
  if (waves * kblocks <= per + 8) per = waves * kblocks;
  *partial = per % kblocks != 0;
  return per;
}

static int launch_streamk(const liger_gemm_args& a, const GemmParams& p, const DeviceInfo* dev, cudaStream_t stream,
                          const CUtensorMap& tm_w, const CUtensorMap& tm_x) {
  const int tiles_full = (a.n + kSmFeat - 1) / kSmFeat;
  bool partial;
  const int per = streamk_units_per_cta(tiles_full, p.kblocks, dev->sm_count, &partial);
  const int ctas_full = (tiles_full * p.kblocks + per - 1) / per;
  StreamK sk;
  sk.per = per;
  sk.tile_begin = a.n_begin / kSmFeat;
  sk.tile_end = (a.n_end + kSmFeat - 1) / kSmFeat;
  sk.cta_begin = (sk.tile_begin * p.kblocks) / per;
  const int cta_end = (sk.tile_end * p.kblocks - 1) / per + 1;
  StreamKWorkspace* w = nullptr;
  int rc = streamk_workspace(dev->device, stream, ctas_full, &w);
  if (rc != LIGER_OK) return rc;
  sk.ws = w->ws;
  sk.counters = w->counters + (size_t)w->flip * kSkMaxTiles;
  sk.counters_next = w->counters + (size_t)(w->flip ^ 1) * kSkMaxTiles;
  w->flip ^= 1;
  constexpr int smem = kSmSmemBytes;
  LIGER_CUDA_TRY(cudaFuncSetAttribute(gemm_smallm_streamk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  gemm_smallm_streamk_kernel<<<cta_end - sk.cta_begin, kGemmThreads, smem, stream>>>(tm_w, tm_x, p, sk);
  return check_launch("gemm_smallm_streamk_kernel");
}

// Which kernel a few-row GEMM over an [n, k] weight takes, and with what split.  A pure function of the whole
// weight, the SM count and conc[s] = clusters of s CTAs that run at once, so that every slice [n_begin, n_end) of
// a weight takes the same kernel, the same k-ranges and the same summation order.  Costs are in k-block times.
struct SmallmPlan {
  bool stream_k;      // false: cluster kernel with `splits` CTAs per tile
  int splits;
  int per;            // stream-K: k-blocks per CTA
  bool partial;       // stream-K: some tile is shared between CTAs
  long cluster_cost, stream_k_cost;
};

static SmallmPlan smallm_plan(int n, int k, int sm_count, const int* conc, int mode, int forced_splits) {
  SmallmPlan pl = {};
  const int kblocks = (k + BK - 1) / BK;
  const int tiles_full = (n + kSmFeat - 1) / kSmFeat;
  // Above about 0.9 x sm_count streaming CTAs HBM, not the SM, sets the pace: no schedule streams the weight in
  // fewer k-block times than this floor.
  const long hbm_floor = (long)tiles_full * kblocks * 11 / (10L * sm_count);
  // Cluster kernel: waves x (k-blocks per CTA + a set-up / drain term).  Measured on B200 a CTA streams a 16 KB
  // k-block in about 0.34 us and spends about 8 us outside its main loop; a cluster of s CTAs needs s free SMs in
  // one GPC, so fewer clusters than sm_count / s run at once, and a second wave of clusters starts raggedly
  // (x 1.4, fitted to the GLM-130B decode shapes).
  pl.splits = 1;
  pl.cluster_cost = -1;
  for (int s = 1; s <= kSmMaxSplits && s <= kblocks; ++s) {
    const long c = conc[s] > 0 ? conc[s] : 1;
    const long waves = (tiles_full + c - 1) / c;
    long cost = std::max(waves * ((kblocks + s - 1) / s), hbm_floor) + waves * 24;
    if (waves > 1) cost += cost * 2 / 5;
    if (pl.cluster_cost < 0 || cost < pl.cluster_cost) { pl.cluster_cost = cost; pl.splits = s; }
  }
  if (forced_splits > 0 && forced_splits <= kSmMaxSplits && forced_splits <= kblocks) pl.splits = forced_splits;
  // Stream-K kernel: every SM streams `per` k-blocks; handing partial tiles over through L2 costs about 9 us more
  // than a kernel that finishes whole tiles (measured at the same shapes).
  const bool possible = tiles_full <= kSkMaxTiles && (long)tiles_full * kblocks < (1l << 24);
  if (possible) {
    pl.per = streamk_units_per_cta(tiles_full, kblocks, sm_count, &pl.partial);
    pl.stream_k_cost = std::max((long)pl.per, hbm_floor) + (pl.partial ? 46 : 20);
  }
  pl.stream_k = possible && (mode == 3 || (mode != 2 && pl.stream_k_cost < pl.cluster_cost));
  return pl;
}

// Returns LIGER_ERR_UNSUPPORTED (error text untouched) when the shape is not this kernel's.
int launch_gemm_smallm(const liger_gemm_args& a, const GemmParams& p0, const DeviceInfo* dev, cudaStream_t stream) {
  const int mode = smallm_mode();
  if (mode == 0 || a.m > kSmTok || a.epilogue == LIGER_EPI_SCATTER) return LIGER_ERR_UNSUPPORTED;
  GemmParams p = p0;
  p.kblocks = (a.k + BK - 1) / BK;
  const int tiles = (a.n_end - a.n_begin + kSmFeat - 1) / kSmFeat;
  int conc[kSmMaxSplits + 1] = {0};
  for (int s = 1; s <= kSmMaxSplits; ++s) conc[s] = smallm_max_clusters(dev->device, dev->sm_count, s);
  static int forced = -1;
  if (forced < 0) { const char* e = getenv("LIGER_GEMM_SMALLM_SPLITS"); forced = e ? atoi(e) : 0; }
  const SmallmPlan plan = smallm_plan(a.n, a.k, dev->sm_count, conc, mode, forced);
  const int best = plan.splits;
  const bool use_sk = plan.stream_k;
  if (!use_sk && a.epilogue == LIGER_EPI_GEGLU && a.n_begin % 128) return LIGER_ERR_UNSUPPORTED;  // gate / value pairs per tile
  CUtensorMap tm_w, tm_x;
  int rc;
  if ((rc = make_tmap_2d_f16(&tm_w, a.wt, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldw, BK, kSmFeat)) != LIGER_OK) return rc;
  if ((rc = make_tmap_2d_f16(&tm_x, a.a, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, kSmTok)) != LIGER_OK) return rc;
  if (use_sk) return launch_streamk(a, p, dev, stream, tm_w, tm_x);
  LIGER_CUDA_TRY(cudaFuncSetAttribute(gemm_smallm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmSmemBytes));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * best));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kSmSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = (unsigned)best; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  LIGER_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_smallm_kernel, tm_w, tm_x, p));
  return check_launch("gemm_smallm_kernel");
}

}  // namespace liger

extern "C" int liger_gemm_smallm_plan(int n, int k, int sm_count, int out[4]) {
  using namespace liger;
  if (n <= 0 || k <= 0 || sm_count <= 0 || !out) return set_error(LIGER_ERR_INVALID, "gemm_smallm_plan: bad argument");
  // clusters that run at once by GPC geometry alone (8 GPCs); a launch asks the device as well
  int conc[kSmMaxSplits + 1] = {0};
  for (int s = 1; s <= kSmMaxSplits; ++s) conc[s] = s < 3 ? sm_count / s : 8 * ((sm_count / 8) / s);
  const SmallmPlan pl = smallm_plan(n, k, sm_count, conc, 1, 0);
  const int kblocks = (k + BK - 1) / BK, tiles = (n + kSmFeat - 1) / kSmFeat;
  out[0] = pl.stream_k ? 3 : 2;
  out[1] = pl.stream_k ? 1 : pl.splits;
  out[2] = pl.stream_k ? pl.per : (kblocks + pl.splits - 1) / pl.splits;
  out[3] = pl.stream_k ? (tiles * kblocks + pl.per - 1) / pl.per : tiles * pl.splits;
  return LIGER_OK;
}
