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
//   * K is split over the CTAs of a thread-block cluster (1..8), so that even a weight shard with
//     few feature blocks puts a CTA on every SM; the partial accumulators are summed through
//     distributed shared memory in a fixed order (deterministic), rank r of the cluster finishing
//     the tokens t = r, r + S, ... with bias / activation / layout applied to rows of 128 contiguous
//     features (16-byte stores).
//
// Roles per CTA (6 warps): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 drain the
// accumulator and run the reduction + epilogue.  Every mbarrier wait is bounded; a CTA that gives up
// still arrives at both cluster barriers, so its partners never wait for it without limit.
#include <cstdlib>

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
    const int tid = threadIdx.x - 64;  // 0..127
    const bool geglu = p.epilogue == LIGER_EPI_GEGLU;
    const int groups = geglu ? 8 : 16;                         // 8-feature output groups per token
    const int my_tokens = (p.m - split + splits - 1) / splits;  // tokens t < m with t % splits == split
    const uint32_t partial_local = smem_u32(partial);
    for (int item = tid; item < my_tokens * groups; item += 128) {
      const int t = split + splits * (item / groups);
      const int g = item % groups;
      // features of this item inside the tile: plain kinds 8g..8g+7; GeGLU: gates 64b+8q.., values 64b+32+8q..
      const int fa = geglu ? (g >> 2) * 64 + (g & 3) * 8 : g * 8;
      const int n = f0 + fa;  // accumulator column (row of W^T)
      if (n >= p.n_end) continue;
      float a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, u[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int s = 0; s < splits; ++s) {  // fixed order: the result does not depend on timing
        const uint32_t base = sm_map_to_cta(partial_local, (uint32_t)s) + (uint32_t)((t * kSmFeat + fa) * 4);
        const float4 x0 = sm_ld_cluster_f4(base), x1 = sm_ld_cluster_f4(base + 16);
        a[0] += x0.x; a[1] += x0.y; a[2] += x0.z; a[3] += x0.w; a[4] += x1.x; a[5] += x1.y; a[6] += x1.z; a[7] += x1.w;
        if (geglu) {
          const float4 y0 = sm_ld_cluster_f4(base + 128), y1 = sm_ld_cluster_f4(base + 144);
          u[0] += y0.x; u[1] += y0.y; u[2] += y0.z; u[3] += y0.w; u[4] += y1.x; u[5] += y1.y; u[6] += y1.z; u[7] += y1.w;
        }
      }
      if (p.bias != nullptr) {
        float b[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.bias + n)), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += b[i];
        if (geglu) {
          unpack8(__ldg(reinterpret_cast<const uint4*>(p.bias + n + 32)), b);
#pragma unroll
          for (int i = 0; i < 8; ++i) u[i] += b[i];
        }
      }
      int out_col = n;
      if (geglu) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = gelu_tanh(a[i]) * u[i];
        out_col = (f0 >> 1) + (g >> 2) * 32 + (g & 3) * 8;
      } else if (p.epilogue == LIGER_EPI_GELU) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = gelu_tanh(a[i]);
      } else if (p.epilogue == LIGER_EPI_RESIDUAL) {
        float b[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.residual + (size_t)t * p.ldr + n)), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += b[i];
      }
      uint4 o;
      o.x = pack_half2(a[0], a[1]); o.y = pack_half2(a[2], a[3]); o.z = pack_half2(a[4], a[5]); o.w = pack_half2(a[6], a[7]);
      *reinterpret_cast<uint4*>(epilogue_dst(p, t, out_col)) = o;
    }
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

// LIGER_GEMM_SMALLM = 0 keeps small-M launches on the big-tile kernels.
static bool smallm_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("LIGER_GEMM_SMALLM"); v = e ? atoi(e) : 1; }
  return v != 0;
}

// Returns LIGER_ERR_UNSUPPORTED (error text untouched) when the shape is not this kernel's.
int launch_gemm_smallm(const liger_gemm_args& a, const GemmParams& p0, const DeviceInfo* dev, cudaStream_t stream) {
  if (!smallm_enabled() || a.m > kSmTok || a.epilogue == LIGER_EPI_SCATTER) return LIGER_ERR_UNSUPPORTED;
  if (a.epilogue == LIGER_EPI_GEGLU && a.n_begin % 128) return LIGER_ERR_UNSUPPORTED;  // gate / value pairs per tile
  GemmParams p = p0;
  p.kblocks = (a.k + BK - 1) / BK;
  const int tiles = (a.n_end - a.n_begin + kSmFeat - 1) / kSmFeat;
  // The split count is chosen from the whole weight (a.n), not from the slice being computed, so that
  // a decomposed launch [n_begin, n_end) gives the bits of the whole launch.
  const int tiles_full = (a.n + kSmFeat - 1) / kSmFeat;
  // Cost of a split count, in k-block times: waves x (k-blocks per CTA + a set-up / drain term).  Measured on B200 a
  // CTA streams a 16 KB k-block in about 0.34 us and spends about 8 us outside its main loop, and a cluster of s
  // CTAs needs s free SMs in one GPC, so fewer clusters than sm_count / s run at once (the occupancy query knows).
  static int forced = -1;
  if (forced < 0) { const char* e = getenv("LIGER_GEMM_SMALLM_SPLITS"); forced = e ? atoi(e) : 0; }
  int best = 1;
  long best_cost = -1;
  for (int s = 1; s <= kSmMaxSplits && s <= p.kblocks; ++s) {
    const long conc = smallm_max_clusters(dev->device, dev->sm_count, s);
    const long waves = (tiles_full + conc - 1) / conc;
    const long cost = waves * ((p.kblocks + s - 1) / s + 24);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
  }
  if (forced > 0 && forced <= kSmMaxSplits && forced <= p.kblocks) best = forced;
  CUtensorMap tm_w, tm_x;
  int rc;
  if ((rc = make_tmap_2d_f16(&tm_w, a.wt, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldw, BK, kSmFeat)) != LIGER_OK) return rc;
  if ((rc = make_tmap_2d_f16(&tm_x, a.a, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, kSmTok)) != LIGER_OK) return rc;
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
