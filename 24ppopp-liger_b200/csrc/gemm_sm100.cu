// fp16 GEMM for sm_100a: C[M, n_begin:n_end] = epilogue(A[M,K] * W[K,N]), fp32 accumulation.
//
// Replaces the reference's cublasGemmEx calls (GemmEx, src/layer/func_wrapper.h:20-27, bound by
// Linear_Col / Linear_Row at src/layer/linear.h:47-53,99-105) and, through its epilogues, the
// element-wise kernels that follow them (add_QKV_bias, add_bias_gelu).
//
// Structure (one persistent CTA per SM, 6 warps):
//   warp 0  : TMA producer  -- one thread streams 128x64 A tiles and BNx64 W^T tiles into a
//             STAGES-deep shared-memory ring (128-byte swizzle), signalling `full` mbarriers.
//   warp 1  : MMA issuer    -- one thread issues tcgen05.mma (M=128, N=BN, K=16) x4 per stage into
//             one of two TMEM accumulators; tcgen05.commit releases the stage (`empty`) and,
//             after the last k-block, hands the accumulator to the epilogue (`tmem_full`).
//   warps 2-5: epilogue     -- tcgen05.ld 32 columns at a time (thread = row), bias / activation /
//             scatter in registers, 16-byte fp16 stores; then `tmem_empty` lets the MMA warp
//             reuse the accumulator, so the epilogue of tile i overlaps the MMAs of tile i+1.
// All waits are bounded (common.cuh); a timeout sets the sticky status word and the CTA unwinds.
#include <cmath>
#include <cstdlib>

#include "gemm_epilogue.cuh"

LIGER_REGISTER_WAIT_BUDGET()

namespace liger {

template <int BN, int STAGES>
struct GemmCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kEpiW = BN < 128 ? BN : 128;             // accumulator columns staged per pass
  static constexpr int kEpiBytesPerWarp = 32 * kEpiW * 2;       // fp16 staging tile of one epilogue warp
  static constexpr int kEpiBytes = 4 * kEpiBytesPerWarp;
  static constexpr int kSmemBytes = STAGES * kStageBytes + kEpiBytes + kBarrierBytes + 1024;  // + alignment slack
  static constexpr int kTmemCols = 2 * BN;
};

// ---- the kernel -------------------------------------------------------------------------------
template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
  using Cfg = GemmCfg<BN, STAGES>;
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

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t armed_mask = 0, armed_phase = 0;  // which stages have a load in flight, and its parity
      bool ok = true;
      const uint64_t hint_a = !p.use_hints ? kL2EvictNormal : p.stationary == 0 ? kL2EvictLast : kL2EvictFirst;
      const uint64_t hint_b = !p.use_hints ? kL2EvictNormal : p.stationary == 0 ? kL2EvictFirst : kL2EvictLast;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(p, t, tm, tn);
        const int m0 = tm * BM;
        const int n0 = p.n_begin + tn * BN;
        if (!wait_rows_ready(p, m0, BM, abort_flag)) { ok = false; break; }
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d_hint(sa, &tmap_a, &full_bar[stage], kb * BK, m0, hint_a);
          tma_load_2d_hint(sa + Cfg::kABytes, &tmap_b, &full_bar[stage], kb * BK, n0, hint_b);
          armed_mask |= 1u << stage;
          armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // unwinding: give the copies already issued a bounded time to land before the CTA exits
        for (int s = 0; s < STAGES; ++s)
          if (armed_mask & (1u << s))
            for (int spin = 0; spin < (1 << 16) && !mbar_test(&full_bar[s], (armed_phase >> s) & 1u); ++spin) {}
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer =====
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(BM, BN);
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
        if (!mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t da = make_sw128_kmajor_desc(sa);
          const uint64_t db = make_sw128_kmajor_desc(sa + Cfg::kABytes);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            // advancing 16 fp16 along K inside the 128-byte swizzle atom = +32 bytes = +2 in the
            // descriptor's (address >> 4) field
            umma_f16(d_tmem, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb | k4) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ===== epilogue: warps 2..5, TMEM lane quadrant = warp % 4 =====
    const int quad = warp & 3;
    uint32_t it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
      int tm, tn;
      tile_coords(p, t, tm, tn);
      const int m0 = tm * BM;
      const int n0 = p.n_begin + tn * BN;
      if (!mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      epilogue_tile<BN>(p, tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16),
                        epi_stage + (warp - 2) * Cfg::kEpiBytesPerWarp, m0 + quad * 32, n0, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  // ===== teardown =====
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) report_failure(p.status, LIGER_DEV_TIMEOUT, 0x100u, blockIdx.x, 0);
}

template <int BN, int STAGES>
static int launch_gemm(const liger_gemm_args& a, const GemmParams& p0, int sm_count, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, STAGES>;
  GemmParams p = p0;
  p.tiles_m = (a.m + BM - 1) / BM;
  p.tiles_n = (a.n_end - a.n_begin + BN - 1) / BN;
  p.kblocks = (a.k + BK - 1) / BK;
  choose_tile_order(p, a, BM, BN);
  choose_arrival_order(p, BM);
  CUtensorMap tm_a, tm_b;
  int rc;
  if ((rc = make_tmap_2d_f16(&tm_a, a.a, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, BM)) != LIGER_OK) return rc;
  if ((rc = make_tmap_2d_f16(&tm_b, a.wt, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldw, BK, BN)) != LIGER_OK) return rc;
  static bool attr_set = false;  // per template instantiation
  if (!attr_set) {
    LIGER_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg::kSmemBytes));
    attr_set = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;
  gemm_tcgen05_kernel<BN, STAGES><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tm_a, tm_b, p);
  return check_launch("gemm_tcgen05_kernel");
}

// Panel choice for tile_coords: keep the operand whose re-streaming would cost more resident.
// cost(A stationary) = A + B * panels(A); cost(B stationary) = B + A * panels(B).
// Measured on B200 (GLM-130B shapes, power-capped and not): the plain order -- m fastest over the whole
// matrix, so that the CTAs of a wave share few W^T tiles and walk K in step -- beats M- or N-panels sized
// to half of L2, with or without eviction-priority hints (by 5 % and 9 % on the 4-layer step), although
// the panels cut DRAM traffic: the kernel is limited by power and the tensor pipe, not by DRAM.  The panel
// orders stay selectable (LIGER_GEMM_ORDER = 1: panels, 2: panels + hints) for other shapes.
void choose_tile_order(GemmParams& p, const liger_gemm_args& a, int tile_m, int tile_n) {
  static int order = -1, hints = -1;
  static double cap = 0.0;
  if (order < 0) {
    const char* e = getenv("LIGER_GEMM_ORDER");
    order = e ? atoi(e) : 0;
    e = getenv("LIGER_GEMM_HINTS");
    hints = e ? atoi(e) : (order == 2 ? 1 : 0);
    e = getenv("LIGER_GEMM_PANEL_MB");
    cap = (e ? atof(e) : 56.0) * 1e6;  // bytes of L2 a resident panel may take
  }
  p.use_hints = hints;
  if (order == 0) {  // plain m-fastest order over the whole matrix
    p.stationary = 0;
    p.panel_tiles = p.tiles_m;
    return;
  }
  const double row_bytes = 2.0 * a.k;
  const double a_bytes = (double)a.m * row_bytes, b_bytes = (double)(a.n_end - a.n_begin) * row_bytes;
  const int pa = (int)ceil(a_bytes / cap), pb = (int)ceil(b_bytes / cap);
  const double cost_a = a_bytes + b_bytes * (pa < 1 ? 1 : pa), cost_b = b_bytes + a_bytes * (pb < 1 ? 1 : pb);
  if (cost_a <= cost_b) {
    p.stationary = 0;
    int rows = (int)(cap / row_bytes);
    int t = rows / tile_m;
    if (t < 1) t = 1;
    p.panel_tiles = t > p.tiles_m ? p.tiles_m : t;
    const int panels = (p.tiles_m + p.panel_tiles - 1) / p.panel_tiles;
    p.panel_tiles = (p.tiles_m + panels - 1) / panels;
  } else {
    p.stationary = 1;
    int rows = (int)(cap / row_bytes);
    int t = rows / tile_n;
    if (t < 1) t = 1;
    p.panel_tiles = t > p.tiles_n ? p.tiles_n : t;
    const int panels = (p.tiles_n + p.panel_tiles - 1) / p.panel_tiles;
    p.panel_tiles = (p.tiles_n + panels - 1) / panels;
  }
}

// A arrives by liger_allgather_push: walk the row tiles (tile_m rows each) in the order their rows land -- this
// rank's own rows first, then, row block by row block, the blocks of ranks rank+1, rank+2, ... -- in panels of a
// few row tiles, so that a wave of CTAs needs only the rows that are already there or arrive next.  Launches with
// more row tiles than the order table holds fall back to the plain order (every tile still waits for its rows).
void choose_arrival_order(GemmParams& p, int tile_m) {
  if (p.ready_flags == nullptr) return;
  const int tiles_m = p.tiles_m;
  p.tm_order_on = 0;
  if (tiles_m > kTmOrderMax) return;
  p.tm_order_on = 1;
  const int ws = (p.m + p.ready_rpr - 1) / p.ready_rpr;
  const int steps_per_block = ws > 1 ? ws - 1 : 1;
  auto step_of_row = [&](int row) -> int {
    if (row >= p.m) row = p.m - 1;
    const int owner = row / p.ready_rpr;
    if (owner == p.ready_rank) return -1;
    const int blk = (row - owner * p.ready_rpr) / p.ready_block_rows;
    int k = owner - p.ready_rank;
    if (k < 0) k += ws;
    return blk * steps_per_block + (k - 1);
  };
  int key[kTmOrderMax];
  for (int t = 0; t < tiles_m; ++t) {
    const int a0 = step_of_row(t * tile_m), a1 = step_of_row(t * tile_m + tile_m - 1);
    key[t] = a0 > a1 ? a0 : a1;
    p.tm_order[t] = (uint8_t)t;
  }
  for (int i = 1; i < tiles_m; ++i) {  // stable insertion sort by arrival step
    const uint8_t v = p.tm_order[i];
    int j = i - 1;
    while (j >= 0 && key[p.tm_order[j]] > key[v]) { p.tm_order[j + 1] = p.tm_order[j]; --j; }
    p.tm_order[j + 1] = v;
  }
  // panels of as many row tiles as one rank owns (at least 2): m runs fastest inside a panel
  int per_rank = p.ready_rpr / tile_m;
  if (per_rank < 2) per_rank = 2;
  if (per_rank > 8) per_rank = 8;
  p.stationary = 0;
  p.panel_tiles = per_rank < tiles_m ? per_rank : tiles_m;
}

int launch_gemm_2cta(const liger_gemm_args& a, const GemmParams& p0, int sm_count, cudaStream_t stream);
int launch_gemm_smallm(const liger_gemm_args& a, const GemmParams& p0, const DeviceInfo* dev, cudaStream_t stream);

// 0 = choose automatically, 1 = 1-CTA kernel only, 2 = 2-CTA kernel whenever the shape allows
static int g_gemm_variant = -1;
static int gemm_variant() {
  if (g_gemm_variant < 0) {
    const char* e = getenv("LIGER_GEMM_VARIANT");
    g_gemm_variant = e ? atoi(e) : 0;
  }
  return g_gemm_variant;
}

}  // namespace liger

extern "C" int liger_gemm_fp16(const liger_gemm_args* args, void* stream) {
  using namespace liger;
  if (!args) return set_error(LIGER_ERR_INVALID, "liger_gemm_fp16: null args");
  const liger_gemm_args& a = *args;
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return set_error(LIGER_ERR_INVALID, "gemm: m, n, k must be positive");
  if (!a.a || !a.wt) return set_error(LIGER_ERR_INVALID, "gemm: null operand");
  if (a.k % 8 || a.lda % 8 || a.ldw % 8 || a.lda < a.k || a.ldw < a.k)
    return set_error(LIGER_ERR_INVALID, "gemm: k, lda, ldw must be multiples of 8 and lda, ldw >= k");
  if (a.n_begin < 0 || a.n_end > a.n || a.n_begin >= a.n_end || a.n_begin % 8 || a.n_end % 8)
    return set_error(LIGER_ERR_INVALID, "gemm: bad feature slice [%d, %d) of %d (bounds must be multiples of 8)",
                     a.n_begin, a.n_end, a.n);
  if (a.bias && ((uintptr_t)a.bias & 15u)) return set_error(LIGER_ERR_INVALID, "gemm: bias must be 16-byte aligned");
  GemmParams p{};
  p.c = (__half*)a.c;
  p.bias = (const __half*)a.bias;
  p.residual = (const __half*)a.residual;
  p.m = a.m; p.n_begin = a.n_begin; p.n_end = a.n_end;
  p.ldc = a.ldc; p.ldr = a.ldr;
  p.epilogue = a.epilogue;
  switch (a.epilogue) {
    case LIGER_EPI_STORE:
    case LIGER_EPI_GELU:
    case LIGER_EPI_RESIDUAL:
    case LIGER_EPI_GEGLU:
      if (!a.c || ((uintptr_t)a.c & 15u) || a.ldc % 8)
        return set_error(LIGER_ERR_INVALID, "gemm: c must be 16-byte aligned with ldc %% 8 == 0");
      if (a.epilogue == LIGER_EPI_RESIDUAL && (!a.residual || ((uintptr_t)a.residual & 15u) || a.ldr % 8))
        return set_error(LIGER_ERR_INVALID, "gemm: residual must be 16-byte aligned with ldr %% 8 == 0");
      if (a.epilogue == LIGER_EPI_GEGLU && (a.n % 64 || a.n_begin % 64 || a.n_end % 64))
        return set_error(LIGER_ERR_INVALID, "gemm: GeGLU needs n, n_begin, n_end to be multiples of 64");
      break;
    case LIGER_EPI_QKV_SPLIT:
      if (!a.q_out || !a.k_out || !a.v_out || a.seq_len <= 0 || a.heads <= 0 || a.head_dim <= 0)
        return set_error(LIGER_ERR_INVALID, "gemm: QKV split needs q/k/v outputs and seq_len, heads, head_dim");
      if (a.n != 3 * a.heads * a.head_dim || a.head_dim % 8 || a.m % a.seq_len)
        return set_error(LIGER_ERR_INVALID, "gemm: QKV split needs n == 3*heads*head_dim, head_dim %% 8 == 0, m %% seq_len == 0");
      if (((uintptr_t)a.q_out | (uintptr_t)a.k_out | (uintptr_t)a.v_out) & 15u)
        return set_error(LIGER_ERR_INVALID, "gemm: q/k/v outputs must be 16-byte aligned");
      p.qkv[0] = (__half*)a.q_out; p.qkv[1] = (__half*)a.k_out; p.qkv[2] = (__half*)a.v_out;
      if (a.kv_stride < 0 || a.kv_pos < 0 || (a.kv_stride > 0 && a.kv_pos + a.seq_len > a.kv_stride))
        return set_error(LIGER_ERR_INVALID, "gemm: kv_pos + seq_len must fit in kv_stride");
      p.seq_len = a.seq_len; p.heads = a.heads; p.head_dim = a.head_dim;
      p.kv_stride = a.kv_stride; p.kv_pos = a.kv_pos;
      break;
    case LIGER_EPI_SCATTER: {
      liger_comm* c = a.scatter_comm;
      if (!c || !c->connected) return set_error(LIGER_ERR_INVALID, "gemm: scatter epilogue needs a connected communicator");
      const int rpr = (a.m + c->ws - 1) / c->ws;
      const size_t need = (size_t)c->ws * rpr * a.n * 2;
      if (a.scatter_off % 16 || a.scatter_off + need > c->data_bytes)
        return set_error(LIGER_ERR_INVALID, "gemm: scatter region [%zu, +%zu) must be 16-byte aligned and inside the %zu-byte data region",
                         a.scatter_off, need, c->data_bytes);
      for (int r = 0; r < kMaxRanks; ++r) p.peer[r] = r < c->ws ? c->peer[r] : nullptr;
      p.scatter_off = kFlagRegionBytes + a.scatter_off;
      p.rank = c->rank; p.rows_per_rank = rpr; p.ldc = a.n;
      break;
    }
    default:
      return set_error(LIGER_ERR_INVALID, "gemm: unknown epilogue %d", a.epilogue);
  }
  const DeviceInfo* dev;
  int rc = require_sm100(&dev);
  if (rc != LIGER_OK) return rc;
  p.status = dev->status_dev;
  if (a.gather_comm != nullptr) {
    liger_comm* c = a.gather_comm;
    if (!c->connected || a.gather_channel < 0 || a.gather_channel >= c->channels || c->ready_block_rows[a.gather_channel] <= 0)
      return set_error(LIGER_ERR_INVALID, "gemm: gather_comm / gather_channel must name a channel liger_allgather_push has used");
    p.ready_flags = reinterpret_cast<const uint32_t*>(c->local) + (size_t)a.gather_channel * kMaxRanks * kFlagStrideWords;
    p.ready_epoch = c->epoch[a.gather_channel];
    p.ready_rpr = (a.m + c->ws - 1) / c->ws;
    p.ready_rank = c->rank;
    p.ready_block_rows = c->ready_block_rows[a.gather_channel];
    // 256x256 tiles for a consumer of a gather: a wave of them spans half as many row blocks as a wave of 256x512
    // tiles, so the first wave waits for two ranks' rows instead of six (LIGER_GATHER_WIDE=1 allows the wide kernel)
    static int gather_wide = -1;
    if (gather_wide < 0) { const char* e = getenv("LIGER_GATHER_WIDE"); gather_wide = e ? atoi(e) : 0; }
    p.no_wide = gather_wide ? 0 : 1;
  }

  // Tile-width choice: fewest (waves x per-tile cost); per-tile cost ~ (BM + BN) (operand bytes per
  // k-block and MMA time are both linear in BN).  GeGLU pairs 32-column chunks, so BN >= 64 there.
  const int tiles_m = (a.m + BM - 1) / BM;
  const int span = a.n_end - a.n_begin;
  int best_bn = 256;
  long best_cost = -1;
  const int cands[4] = {256, 128, 64, 32};
  for (int i = 0; i < 4; ++i) {
    const int bn = cands[i];
    if (a.epilogue == LIGER_EPI_GEGLU && bn < 64) continue;
    const long tiles = (long)tiles_m * ((span + bn - 1) / bn);
    const long waves = (tiles + dev->sm_count - 1) / dev->sm_count;
    const long cost = waves * (BM + bn);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_bn = bn; }
  }
  cudaStream_t s = (cudaStream_t)stream;
  // a handful of rows (decode): the weight-streaming kernel with swapped operand roles and split K
  if (a.m <= 32 && p.ready_flags == nullptr) {
    const int rcs = launch_gemm_smallm(a, p, dev, s);
    if (rcs != LIGER_ERR_UNSUPPORTED) return rcs;
  }
  // 2-CTA 256x256 tiles when there is at least one full wave of them (one tile per SM pair)
  const long tiles2 = (long)((a.m + 255) / 256) * ((span + 255) / 256);
  const int variant = gemm_variant();
  if (variant != 1 && a.m >= 256 && (variant == 2 || tiles2 >= dev->sm_count / 2)) {
    const int rc2 = launch_gemm_2cta(a, p, dev->sm_count, s);
    if (rc2 != LIGER_ERR_UNSUPPORTED) return rc2;
  }
  switch (best_bn) {
    case 256: return launch_gemm<256, 4>(a, p, dev->sm_count, s);
    case 128: return launch_gemm<128, 6>(a, p, dev->sm_count, s);
    case 64: return launch_gemm<64, 8>(a, p, dev->sm_count, s);
    default: return launch_gemm<32, 8>(a, p, dev->sm_count, s);
  }
}
