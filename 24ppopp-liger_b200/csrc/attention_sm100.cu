// Prefill attention on the tcgen05 tensor cores (head_dim 128, no mask tensor).
//
// One persistent CTA per SM walks work items (128 query rows of one (batch, head)), heaviest
// first.  Per 128-key block:  S = Q K^T  (tcgen05.mma, M=128 N=128 K=128, fp32 in TMEM)  ->  softmax
// warps read their rows from TMEM (thread = row: row max and row sum need no shuffles) and write
// P = exp(x - m) as fp16 into shared memory in the 128-byte-swizzled K-major layout  ->
// O += P V  (tcgen05.mma accumulating in TMEM over the blocks of the item; V is consumed as the TMA
// stored it, head_dim contiguous, i.e. an MN-major B operand).
//
// The running maximum m is updated lazily: a row keeps its reference maximum while the block's
// maximum exceeds it by less than 8 in log2 units (p stays below 256, harmless in fp16 with fp32
// sums), so the accumulator in TMEM only has to be rescaled (read, multiply, write back) on the
// rare blocks where some row's maximum jumps; sum and output stay consistent because both are kept
// relative to the same m.  S and the K / V stages are double-buffered, and consecutive items
// alternate between two O accumulators, so the MMAs run under the softmax; the softmax warps (the
// exp unit in particular) are the critical resource.
//
// Arithmetic as the mma.sync kernel and the reference (src/cuda/attention_kernels.cu:543-573): scores
// scaled in fp32, masked positions get -10000 added, p = exp(x - m) / (sum + 1e-6), P rounded to
// fp16 before the second product, fp32 accumulation.
//
// Warps: 0 = TMA producer (one lane), 1 = MMA issuer (one lane) and TMEM owner, 2-17 = softmax /
// output.  A softmax warp can only read the TMEM lanes (rows) 32 (w % 4) .. +31, so the 16 warps split
// the columns: warp w handles rows 32 (w % 4) .. +31 and the 32 keys (and 32 output columns)
// 32 ((w - 2) / 4) .. +31 of every block; the four threads of a row exchange their maxima (per
// block) and their sums (per item) through shared memory.  Four warps per scheduler hide the TMEM
// and special-function latencies that a single warp per scheduler leaves exposed (measured: 4x).
// Every wait is bounded.
#include "runtime.h"

LIGER_REGISTER_WAIT_BUDGET()

namespace liger {

namespace {

constexpr int kTcThreads = 576;  // 18 warps
constexpr int kBoxBytes = 128 * 64 * 2;   // one swizzled box: 128 rows x 64 fp16
constexpr int kTileBytes = 2 * kBoxBytes; // a [128 x 128] fp16 tile = two boxes (columns 0-63, 64-127)
constexpr int kExchBytes = (2 * 4 + 2 * 4) * 128 * 4;  // row maxima [2 stages][4 column groups][128 rows], row sums [2 items][4][128]
constexpr int kOutScratchBytes = 16 * 512;  // per softmax warp: 8 rows x 64 B of output being regrouped for coalesced stores
constexpr int kTcSmemBytes = 6 * kTileBytes /* Q, K x2, V x2, P */ + kExchBytes + kOutScratchBytes + 512 + 1024;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnTcParams {
  __half* out;
  int S, heads, ldo, causal;
  int nq;        // query tiles per (batch, head)
  int nkb;       // key blocks per (batch, head)
  int items;     // nq * batch * heads
  float scale;
  DeviceStatus* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// V tile as B operand of P*V: N = head_dim runs along the 128-byte rows (MN-major), K = keys across
// rows.  Swizzle atoms are 64 head_dim elements x 8 keys (1024 B): `sbo` is the distance between
// 8-key groups, `lbo` the distance between the two 64-column boxes.
__device__ __forceinline__ uint64_t make_v_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// which item / block a role is at; every role advances through the same sequence.
// Item order: the query tiles of one (batch, head) are adjacent, so that the CTAs working on them run
// at the same time and its K / V blocks are fetched from DRAM once and hit in L2 for the other
// tiles; in round k a CTA takes slot (blockIdx.x + k) mod gridDim.x of the round, so that under a
// causal mask (tiles of very different cost) every CTA sees all tile positions in turn.
struct Cursor {
  int round, j, nblk, qt, bh;
  uint32_t g, item;
  bool valid;
};
__device__ __forceinline__ void cursor_load(const AttnTcParams& p, Cursor& c) {
  const int w = c.round * (int)gridDim.x + (int)((blockIdx.x + (unsigned)c.round) % gridDim.x);
  c.valid = w < p.items;
  if (!c.valid) {
    // a later slot of the last, partial round may still be in range for other CTAs but not for this one
    return;
  }
  c.bh = w / p.nq;
  c.qt = p.nq - 1 - w % p.nq;  // heavy (late) query tiles first within a head
  c.nblk = p.causal ? min(p.nkb, c.qt + 1) : p.nkb;
  c.j = 0;
}
__device__ __forceinline__ void cursor_init(const AttnTcParams& p, Cursor& c) {
  c.round = 0;
  c.g = 0;
  c.item = 0;
  cursor_load(p, c);
}
__device__ __forceinline__ void cursor_next(const AttnTcParams& p, Cursor& c) {
  ++c.g;
  if (++c.j < c.nblk) return;
  ++c.round;
  ++c.item;
  cursor_load(p, c);
}

__global__ void __launch_bounds__(kTcThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, const AttnTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTileBytes;      // [2]
  uint8_t* sV = sK + 2 * kTileBytes;  // [2]
  uint8_t* sP = sV + 2 * kTileBytes;
  float* xmax = reinterpret_cast<float*>(sP + kTileBytes);  // [2][4][128]
  float* lsum = xmax + 2 * 4 * 128;                         // [2][4][128]
  uint8_t* out_scratch = reinterpret_cast<uint8_t*>(lsum + 2 * 4 * 128);  // [16 warps][512 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_scratch + kOutScratchBytes);
  uint64_t* q_full = bars;        // [1]
  uint64_t* q_empty = bars + 1;   // [1]
  uint64_t* k_full = bars + 2;    // [2]
  uint64_t* k_empty = bars + 4;   // [2]
  uint64_t* v_full = bars + 6;    // [2]
  uint64_t* v_empty = bars + 8;   // [2]
  uint64_t* s_full = bars + 10;   // [2]
  uint64_t* s_empty = bars + 12;  // [2]
  uint64_t* o_empty = bars + 14;  // [2]: the output of the item that used accumulator i has been read
  uint64_t* p_full = bars + 16;   // [1]: P written (and O rescaled where needed) for the next PV product
  uint64_t* pv_done = bars + 17;  // [1]: a PV product has completed (P may be overwritten, O may be touched)
  uint64_t* x_bar = bars + 18;    // [2][4]: the four column groups of a row quarter have published their maxima
  uint64_t* l_bar = bars + 26;    // [4]: ... their sums
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 30);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 16);
      mbar_init(&o_empty[i], 16);
    }
    mbar_init(p_full, 16);
    mbar_init(pv_done, 1);
    for (int i = 0; i < 8; ++i) mbar_init(&x_bar[i], 4);
    for (int i = 0; i < 4; ++i) mbar_init(&l_bar[i], 4);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);  // S[2] at columns 0 / 128, O[2] at 256 / 384
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  Cursor c;
  cursor_init(p, c);

  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      bool ok = true;
      while (c.valid && ok) {
        if (!mbar_wait_bounded(q_empty, (c.item & 1u) ^ 1u, abort_flag)) break;
        mbar_arrive_expect_tx(q_full, kTileBytes);
        tma_load_3d(sQ, &tmap_q, q_full, 0, c.qt * 128, c.bh);
        tma_load_3d(sQ + kBoxBytes, &tmap_q, q_full, 64, c.qt * 128, c.bh);
        const uint32_t item = c.item;
        while (c.valid && c.item == item) {
          const uint32_t st = c.g & 1u, ph = (c.g >> 1) & 1u;
          if (!mbar_wait_bounded(&k_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&k_full[st], kTileBytes);
          tma_load_3d(sK + st * kTileBytes, &tmap_k, &k_full[st], 0, c.j * 128, c.bh);
          tma_load_3d(sK + st * kTileBytes + kBoxBytes, &tmap_k, &k_full[st], 64, c.j * 128, c.bh);
          if (!mbar_wait_bounded(&v_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&v_full[st], kTileBytes);
          tma_load_3d(sV + st * kTileBytes, &tmap_v, &v_full[st], 0, c.j * 128, c.bh);
          tma_load_3d(sV + st * kTileBytes + kBoxBytes, &tmap_v, &v_full[st], 64, c.j * 128, c.bh);
          cursor_next(p, c);
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer: QK^T of block g+1 is issued ahead of the PV product of block g =====
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(128, 128);
      constexpr uint32_t idesc_pv = make_idesc_f16(128, 128) | (1u << 16);  // B operand MN-major
      bool ok = true;
      auto issue_qk = [&](const Cursor& a) {
        const uint32_t st = a.g & 1u, ph = (a.g >> 1) & 1u;
        if (a.j == 0 && !mbar_wait_bounded(q_full, a.item & 1u, abort_flag)) { ok = false; return; }
        if (!mbar_wait_bounded(&k_full[st], ph, abort_flag)) { ok = false; return; }
        if (!mbar_wait_bounded(&s_empty[st], ph ^ 1u, abort_flag)) { ok = false; return; }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + st * kTileBytes);
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {
          const uint64_t da = make_sw128_kmajor_desc(qa + (k8 >> 2) * kBoxBytes) + (uint64_t)((k8 & 3) * 2);
          const uint64_t db = make_sw128_kmajor_desc(ka + (k8 >> 2) * kBoxBytes) + (uint64_t)((k8 & 3) * 2);
          umma_f16(tmem_base + st * 128, da, db, idesc_qk, k8 != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
        if (a.j == a.nblk - 1) umma_commit(q_empty);
      };
      auto issue_pv = [&](const Cursor& b) {
        const uint32_t st = b.g & 1u, ph = (b.g >> 1) & 1u, ob = b.item & 1u;
        if (!mbar_wait_bounded(&v_full[st], ph, abort_flag)) { ok = false; return; }
        if (!mbar_wait_bounded(p_full, b.g & 1u, abort_flag)) { ok = false; return; }
        if (b.j == 0 && !mbar_wait_bounded(&o_empty[ob], ((b.item >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; return; }
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + st * kTileBytes);
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {  // 16 keys per MMA
          const uint64_t da = make_sw128_kmajor_desc(pa + (k8 >> 2) * kBoxBytes) + (uint64_t)((k8 & 3) * 2);
          const uint64_t db = make_v_desc(va + k8 * 2048, kBoxBytes, 1024);
          umma_f16(tmem_base + 256 + ob * 128, da, db, idesc_pv, (b.j | k8) != 0 ? 1u : 0u);
        }
        umma_commit(pv_done);
        umma_commit(&v_empty[st]);
      };
      Cursor a = c;
      if (a.valid) { issue_qk(a); cursor_next(p, a); }
      while (c.valid && ok) {
        if (a.valid) { issue_qk(a); if (!ok) break; cursor_next(p, a); }
        issue_pv(c);
        cursor_next(p, c);
      }
    }
  } else {
    // ===== softmax + output: thread = (query row, group of 32 keys / output columns) =====
    const int quad = warp & 3;            // TMEM lane quarter = rows 32 quad .. +31
    const int cg = (warp - 2) >> 2;       // column group 0..3
    const int r = quad * 32 + lane;       // row inside the tile
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    bool ok = true;

    // The output of an item is written after the first block of the NEXT item has been handed to the
    // tensor core, so that it is off the critical path (the next item accumulates into the other O buffer).
    struct Pending { int qi, bh; uint32_t item; bool valid; } pend = {0, 0, 0, false};
    auto write_output = [&](const Pending& q) {  // all PV products of item q must be known complete
      const float* ls = lsum + (q.item & 1u) * 512;
      if (!mbar_wait_bounded(&l_bar[quad], q.item & 1u, abort_flag)) { ok = false; return; }
      const float l_tot = (ls[r] + ls[128 + r]) + (ls[256 + r] + ls[384 + r]);
      const uint32_t ob = q.item & 1u;
      tc_fence_after();
      uint32_t t[32];
      tmem_ld_32x32(tmem_base + 256 + ob * 128 + cg * 32 + lane_sel, t);
      tmem_ld_wait_regs(t);
      // thread = row holds 64 contiguous output bytes; a warp store of one 16-byte piece per row would touch
      // 32 different lines.  Regroup 8 rows at a time through 512 B of shared memory so that every store
      // instruction writes 8 rows x 64 contiguous bytes.
      const float inv = 1.0f / (l_tot + 1e-6f);
      uint4 u[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        u[q4].x = pack_half2(__uint_as_float(t[q4 * 8 + 0]) * inv, __uint_as_float(t[q4 * 8 + 1]) * inv);
        u[q4].y = pack_half2(__uint_as_float(t[q4 * 8 + 2]) * inv, __uint_as_float(t[q4 * 8 + 3]) * inv);
        u[q4].z = pack_half2(__uint_as_float(t[q4 * 8 + 4]) * inv, __uint_as_float(t[q4 * 8 + 5]) * inv);
        u[q4].w = pack_half2(__uint_as_float(t[q4 * 8 + 6]) * inv, __uint_as_float(t[q4 * 8 + 7]) * inv);
      }
      uint8_t* scr = out_scratch + (warp - 2) * 512;
      const int b = q.bh / p.heads, head = q.bh - b * p.heads;
      const int q_row0 = q.qi - lane;  // first row of this warp's 32
      __half* obase = p.out + (size_t)b * p.S * p.ldo + (size_t)head * 128 + cg * 32 + (lane & 3) * 8;
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        if ((lane >> 3) == pass) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) *reinterpret_cast<uint4*>(scr + (lane & 7) * 64 + q4 * 16) = u[q4];
        }
        __syncwarp();
        const uint4 piece = *reinterpret_cast<const uint4*>(scr + lane * 16);
        const int row = q_row0 + pass * 8 + (lane >> 2);
        if (row < p.S) *reinterpret_cast<uint4*>(obase + (size_t)row * p.ldo) = piece;
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_empty[ob]);
    };

    uint32_t g_last = 0;
    while (c.valid && ok) {
      const int qi = c.qt * 128 + r;
      const int nblk = c.nblk, bh = c.bh, qt = c.qt;
      const uint32_t item = c.item, ob = item & 1u;
      const uint32_t o_addr = tmem_base + 256 + ob * 128 + cg * 32 + lane_sel;
      float m_ref = -INFINITY, l_run = 0.0f;

      for (int j = 0; j < nblk && ok; ++j) {
        const uint32_t g = c.g, st = g & 1u, ph = (g >> 1) & 1u;
        const int k0 = j * 128;
        // keys of this block with index > cmask get -10000 (causal diagonal block); index >= cinf do not
        // exist (past the sequence end)
        const bool diag = p.causal && j == qt;
        const bool need_mask = diag || (k0 + 128 > p.S);
        const int cmask = diag ? r : 1 << 30;
        const int cinf = p.S - k0;
        if (!mbar_wait_bounded(&s_full[st], ph, abort_flag)) { ok = false; break; }
        tc_fence_after();

        uint32_t v[32];
        tmem_ld_32x32(tmem_base + st * 128 + cg * 32 + lane_sel, v);
        tmem_ld_wait_regs(v);

        // row maximum of x = s * scale (+ mask) over this thread's 32 keys, then over the four groups
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int ci = cg * 32 + i;
            float x = __uint_as_float(v[i]) * p.scale;
            x = ci > cmask ? x - 10000.0f : x;
            x = ci >= cinf ? -INFINITY : x;
            mx4[i & 3] = fmaxf(mx4[i & 3], x);
          }
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        if (!need_mask) mx *= p.scale;  // scale > 0: max(s) * scale == max(s * scale)
        float* xm = xmax + st * 512;
        xm[cg * 128 + r] = mx;
        __syncwarp();
        if (lane == 0) mbar_arrive(&x_bar[st * 4 + quad]);
        if (!mbar_wait_bounded(&x_bar[st * 4 + quad], ph, abort_flag)) { ok = false; break; }
        mx = fmaxf(fmaxf(xm[r], xm[128 + r]), fmaxf(xm[256 + r], xm[384 + r]));

        // lazy reference maximum (identical in the four threads of a row: same inputs, same arithmetic)
        const bool grow = (mx - m_ref) * kLog2e > 8.0f;  // always true for the first block (m_ref = -inf)
        const float m_new = grow ? mx : m_ref;
        const float alpha = grow ? fast_exp2((m_ref - m_new) * kLog2e) : 1.0f;
        m_ref = m_new;
        const float ml2 = m_new * kLog2e;

        // p = exp(x - m) and the partial row sum, in registers: the previous PV product (which still reads
        // the single P tile) runs underneath
        float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint32_t pk[16];
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float a0 = fast_exp2(fmaf(__uint_as_float(v[i]), sl2, -ml2));
            const float a1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), sl2, -ml2));
            sum4[i & 3] += a0;
            sum4[(i + 1) & 3] += a1;
            pk[i >> 1] = pack_half2(a0, a1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float a[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int ci = cg * 32 + i + e;
              float t = fmaf(__uint_as_float(v[i + e]), sl2, -ml2);
              t = ci > cmask ? t - 10000.0f * kLog2e : t;
              t = ci >= cinf ? -INFINITY : t;
              a[e] = fast_exp2(t);
            }
            sum4[i & 3] += a[0];
            sum4[(i + 1) & 3] += a[1];
            pk[i >> 1] = pack_half2(a[0], a[1]);
          }
        }
        l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));

        // P is single-buffered and O must be quiet for a rescale: the previous PV product has to be complete
        if (g > 0 && !mbar_wait_bounded(pv_done, (g - 1) & 1u, abort_flag)) { ok = false; break; }
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          tc_fence_after();
          uint32_t t[32];
          tmem_ld_32x32(o_addr, t);
          tmem_ld_wait_regs(t);
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
          tmem_st_32x32(o_addr, t);
          tmem_st_wait();
        }
        uint8_t* prow = sP + (cg >> 1) * kBoxBytes + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int kc = (cg & 1) * 4 + q4;  // 16-byte chunk (8 keys) inside the 64-key box
          *reinterpret_cast<uint4*>(prow + ((kc ^ (r & 7)) << 4)) =
              make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
        }
        tc_fence_before();
        fence_proxy_async();  // the P tile is read by the tensor core (async proxy)
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&s_empty[st]);
          mbar_arrive(p_full);
        }
        if (j == 0 && pend.valid) {  // the wait on pv_done above covered the last PV product of the previous item
          write_output(pend);
          pend.valid = false;
        }
        g_last = g;
        cursor_next(p, c);
      }
      if (!ok) break;

      // publish this thread's share of the row sum; the output is written later
      lsum[(item & 1u) * 512 + cg * 128 + r] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(&l_bar[quad]);
      pend.qi = qi; pend.bh = bh; pend.item = item; pend.valid = true;
    }
    if (ok && pend.valid && mbar_wait_bounded(pv_done, g_last & 1u, abort_flag)) write_output(pend);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) report_failure(p.status, LIGER_DEV_TIMEOUT, 0x200u, blockIdx.x, 0);
}

}  // namespace

// Returns LIGER_ERR_UNSUPPORTED (error text untouched) when the shape is not one this kernel takes.
int launch_attention_prefill_tc(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len,
                                int ldo, float scale, int causal, cudaStream_t stream) {
  const DeviceInfo* dev = nullptr;
  int rc = require_sm100(&dev);
  if (rc != LIGER_OK) return rc;
  if (ldo % 8 != 0 || ((uintptr_t)out & 15u) != 0 || !(scale > 0.0f)) return LIGER_ERR_UNSUPPORTED;
  AttnTcParams p{};
  p.out = (__half*)out;
  p.S = seq_len;
  p.heads = heads;
  p.ldo = ldo;
  p.causal = causal;
  p.nq = (seq_len + 127) / 128;
  p.nkb = (seq_len + 127) / 128;
  p.items = p.nq * batch * heads;
  p.scale = scale;
  p.status = dev->status_dev;
  CUtensorMap tq, tk, tv;
  const uint64_t bh = (uint64_t)batch * heads;
  if ((rc = make_tmap_3d_f16(&tq, q, 128, (uint64_t)seq_len, bh, 64, 128)) != LIGER_OK) return rc;
  if ((rc = make_tmap_3d_f16(&tk, k, 128, (uint64_t)seq_len, bh, 64, 128)) != LIGER_OK) return rc;
  if ((rc = make_tmap_3d_f16(&tv, v, 128, (uint64_t)seq_len, bh, 64, 128)) != LIGER_OK) return rc;
  LIGER_CUDA_TRY(cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes));
  const int grid = p.items < dev->sm_count ? p.items : dev->sm_count;
  attention_prefill_tc_kernel<<<grid, kTcThreads, kTcSmemBytes, stream>>>(tq, tk, tv, p);
  return check_launch("attention_prefill_tc_kernel");
}

}  // namespace liger
