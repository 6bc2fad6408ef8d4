// Shared by the 1-CTA and 2-CTA tcgen05 GEMM kernels: launch parameters and the epilogue (TMEM ->
// registers -> bias / activation -> shared-memory staging -> row-contiguous 16-byte stores).
#pragma once
#include "comm_internal.h"
#include "runtime.h"

namespace liger {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kGemmThreads = 192;
constexpr int kTmOrderMax = 128;  // row tiles a launch may have for the arrival-order walk (otherwise: plain order)

struct GemmParams {
  __half* c;
  const __half* bias;
  const __half* residual;
  __half* qkv[3];
  int m, n_begin, n_end;
  int ldc, ldr;
  int epilogue;
  int seq_len, heads, head_dim;
  int kv_stride, kv_pos;
  int tiles_m, tiles_n, kblocks;
  // Tile order (see tile_coords): the smaller-footprint operand is kept L2-resident in panels
  int panel_tiles;   // tiles of the stationary operand per panel
  int stationary;    // 0: panels over M (A rows stay in L2, W^T streams), 1: panels over N
  int use_hints;     // 1: L2 eviction-priority hints on the TMA loads
  // LIGER_EPI_SCATTER: row r goes to rank r / rows_per_rank, into that rank's receive slot for this rank
  uint8_t* peer[kMaxRanks];
  size_t scatter_off;
  int rank, rows_per_rank;
  // 256x512 kernel: tiles [tail_start, tiles) form the last, partly filled wave; with tail_split they
  // run as 256x256 halves, one per CTA pair, which ends that wave in half the time
  int tail_start, tail_split;
  // A is the result of an all-gather that may still be in flight (liger_allgather_push): row block b of rank o has
  // landed when word b of flag line o of ready_flags holds ready_epoch or more.  Row tiles are visited in the
  // order tm_order[] (own rows first, then in arrival order) instead of 0, 1, 2, ...
  const uint32_t* ready_flags;  // nullptr: A is complete
  uint32_t ready_epoch;
  int ready_rpr, ready_rank, ready_block_rows;
  int tm_order_on;
  int no_wide;  // host only: keep this launch off the 256x512 kernel
  uint8_t tm_order[kTmOrderMax];
  DeviceStatus* status;
};

// The TMA producer of a tile calls this before its first load of A rows [m0, m0 + rows): waits (bounded) until
// the ranks that own those rows have delivered them.  The flags are written by another GPU's kernel with a
// system-scope release after its data stores; the acquire load here, followed by a proxy fence, orders this
// thread's TMA loads (async proxy) behind them.
__device__ __forceinline__ bool wait_rows_ready(const GemmParams& p, int m0, int rows, volatile uint32_t* abort_flag) {
  if (p.ready_flags == nullptr || m0 >= p.m) return true;
  const int last = (m0 + rows < p.m ? m0 + rows : p.m) - 1;
  bool waited = false;
  for (int row = m0;;) {
    const int owner = row / p.ready_rpr;
    const int blk = (row - owner * p.ready_rpr) / p.ready_block_rows;
    if (owner != p.ready_rank) {
      const uint32_t* f = p.ready_flags + (size_t)owner * kFlagStrideWords + blk;
      unsigned long long t0 = 0;
      uint32_t spins = 0;
      while ((int32_t)(ld_acquire_sys(f) - p.ready_epoch) < 0) {
        if ((++spins & 0x3fu) == 0) {
          if (*abort_flag) return false;
          const unsigned long long now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > g_wait_budget_ns) { *abort_flag = 1u; return false; }
        }
      }
      waited = true;
    }
    // first row of the next (owner, block) piece
    const int next = owner * p.ready_rpr + (blk + 1) * p.ready_block_rows;
    const int next_owner = (owner + 1) * p.ready_rpr;
    row = next < next_owner ? next : next_owner;
    if (row > last) break;
  }
  if (waited) asm volatile("fence.proxy.async;" ::: "memory");
  return true;
}

// host side (gemm_sm100.cu): fills p.stationary / p.panel_tiles; and, for an A operand that is still being
// gathered, p.tm_order / p.tm_order_on
void choose_tile_order(GemmParams& p, const liger_gemm_args& a, int tile_m, int tile_n);
void choose_arrival_order(GemmParams& p, int tile_m);

// Tile t of the launch -> (m tile, n tile).  All CTAs walk K in step, so the DRAM traffic of a GEMM
// is decided by which operand rows the concurrently running tiles share and by what survives in L2
// from one wave to the next.  Tiles are ordered in panels of `panel_tiles` tiles of the stationary
// operand (sized on the host to about half of L2); inside a panel the stationary index runs
// fastest, so every wave re-uses the same resident panel while the other operand streams through
// once per panel.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int t, int& tm, int& tn) {
  if (p.stationary == 0) {
    const int per_panel = p.panel_tiles * p.tiles_n;
    const int panel = t / per_panel;
    const int within = t - panel * per_panel;
    const int rows = min(p.panel_tiles, p.tiles_m - panel * p.panel_tiles);  // last panel may be short
    tn = within / rows;
    tm = panel * p.panel_tiles + (within - tn * rows);
  } else {
    const int per_panel = p.panel_tiles * p.tiles_m;
    const int panel = t / per_panel;
    const int within = t - panel * per_panel;
    const int cols = min(p.panel_tiles, p.tiles_n - panel * p.panel_tiles);
    tm = within / cols;
    tn = panel * p.panel_tiles + (within - tm * cols);
  }
  if (p.tm_order_on) tm = p.tm_order[tm];
}

// L2 eviction-priority descriptors for TMA loads (the fixed encodings CUDA's createpolicy produces
// for fraction 1.0): the stationary operand is loaded evict_last, the streaming one evict_first.
constexpr uint64_t kL2EvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kL2EvictLast = 0x14F0000000000000ull;
constexpr uint64_t kL2EvictNormal = 0x1000000000000000ull;

// ---- epilogue helpers -------------------------------------------------------------------------
// 32 accumulator columns [col0, col0+32) of one row -> bias / activation -> 32 fp16 values in o[4].
__device__ __forceinline__ void epilogue_math(const GemmParams& p, int row, int col0, const uint32_t (&r)[32],
                                              uint4 (&o)[4]) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int col = col0 + g * 8;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]);
    if (col < p.n_end) {
      if (p.bias != nullptr) {
        float b[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.bias + col)), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += b[i];
      }
      if (p.epilogue == LIGER_EPI_GELU) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = gelu_tanh(v[i]);
      } else if (p.epilogue == LIGER_EPI_RESIDUAL) {
        float b[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.residual + (size_t)row * p.ldr + col)), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += b[i];
      }
    }
    o[g].x = pack_half2(v[0], v[1]);
    o[g].y = pack_half2(v[2], v[3]);
    o[g].z = pack_half2(v[4], v[5]);
    o[g].w = pack_half2(v[6], v[7]);
  }
}

// gate chunk (acc columns col0..col0+31) + value chunk (col0+32..col0+63) -> 32 outputs gelu(gate + b) * (value + b)
__device__ __forceinline__ void epilogue_math_geglu(const GemmParams& p, int col0, const uint32_t (&g)[32],
                                                    const uint32_t (&u)[32], uint4 (&o)[4]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float gv[8], uv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      gv[i] = __uint_as_float(g[q * 8 + i]);
      uv[i] = __uint_as_float(u[q * 8 + i]);
    }
    if (p.bias != nullptr && col0 < p.n_end) {
      float b[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(p.bias + col0 + q * 8)), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) gv[i] += b[i];
      unpack8(__ldg(reinterpret_cast<const uint4*>(p.bias + col0 + 32 + q * 8)), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) uv[i] += b[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) gv[i] = gelu_tanh(gv[i]) * uv[i];
    o[q].x = pack_half2(gv[0], gv[1]);
    o[q].y = pack_half2(gv[2], gv[3]);
    o[q].z = pack_half2(gv[4], gv[5]);
    o[q].w = pack_half2(gv[6], gv[7]);
  }
}

// Where 8 consecutive outputs of (row, out_col) go.  out_col is in output-column space (for GeGLU
// already halved).
__device__ __forceinline__ __half* epilogue_dst(const GemmParams& p, int row, int out_col) {
  if (p.epilogue == LIGER_EPI_QKV_SPLIT) {
    const int hd = p.heads * p.head_dim;
    const int which = out_col / hd;
    const int rem = out_col - which * hd;
    const int head = rem / p.head_dim;
    const int d = rem - head * p.head_dim;
    const int b = row / p.seq_len;
    const int s = row - b * p.seq_len;
    __half* base = which == 0 ? p.qkv[0] : which == 1 ? p.qkv[1] : p.qkv[2];
    if (which != 0 && p.kv_stride > 0)
      return base + (((size_t)b * p.heads + head) * p.kv_stride + p.kv_pos + s) * p.head_dim + d;
    return base + (((size_t)b * p.heads + head) * p.seq_len + s) * p.head_dim + d;
  }
  if (p.epilogue == LIGER_EPI_SCATTER) {
    const int owner = row / p.rows_per_rank;
    const int local_row = p.rank * p.rows_per_rank + (row - owner * p.rows_per_rank);
    return reinterpret_cast<__half*>(p.peer[owner] + p.scatter_off) + (size_t)local_row * p.ldc + out_col;
  }
  return p.c + (size_t)row * p.ldc + out_col;
}

// Per-warp staging tile in shared memory: 32 rows x W output columns (fp16), 16-byte chunks XOR-swizzled
// by row so that both the row-per-thread writes and the row-contiguous reads are conflict-light.
template <int W>
__device__ __forceinline__ uint4* stage_slot(uint8_t* stage, int r, int chunk) {
  constexpr int NCH = W / 8;                       // 16-byte chunks per row
  constexpr int MASK = (NCH < 8 ? NCH : 8) - 1;
  return reinterpret_cast<uint4*>(stage + (size_t)r * (W * 2) + (size_t)((chunk ^ (r & MASK)) * 16));
}

// Write the staged [32 x W] tile out with row-contiguous 16-byte stores: a warp instruction covers
// 32/NCH rows of W*2 contiguous bytes each (256 B for W = 128), which is what both HBM sectors and
// NVLink write packets want -- row-per-thread stores would issue 32 separate 16-byte writes.
template <int W>
__device__ __forceinline__ void stage_writeout(const GemmParams& p, uint8_t* stage, int row0, int out_col0, int out_end,
                                               int lane) {
  constexpr int NCH = W / 8;
#pragma unroll 4
  for (int i = 0; i < NCH; ++i) {
    const int idx = i * 32 + lane;
    const int r = idx / NCH, ch = idx % NCH;
    const int row = row0 + r, col = out_col0 + ch * 8;
    if (row < p.m && col < out_end) *reinterpret_cast<uint4*>(epilogue_dst(p, row, col)) = *stage_slot<W>(stage, r, ch);
  }
}


// Epilogue of one accumulator tile for one warp: TMEM lanes [taddr.lane, +32) x BN columns -> rows
// [row0, row0+32), accumulator columns [n0, n0+BN).  `stage` is this warp's staging tile.
template <int BN>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t taddr, uint8_t* stage, int row0, int n0,
                                              int lane) {
  constexpr int W = BN < 128 ? BN : 128;
  const int row = row0 + lane;
#pragma unroll 1
  for (int pass = 0; pass < BN / W; ++pass) {
    const int pcol0 = n0 + pass * W;  // first accumulator column of this pass
    if (pcol0 >= p.n_end) break;
    if (p.epilogue == LIGER_EPI_GEGLU) {
      if constexpr (W >= 64) {
#pragma unroll 1
        for (int c = 0; c < W / 64; ++c) {
          const int col0 = pcol0 + c * 64;
          if (col0 >= p.n_end) break;
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + pass * W + c * 64, g);
          tmem_ld_32x32(taddr + pass * W + c * 64 + 32, u);
          tmem_ld_wait();
          uint4 o[4];
          epilogue_math_geglu(p, col0, g, u, o);
#pragma unroll
          for (int j = 0; j < 4; ++j) *stage_slot<W / 2>(stage, lane, c * 4 + j) = o[j];
        }
        __syncwarp();
        stage_writeout<W / 2>(p, stage, row0, pcol0 >> 1, p.n_end >> 1, lane);
      }
    } else {
#pragma unroll 1
      for (int c = 0; c < W / 32; ++c) {
        const int col0 = pcol0 + c * 32;
        if (col0 >= p.n_end) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + pass * W + c * 32, r);
        tmem_ld_wait();
        uint4 o[4];
        epilogue_math(p, row < p.m ? row : 0, col0, r, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) *stage_slot<W>(stage, lane, c * 4 + j) = o[j];
      }
      __syncwarp();
      stage_writeout<W>(p, stage, row0, pcol0, p.n_end, lane);
    }
    __syncwarp();  // the staging tile is reused by the next pass
  }
}

// ---- pipelined epilogue ------------------------------------------------------------------------------
// Used where the epilogue is not hidden behind the next tile's MMAs (the 256x512 kernel, whose tile
// owns all of TMEM).  Differences from epilogue_tile: the TMEM load (and the residual load) of unit
// u+1 is in flight while unit u is converted; the bias lines are prefetched into L1 before the accumulator
// is ready and read with broadcast loads; destination addresses are split into a per-lane column part computed once
// per pass and a row part advanced without divisions.

// Staged [32 x 64] output tile -> global memory; a warp instruction stores 4 rows of 128 contiguous bytes.
template <int EPI>
__device__ __forceinline__ void stage_writeout64(const GemmParams& p, uint8_t* stage, int row0, int out_col0, int out_end,
                                                 int lane) {
  const int ch = lane & 7, rsub = lane >> 3;
  const int col = out_col0 + ch * 8;
  if (col >= out_end) return;
  int row = row0 + rsub;
  if constexpr (EPI == LIGER_EPI_QKV_SPLIT) {
    const int hd = p.heads * p.head_dim;
    const int which = col / hd;
    const int rem = col - which * hd;
    const int head = rem / p.head_dim;
    const int d = rem - head * p.head_dim;
    const bool cache = which != 0 && p.kv_stride > 0;
    const size_t S = cache ? (size_t)p.kv_stride : (size_t)p.seq_len;
    __half* base = (which == 0 ? p.qkv[0] : which == 1 ? p.qkv[1] : p.qkv[2]) +
                   ((size_t)head * S + (cache ? (size_t)p.kv_pos : 0)) * p.head_dim + d;
    // rows advance by 4: the destination moves by 4 tokens inside a sequence and jumps to the next
    // batch entry's block when the sequence ends
    const int b = row / p.seq_len;
    int s = row - b * p.seq_len;
    const size_t batch_step = (size_t)p.heads * S * p.head_dim;
    __half* dst = base + (size_t)b * batch_step + (size_t)s * p.head_dim;
    const int row_step = 4 * p.head_dim;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (row < p.m) *reinterpret_cast<uint4*>(dst) = *stage_slot<64>(stage, rsub + i * 4, ch);
      row += 4;
      s += 4;
      dst += row_step;
      while (s >= p.seq_len) {
        s -= p.seq_len;
        dst += batch_step - (size_t)p.seq_len * p.head_dim;
      }
    }
  } else if constexpr (EPI == LIGER_EPI_SCATTER) {
    int owner = row / p.rows_per_rank, lr = row - owner * p.rows_per_rank;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (row < p.m)
        *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.peer[owner] + p.scatter_off) +
                                  (size_t)(p.rank * p.rows_per_rank + lr) * p.ldc + col) =
            *stage_slot<64>(stage, rsub + i * 4, ch);
      row += 4;
      lr += 4;
      while (lr >= p.rows_per_rank) { lr -= p.rows_per_rank; ++owner; }
    }
  } else {
    __half* dst = p.c + (size_t)row * p.ldc + col;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (row < p.m) *reinterpret_cast<uint4*>(dst) = *stage_slot<64>(stage, rsub + i * 4, ch);
      row += 4;
      dst += (size_t)4 * p.ldc;
    }
  }
}

// Bias of the warp's 256-column range: `ptr` points at its first column, groups (of 8 columns) at or past
// `groups` do not exist (past n_end, or no bias vector at all).  Every lane needs the same values, so a
// group is one broadcast 16-byte load; the lines are in L1 after epilogue_bias8's prefetch.  (Handing the
// values round with shuffles instead costs 16 shuffles per 32 columns and was a quarter of the epilogue.)
struct BiasRef {
  const __half* ptr;
  int groups;
};
__device__ __forceinline__ uint4 bias_group(const BiasRef& b, int group) {
  return group < b.groups ? __ldg(reinterpret_cast<const uint4*>(b.ptr) + group) : make_uint4(0u, 0u, 0u, 0u);
}

// 32 accumulator columns of one row (columns [cl, cl+32) of the warp's range) + bias [+ residual /
// GELU] -> 32 fp16 values
template <int EPI>
__device__ __forceinline__ void unit_math(const BiasRef& bias8, int cl, const uint32_t (&r)[32], const uint4 (&res)[4],
                                          uint4 (&o)[4]) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float v[8], b[8];
    unpack8(bias_group(bias8, (cl >> 3) + g), b);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]) + b[i];
    if constexpr (EPI == LIGER_EPI_GELU) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = gelu_tanh(v[i]);
    } else if constexpr (EPI == LIGER_EPI_RESIDUAL) {
      unpack8(res[g], b);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += b[i];
    }
    o[g].x = pack_half2(v[0], v[1]);
    o[g].y = pack_half2(v[2], v[3]);
    o[g].z = pack_half2(v[4], v[5]);
    o[g].w = pack_half2(v[6], v[7]);
  }
}

__device__ __forceinline__ void unit_math_geglu(const BiasRef& bias8, int cl, const uint32_t (&gt)[32],
                                                const uint32_t (&up)[32], uint4 (&o)[4]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float gv[8], uv[8], b[8];
    unpack8(bias_group(bias8, (cl >> 3) + q), b);
#pragma unroll
    for (int i = 0; i < 8; ++i) gv[i] = __uint_as_float(gt[q * 8 + i]) + b[i];
    unpack8(bias_group(bias8, (cl >> 3) + 4 + q), b);
#pragma unroll
    for (int i = 0; i < 8; ++i) uv[i] = __uint_as_float(up[q * 8 + i]) + b[i];
#pragma unroll
    for (int i = 0; i < 8; ++i) gv[i] = gelu_tanh(gv[i]) * uv[i];
    o[q].x = pack_half2(gv[0], gv[1]);
    o[q].y = pack_half2(gv[2], gv[3]);
    o[q].z = pack_half2(gv[4], gv[5]);
    o[q].w = pack_half2(gv[6], gv[7]);
  }
}

// Called before the accumulator is ready: touches the warp's bias lines (one 16-byte piece per lane) so that
// the broadcast loads of the epilogue proper hit in L1, and returns the reference the epilogue uses.
__device__ __forceinline__ BiasRef epilogue_bias8(const GemmParams& p, int n0, int lane) {
  BiasRef b;
  b.ptr = p.bias != nullptr ? p.bias + n0 : nullptr;
  b.groups = (p.bias != nullptr && n0 < p.n_end) ? min(32, (p.n_end - n0 + 7) >> 3) : 0;
  if (lane < b.groups) asm volatile("prefetch.global.L1 [%0];" ::"l"(b.ptr + lane * 8));
  return b;
}

// One warp's share of an accumulator: TMEM lanes [taddr.lane, +32) x 256 columns starting at
// accumulator column n0 -> rows [row0, row0+32).  `stage` is the warp's [32 x 64] staging tile,
// `bias8` the warp's bias reference (see epilogue_bias8).
template <int EPI>
__device__ __forceinline__ void epilogue_warp_pipelined(const GemmParams& p, uint32_t taddr, uint8_t* stage,
                                                        const BiasRef& bias8, int row0, int n0, int lane) {
  if (n0 >= p.n_end) return;
  const int row = row0 + lane;
  if constexpr (EPI == LIGER_EPI_GEGLU) {
    // unit = 32 gate + 32 value columns -> 32 outputs; two units fill the staging tile
    const int nu = min(4, (p.n_end - n0 + 63) / 64);
    uint32_t g0[32], u0[32], g1[32], u1[32];
    tmem_ld_32x32(taddr, g0);
    tmem_ld_32x32(taddr + 32, u0);
#pragma unroll 1
    for (int u = 0; u < nu; u += 2) {
      uint4 o[4];
      tmem_ld_wait_regs(g0);
      tmem_ld_wait_regs(u0);
      if (u + 1 < nu) {
        tmem_ld_32x32(taddr + (u + 1) * 64, g1);
        tmem_ld_32x32(taddr + (u + 1) * 64 + 32, u1);
      }
      unit_math_geglu(bias8, u * 64, g0, u0, o);
#pragma unroll
      for (int j = 0; j < 4; ++j) *stage_slot<64>(stage, lane, j) = o[j];
      if (u + 1 < nu) {
        tmem_ld_wait_regs(g1);
        tmem_ld_wait_regs(u1);
        if (u + 2 < nu) {
          tmem_ld_32x32(taddr + (u + 2) * 64, g0);
          tmem_ld_32x32(taddr + (u + 2) * 64 + 32, u0);
        }
        unit_math_geglu(bias8, (u + 1) * 64, g1, u1, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) *stage_slot<64>(stage, lane, 4 + j) = o[j];
      }
      __syncwarp();
      stage_writeout64<EPI>(p, stage, row0, (n0 + u * 64) >> 1, p.n_end >> 1, lane);
      __syncwarp();
    }
  } else {
    const int nu = min(8, (p.n_end - n0 + 31) / 32);
    uint32_t r0[32], r1[32];
    uint4 q[4] = {};
    // RESIDUAL: the residual tile of a pass (32 rows x 64 columns) is read with row-contiguous loads (4 rows x
    // 128 B per instruction, the write-out mapping) one pass ahead, parked in registers, and dropped into the
    // staging tile before the pass's math, which picks its row's values up from there.  Row-per-thread
    // loads would touch 32 lines per instruction and cost more than the rest of the epilogue together.
    uint4 rs[8];
    const int wch = lane & 7, wrsub = lane >> 3;
    auto load_residual = [&](int u) {  // pass starting at unit u
      if constexpr (EPI == LIGER_EPI_RESIDUAL) {
        const int col = n0 + u * 32 + wch * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = row0 + wrsub + i * 4;
          rs[i] = (rr < p.m && col < p.n_end) ? __ldg(reinterpret_cast<const uint4*>(p.residual + (size_t)rr * p.ldr + col))
                                              : make_uint4(0u, 0u, 0u, 0u);
        }
      }
    };
    load_residual(0);
    tmem_ld_32x32(taddr, r0);
#pragma unroll 1
    for (int u = 0; u < nu; u += 2) {
      uint4 o[4];
      if constexpr (EPI == LIGER_EPI_RESIDUAL) {
#pragma unroll
        for (int i = 0; i < 8; ++i) *stage_slot<64>(stage, wrsub + i * 4, wch) = rs[i];
        __syncwarp();
        if (u + 2 < nu) load_residual(u + 2);
      }
      tmem_ld_wait_regs(r0);
      if (u + 1 < nu) tmem_ld_32x32(taddr + (u + 1) * 32, r1);
      if constexpr (EPI == LIGER_EPI_RESIDUAL) {
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = *stage_slot<64>(stage, lane, j);
      }
      unit_math<EPI>(bias8, u * 32, r0, q, o);
#pragma unroll
      for (int j = 0; j < 4; ++j) *stage_slot<64>(stage, lane, j) = o[j];
      if (u + 1 < nu) {
        tmem_ld_wait_regs(r1);
        if (u + 2 < nu) tmem_ld_32x32(taddr + (u + 2) * 32, r0);
        if constexpr (EPI == LIGER_EPI_RESIDUAL) {
#pragma unroll
          for (int j = 0; j < 4; ++j) q[j] = *stage_slot<64>(stage, lane, 4 + j);
        }
        unit_math<EPI>(bias8, (u + 1) * 32, r1, q, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) *stage_slot<64>(stage, lane, 4 + j) = o[j];
      }
      __syncwarp();
      stage_writeout64<EPI>(p, stage, row0, n0 + u * 32, p.n_end, lane);
      __syncwarp();
    }
  }
}

}  // namespace liger
