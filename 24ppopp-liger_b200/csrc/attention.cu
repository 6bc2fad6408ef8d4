// Attention for sm_100a.
//
// Prefill: one kernel replaces the reference's QK^T batched GEMM, masked softmax, P*V batched GEMM
// and head-merge transpose (src/layer/bert_layer.h:145-168; src/cuda/attention_kernels.cu:543-573,
// 693-710).  Each CTA owns 64 query rows of one (batch, head); K/V stream through shared memory
// in 64-key blocks; scores stay in registers and the softmax is an online, warp-level one
// (running row max / row sum kept per quad of lanes), in fp32.
//
// Decode: one query token per sequence against a KV cache, split over the KV length so that the
// cache streams at HBM rate; a second kernel merges the split partials.
#include <cstdlib>
#include <mutex>

#include "runtime.h"

namespace liger {

// ---- mma.sync / ldmatrix helpers -----------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kBr = 64;  // query rows per CTA
constexpr int kBc = 64;  // keys per block
constexpr int kAttnThreads = 128;

// element offset of (row, col) in a [rows][D] fp16 tile whose 16-byte chunks are XOR-swizzled by row
template <int D>
__device__ __forceinline__ int swz(int row, int col) {
  return row * D + ((((col >> 3) ^ (row & 7)) << 3) | (col & 7));
}

// asynchronous copy of a [64][D] tile (rows r0.. of a [nrows][D] matrix, zero-filled past nrows) into
// shared memory: 16-byte cp.async per chunk, completion tracked by the caller's commit / wait groups
template <int D>
__device__ __forceinline__ void load_tile_async(__half* s, const __half* __restrict__ g, int r0, int nrows) {
  constexpr int CPR = D / 8;
  for (int i = threadIdx.x; i < 64 * CPR; i += kAttnThreads) {
    const int r = i / CPR, c = i % CPR;
    const bool ok = r0 + r < nrows;
    const __half* src = ok ? g + (size_t)(r0 + r) * D + c * 8 : g;
    const uint32_t dst = smem_u32(s + swz<D>(r, c * 8));
    const int bytes = ok ? 16 : 0;  // src-size 0: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
  }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D>
__global__ void __launch_bounds__(kAttnThreads)
attention_prefill_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                         const __half* __restrict__ mask, __half* __restrict__ out, int S, int heads, int ldo,
                         float scale, int causal) {
  extern __shared__ __align__(16) uint8_t smem_attn[];
  __half* sQ = reinterpret_cast<__half*>(smem_attn);
  __half* sKbuf = sQ + kBr * D;           // two K stages
  __half* sVbuf = sKbuf + 2 * kBc * D;    // two V stages

  const int q0 = blockIdx.x * kBr;
  const int head = blockIdx.y;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const size_t bh = ((size_t)b * heads + head) * (size_t)S * D;
  const __half* qg = q + bh;
  const __half* kg = k + bh;
  const __half* vg = v + bh;

  int nblocks = (S + kBc - 1) / kBc;
  if (causal && mask == nullptr) {
    const int last = (q0 + kBr - 1) / kBc + 1;  // blocks past the diagonal contribute exp(-10000 - max) == 0
    if (last < nblocks) nblocks = last;
  }
  // prologue: Q and the first K/V block in flight together
  load_tile_async<D>(sQ, qg, q0, S);
  load_tile_async<D>(sKbuf, kg, 0, S);
  load_tile_async<D>(sVbuf, vg, 0, S);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  // Q fragments for this warp's 16 rows
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int row = warp * 16 + (lane & 15);
    const int col = kk * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qf[kk], smem_u32(sQ + swz<D>(row, col)));
  }

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};

  for (int jb = 0; jb < nblocks; ++jb) {
    // double buffering: block jb sits in stage jb & 1; start fetching block jb + 1 into the other stage
    // (every warp finished reading that stage at the barrier that ended iteration jb - 1)
    const __half* sK = sKbuf + (jb & 1) * kBc * D;
    const __half* sV = sVbuf + (jb & 1) * kBc * D;
    if (jb + 1 < nblocks) {
      load_tile_async<D>(sKbuf + ((jb + 1) & 1) * kBc * D, kg, (jb + 1) * kBc, S);
      load_tile_async<D>(sVbuf + ((jb + 1) & 1) * kBc * D, vg, (jb + 1) * kBc, S);
    }
    cp_async_commit();
    if (jb > 0) {
      cp_async_wait<1>();  // everything but the group just committed has landed: block jb is complete
      __syncthreads();
    }

    float s[kBc / 8][4];
#pragma unroll
    for (int j = 0; j < kBc / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int jp = 0; jp < kBc / 16; ++jp) {
        uint32_t kf[4];
        const int row = jp * 16 + (lane & 7) + (lane >> 4) * 8;
        const int col = kk * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(kf, smem_u32(sK + swz<D>(row, col)));
        mma_16816(s[2 * jp], qf[kk], kf[0], kf[1]);
        mma_16816(s[2 * jp + 1], qf[kk], kf[2], kf[3]);
      }
    }

    // scale, mask, running max
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < kBc / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int qi = q0 + warp * 16 + g + r * 8;
        const int kj = jb * kBc + j * 8 + 2 * t + (e & 1);
        float x = s[j][e] * scale;
        if (kj >= S) {
          x = -INFINITY;
        } else if (mask != nullptr) {
          if (qi < S) x += (1.0f - __half2float(__ldg(mask + ((size_t)b * S + qi) * S + kj))) * -10000.0f;
        } else if (causal && kj > qi) {
          x += -10000.0f;
        }
        s[j][e] = x;
        mx[r] = fmaxf(mx[r], x);
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      alpha[r] = __expf(m_run[r] - m_new);
      m_run[r] = m_new;
      l_run[r] *= alpha[r];
    }
#pragma unroll
    for (int j = 0; j < kBc / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float p = __expf(s[j][e] - m_run[r]);
        s[j][e] = p;
        l_run[r] += p;
      }
    }
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
      o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
    }

    // O += P * V
#pragma unroll
    for (int kk = 0; kk < kBc / 16; ++kk) {
      uint32_t pf[4];
      pf[0] = pack_half2(s[2 * kk][0], s[2 * kk][1]);
      pf[1] = pack_half2(s[2 * kk][2], s[2 * kk][3]);
      pf[2] = pack_half2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pf[3] = pack_half2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t vf[4];
        const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int col = dp * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vf, smem_u32(sV + swz<D>(row, col)));
        mma_16816(o[2 * dp], pf, vf[0], vf[1]);
        mma_16816(o[2 * dp + 1], pf, vf[2], vf[3]);
      }
    }
    __syncthreads();  // all warps are done with stage jb & 1 before iteration jb + 1 refills it
  }
  cp_async_wait<0>();

  // normalise: p = exp(t - max) / (sum + 1e-6)   (src/cuda/attention_kernels.cu:567-568)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float inv = 1.0f / (l + 1e-6f);
    const int qi = q0 + warp * 16 + g + r * 8;
    if (qi < S) {
      __half* dst = out + ((size_t)b * S + qi) * ldo + head * D;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t) = pack_half2(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
      }
    }
  }
}

// ---- decode ---------------------------------------------------------------------------------------
constexpr int kDecThreads = 128;
constexpr int kDecChunk = 256;  // keys per CTA

__host__ __device__ inline int decode_splits(int kv_len) { return (kv_len + kDecChunk - 1) / kDecChunk; }

// partial layout per (b, head, split): [m, l, acc[D]] floats
template <int D, int U>
__global__ void __launch_bounds__(kDecThreads)
attention_decode_partial_kernel(const __half* __restrict__ q, const __half* __restrict__ kc, const __half* __restrict__ vc,
                                float* __restrict__ scratch, int heads, int kv_len, int kv_stride, float scale) {
  constexpr int LPK = D / 8;        // lanes per key (16 B each)
  constexpr int KPW = 32 / LPK;     // keys per warp per step
  __shared__ float s_m[kDecThreads / 32][KPW];
  __shared__ float s_l[kDecThreads / 32][KPW];
  __shared__ float s_acc[kDecThreads / 32][KPW][D];

  const int split = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int nsplit = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK, li = lane % LPK;
  const size_t bh = (size_t)b * heads + head;
  const __half* kbase = kc + bh * (size_t)kv_stride * D;
  const __half* vbase = vc + bh * (size_t)kv_stride * D;

  float qv[8];
  {
    uint4 u = __ldg(reinterpret_cast<const uint4*>(q + bh * D + li * 8));
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __half22float2(h[j]);
      qv[2 * j] = f.x * scale;
      qv[2 * j + 1] = f.y * scale;
    }
  }
  float m = -INFINITY, l = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int k_begin = split * kDecChunk;
  const int k_end = min(kv_len, k_begin + kDecChunk);
  // Every lane of a warp runs the same number of steps (the shuffles need the full warp).  A step
  // fetches U keys and values per lane group before it uses any of them -- U x 32 bytes in flight per
  // thread is what keeps HBM busy -- and folds them into the running state with one rescale.
  constexpr int STEP = (kDecThreads / 32) * KPW;  // keys the CTA covers per unrolled slot
  for (int base = k_begin + warp * KPW; base < k_end; base += STEP * U) {
    uint4 ku[U], vu[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int key = base + u * STEP + sub;
      valid[u] = key < k_end;
      ku[u] = make_uint4(0, 0, 0, 0);
      vu[u] = make_uint4(0, 0, 0, 0);
      if (valid[u]) {
        ku[u] = __ldcs(reinterpret_cast<const uint4*>(kbase + (size_t)key * D + li * 8));
        vu[u] = __ldcs(reinterpret_cast<const uint4*>(vbase + (size_t)key * D + li * 8));
      }
    }
    float dot[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const __half2* kh = reinterpret_cast<const __half2*>(&ku[u]);
      float d = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __half22float2(kh[j]);
        d += qv[2 * j] * f.x + qv[2 * j + 1] * f.y;
      }
      dot[u] = d;
    }
#pragma unroll
    for (int o = LPK / 2; o > 0; o >>= 1) {
#pragma unroll
      for (int u = 0; u < U; ++u) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
    }
    float m_new = m;
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (valid[u]) m_new = fmaxf(m_new, dot[u]);
    if (m_new != -INFINITY) {  // false only while this lane group has seen no key at all
      const float alpha = (m == -INFINITY) ? 0.0f : __expf(m - m_new);
      float pr[U], psum = 0.0f;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        pr[u] = valid[u] ? __expf(dot[u] - m_new) : 0.0f;
        psum += pr[u];
      }
      l = l * alpha + psum;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= alpha;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const __half2* vh = reinterpret_cast<const __half2*>(&vu[u]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __half22float2(vh[j]);
          acc[2 * j] += pr[u] * f.x;
          acc[2 * j + 1] += pr[u] * f.y;
        }
      }
      m = m_new;
    }
  }
  if (li == 0) { s_m[warp][sub] = m; s_l[warp][sub] = l; }
#pragma unroll
  for (int j = 0; j < 8; ++j) s_acc[warp][sub][li * 8 + j] = acc[j];
  __syncthreads();
  // merge the (warps x KPW) partial states; thread d < D owns one output column
  if (threadIdx.x < D) {
    float mm = -INFINITY;
    for (int w = 0; w < kDecThreads / 32; ++w)
      for (int s2 = 0; s2 < KPW; ++s2) mm = fmaxf(mm, s_m[w][s2]);
    float ll = 0.0f, a = 0.0f;
    for (int w = 0; w < kDecThreads / 32; ++w)
      for (int s2 = 0; s2 < KPW; ++s2) {
        const float mw = s_m[w][s2];
        const float sc = (mw == -INFINITY) ? 0.0f : __expf(mw - mm);
        ll += s_l[w][s2] * sc;
        a += s_acc[w][s2][threadIdx.x] * sc;
      }
    float* dst = scratch + (bh * nsplit + split) * (size_t)(D + 2);
    if (threadIdx.x == 0) { dst[0] = mm; dst[1] = ll; }
    dst[2 + threadIdx.x] = a;
  }
}

template <int D>
__global__ void attention_decode_merge_kernel(const float* __restrict__ scratch, __half* __restrict__ out, int heads,
                                              int nsplit, int ldo) {
  const int head = blockIdx.x, b = blockIdx.y;
  const size_t bh = (size_t)b * heads + head;
  const float* src = scratch + bh * nsplit * (size_t)(D + 2);
  const int d = threadIdx.x;
  float mm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, src[(size_t)s * (D + 2)]);
  float ll = 0.0f, a = 0.0f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = src[(size_t)s * (D + 2)];
    const float sc = (ms == -INFINITY) ? 0.0f : __expf(ms - mm);
    ll += src[(size_t)s * (D + 2) + 1] * sc;
    a += src[(size_t)s * (D + 2) + 2 + d] * sc;
  }
  out[(size_t)b * ldo + head * D + d] = __float2half_rn(a / (ll + 1e-6f));
}

// Keys each lane group fetches before it uses them (LIGER_DEC_UNROLL = 1, 2, 4 or 8 overrides the default).
static int decode_unroll() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LIGER_DEC_UNROLL");
    const int u = e ? atoi(e) : 4;
    v = (u == 1 || u == 2 || u == 4 || u == 8) ? u : 4;
  }
  return v;
}

template <int D>
static void launch_decode_partial(dim3 grid, cudaStream_t s, const __half* q, const __half* kc, const __half* vc, float* scratch,
                                  int heads, int kv_len, int kv_stride, float scale) {
  switch (decode_unroll()) {
    case 1: attention_decode_partial_kernel<D, 1><<<grid, kDecThreads, 0, s>>>(q, kc, vc, scratch, heads, kv_len, kv_stride, scale); break;
    case 2: attention_decode_partial_kernel<D, 2><<<grid, kDecThreads, 0, s>>>(q, kc, vc, scratch, heads, kv_len, kv_stride, scale); break;
    case 8: attention_decode_partial_kernel<D, 8><<<grid, kDecThreads, 0, s>>>(q, kc, vc, scratch, heads, kv_len, kv_stride, scale); break;
    default: attention_decode_partial_kernel<D, 4><<<grid, kDecThreads, 0, s>>>(q, kc, vc, scratch, heads, kv_len, kv_stride, scale); break;
  }
}

// attention_sm100.cu: the tcgen05 kernel (head_dim 128, no mask tensor)
int launch_attention_prefill_tc(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len,
                                int ldo, float scale, int causal, cudaStream_t stream);
static bool tc_attention_enabled() {
  static int on = -1;  // LIGER_ATTN_TC=0 keeps every shape on the mma.sync kernel
  if (on < 0) { const char* e = getenv("LIGER_ATTN_TC"); on = (e && atoi(e) == 0) ? 0 : 1; }
  return on != 0;
}

template <int D>
static int launch_prefill(const void* q, const void* k, const void* v, const void* mask, void* out, int batch, int heads,
                          int S, int ldo, float scale, int causal, cudaStream_t stream) {
  const int smem = (kBr + 4 * kBc) * D * 2;
  LIGER_CUDA_TRY(cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((S + kBr - 1) / kBr, heads, batch);
  attention_prefill_kernel<D><<<grid, kAttnThreads, smem, stream>>>((const __half*)q, (const __half*)k, (const __half*)v,
                                                                   (const __half*)mask, (__half*)out, S, heads, ldo,
                                                                   scale, causal);
  return check_launch("attention_prefill_kernel");
}

}  // namespace liger

using namespace liger;

extern "C" int liger_attention_prefill(const void* q, const void* k, const void* v, const void* mask, void* out, int batch,
                                       int heads, int seq_len, int head_dim, int ldo, float scale, int causal,
                                       void* stream) {
  if (!q || !k || !v || !out || batch <= 0 || heads <= 0 || seq_len <= 0)
    return set_error(LIGER_ERR_INVALID, "attention_prefill: bad argument");
  if (ldo < heads * head_dim || ldo % 2) return set_error(LIGER_ERR_INVALID, "attention_prefill: ldo must be even and >= heads*head_dim");
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15u || ((uintptr_t)out & 3u))
    return set_error(LIGER_ERR_INVALID, "attention_prefill: q/k/v must be 16-byte aligned");
  if (batch > 65535 || heads > 65535) return set_error(LIGER_ERR_UNSUPPORTED, "attention_prefill: batch, heads <= 65535");
  if (!current_device()) return LIGER_ERR_CUDA;
  cudaStream_t s = (cudaStream_t)stream;
  if (head_dim == 128 && mask == nullptr && seq_len >= 128 && tc_attention_enabled()) {
    const int rc = launch_attention_prefill_tc(q, k, v, out, batch, heads, seq_len, ldo, scale, causal, s);
    if (rc != LIGER_ERR_UNSUPPORTED) return rc;
  }
  if (head_dim == 64) return launch_prefill<64>(q, k, v, mask, out, batch, heads, seq_len, ldo, scale, causal, s);
  if (head_dim == 128) return launch_prefill<128>(q, k, v, mask, out, batch, heads, seq_len, ldo, scale, causal, s);
  return set_error(LIGER_ERR_UNSUPPORTED, "attention_prefill: head_dim %d (64 and 128 are implemented)", head_dim);
}

extern "C" size_t liger_attention_decode_scratch_bytes(int batch, int heads, int head_dim, int kv_len) {
  if (batch <= 0 || heads <= 0 || head_dim <= 0 || kv_len <= 0) return 0;
  return (size_t)batch * heads * decode_splits(kv_len) * (size_t)(head_dim + 2) * sizeof(float);
}

extern "C" int liger_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, void* scratch,
                                      int batch, int heads, int kv_len, int kv_stride, int head_dim, int ldo, float scale,
                                      void* stream) {
  if (!q || !k_cache || !v_cache || !out || !scratch || batch <= 0 || heads <= 0 || kv_len <= 0 || kv_stride < kv_len)
    return set_error(LIGER_ERR_INVALID, "attention_decode: bad argument");
  if (head_dim <= 0 || ldo < heads * head_dim)
    return set_error(LIGER_ERR_INVALID, "attention_decode: ldo = %d must be >= heads * head_dim = %d", ldo, heads * head_dim);
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15u)
    return set_error(LIGER_ERR_INVALID, "attention_decode: q / caches must be 16-byte aligned");
  if (((uintptr_t)scratch & 3u) || ((uintptr_t)out & 1u))
    return set_error(LIGER_ERR_INVALID, "attention_decode: scratch must be 4-byte aligned, out 2-byte aligned");
  if (batch > 65535 || heads > 65535) return set_error(LIGER_ERR_UNSUPPORTED, "attention_decode: batch, heads <= 65535");
  if (!current_device()) return LIGER_ERR_CUDA;
  cudaStream_t s = (cudaStream_t)stream;
  const int ns = decode_splits(kv_len);
  dim3 grid(ns, heads, batch), mgrid(heads, batch);
  if (head_dim == 128) {
    launch_decode_partial<128>(grid, s, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, (float*)scratch, heads, kv_len,
                               kv_stride, scale);
    int rc = check_launch("attention_decode_partial_kernel");
    if (rc != LIGER_OK) return rc;
    attention_decode_merge_kernel<128><<<mgrid, 128, 0, s>>>((const float*)scratch, (__half*)out, heads, ns, ldo);
  } else if (head_dim == 64) {
    launch_decode_partial<64>(grid, s, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, (float*)scratch, heads, kv_len,
                               kv_stride, scale);
    int rc = check_launch("attention_decode_partial_kernel");
    if (rc != LIGER_OK) return rc;
    attention_decode_merge_kernel<64><<<mgrid, 64, 0, s>>>((const float*)scratch, (__half*)out, heads, ns, ldo);
  } else {
    return set_error(LIGER_ERR_UNSUPPORTED, "attention_decode: head_dim %d (64 and 128 are implemented)", head_dim);
  }
  return check_launch("attention_decode_merge_kernel");
}


// ---- decode attention without any allocation ---------------------------------------------------------
// Split-KV partials of liger_attention_decode_noalloc live in this file-scope device array instead of
// caller-provided scratch.  Every device that loads the library holds these 16 MiB until the process
// exits.  All calls on a device share it.
namespace liger {
constexpr size_t kStaticScratchFloats = (size_t)4 << 20;  // 4 Mi floats = 16 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

constexpr int kStaticMaxDevices = 64;
static float* g_decode_scratch_addr[kStaticMaxDevices];  // device address of the array, per device
static std::mutex g_decode_scratch_mu;

// Device address of g_decode_scratch on the current device.  In host code the array's name is only a
// handle: the address a kernel can use has to be asked for, once per device, with that device current.
static int static_scratch_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices)
    return set_error(LIGER_ERR_CUDA, "attention_decode_noalloc: no usable CUDA device: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lk(g_decode_scratch_mu);
  if (g_decode_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return set_error(LIGER_ERR_CUDA, "attention_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                       cudaGetErrorString(e));
    }
    g_decode_scratch_addr[dev] = (float*)p;
  }
  *out = g_decode_scratch_addr[dev];
  return LIGER_OK;
}
}  // namespace liger

extern "C" size_t liger_attention_decode_noalloc_max_bytes(void) { return liger::kStaticScratchFloats * sizeof(float); }

extern "C" int liger_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, int batch,
                                              int heads, int kv_len, int kv_stride, int head_dim, int ldo, float scale,
                                              void* stream) {
  if (!q || !k_cache || !v_cache || !out || batch <= 0 || heads <= 0 || kv_len <= 0 || kv_stride < kv_len)
    return set_error(LIGER_ERR_INVALID, "attention_decode_noalloc: bad argument");
  if (head_dim != 64 && head_dim != 128)
    return set_error(LIGER_ERR_UNSUPPORTED, "attention_decode_noalloc: head_dim %d (64 and 128 are implemented)", head_dim);
  if (ldo < heads * head_dim)
    return set_error(LIGER_ERR_INVALID, "attention_decode_noalloc: ldo = %d must be >= heads * head_dim = %d", ldo,
                     heads * head_dim);
  if ((uintptr_t)out & 1u) return set_error(LIGER_ERR_INVALID, "attention_decode_noalloc: out must be 2-byte aligned");
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15u)
    return set_error(LIGER_ERR_INVALID, "attention_decode_noalloc: q / caches must be 16-byte aligned");
  if (batch > 65535 || heads > 65535) return set_error(LIGER_ERR_UNSUPPORTED, "attention_decode_noalloc: batch, heads <= 65535");
  const size_t need = liger_attention_decode_scratch_bytes(batch, heads, head_dim, kv_len);
  if (need > kStaticScratchFloats * sizeof(float))
    return set_error(LIGER_ERR_TOO_LARGE,
                     "attention_decode_noalloc: batch %d x heads %d x kv_len %d needs %zu bytes of split-KV partials; the built-in "
                     "buffer holds %zu (use liger_attention_decode with caller scratch)",
                     batch, heads, kv_len, need, kStaticScratchFloats * sizeof(float));
  float* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != LIGER_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int ns = decode_splits(kv_len);
  dim3 grid(ns, heads, batch), mgrid(heads, batch);
  // every partial that the merge kernel reads is written by the partial kernel of the same call, so
  // nothing left over from an earlier call is ever consumed and nothing needs clearing
  if (head_dim == 128) {
    launch_decode_partial<128>(grid, s, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, scratch, heads, kv_len,
                               kv_stride, scale);
    if ((rc = check_launch("attention_decode_partial_kernel")) != LIGER_OK) return rc;
    attention_decode_merge_kernel<128><<<mgrid, 128, 0, s>>>(scratch, (__half*)out, heads, ns, ldo);
  } else {
    launch_decode_partial<64>(grid, s, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, scratch, heads, kv_len,
                               kv_stride, scale);
    if ((rc = check_launch("attention_decode_partial_kernel")) != LIGER_OK) return rc;
    attention_decode_merge_kernel<64><<<mgrid, 64, 0, s>>>(scratch, (__half*)out, heads, ns, ldo);
  }
  return check_launch("attention_decode_merge_kernel");
}
