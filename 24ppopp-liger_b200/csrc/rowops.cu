// HBM-bound row-wise operators and layout kernels: LayerNorm, residual + bias (+ LayerNorm),
// bias + GELU, bias + head split, head merge, weight transpose, seeded fill.
// All move 16 bytes per thread per access and keep a row in registers where a row is reused.
#include "../../include/liger_rng.h"
#include "runtime.h"

namespace liger {

constexpr int kLnThreads = 256;
constexpr int kLnMaxVec = 8;  // uint4 per thread held in registers -> rows up to 256*8*8 = 16384

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // protect `red` from the previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.0f;
  return warp_sum(t);
}

// y = LN(x); optionally x := in + x + bias first (stored back in fp16, then re-read as fp16 for
// the variance and the normalisation exactly as add_bias_input_layernorm_2 does,
// src/cuda/cuda_kernels.cu:360-409; plain LayerNorm follows :463-508).
template <bool kResidual>
__global__ void __launch_bounds__(kLnThreads)
layernorm_kernel(const __half* __restrict__ x_in, const __half* __restrict__ res_in, const __half* __restrict__ bias,
                 const __half* __restrict__ gamma, const __half* __restrict__ beta, __half* __restrict__ out_sum,
                 __half* __restrict__ y, int n) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nvec = n >> 3;
  const size_t base = (size_t)row * n;
  // The row stays in registers as the fp16 values it is (8 per uint4) and is widened on the fly in each of
  // the three passes: half the registers of an fp32 copy, twice the resident CTAs, same arithmetic.
  uint4 v[kLnMaxVec];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kLnMaxVec; ++i) {
    const int idx = threadIdx.x + i * kLnThreads;
    if (idx < nvec) {
      v[i] = *reinterpret_cast<const uint4*>(x_in + base + (size_t)idx * 8);
      if (kResidual) {
        float x[8], r[8], b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        unpack8(v[i], x);
        unpack8(__ldg(reinterpret_cast<const uint4*>(res_in + base + (size_t)idx * 8)), r);
        if (bias != nullptr) unpack8(__ldg(reinterpret_cast<const uint4*>(bias + (size_t)idx * 8)), b);
        uint32_t* ow = reinterpret_cast<uint32_t*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float t0 = r[2 * j] + x[2 * j] + b[2 * j];
          const float t1 = r[2 * j + 1] + x[2 * j + 1] + b[2 * j + 1];
          sum += t0 + t1;
          ow[j] = pack_half2(t0, t1);  // stored in fp16 and used from here on as the fp16 value
        }
        *reinterpret_cast<uint4*>(out_sum + base + (size_t)idx * 8) = v[i];
      } else {
        float x[8];
        unpack8(v[i], x);
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += x[j];
      }
    }
  }
  if (y == nullptr) return;
  const float mean = block_sum(sum, red) / (float)n;
  float vs = 0.0f;
#pragma unroll
  for (int i = 0; i < kLnMaxVec; ++i) {
    const int idx = threadIdx.x + i * kLnThreads;
    if (idx < nvec) {
      float x[8];
      unpack8(v[i], x);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = x[j] - mean;
        vs += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(vs, red) / (float)n + 1e-6f);
#pragma unroll
  for (int i = 0; i < kLnMaxVec; ++i) {
    const int idx = threadIdx.x + i * kLnThreads;
    if (idx < nvec) {
      float x[8], g[8], b[8];
      unpack8(v[i], x);
      unpack8(__ldg(reinterpret_cast<const uint4*>(gamma + (size_t)idx * 8)), g);
      unpack8(__ldg(reinterpret_cast<const uint4*>(beta + (size_t)idx * 8)), b);
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        ow[j] = pack_half2((x[2 * j] - mean) * rstd * g[2 * j] + b[2 * j], (x[2 * j + 1] - mean) * rstd * g[2 * j + 1] + b[2 * j + 1]);
      *reinterpret_cast<uint4*>(y + base + (size_t)idx * 8) = o;
    }
  }
}

// x = gelu(x + bias), 8 elements per thread (src/cuda/cuda_kernels.cu:71-84)
__global__ void add_bias_gelu_kernel(__half* __restrict__ x, const __half* __restrict__ bias, size_t total_vec, int nvec) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total_vec; i += (size_t)gridDim.x * blockDim.x) {
    uint4 u = *reinterpret_cast<uint4*>(x + i * 8);
    const int c = (int)(i % nvec);
    uint4 b = bias ? __ldg(reinterpret_cast<const uint4*>(bias + (size_t)c * 8)) : make_uint4(0, 0, 0, 0);
    const __half2* uh = reinterpret_cast<const __half2*>(&u);
    const __half2* bh = reinterpret_cast<const __half2*>(&b);
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __half22float2(uh[j]);
      float2 g = __half22float2(bh[j]);
      ow[j] = pack_half2(gelu_tanh(f.x + g.x), gelu_tanh(f.y + g.y));
    }
    *reinterpret_cast<uint4*>(x + i * 8) = o;
  }
}

// bias + head split for Q, K, V at once (src/cuda/attention_kernels.cu:133-163)
__global__ void add_qkv_bias_transpose_kernel(__half* __restrict__ qo, __half* __restrict__ ko, __half* __restrict__ vo,
                                              const __half* __restrict__ q, const __half* __restrict__ bq,
                                              const __half* __restrict__ k, const __half* __restrict__ bk,
                                              const __half* __restrict__ v, const __half* __restrict__ bv, int B, int S,
                                              int h, int D) {
  const int dv = D >> 3;
  const size_t total = (size_t)B * S * h * dv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total * 3; i += (size_t)gridDim.x * blockDim.x) {
    const int which = (int)(i / total);
    size_t r = i - (size_t)which * total;
    const int d8 = (int)(r % dv); r /= dv;
    const int hh = (int)(r % h); r /= h;
    const int s = (int)(r % S);
    const int b = (int)(r / S);
    const __half* src = which == 0 ? q : which == 1 ? k : v;
    const __half* bias = which == 0 ? bq : which == 1 ? bk : bv;
    __half* dst = which == 0 ? qo : which == 1 ? ko : vo;
    uint4 u = __ldg(reinterpret_cast<const uint4*>(src + ((size_t)b * S + s) * (size_t)(h * D) + hh * D + d8 * 8));
    uint4 bb = bias ? __ldg(reinterpret_cast<const uint4*>(bias + hh * D + d8 * 8)) : make_uint4(0, 0, 0, 0);
    const __half2* uh = reinterpret_cast<const __half2*>(&u);
    const __half2* bh = reinterpret_cast<const __half2*>(&bb);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __hadd2(uh[j], bh[j]);
    *reinterpret_cast<uint4*>(dst + (((size_t)b * h + hh) * S + s) * D + d8 * 8) = o;
  }
}

// head merge (src/cuda/attention_kernels.cu:693-710)
__global__ void transpose_heads_kernel(__half* __restrict__ dst, const __half* __restrict__ src, int B, int S, int h,
                                       int D) {
  const int dv = D >> 3;
  const size_t total = (size_t)B * S * h * dv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i;
    const int d8 = (int)(r % dv); r /= dv;
    const int hh = (int)(r % h); r /= h;
    const int s = (int)(r % S);
    const int b = (int)(r / S);
    uint4 u = __ldg(reinterpret_cast<const uint4*>(src + (((size_t)b * h + hh) * S + s) * D + d8 * 8));
    *reinterpret_cast<uint4*>(dst + ((size_t)b * S + s) * (size_t)(h * D) + hh * D + d8 * 8) = u;
  }
}

// dst[n][k] = src[k][n] through a 32x32 shared-memory tile; optional 32-row block interleave
__global__ void transpose_weight_kernel(const __half* __restrict__ src, __half* __restrict__ dst, int K, int N,
                                        int interleave32) {
  __shared__ __half tile[32][34];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int k = k0 + i, n = n0 + threadIdx.x;
    tile[i][threadIdx.x] = (k < K && n < N) ? src[(size_t)k * N + n] : __float2half(0.0f);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int n = n0 + i, k = k0 + threadIdx.x;
    if (n < N && k < K) {
      int row = n;
      if (interleave32) {
        const int half_n = N >> 1;
        const int hsel = n >= half_n ? 1 : 0;
        const int j = n - hsel * half_n;
        row = (j >> 5) * 64 + hsel * 32 + (j & 31);
      }
      dst[(size_t)row * K + k] = tile[threadIdx.x][i];
    }
  }
}

// seeded fill; mode: 0 plain, 1 transposed, 2 / 3 transposed into the gate / value rows of the
// 32-row interleaved layout
__global__ void fill_normal_kernel(__half* __restrict__ dst, int rows, int cols, int dst_ld, int row0, int col0, int src_ld,
                                   uint32_t seed, uint32_t tensor_id, float mean, float std, int mode) {
  const size_t total = (size_t)rows * cols;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    int r, c;
    size_t off;
    if (mode == 0) {
      r = (int)(i / cols);
      c = (int)(i % cols);
      off = (size_t)r * dst_ld + c;
    } else {
      c = (int)(i / rows);
      r = (int)(i % rows);
      int orow = c;
      if (mode >= 2) orow = (c >> 5) * 64 + (mode == 3 ? 32 : 0) + (c & 31);
      off = (size_t)orow * dst_ld + r;
    }
    const uint64_t idx = (uint64_t)(row0 + r) * (uint64_t)src_ld + (uint64_t)(col0 + c);
    reinterpret_cast<uint16_t*>(dst)[off] = lg_normal_half_bits(seed, tensor_id, idx, mean, std);
  }
}

static inline int grid_for(size_t work_items, int threads, int sm_count) {
  size_t blocks = (work_items + threads - 1) / threads;
  size_t cap = (size_t)sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace liger

using namespace liger;

extern "C" int liger_layernorm(const void* x, const void* gamma, const void* beta, void* y, int m, int n, void* stream) {
  if (!x || !gamma || !beta || !y || m <= 0 || n <= 0) return set_error(LIGER_ERR_INVALID, "layernorm: bad argument");
  if (n % 8 || n > kLnThreads * kLnMaxVec * 8)
    return set_error(LIGER_ERR_UNSUPPORTED, "layernorm: n = %d must be a multiple of 8 and <= %d", n,
                     kLnThreads * kLnMaxVec * 8);
  if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)gamma | (uintptr_t)beta) & 15u)
    return set_error(LIGER_ERR_INVALID, "layernorm: pointers must be 16-byte aligned");
  if (!current_device()) return LIGER_ERR_CUDA;
  layernorm_kernel<false><<<m, kLnThreads, 0, (cudaStream_t)stream>>>((const __half*)x, nullptr, nullptr,
                                                                      (const __half*)gamma, (const __half*)beta, nullptr,
                                                                      (__half*)y, n);
  return check_launch("layernorm_kernel");
}

extern "C" int liger_add_bias_input_layernorm(const void* in, const void* gamma, const void* beta, const void* bias,
                                              void* out, void* norm, int m, int n, void* stream) {
  if (!in || !out || m <= 0 || n <= 0) return set_error(LIGER_ERR_INVALID, "add_bias_input_layernorm: bad argument");
  if (norm && (!gamma || !beta)) return set_error(LIGER_ERR_INVALID, "add_bias_input_layernorm: norm needs gamma and beta");
  if (n % 8 || n > kLnThreads * kLnMaxVec * 8)
    return set_error(LIGER_ERR_UNSUPPORTED, "add_bias_input_layernorm: n = %d must be a multiple of 8 and <= %d", n,
                     kLnThreads * kLnMaxVec * 8);
  if (((uintptr_t)in | (uintptr_t)out | (uintptr_t)norm | (uintptr_t)gamma | (uintptr_t)beta | (uintptr_t)bias) & 15u)
    return set_error(LIGER_ERR_INVALID, "add_bias_input_layernorm: pointers must be 16-byte aligned");
  if (!current_device()) return LIGER_ERR_CUDA;
  layernorm_kernel<true><<<m, kLnThreads, 0, (cudaStream_t)stream>>>((const __half*)out, (const __half*)in,
                                                                     (const __half*)bias, (const __half*)gamma,
                                                                     (const __half*)beta, (__half*)out, (__half*)norm, n);
  return check_launch("layernorm_kernel<residual>");
}

extern "C" int liger_add_bias_gelu(void* x, const void* bias, int m, int n, void* stream) {
  if (!x || m <= 0 || n <= 0 || n % 8) return set_error(LIGER_ERR_INVALID, "add_bias_gelu: bad argument (n %% 8 == 0)");
  if (((uintptr_t)x | (uintptr_t)bias) & 15u) return set_error(LIGER_ERR_INVALID, "add_bias_gelu: pointers must be 16-byte aligned");
  const DeviceInfo* d = current_device();
  if (!d) return LIGER_ERR_CUDA;
  const size_t total = (size_t)m * n / 8;
  add_bias_gelu_kernel<<<grid_for(total, 256, d->sm_count), 256, 0, (cudaStream_t)stream>>>((__half*)x, (const __half*)bias,
                                                                                            total, n / 8);
  return check_launch("add_bias_gelu_kernel");
}

extern "C" int liger_add_qkv_bias_transpose(void* q_out, void* k_out, void* v_out, const void* q, const void* bq,
                                            const void* k, const void* bk, const void* v, const void* bv, int batch,
                                            int seq_len, int heads, int head_dim, void* stream) {
  if (!q_out || !k_out || !v_out || !q || !k || !v || batch <= 0 || seq_len <= 0 || heads <= 0 || head_dim <= 0 ||
      head_dim % 8)
    return set_error(LIGER_ERR_INVALID, "add_qkv_bias_transpose: bad argument (head_dim %% 8 == 0)");
  if (((uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)v_out | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)bq |
       (uintptr_t)bk | (uintptr_t)bv) & 15u)
    return set_error(LIGER_ERR_INVALID, "add_qkv_bias_transpose: pointers must be 16-byte aligned");
  const DeviceInfo* d = current_device();
  if (!d) return LIGER_ERR_CUDA;
  const size_t total = (size_t)3 * batch * seq_len * heads * (head_dim / 8);
  add_qkv_bias_transpose_kernel<<<grid_for(total, 256, d->sm_count), 256, 0, (cudaStream_t)stream>>>(
      (__half*)q_out, (__half*)k_out, (__half*)v_out, (const __half*)q, (const __half*)bq, (const __half*)k,
      (const __half*)bk, (const __half*)v, (const __half*)bv, batch, seq_len, heads, head_dim);
  return check_launch("add_qkv_bias_transpose_kernel");
}

extern "C" int liger_transpose_heads(void* dst, const void* src, int batch, int seq_len, int heads, int head_dim,
                                     void* stream) {
  if (!dst || !src || batch <= 0 || seq_len <= 0 || heads <= 0 || head_dim <= 0 || head_dim % 8)
    return set_error(LIGER_ERR_INVALID, "transpose_heads: bad argument (head_dim %% 8 == 0)");
  if (((uintptr_t)dst | (uintptr_t)src) & 15u) return set_error(LIGER_ERR_INVALID, "transpose_heads: pointers must be 16-byte aligned");
  const DeviceInfo* d = current_device();
  if (!d) return LIGER_ERR_CUDA;
  const size_t total = (size_t)batch * seq_len * heads * (head_dim / 8);
  transpose_heads_kernel<<<grid_for(total, 256, d->sm_count), 256, 0, (cudaStream_t)stream>>>(
      (__half*)dst, (const __half*)src, batch, seq_len, heads, head_dim);
  return check_launch("transpose_heads_kernel");
}

extern "C" int liger_transpose_weight(const void* src, void* dst, int k, int n, int interleave32, void* stream) {
  if (!src || !dst || k <= 0 || n <= 0) return set_error(LIGER_ERR_INVALID, "transpose_weight: bad argument");
  if (interleave32 && n % 64) return set_error(LIGER_ERR_INVALID, "transpose_weight: interleave needs n %% 64 == 0");
  if (!current_device()) return LIGER_ERR_CUDA;
  dim3 grid((n + 31) / 32, (k + 31) / 32), block(32, 8);
  transpose_weight_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((const __half*)src, (__half*)dst, k, n, interleave32);
  return check_launch("transpose_weight_kernel");
}

extern "C" int liger_fill_normal(void* dst, int rows, int cols, int dst_ld, int row0, int col0, int src_ld, uint32_t seed,
                                 uint32_t tensor_id, float mean, float std, int transpose, void* stream) {
  if (!dst || rows <= 0 || cols <= 0 || dst_ld <= 0 || src_ld <= 0 || transpose < 0 || transpose > 3)
    return set_error(LIGER_ERR_INVALID, "fill_normal: bad argument");
  if (transpose >= 2 && cols % 32) return set_error(LIGER_ERR_INVALID, "fill_normal: interleaved modes need cols %% 32 == 0");
  const DeviceInfo* d = current_device();
  if (!d) return LIGER_ERR_CUDA;
  const size_t total = (size_t)rows * cols;
  fill_normal_kernel<<<grid_for(total, 256, d->sm_count), 256, 0, (cudaStream_t)stream>>>(
      (__half*)dst, rows, cols, dst_ld, row0, col0, src_ld, seed, tensor_id, mean, std, transpose);
  return check_launch("fill_normal_kernel");
}
