/*
 * liger_oracle.c -- TEST INFRASTRUCTURE, not product code.
 *
 * An fp32 host restatement of the arithmetic of Liger's tensor-parallel transformer-layer
 * path.  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may build, load
 * or call this file; the product library never links or calls it.
 *
 * PARITY PINNED TO THE REFERENCE'S OWN OUTPUT.  The reference ships no golden vectors, known-answer tests or CPU
 * path for this arithmetic (src/test_model.h is timing-only; weights and inputs are never initialised, outputs
 * never read back), and its dense contractions and reductions live in cuBLAS (cublasGemmEx /
 * cublasGemmStridedBatchedEx, call sites src/layer/func_wrapper.h:25,35) and NCCL (ncclAllReduce,
 * src/layer/func_wrapper.h:42), closed libraries outside the reference tree.  So the reference itself is run: its
 * unmodified sources, compiled with a harness (oracle/ref_harness/) into oracle/_ref/, execute each of its kernels
 * and its whole layer stack on seeded inputs on the GPU, and tests/test_reference_parity.py compares those outputs
 * with the functions below (per operator within 1e-2, data movement bit for bit; whole stacks within 2e-2, the
 * reference accumulating its GEMMs in fp16).  Each function follows the reference's call sites and CUDA kernels,
 * cited per function, and computes in plain fp32.
 *
 * Conventions: every tensor is a dense row-major float array whose values are fp16
 * representable on entry.  Weights use the reference orientation W[k][n] with Y = X * W
 * (src/layer/linear.h:47-53,99-105 are the column-major cuBLAS spellings of that product).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#endif
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/liger_rng.h"

#define LO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------ */
/* seeded tensors                                                                             */
/* ------------------------------------------------------------------------------------------ */

LO_API int lo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Seconds spent generating seeded tensors since the last reset: lets a caller that times the stack
 * separate the arithmetic from the cost of materialising the weights. */
static double g_fill_seconds = 0.0;
static double now_seconds(void) {
#ifdef _OPENMP
  return omp_get_wtime();
#else
  return 0.0;
#endif
}
LO_API double lo_fill_seconds(int reset) {
  double v = g_fill_seconds;
  if (reset) g_fill_seconds = 0.0;
  return v;
}

/* dst[i] = value of element (idx0 + i) of seeded tensor `tensor_id`, as fp16 bits */
LO_API void lo_fill_normal_f16(uint16_t* dst, uint64_t n, uint32_t seed, uint32_t tensor_id, uint64_t idx0,
                               float mean, float std) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) dst[i] = lg_normal_half_bits(seed, tensor_id, idx0 + (uint64_t)i, mean, std);
}

/* the same values widened to float */
LO_API void lo_fill_normal_f32(float* dst, uint64_t n, uint32_t seed, uint32_t tensor_id, uint64_t idx0, float mean,
                               float std) {
  const double t0 = now_seconds();
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i)
    dst[i] = lg_half_bits_to_float(lg_normal_half_bits(seed, tensor_id, idx0 + (uint64_t)i, mean, std));
  g_fill_seconds += now_seconds() - t0;
}

/* a [rows x cols] window (row0.., col0..) of a seeded logical matrix with `ld` columns */
LO_API void lo_fill_normal_window_f32(float* dst, int rows, int cols, int row0, int col0, int ld, uint32_t seed,
                                      uint32_t tensor_id, float mean, float std) {
  const double t0 = now_seconds();
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c)
      dst[(size_t)r * cols + c] = lg_half_bits_to_float(
          lg_normal_half_bits(seed, tensor_id, (uint64_t)(row0 + r) * (uint64_t)ld + (uint64_t)(col0 + c), mean, std));
  g_fill_seconds += now_seconds() - t0;
}

LO_API void lo_half_to_float(const uint16_t* src, float* dst, uint64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) dst[i] = lg_half_bits_to_float(src[i]);
}
LO_API void lo_float_to_half(const float* src, uint16_t* dst, uint64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) dst[i] = lg_float_to_half_bits(src[i]);
}
/* round every element to the nearest fp16 value (what a GPU kernel's fp16 store does) */
LO_API void lo_round_fp16(float* x, uint64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) x[i] = lg_half_bits_to_float(lg_float_to_half_bits(x[i]));
}

/* ------------------------------------------------------------------------------------------ */
/* linear layers: src/layer/linear.h:43-63 (row-parallel) and :95-108 (column-parallel)       */
/* Y[M,N] = X[M,K] * W[K,N]; ldx / ldw / ldy are row strides so that a rank's slice of the      */
/* full weight can be addressed in place.                                                     */
/* ------------------------------------------------------------------------------------------ */
/* one task: rows [i0,i1) x columns [j0,j1), full K, accumulating into Y in k-blocks of 256 so that the
 * W sub-block (256 x 64 floats) and the X sub-block stay in cache */
static void gemm_task(const float* X, int ldx, const float* W, int ldw, float* Y, int ldy, int i0, int i1, int j0, int j1,
                      int K) {
  const int KB = 256;
  for (int i = i0; i < i1; ++i) memset(Y + (size_t)i * ldy + j0, 0, sizeof(float) * (size_t)(j1 - j0));
  for (int kb = 0; kb < K; kb += KB) {
    const int ke = kb + KB < K ? kb + KB : K;
    int i = i0;
#if defined(__AVX2__) && defined(__FMA__)
    for (; i + 4 <= i1; i += 4) {
      int j = j0;
      for (; j + 16 <= j1; j += 16) {
        float* y0 = Y + (size_t)(i + 0) * ldy + j;
        float* y1 = Y + (size_t)(i + 1) * ldy + j;
        float* y2 = Y + (size_t)(i + 2) * ldy + j;
        float* y3 = Y + (size_t)(i + 3) * ldy + j;
        __m256 a00 = _mm256_loadu_ps(y0), a01 = _mm256_loadu_ps(y0 + 8);
        __m256 a10 = _mm256_loadu_ps(y1), a11 = _mm256_loadu_ps(y1 + 8);
        __m256 a20 = _mm256_loadu_ps(y2), a21 = _mm256_loadu_ps(y2 + 8);
        __m256 a30 = _mm256_loadu_ps(y3), a31 = _mm256_loadu_ps(y3 + 8);
        for (int k = kb; k < ke; ++k) {
          const float* w = W + (size_t)k * ldw + j;
          __m256 w0 = _mm256_loadu_ps(w), w1 = _mm256_loadu_ps(w + 8);
          __m256 x0 = _mm256_broadcast_ss(X + (size_t)(i + 0) * ldx + k);
          __m256 x1 = _mm256_broadcast_ss(X + (size_t)(i + 1) * ldx + k);
          __m256 x2 = _mm256_broadcast_ss(X + (size_t)(i + 2) * ldx + k);
          __m256 x3 = _mm256_broadcast_ss(X + (size_t)(i + 3) * ldx + k);
          a00 = _mm256_fmadd_ps(x0, w0, a00); a01 = _mm256_fmadd_ps(x0, w1, a01);
          a10 = _mm256_fmadd_ps(x1, w0, a10); a11 = _mm256_fmadd_ps(x1, w1, a11);
          a20 = _mm256_fmadd_ps(x2, w0, a20); a21 = _mm256_fmadd_ps(x2, w1, a21);
          a30 = _mm256_fmadd_ps(x3, w0, a30); a31 = _mm256_fmadd_ps(x3, w1, a31);
        }
        _mm256_storeu_ps(y0, a00); _mm256_storeu_ps(y0 + 8, a01);
        _mm256_storeu_ps(y1, a10); _mm256_storeu_ps(y1 + 8, a11);
        _mm256_storeu_ps(y2, a20); _mm256_storeu_ps(y2 + 8, a21);
        _mm256_storeu_ps(y3, a30); _mm256_storeu_ps(y3 + 8, a31);
      }
      for (; j < j1; ++j)
        for (int r = 0; r < 4; ++r) {
          float acc = Y[(size_t)(i + r) * ldy + j];
          for (int k = kb; k < ke; ++k) acc += X[(size_t)(i + r) * ldx + k] * W[(size_t)k * ldw + j];
          Y[(size_t)(i + r) * ldy + j] = acc;
        }
    }
#endif
    for (; i < i1; ++i) {
      float* y = Y + (size_t)i * ldy;
      for (int k = kb; k < ke; ++k) {
        const float x = X[(size_t)i * ldx + k];
        const float* w = W + (size_t)k * ldw;
        for (int j = j0; j < j1; ++j) y[j] += x * w[j];
      }
    }
  }
}

LO_API void lo_linear(const float* X, int ldx, const float* W, int ldw, float* Y, int ldy, int M, int N, int K) {
  const int RB = 128, CB = 64;
  const int nrb = (M + RB - 1) / RB, ncb = (N + CB - 1) / CB;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int rb = 0; rb < nrb; ++rb)
    for (int cb = 0; cb < ncb; ++cb) {
      const int i0 = rb * RB, i1 = i0 + RB < M ? i0 + RB : M;
      const int j0 = cb * CB, j1 = j0 + CB < N ? j0 + CB : N;
      gemm_task(X, ldx, W, ldw, Y, ldy, i0, i1, j0, j1, K);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* bias + head split: src/cuda/attention_kernels.cu:133-163 (add_QKV_bias<half>)              */
/* dst[b][h][s][d] = src[(b*S+s)][h*D+d] + bias[h*D+d]                                        */
/* ------------------------------------------------------------------------------------------ */
LO_API void lo_add_bias_split_heads(const float* src, int ld, const float* bias, float* dst, int B, int S, int h,
                                    int D) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b)
    for (int s = 0; s < S; ++s)
      for (int hh = 0; hh < h; ++hh)
        for (int d = 0; d < D; ++d)
          dst[(((size_t)b * h + hh) * S + s) * D + d] =
              src[((size_t)b * S + s) * ld + hh * D + d] + (bias ? bias[hh * D + d] : 0.0f);
}

/* head merge: src/cuda/attention_kernels.cu:693-710 (transpose<half>) [B,h,S,D] -> [B*S, h*D] */
LO_API void lo_merge_heads(const float* src, float* dst, int ld, int B, int S, int h, int D) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b)
    for (int s = 0; s < S; ++s)
      for (int hh = 0; hh < h; ++hh)
        for (int d = 0; d < D; ++d)
          dst[((size_t)b * S + s) * ld + hh * D + d] = src[(((size_t)b * h + hh) * S + s) * D + d];
}

/* ------------------------------------------------------------------------------------------ */
/* attention core: QK^T (src/layer/bert_layer.h:145-150), masked softmax                     */
/* (src/cuda/attention_kernels.cu:543-573: p = exp(t - max t) / (sum + 1e-6) with              */
/*  t = scale*s + (1-mask)*(-10000)), then P*V (src/layer/bert_layer.h:158-163).              */
/* q,k,v,out are [B,h,S,D]; mask is [B,Sq,Skv] of 0/1 shared over heads; with mask == NULL the   */
/* mask is causal (mask[q][k] = k <= Skv-Sq+q; Skv may exceed Sq for decode) when `causal` is    */
/* set, else all ones.                                                                         */
/* ------------------------------------------------------------------------------------------ */
LO_API void lo_attention(const float* q, const float* k, const float* v, const float* mask, int causal, float* out,
                         int B, int h, int Sq, int Skv, int D, float scale) {
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < B; ++b)
    for (int hh = 0; hh < h; ++hh) {
      float* t = (float*)malloc(sizeof(float) * (size_t)Skv);
      const float* qh = q + ((size_t)b * h + hh) * Sq * D;
      const float* kh = k + ((size_t)b * h + hh) * Skv * D;
      const float* vh = v + ((size_t)b * h + hh) * Skv * D;
      float* oh = out + ((size_t)b * h + hh) * Sq * D;
      for (int i = 0; i < Sq; ++i) {
        float mx = -1e20f;
        for (int j = 0; j < Skv; ++j) {
          float s = 0.0f;
          for (int d = 0; d < D; ++d) s += qh[(size_t)i * D + d] * kh[(size_t)j * D + d];
          float m = mask ? mask[((size_t)b * Sq + i) * Skv + j] : (!causal || j <= Skv - Sq + i ? 1.0f : 0.0f);
          t[j] = scale * s + (1.0f - m) * -10000.0f;
          if (t[j] > mx) mx = t[j];
        }
        float sum = 0.0f;
        for (int j = 0; j < Skv; ++j) { t[j] = expf(t[j] - mx); sum += t[j]; }
        const float inv = 1.0f / (sum + 1e-6f);
        for (int d = 0; d < D; ++d) oh[(size_t)i * D + d] = 0.0f;
        for (int j = 0; j < Skv; ++j) {
          const float p = t[j] * inv;
          if (p == 0.0f) continue;
          for (int d = 0; d < D; ++d) oh[(size_t)i * D + d] += p * vh[(size_t)j * D + d];
        }
      }
      free(t);
    }
}

/* The masked softmax alone, in place on scores [B,h,S,S]: src/cuda/attention_kernels.cu:543-573,620-680
 * (attn_softmax_kernelLauncher): p = exp(t - max t) / (sum + 1e-6), t = scale*s + (1-mask)*(-10000),
 * mask [B,S,S] of 0/1 shared over heads.  The same arithmetic as inside lo_attention. */
LO_API void lo_masked_softmax(float* scores, const float* mask, int B, int h, int S, float scale) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b)
    for (int hh = 0; hh < h; ++hh)
      for (int i = 0; i < S; ++i) {
        float* t = scores + (((size_t)b * h + hh) * S + i) * S;
        float mx = -1e20f;
        for (int j = 0; j < S; ++j) {
          const float m = mask ? mask[((size_t)b * S + i) * S + j] : 1.0f;
          t[j] = scale * t[j] + (1.0f - m) * -10000.0f;
          if (t[j] > mx) mx = t[j];
        }
        float sum = 0.0f;
        for (int j = 0; j < S; ++j) { t[j] = expf(t[j] - mx); sum += t[j]; }
        const float inv = 1.0f / (sum + 1e-6f);
        for (int j = 0; j < S; ++j) t[j] *= inv;
      }
}

/* ------------------------------------------------------------------------------------------ */
/* bias + GELU (tanh form): src/cuda/cuda_kernels.cu:9-29,71-84                                */
/* ------------------------------------------------------------------------------------------ */
static inline float gelu_tanh(float x) {
  return x * 0.5f * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
LO_API void lo_add_bias_gelu(float* x, const float* bias, int M, int N) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) x[(size_t)i * N + j] = gelu_tanh(x[(size_t)i * N + j] + (bias ? bias[j] : 0.0f));
}
/* GeGLU: out[i][j] = gelu(u[i][j] + b[j]) * (u[i][F+j] + b[F+j]); u is [M, 2F] (gate | value).  No
 * reference source: the gated form is defined by the benchmark configuration only. */
LO_API void lo_add_bias_geglu(const float* u, const float* bias, float* out, int M, int F) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < F; ++j) {
      float g = u[(size_t)i * 2 * F + j] + (bias ? bias[j] : 0.0f);
      float val = u[(size_t)i * 2 * F + F + j] + (bias ? bias[F + j] : 0.0f);
      out[(size_t)i * F + j] = gelu_tanh(g) * val;
    }
}

/* ------------------------------------------------------------------------------------------ */
/* LayerNorm: src/cuda/cuda_kernels.cu:463-508 (two-pass mean / biased variance, eps 1e-6)     */
/* ------------------------------------------------------------------------------------------ */
LO_API void lo_layernorm(const float* x, const float* gamma, const float* beta, float* y, int M, int N) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; ++i) {
    const float* r = x + (size_t)i * N;
    float s = 0.0f;
    for (int j = 0; j < N; ++j) s += r[j];
    const float mean = s / N;
    float vs = 0.0f;
    for (int j = 0; j < N; ++j) { float d = r[j] - mean; vs += d * d; }
    const float rstd = 1.0f / sqrtf(vs / N + 1e-6f);
    for (int j = 0; j < N; ++j) y[(size_t)i * N + j] = (r[j] - mean) * rstd * gamma[j] + beta[j];
  }
}

/* residual + bias, then LayerNorm: src/cuda/cuda_kernels.cu:360-409 (add_bias_input_layernorm_2)
 * out[i][j] = in[i][j] + out[i][j] + bias[j]  (stored; rounded to fp16 when round16 != 0, as the
 * kernel stores T before re-reading it), norm = LN(out).  norm may be NULL. */
LO_API void lo_add_bias_input_layernorm_2(const float* in, const float* gamma, const float* beta, const float* bias,
                                          float* out, float* norm, int M, int N, int round16) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; ++i) {
    float* o = out + (size_t)i * N;
    const float* a = in + (size_t)i * N;
    for (int j = 0; j < N; ++j) {
      float t = a[j] + o[j] + (bias ? bias[j] : 0.0f);
      o[j] = round16 ? lg_half_bits_to_float(lg_float_to_half_bits(t)) : t;
    }
  }
  if (norm) lo_layernorm(out, gamma, beta, norm, M, N);
}

/* all-reduce (sum) of `ws` rank-partials laid out back to back: src/layer/linear.h:55-60.
 * Partials are added in rank order 0..ws-1 in fp32. */
LO_API void lo_allreduce_sum(const float* partials, float* out, int ws, uint64_t count) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)count; ++i) {
    float s = 0.0f;
    for (int r = 0; r < ws; ++r) s += partials[(size_t)r * count + i];
    out[i] = s;
  }
}

/* ------------------------------------------------------------------------------------------ */
/* the layer stack                                                                            */
/* ------------------------------------------------------------------------------------------ */
typedef struct {
  int hidden;      /* H = heads * head_dim */
  int heads;       /* global head count */
  int head_dim;    /* D */
  int ffn_inner;   /* F: 4H in the reference (src/layer/bert_layer.h:23), 32768 for the gated form */
  int layers;
  int tp;          /* world size ws */
  int graph;       /* 0 = reference graph  MHA -> AR -> LN -> MLP -> AR -> LN, no residual
                          (src/layer/bert.h:59-79);
                      1 = pre-LayerNorm graph with residual adds (the semantics of
                          add_bias_input_layernorm_2, src/cuda/cuda_kernels.cu:360-409) */
  int act;         /* 0 = bias + GELU, 1 = GeGLU (gate | value) */
  int causal;      /* 1: causal mask by construction; 0: use the mask tensor passed in */
  int round16;     /* 1: round to fp16 wherever the GPU path stores an fp16 tensor */
  uint32_t seed;
} lo_config;

/* tensor ids of the seeded parameters of layer l: id = l * 32 + kind */
enum {
  LO_WQ = 0, LO_WK = 1, LO_WV = 2, LO_WO = 3, LO_WUP = 4, LO_WDOWN = 5, LO_BQ = 6, LO_BK = 7, LO_BV = 8, LO_BUP = 9,
  LO_LN1_G = 10, LO_LN1_B = 11, LO_LN2_G = 12, LO_LN2_B = 13, LO_BO = 14, LO_BDOWN = 15,
  LO_INPUT = 0x10000, LO_KCACHE = 0x10001, LO_VCACHE = 0x10002
};
#define LO_W_STD 0.02f

static float* falloc(size_t n) { return (float*)malloc(sizeof(float) * (n ? n : 1)); }
static void maybe_round(float* x, size_t n, int on) { if (on) lo_round_fp16(x, n); }

/*
 * One forward pass of `layers` layers over x[M = B*S, H] -> out[M, H].
 *
 * Tensor parallelism is simulated rank by rank exactly as the reference shards it
 * (src/layer/linear.h:16-109, src/layer/bert_layer.h:98-101): Q/K/V and FFN-up are column
 * parallel (rank r owns output features [r*n/ws, (r+1)*n/ws), i.e. heads/ws whole heads; for the
 * gated form the gate and value columns of one inner unit live on the same rank); attention is
 * head-local; out-proj and FFN-down are row parallel and their partial sums are all-reduced.
 */
LO_API void lo_stack_forward(const lo_config* cfg, const float* x, const float* mask, float* out, int B, int S) {
  const int H = cfg->hidden, D = cfg->head_dim, ws = cfg->tp, F = cfg->ffn_inner;
  const int hl = cfg->heads / ws, Hl = H / ws, Fl = F / ws;
  const int M = B * S;
  const int upw = cfg->act ? 2 * F : F; /* full width of W_up */
  const float scale = 1.0f / sqrtf((float)D);
  const int r16 = cfg->round16;

  float* hbuf = falloc((size_t)M * H);      /* residual stream / layer input */
  float* nbuf = falloc((size_t)M * H);      /* normed activations */
  float* part = falloc((size_t)ws * M * H); /* row-parallel partials of every rank */
  float* red = falloc((size_t)M * H);
  const int wmax = Fl > Hl ? Fl : Hl;
  const int linmax = 2 * Fl > Hl ? 2 * Fl : Hl;
  float* W = falloc((size_t)H * wmax);
  float* W2 = falloc((size_t)wmax * H);
  float* lin = falloc((size_t)M * linmax);
  float* qb = falloc((size_t)M * Hl); float* kb = falloc((size_t)M * Hl); float* vb = falloc((size_t)M * Hl);
  float* ab = falloc((size_t)M * Hl); float* am = falloc((size_t)M * Hl);
  float* act = falloc((size_t)M * Fl);
  float* bias = falloc((size_t)(2 * F > H ? 2 * F : H));
  float* g = falloc(H); float* be = falloc(H);
  memcpy(hbuf, x, sizeof(float) * (size_t)M * H);

  for (int l = 0; l < cfg->layers; ++l) {
    const uint32_t id0 = (uint32_t)l * 32u;
    const float* attn_in = hbuf;
    if (cfg->graph == 1) { /* pre-LN */
      lo_fill_normal_f32(g, H, cfg->seed, id0 + LO_LN1_G, 0, 1.0f, LO_W_STD);
      lo_fill_normal_f32(be, H, cfg->seed, id0 + LO_LN1_B, 0, 0.0f, LO_W_STD);
      lo_layernorm(hbuf, g, be, nbuf, M, H);
      maybe_round(nbuf, (size_t)M * H, r16);
      attn_in = nbuf;
    }
    /* ---- attention block, rank by rank (src/layer/bert_layer.h:121-175) ---- */
    for (int r = 0; r < ws; ++r) {
      const uint32_t wid[3] = {LO_WQ, LO_WK, LO_WV}, bid[3] = {LO_BQ, LO_BK, LO_BV};
      float* dst[3] = {qb, kb, vb};
      for (int t = 0; t < 3; ++t) {
        lo_fill_normal_window_f32(W, H, Hl, 0, r * Hl, H, cfg->seed, id0 + wid[t], 0.0f, LO_W_STD);
        lo_linear(attn_in, H, W, Hl, lin, Hl, M, Hl, H);
        lo_fill_normal_f32(bias, Hl, cfg->seed, id0 + bid[t], (uint64_t)r * Hl, 0.0f, LO_W_STD);
        lo_add_bias_split_heads(lin, Hl, bias, dst[t], B, S, hl, D);
        maybe_round(dst[t], (size_t)M * Hl, r16);
      }
      lo_attention(qb, kb, vb, cfg->causal ? NULL : mask, cfg->causal, ab, B, hl, S, S, D, scale);
      lo_merge_heads(ab, am, Hl, B, S, hl, D);
      maybe_round(am, (size_t)M * Hl, r16);
      lo_fill_normal_window_f32(W2, Hl, H, r * Hl, 0, H, cfg->seed, id0 + LO_WO, 0.0f, LO_W_STD);
      lo_linear(am, Hl, W2, H, part + (size_t)r * M * H, H, M, H, Hl);
      maybe_round(part + (size_t)r * M * H, (size_t)M * H, r16);
    }
    lo_allreduce_sum(part, red, ws, (uint64_t)M * H);
    const float* mlp_in;
    if (cfg->graph == 0) { /* post-LN, no residual, no out-proj bias (src/layer/bert.h:65-69) */
      maybe_round(red, (size_t)M * H, r16);
      lo_fill_normal_f32(g, H, cfg->seed, id0 + LO_LN1_G, 0, 1.0f, LO_W_STD);
      lo_fill_normal_f32(be, H, cfg->seed, id0 + LO_LN1_B, 0, 0.0f, LO_W_STD);
      lo_layernorm(red, g, be, nbuf, M, H);
      maybe_round(nbuf, (size_t)M * H, r16);
      mlp_in = nbuf;
    } else { /* h = h + o + b_o ; n = LN2(h) */
      lo_fill_normal_f32(bias, H, cfg->seed, id0 + LO_BO, 0, 0.0f, LO_W_STD);
      lo_fill_normal_f32(g, H, cfg->seed, id0 + LO_LN2_G, 0, 1.0f, LO_W_STD);
      lo_fill_normal_f32(be, H, cfg->seed, id0 + LO_LN2_B, 0, 0.0f, LO_W_STD);
      lo_add_bias_input_layernorm_2(red, g, be, bias, hbuf, nbuf, M, H, r16);
      maybe_round(nbuf, (size_t)M * H, r16);
      mlp_in = nbuf;
    }
    /* ---- MLP block (src/layer/bert_layer.h:48-62) ---- */
    for (int r = 0; r < ws; ++r) {
      if (cfg->act == 0) {
        lo_fill_normal_window_f32(W, H, Fl, 0, r * Fl, upw, cfg->seed, id0 + LO_WUP, 0.0f, LO_W_STD);
        lo_linear(mlp_in, H, W, Fl, lin, Fl, M, Fl, H);
        lo_fill_normal_f32(bias, Fl, cfg->seed, id0 + LO_BUP, (uint64_t)r * Fl, 0.0f, LO_W_STD);
        lo_add_bias_gelu(lin, bias, M, Fl);
        memcpy(act, lin, sizeof(float) * (size_t)M * Fl);
      } else {
        /* rank r owns gate columns [r*Fl,(r+1)*Fl) and value columns F + the same range */
        lo_fill_normal_window_f32(W, H, Fl, 0, r * Fl, upw, cfg->seed, id0 + LO_WUP, 0.0f, LO_W_STD);
        for (int i = 0; i < M; ++i) memset(lin + (size_t)i * 2 * Fl, 0, sizeof(float) * 2 * Fl);
        lo_linear(mlp_in, H, W, Fl, lin, 2 * Fl, M, Fl, H);
        lo_fill_normal_window_f32(W, H, Fl, 0, F + r * Fl, upw, cfg->seed, id0 + LO_WUP, 0.0f, LO_W_STD);
        lo_linear(mlp_in, H, W, Fl, lin + Fl, 2 * Fl, M, Fl, H);
        lo_fill_normal_f32(bias, Fl, cfg->seed, id0 + LO_BUP, (uint64_t)r * Fl, 0.0f, LO_W_STD);
        lo_fill_normal_f32(bias + Fl, Fl, cfg->seed, id0 + LO_BUP, (uint64_t)F + (uint64_t)r * Fl, 0.0f, LO_W_STD);
        lo_add_bias_geglu(lin, bias, act, M, Fl);
      }
      maybe_round(act, (size_t)M * Fl, r16);
      lo_fill_normal_window_f32(W2, Fl, H, r * Fl, 0, H, cfg->seed, id0 + LO_WDOWN, 0.0f, LO_W_STD);
      lo_linear(act, Fl, W2, H, part + (size_t)r * M * H, H, M, H, Fl);
      maybe_round(part + (size_t)r * M * H, (size_t)M * H, r16);
    }
    lo_allreduce_sum(part, red, ws, (uint64_t)M * H);
    if (cfg->graph == 0) { /* second post-LN (src/layer/bert.h:75) becomes the next layer's input */
      maybe_round(red, (size_t)M * H, r16);
      lo_fill_normal_f32(g, H, cfg->seed, id0 + LO_LN2_G, 0, 1.0f, LO_W_STD);
      lo_fill_normal_f32(be, H, cfg->seed, id0 + LO_LN2_B, 0, 0.0f, LO_W_STD);
      lo_layernorm(red, g, be, hbuf, M, H);
      maybe_round(hbuf, (size_t)M * H, r16);
    } else { /* h = h + d + b_down */
      lo_fill_normal_f32(bias, H, cfg->seed, id0 + LO_BDOWN, 0, 0.0f, LO_W_STD);
      lo_add_bias_input_layernorm_2(red, NULL, NULL, bias, hbuf, NULL, M, H, r16);
    }
  }
  memcpy(out, hbuf, sizeof(float) * (size_t)M * H);
  free(hbuf); free(nbuf); free(part); free(red); free(W); free(W2); free(lin); free(qb); free(kb); free(vb);
  free(ab); free(am); free(act); free(bias); free(g); free(be);
}


/*
 * One decode step: a single new token per sequence (x is [B, H]) against a seeded KV cache holding
 * kv_len positions per sequence, on the pre-LayerNorm graph (cfg->graph must be 1).  The reference
 * has no KV cache or decode path; the step is defined by the benchmark configuration: per layer the
 * new token's K and V are appended at position kv_len and the query attends to positions 0..kv_len.
 * The cache of layer l is the seeded tensor LO_KCACHE + 2*l (keys) / LO_VCACHE + 2*l (values) with
 * logical layout [B][heads][kv_cap][head_dim], N(0,1); rank r owns heads [r*h/ws, (r+1)*h/ws).
 */
LO_API void lo_stack_decode(const lo_config* cfg, const float* x, float* out, int B, int kv_len, int kv_cap) {
  const int H = cfg->hidden, D = cfg->head_dim, ws = cfg->tp, F = cfg->ffn_inner, heads = cfg->heads;
  const int hl = heads / ws, Hl = H / ws, Fl = F / ws;
  const int M = B, L = kv_len + 1;
  const int upw = cfg->act ? 2 * F : F;
  const float scale = 1.0f / sqrtf((float)D);
  const int r16 = cfg->round16;
  float* hbuf = falloc((size_t)M * H); float* nbuf = falloc((size_t)M * H);
  float* part = falloc((size_t)ws * M * H); float* red = falloc((size_t)M * H);
  const int wmax = Fl > Hl ? Fl : Hl, linmax = 2 * Fl > Hl ? 2 * Fl : Hl;
  float* W = falloc((size_t)H * wmax); float* W2 = falloc((size_t)wmax * H); float* lin = falloc((size_t)M * linmax);
  float* qb = falloc((size_t)M * Hl); float* kn = falloc((size_t)M * Hl); float* vn = falloc((size_t)M * Hl);
  float* kc = falloc((size_t)B * hl * L * D); float* vc = falloc((size_t)B * hl * L * D);
  float* ab = falloc((size_t)M * Hl); float* act = falloc((size_t)M * Fl);
  float* bias = falloc((size_t)(2 * F > H ? 2 * F : H)); float* g = falloc(H); float* be = falloc(H);
  memcpy(hbuf, x, sizeof(float) * (size_t)M * H);
  for (int l = 0; l < cfg->layers; ++l) {
    const uint32_t id0 = (uint32_t)l * 32u;
    lo_fill_normal_f32(g, H, cfg->seed, id0 + LO_LN1_G, 0, 1.0f, LO_W_STD);
    lo_fill_normal_f32(be, H, cfg->seed, id0 + LO_LN1_B, 0, 0.0f, LO_W_STD);
    lo_layernorm(hbuf, g, be, nbuf, M, H);
    maybe_round(nbuf, (size_t)M * H, r16);
    for (int r = 0; r < ws; ++r) {
      const uint32_t wid[3] = {LO_WQ, LO_WK, LO_WV}, bid[3] = {LO_BQ, LO_BK, LO_BV};
      float* dst[3] = {qb, kn, vn};
      for (int t = 0; t < 3; ++t) {
        lo_fill_normal_window_f32(W, H, Hl, 0, r * Hl, H, cfg->seed, id0 + wid[t], 0.0f, LO_W_STD);
        lo_linear(nbuf, H, W, Hl, lin, Hl, M, Hl, H);
        lo_fill_normal_f32(bias, Hl, cfg->seed, id0 + bid[t], (uint64_t)r * Hl, 0.0f, LO_W_STD);
        lo_add_bias_split_heads(lin, Hl, bias, dst[t], B, 1, hl, D);   /* [B, hl, 1, D] */
        maybe_round(dst[t], (size_t)M * Hl, r16);
      }
      /* this rank's heads of the cache, positions 0..kv_len-1, then the new token's K / V */
      for (int b = 0; b < B; ++b)
        for (int hh = 0; hh < hl; ++hh) {
          const uint64_t base = (((uint64_t)b * heads + (uint64_t)(r * hl + hh)) * kv_cap) * D;
          float* kd = kc + ((size_t)b * hl + hh) * L * D;
          float* vd = vc + ((size_t)b * hl + hh) * L * D;
          lo_fill_normal_f32(kd, (uint64_t)kv_len * D, cfg->seed, LO_KCACHE + 2u * (uint32_t)l, base, 0.0f, 1.0f);
          lo_fill_normal_f32(vd, (uint64_t)kv_len * D, cfg->seed, LO_VCACHE + 2u * (uint32_t)l, base, 0.0f, 1.0f);
          memcpy(kd + (size_t)kv_len * D, kn + ((size_t)b * hl + hh) * D, sizeof(float) * D);
          memcpy(vd + (size_t)kv_len * D, vn + ((size_t)b * hl + hh) * D, sizeof(float) * D);
        }
      lo_attention(qb, kc, vc, NULL, 1, ab, B, hl, 1, L, D, scale);   /* [B, hl, 1, D] == [B, hl*D] */
      maybe_round(ab, (size_t)M * Hl, r16);
      lo_fill_normal_window_f32(W2, Hl, H, r * Hl, 0, H, cfg->seed, id0 + LO_WO, 0.0f, LO_W_STD);
      lo_linear(ab, Hl, W2, H, part + (size_t)r * M * H, H, M, H, Hl);
      maybe_round(part + (size_t)r * M * H, (size_t)M * H, r16);
    }
    lo_allreduce_sum(part, red, ws, (uint64_t)M * H);
    lo_fill_normal_f32(bias, H, cfg->seed, id0 + LO_BO, 0, 0.0f, LO_W_STD);
    lo_fill_normal_f32(g, H, cfg->seed, id0 + LO_LN2_G, 0, 1.0f, LO_W_STD);
    lo_fill_normal_f32(be, H, cfg->seed, id0 + LO_LN2_B, 0, 0.0f, LO_W_STD);
    lo_add_bias_input_layernorm_2(red, g, be, bias, hbuf, nbuf, M, H, r16);
    maybe_round(nbuf, (size_t)M * H, r16);
    for (int r = 0; r < ws; ++r) {
      if (cfg->act == 0) {
        lo_fill_normal_window_f32(W, H, Fl, 0, r * Fl, upw, cfg->seed, id0 + LO_WUP, 0.0f, LO_W_STD);
        lo_linear(nbuf, H, W, Fl, lin, Fl, M, Fl, H);
        lo_fill_normal_f32(bias, Fl, cfg->seed, id0 + LO_BUP, (uint64_t)r * Fl, 0.0f, LO_W_STD);
        lo_add_bias_gelu(lin, bias, M, Fl);
        memcpy(act, lin, sizeof(float) * (size_t)M * Fl);
      } else {
        lo_fill_normal_window_f32(W, H, Fl, 0, r * Fl, upw, cfg->seed, id0 + LO_WUP, 0.0f, LO_W_STD);
        lo_linear(nbuf, H, W, Fl, lin, 2 * Fl, M, Fl, H);
        lo_fill_normal_window_f32(W, H, Fl, 0, F + r * Fl, upw, cfg->seed, id0 + LO_WUP, 0.0f, LO_W_STD);
        lo_linear(nbuf, H, W, Fl, lin + Fl, 2 * Fl, M, Fl, H);
        lo_fill_normal_f32(bias, Fl, cfg->seed, id0 + LO_BUP, (uint64_t)r * Fl, 0.0f, LO_W_STD);
        lo_fill_normal_f32(bias + Fl, Fl, cfg->seed, id0 + LO_BUP, (uint64_t)F + (uint64_t)r * Fl, 0.0f, LO_W_STD);
        lo_add_bias_geglu(lin, bias, act, M, Fl);
      }
      maybe_round(act, (size_t)M * Fl, r16);
      lo_fill_normal_window_f32(W2, Fl, H, r * Fl, 0, H, cfg->seed, id0 + LO_WDOWN, 0.0f, LO_W_STD);
      lo_linear(act, Fl, W2, H, part + (size_t)r * M * H, H, M, H, Fl);
      maybe_round(part + (size_t)r * M * H, (size_t)M * H, r16);
    }
    lo_allreduce_sum(part, red, ws, (uint64_t)M * H);
    lo_fill_normal_f32(bias, H, cfg->seed, id0 + LO_BDOWN, 0, 0.0f, LO_W_STD);
    lo_add_bias_input_layernorm_2(red, NULL, NULL, bias, hbuf, NULL, M, H, r16);
  }
  memcpy(out, hbuf, sizeof(float) * (size_t)M * H);
  free(hbuf); free(nbuf); free(part); free(red); free(W); free(W2); free(lin); free(qb); free(kn); free(vn);
  free(kc); free(vc); free(ab); free(act); free(bias); free(g); free(be);
}
