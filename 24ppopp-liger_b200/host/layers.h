// Layers and function assembly: every layer's forward() returns the vector of kernel launches
// (FuncWrap closures) it consists of, and Bert_Model::forward concatenates them for the whole
// stack -- the reference's "function assembly" (src/layer/linear.h, operator.h, bert_layer.h,
// bert.h).  Class names follow the reference; what differs is what a closure launches:
//
//   reference layer (16 kernels, src/layer/bert.h:59-79)      this implementation (7 kernels)
//   0-2  Q, K, V cuBLAS GEMMs        }                        0 GEMM  fused QKV tcgen05 GEMM, epilogue
//   3    bias + head split           }                               adds the bias and stores [B,h,S,D]
//   4-7  QK^T, softmax, PV, merge                             1 COMP  one attention kernel
//   8    out-proj cuBLAS GEMM                                 2 GEMM  out-proj GEMM
//   9,10 ncclAllReduce, LayerNorm                             3 COMM  fused all-reduce (+residual) + LayerNorm
//   11,12 FFN-up GEMM, bias + GELU                            4 GEMM  FFN-up GEMM, epilogue bias + GELU / GeGLU
//   13   FFN-down GEMM                                        5 GEMM  FFN-down GEMM
//   14,15 ncclAllReduce, LayerNorm                            6 COMM  fused all-reduce (+residual) + LayerNorm
//
// With world_size == 1 kernels 3 and 6 are plain LayerNorm COMPUTATION kernels and, in the
// pre-LayerNorm graph, the residual add moves into the GEMM epilogue of kernels 2 and 5.
// The pre-LayerNorm graph has one extra kernel in front of layer 0 (name kPrologueName: the first
// LayerNorm) and, with world_size > 1, one after the last layer (name kEpilogueName: copy of the
// gathered result into the caller's buffer).
#pragma once
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "context.h"

namespace liger_host {

constexpr int kKernelsPerLayer = 7;
constexpr int kPrologueName = 7;
constexpr int kEpilogueName = 8;
constexpr float kWeightStd = 0.02f;

// tensor ids of the seeded parameters of layer l: l * 32 + kind (shared with the test oracle)
enum weight_kind {
  W_Q = 0, W_K = 1, W_V = 2, W_O = 3, W_UP = 4, W_DOWN = 5, B_Q = 6, B_K = 7, B_V = 8, B_UP = 9,
  LN1_G = 10, LN1_B = 11, LN2_G = 12, LN2_B = 13, B_O = 14, B_DOWN = 15
};

inline void host_check(int rc, const char* what) {
  if (rc != LIGER_OK) throw std::runtime_error(std::string(what) + ": " + liger_last_error());
}
inline void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
// While a Bert_Model is under construction on this thread, every device allocation its layers make is
// recorded here, so that the model can free them when it is destroyed (the reference's layers never free
// anything: src/layer/linear.h:40, src/layer/bert_layer.h:115-118).
inline std::vector<void*>*& alloc_sink() {
  static thread_local std::vector<void*>* sink = nullptr;
  return sink;
}
template <typename T>
inline T* device_alloc(size_t count, const char* what) {
  void* p = nullptr;
  cuda_check(cudaMalloc(&p, count * sizeof(T) > 0 ? count * sizeof(T) : 16), what);
  if (alloc_sink()) alloc_sink()->push_back(p);
  return (T*)p;
}
inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int device_count() { int n = 0; if (cudaGetDeviceCount(&n) != cudaSuccess) n = 0; return n; }

typedef uint16_t half_t;  // fp16 storage

// ---- column-parallel linear: Y[M, n/ws] = X[M,k] * W[k, n/ws]  (src/layer/linear.h:68-108) --------
class Linear_Col {
 public:
  int k, n;            // full (unsharded) shape
  int n_local;
  half_t* weights;     // W^T shard, [n_local, k], K contiguous
  StaticNvInitParam SParams;
  Linear_Col(const StaticNvInitParam& sp, int k_, int n_) : k(k_), n(n_), SParams(sp) {
    n_local = n / sp.world_size;
    weights = device_alloc<half_t>((size_t)k * n_local, "Linear_Col weights");
  }
  // argument block of the GEMM; the caller chooses the epilogue
  GEMM_ARGS args(const void* input, void* output, int m, int ldc) const {
    GEMM_ARGS a{};
    a.a = input; a.wt = weights; a.c = output;
    a.m = m; a.n = n_local; a.k = k;
    a.lda = k; a.ldw = k; a.ldc = ldc;
    a.n_begin = 0; a.n_end = n_local;
    a.epilogue = LIGER_EPI_STORE;
    return a;
  }
};

// ---- row-parallel linear: Y[M,n] = X[M, k/ws] * W[k/ws, n] partial sums (src/layer/linear.h:16-64) ----
class Linear_Row {
 public:
  int k, n;
  int k_local;
  half_t* weights;     // W^T shard, [n, k_local]
  StaticNvInitParam SParams;
  Linear_Row(const StaticNvInitParam& sp, int k_, int n_) : k(k_), n(n_), SParams(sp) {
    k_local = k / sp.world_size;
    weights = device_alloc<half_t>((size_t)n * k_local, "Linear_Row weights");
  }
  GEMM_ARGS args(const void* input, void* output, int m) const {
    GEMM_ARGS a{};
    a.a = input; a.wt = weights; a.c = output;
    a.m = m; a.n = n; a.k = k_local;
    a.lda = k_local; a.ldw = k_local; a.ldc = n;
    a.n_begin = 0; a.n_end = n;
    a.epilogue = LIGER_EPI_STORE;
    return a;
  }
};

inline FuncWrap make_gemm(int name, float placeholder_ms, const GEMM_ARGS& a) {
  GEMM_ARGS copy = a;
  return FuncWrap(name, placeholder_ms, GEMM,
                  [copy](const DynamicNvInitParam& d) { return liger_gemm_fp16(&copy, d.stream); }, copy);
}
inline FuncWrap make_comm(int name, float placeholder_ms, const COMM_ARGS& c) {
  COMM_ARGS copy = c;
  return FuncWrap(name, placeholder_ms, COMMUNICATION,
                  [copy](const DynamicNvInitParam& d) {
                    if (copy.copy_engine)
                      return liger_allreduce_ce(copy.comm, copy.channel, copy.partial_off, copy.recv_off, copy.out_off,
                                                copy.residual_in, copy.hidden, copy.bias, copy.gamma, copy.beta, copy.m,
                                                copy.n, copy.row_begin, copy.row_end, d.stream);
                    return liger_allreduce_fused(copy.comm, copy.channel, copy.partial_off, copy.out_off,
                                                 copy.residual_in, copy.hidden, copy.bias, copy.gamma, copy.beta,
                                                 copy.m, copy.n, copy.row_begin, copy.row_end, copy.one_shot, d.stream);
                  },
                  copy);
}

// ---- LayerNorm (src/layer/operator.h:16-40) -------------------------------------------------------
class LayerNorm {
 public:
  int k;
  half_t* gamma;
  half_t* beta;
  LayerNorm(int k_) : k(k_) {
    gamma = device_alloc<half_t>(k, "LayerNorm gamma");
    beta = device_alloc<half_t>(k, "LayerNorm beta");
  }
  FuncWrap forward(int name, const void* input, void* output, int m) const {
    const half_t *g = gamma, *b = beta;
    const int kk = k;
    return FuncWrap(name, 0.1f, COMPUTATION, [=](const DynamicNvInitParam& d) {
      return liger_layernorm(input, g, b, output, m, kk, d.stream);
    });
  }
};

// Per-request activation buffers.  The reference shares one workspace between all in-flight
// requests (src/layer/bert.h:98-101), which races as soon as two requests overlap; here every
// in-flight request gets its own slot.  `partial`, `normed` and `xbuf` live in the symmetric
// segment when world_size > 1 (peers read `partial` and write `normed` / `xbuf`).
struct Workspace {
  half_t* hidden = nullptr;   // residual stream [M, H] (pre-LN graph) / GEMM output staging (TP = 1)
  half_t* partial = nullptr;  // row-parallel GEMM output [M, H]
  half_t* normed = nullptr;   // LayerNorm output [M, H]
  half_t* xbuf = nullptr;     // layer output [M, H] (reference graph) / gathered final result
  half_t* q = nullptr;        // [B, h, S, D]
  half_t* k = nullptr;
  half_t* v = nullptr;
  half_t* attn = nullptr;     // [M, h*D]
  half_t* act = nullptr;      // [M, F/ws]
  float* decode_scratch = nullptr;
  size_t partial_off = 0, normed_off = 0, xbuf_off = 0, recv_off = 0;  // byte offsets inside the comm data region
  // decode: the two all-reduces of a layer read their partials from two different buffers in turn (`partial` and
  // the receive region), which lets the latency-bound one-shot all-reduce drop its exit barrier (mode 6)
  bool alternating_partials = false;
};

// What follows an all-reduce (or, with world_size == 1, the row-parallel GEMM): an optional
// residual add into the residual stream and an optional LayerNorm whose result every rank needs.
struct PostOp {
  const void* residual_in = nullptr;  // non-null: hidden = residual_in + sum + bias
  const half_t* bias = nullptr;
  const half_t* gamma = nullptr;      // non-null: out = LayerNorm(value); null: out = value
  const half_t* beta = nullptr;
  half_t* out = nullptr;              // where the LayerNorm / plain result goes (local address)
  size_t out_off = 0;                 // ... and its offset in the symmetric segment (world_size > 1)
  void* direct_out = nullptr;         // world_size == 1, no LayerNorm: the GEMM writes here
};

struct Shape {
  int batch, seq, slot;
  int M() const { return batch * seq; }
};

// ---- attention block: kernels 0-3 (src/layer/bert_layer.h:65-176) -----------------------------------
class Bert_MHA {
 public:
  int k, n;  // hidden in / out
  BertInitParam BertParams;
  StaticNvInitParam SParam;
  int heads_local, Hl, D;
  float scalar;                 // 1/sqrt(size_per_head), src/layer/bert_layer.h:94
  Linear_Col* linear_qkv_col;   // Q | K | V fused: W^T [3*H/ws, H]
  Linear_Row* linear_w_row;     // out-proj: W^T [H, H/ws]
  half_t* qkv_bias;             // [3*H/ws]
  half_t* w_bias;               // [H]; used by the pre-LN graph only (the reference declares it and never
                                // allocates it, src/layer/bert_layer.h:82)
  const half_t* attr_mask = nullptr;  // [B, S, S] or null = all ones (src/layer/bert_layer.h:118)

  Bert_MHA(const BertInitParam& bp, const StaticNvInitParam& sp, int k_, int n_) : k(k_), n(n_), BertParams(bp), SParam(sp) {
    heads_local = bp.head_num / sp.world_size; D = bp.size_per_head; Hl = heads_local * D;
    scalar = 1.0f / sqrtf((float)D);
    StaticNvInitParam one = sp; one.world_size = 1;  // shapes below are already rank-local
    linear_qkv_col = new Linear_Col(one, k, 3 * Hl);
    linear_w_row = new Linear_Row(one, Hl, n);
    qkv_bias = device_alloc<half_t>(3 * Hl, "qkv_bias");
    w_bias = device_alloc<half_t>(n, "w_bias");
  }
  ~Bert_MHA() { delete linear_qkv_col; delete linear_w_row; }
  Bert_MHA(const Bert_MHA&) = delete;
  Bert_MHA& operator=(const Bert_MHA&) = delete;

  std::vector<FuncWrap> forward(const void* input, Workspace& w, const PostOp& post, const Shape& sh) const {
    std::vector<FuncWrap> vec;
    const int M = sh.M(), ws = SParam.world_size;
    {  // 0: fused QKV GEMM + bias + head split
      GEMM_ARGS a = linear_qkv_col->args(input, nullptr, M, 0);
      a.epilogue = LIGER_EPI_QKV_SPLIT; a.bias = qkv_bias;
      a.q_out = w.q; a.k_out = w.k; a.v_out = w.v;
      a.seq_len = sh.seq; a.heads = heads_local; a.head_dim = D;
      vec.push_back(make_gemm(0, 1.0f, a));
    }
    {  // 1: attention (QK^T, masked softmax, PV, head merge in one kernel)
      const half_t *q = w.q, *kk = w.k, *v = w.v; half_t* o = w.attn;
      const half_t* mk = attr_mask;
      const int hl = heads_local, d = D, ldo = Hl, causal = BertParams.causal, B = sh.batch, S = sh.seq;
      const float sc = scalar;
      vec.push_back(FuncWrap(1, 0.3f, COMPUTATION, [=](const DynamicNvInitParam& dp) {
        return liger_attention_prefill(q, kk, v, mk, o, B, hl, S, d, ldo, sc, causal, dp.stream);
      }));
    }
    {  // 2: out-proj (row parallel)
      GEMM_ARGS a = linear_w_row->args(w.attn, w.partial, M);
      if (ws == 1 && post.residual_in) {  // no all-reduce to fuse the residual into: use the epilogue
        a.epilogue = LIGER_EPI_RESIDUAL; a.bias = post.bias; a.residual = post.residual_in; a.ldr = n;
        a.c = w.hidden;
      } else if (ws > 1 && !is_one_shot(M, n) && !use_copy_engines()) {  // reduce-scatter by the epilogue's own stores
        a.epilogue = LIGER_EPI_SCATTER; a.scatter_comm = SParam.comm; a.scatter_off = w.partial_off;
      }
      vec.push_back(make_gemm(2, 2.0f, a));
    }
    vec.push_back(post_kernel(3, w, post, sh, SParam, n));
    return vec;
  }

  // One decode step (no counterpart in the reference, which has no KV cache): one new token per
  // sequence.  Kernel 0 appends the token's K and V to the cache at position kv_len, kernel 1 is the
  // split-KV decode attention over kv_len + 1 positions; kernels 2-3 are the prefill ones with M = batch.
  std::vector<FuncWrap> forward_decode(const void* input, Workspace& w, const PostOp& post, const Shape& sh, half_t* k_cache,
                                       half_t* v_cache, int kv_len, int kv_cap) const {
    std::vector<FuncWrap> vec;
    const int M = sh.batch, ws = SParam.world_size;
    {
      GEMM_ARGS a = linear_qkv_col->args(input, nullptr, M, 0);
      a.epilogue = LIGER_EPI_QKV_SPLIT; a.bias = qkv_bias;
      a.q_out = w.q; a.k_out = k_cache; a.v_out = v_cache;
      a.seq_len = 1; a.heads = heads_local; a.head_dim = D; a.kv_stride = kv_cap; a.kv_pos = kv_len;
      vec.push_back(make_gemm(0, 1.0f, a));
    }
    {
      const half_t* q = w.q; half_t* o = w.attn; float* scratch = w.decode_scratch;
      const int hl = heads_local, d = D, ldo = Hl, B = sh.batch, L = kv_len + 1;
      const float sc = scalar;
      vec.push_back(FuncWrap(1, 0.3f, COMPUTATION, [=](const DynamicNvInitParam& dp) {
        return liger_attention_decode(q, k_cache, v_cache, o, scratch, B, hl, L, kv_cap, d, ldo, sc, dp.stream);
      }));
    }
    {
      GEMM_ARGS a = linear_w_row->args(w.attn, w.partial, M);
      if (ws == 1 && post.residual_in) {
        a.epilogue = LIGER_EPI_RESIDUAL; a.bias = post.bias; a.residual = post.residual_in; a.ldr = n; a.c = w.hidden;
      } else if (ws > 1 && !is_one_shot(M, n) && !use_copy_engines()) {
        a.epilogue = LIGER_EPI_SCATTER; a.scatter_comm = SParam.comm; a.scatter_off = w.partial_off;
      }
      vec.push_back(make_gemm(2, 2.0f, a));
    }
    Shape flat{sh.batch, 1, sh.slot};
    vec.push_back(post_kernel(3, w, post, flat, SParam, n));
    return vec;
  }

  // kernel 3 / 6: fused all-reduce (+ residual) + LayerNorm, or a plain LayerNorm when world_size == 1
  static FuncWrap post_kernel(int name, Workspace& w, const PostOp& post, const Shape& sh, const StaticNvInitParam& sp,
                              int n) {
    const int M = sh.M();
    if (sp.world_size > 1) {
      COMM_ARGS c;
      c.comm = sp.comm; c.channel = sh.slot; c.partial_off = w.partial_off; c.out_off = post.out_off;
      c.m = M; c.n = n; c.row_begin = 0; c.row_end = M;
      c.one_shot = is_one_shot(M, n) ? (w.alternating_partials ? 6 : 1) : 3;
      if (!is_one_shot(M, n) && use_copy_engines()) { c.copy_engine = 1; c.recv_off = w.recv_off; }
      if (post.residual_in) { c.residual_in = post.residual_in; c.hidden = w.hidden; c.bias = post.bias; }
      c.gamma = post.gamma; c.beta = post.beta;
      return make_comm(name, 2.0f, c);
    }
    const void* src = post.residual_in ? (const void*)w.hidden : (const void*)w.partial;
    const half_t *g = post.gamma, *b = post.beta; half_t* out = post.out;
    return FuncWrap(name, 0.1f, COMPUTATION, [=](const DynamicNvInitParam& d) {
      return liger_layernorm(src, g, b, out, M, n, d.stream);
    });
  }
  // payloads up to 1 MiB (decode) are latency bound: every rank reduces everything itself
  static bool is_one_shot(int M, int n) { return (size_t)M * n * 2 <= ((size_t)1 << 20); }
  // LIGER_COMM_MODE=ce moves the inter-GPU traffic of the two-shot collective to the copy engines
  // (liger_allreduce_ce); the default keeps it in the kernels (GEMM epilogue scatter + fused all-reduce).
  static bool use_copy_engines() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("LIGER_COMM_MODE"); v = (e && std::string(e) == "ce") ? 1 : 0; }
    return v == 1;
  }
};

// ---- MLP block: kernels 4-6 (src/layer/bert_layer.h:19-63) --------------------------------------------
class Bert_MLP {
 public:
  int k, n, intermediate_size;
  BertInitParam BertParams;
  StaticNvInitParam SParam;
  int Fl, up_cols_local;
  Linear_Col* linear_col;  // FFN-up: W^T [F/ws or 2F/ws (gate/value interleaved by 32), H]
  Linear_Row* linear_row;  // FFN-down: W^T [H, F/ws]
  half_t* bias;            // FFN-up bias, same row order as linear_col
  half_t* down_bias;       // [H]; pre-LN graph only

  Bert_MLP(const BertInitParam& bp, const StaticNvInitParam& sp, int k_, int n_) : k(k_), n(n_), BertParams(bp), SParam(sp) {
    intermediate_size = bp.ffn();
    Fl = intermediate_size / sp.world_size;
    up_cols_local = bp.act == ACT_GEGLU ? 2 * Fl : Fl;
    StaticNvInitParam one = sp; one.world_size = 1;
    linear_col = new Linear_Col(one, k, up_cols_local);
    linear_row = new Linear_Row(one, Fl, n);
    bias = device_alloc<half_t>(up_cols_local, "ffn bias");
    down_bias = device_alloc<half_t>(n, "ffn down bias");
  }
  ~Bert_MLP() { delete linear_col; delete linear_row; }
  Bert_MLP(const Bert_MLP&) = delete;
  Bert_MLP& operator=(const Bert_MLP&) = delete;

  // has_post = false only for the last layer of the pre-LN graph with world_size == 1 (nothing follows)
  std::vector<FuncWrap> forward(const void* input, Workspace& w, const PostOp& post, const Shape& sh) const {
    std::vector<FuncWrap> vec;
    const int M = sh.M(), ws = SParam.world_size;
    {  // 4: FFN-up + bias + activation
      GEMM_ARGS a = linear_col->args(input, w.act, M, Fl);
      a.bias = bias;
      a.epilogue = BertParams.act == ACT_GEGLU ? LIGER_EPI_GEGLU : LIGER_EPI_GELU;
      vec.push_back(make_gemm(4, 1.0f, a));
    }
    {  // 5: FFN-down (row parallel)
      GEMM_ARGS a = linear_row->args(w.act, w.partial, M);
      if (ws == 1 && post.residual_in) {
        a.epilogue = LIGER_EPI_RESIDUAL; a.bias = post.bias; a.residual = post.residual_in; a.ldr = n;
        a.c = post.direct_out ? post.direct_out : (void*)w.hidden;
      } else if (ws > 1 && !Bert_MHA::is_one_shot(M, n) && !Bert_MHA::use_copy_engines()) {
        a.epilogue = LIGER_EPI_SCATTER; a.scatter_comm = SParam.comm; a.scatter_off = w.partial_off;
      }
      vec.push_back(make_gemm(5, 2.0f, a));
    }
    if (ws > 1 || post.gamma) vec.push_back(Bert_MHA::post_kernel(6, w, post, sh, SParam, n));
    return vec;
  }
};

// ---- one layer (src/layer/bert.h:18-80) -----------------------------------------------------------------
class Bert_Encoder {
 public:
  Bert_MHA* MHA;
  Bert_MLP* MLP;
  LayerNorm* ln_mha;  // reference graph: after the attention block; pre-LN graph: before it
  LayerNorm* ln_mlp;  // reference graph: after the MLP block;       pre-LN graph: before it
  half_t* k_cache = nullptr;  // [B_max, h, kv_capacity, D]
  half_t* v_cache = nullptr;
  Bert_Encoder(const BertInitParam& bp, const StaticNvInitParam& sp, int k, int n) {
    MHA = new Bert_MHA(bp, sp, k, n);
    MLP = new Bert_MLP(bp, sp, k, n);
    ln_mha = new LayerNorm(k);
    ln_mlp = new LayerNorm(k);
  }
  ~Bert_Encoder() { delete MHA; delete MLP; delete ln_mha; delete ln_mlp; }
  Bert_Encoder(const Bert_Encoder&) = delete;
  Bert_Encoder& operator=(const Bert_Encoder&) = delete;
  // concatenation of the two blocks' kernel vectors (src/layer/bert.h:59-79)
  std::vector<FuncWrap> forward(const void* mha_in, const PostOp& mha_post, const void* mlp_in, const PostOp& mlp_post,
                                Workspace& w, const Shape& sh) const {
    std::vector<FuncWrap> vec = MHA->forward(mha_in, w, mha_post, sh);
    std::vector<FuncWrap> tmp = MLP->forward(mlp_in, w, mlp_post, sh);
    vec.insert(vec.end(), tmp.begin(), tmp.end());
    return vec;
  }
};

// ---- the model: owns weights and workspaces; assembles the kernel vector of a request -------------------
class Bert_Model {
 public:
  int k, n;
  BertInitParam BertParams;
  StaticNvInitParam SParam;
  int H, F, D, heads_local, Hl, Fl;
  std::vector<Bert_Encoder*> encoders;
  std::vector<Workspace> slots;
  int next_slot = 0;
  std::vector<void*> allocations;  // every cudaMalloc made for this model; freed by the destructor

  // Unlike the reference's model (no destructors anywhere), this one owns its device memory: destroying it
  // frees weights, caches and workspaces.  Closures returned by forward() must not outlive it.
  ~Bert_Model() {
    for (auto* e : encoders) delete e;
    for (void* p : allocations) cudaFree(p);
  }
  Bert_Model(const Bert_Model&) = delete;
  Bert_Model& operator=(const Bert_Model&) = delete;

  Bert_Model(const BertInitParam& bp, const StaticNvInitParam& sp) : BertParams(bp), SParam(sp) {
    struct SinkGuard {
      std::vector<void*>* prev;
      explicit SinkGuard(std::vector<void*>* mine) : prev(alloc_sink()) { alloc_sink() = mine; }
      ~SinkGuard() { alloc_sink() = prev; }
    } guard(&allocations);
    const int ws = sp.world_size;
    H = bp.hidden(); F = bp.ffn(); D = bp.size_per_head; k = n = H;
    if (ws < 1 || bp.head_num % ws || F % ws || H % 8 || D % 8)
      throw std::runtime_error("Bert_Model: head_num and ffn_inner must divide by world_size, H and D by 8");
    if (ws > 1 && !sp.comm) throw std::runtime_error("Bert_Model: world_size > 1 needs a communicator");
    heads_local = bp.head_num / ws; Hl = H / ws; Fl = F / ws;
    if (bp.act == ACT_GEGLU && Fl % 32) throw std::runtime_error("Bert_Model: GeGLU needs ffn_inner/world_size % 32 == 0");
    for (int l = 0; l < bp.layer_num; ++l) encoders.push_back(new Bert_Encoder(bp, sp, H, H));
    init_weights();
    init_workspaces();
  }

  size_t tokens_max() const { return (size_t)BertParams.max_batch_size * BertParams.max_seq_len; }

  // bytes of symmetric memory the model needs from the communicator's data region
  static size_t comm_bytes_needed(const BertInitParam& bp) {
    // + kMaxRanks rows: the scattered layout [ws][ceil(M/ws)][H] can exceed M rows by up to ws - 1
    const size_t mh = round_up(((size_t)bp.max_batch_size * bp.max_seq_len + LIGER_COMM_MAX_RANKS) * bp.hidden() * 2, 256);
    return 4 * mh * (size_t)(bp.workspace_slots > 0 ? bp.workspace_slots : 1);
  }

  // The flat kernel vector of one request: layer_num encoders back to back (src/layer/bert.h:104-115).
  // `slot` selects the activation workspace; -1 = round robin.
  std::vector<FuncWrap> forward(const void* input, void* output, int batch_size, int seq_len, int slot = -1) {
    if (batch_size < 1 || seq_len < 1 || (size_t)batch_size * seq_len > tokens_max() ||
        batch_size > BertParams.max_batch_size)
      throw std::runtime_error("Bert_Model::forward: batch/seq outside the configured maximum");
    if (slot < 0) { slot = next_slot; next_slot = (next_slot + 1) % (int)slots.size(); }
    Workspace& w = slots.at(slot);
    const Shape sh{batch_size, seq_len, slot};
    const int ws = SParam.world_size, L = BertParams.layer_num, M = sh.M();
    const bool preln = BertParams.graph == GRAPH_PRELN;
    std::vector<FuncWrap> vec;
    vec.reserve((size_t)L * kKernelsPerLayer + 2);

    if (preln) vec.push_back(encoders[0]->ln_mha->forward(kPrologueName, input, w.normed, M));
    const void* x = input;      // reference graph: the layer's input
    const void* resid = input;  // pre-LN graph: where the residual stream currently lives
    for (int l = 0; l < L; ++l) {
      const Bert_Encoder* e = encoders[l];
      const bool last = (l == L - 1);
      PostOp mha_post, mlp_post;
      if (preln) {
        // h = resid + attn_out + b_o ; normed = LN_mlp(h)
        mha_post.residual_in = resid; mha_post.bias = e->MHA->w_bias;
        mha_post.gamma = e->ln_mlp->gamma; mha_post.beta = e->ln_mlp->beta;
        mha_post.out = w.normed; mha_post.out_off = w.normed_off;
        // h = h + ffn_out + b_down ; normed = LN_mha(next layer)(h), or the final result
        mlp_post.residual_in = w.hidden; mlp_post.bias = e->MLP->down_bias;
        if (!last) {
          mlp_post.gamma = encoders[l + 1]->ln_mha->gamma; mlp_post.beta = encoders[l + 1]->ln_mha->beta;
          mlp_post.out = w.normed; mlp_post.out_off = w.normed_off;
        } else {
          mlp_post.out = w.xbuf; mlp_post.out_off = w.xbuf_off;
          if (ws == 1) mlp_post.direct_out = output;
        }
        std::vector<FuncWrap> t = e->forward(w.normed, mha_post, w.normed, mlp_post, w, sh);
        vec.insert(vec.end(), t.begin(), t.end());
        resid = w.hidden;
      } else {
        // normed = LN_mha(sum) ; x_next = LN_mlp(sum)   (src/layer/bert.h:65-76)
        mha_post.gamma = e->ln_mha->gamma; mha_post.beta = e->ln_mha->beta;
        mha_post.out = w.normed; mha_post.out_off = w.normed_off;
        mlp_post.gamma = e->ln_mlp->gamma; mlp_post.beta = e->ln_mlp->beta;
        mlp_post.out = (last && ws == 1) ? (half_t*)output : w.xbuf; mlp_post.out_off = w.xbuf_off;
        std::vector<FuncWrap> t = e->forward(x, mha_post, w.normed, mlp_post, w, sh);
        vec.insert(vec.end(), t.begin(), t.end());
        x = w.xbuf;
      }
    }
    if (ws > 1) {  // the gathered result sits in the symmetric segment: copy it to the caller's buffer
      const void* src = w.xbuf; const size_t bytes = (size_t)M * H * 2;
      vec.push_back(FuncWrap(kEpilogueName, 0.05f, COMPUTATION, [=](const DynamicNvInitParam& dp) {
        cudaError_t err = cudaMemcpyAsync(output, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)dp.stream);
        return err == cudaSuccess ? LIGER_OK : LIGER_ERR_CUDA;
      }));
    }
    return vec;
  }

  // One decode step for `batch` sequences whose caches hold kv_len positions: input / output are
  // [batch, H]; pre-LayerNorm graph only.  The caches must have been created (kv_capacity > 0).
  std::vector<FuncWrap> forward_decode(const void* input, void* output, int batch_size, int kv_len, int slot = -1) {
    if (BertParams.graph != GRAPH_PRELN) throw std::runtime_error("Bert_Model::forward_decode: pre-LayerNorm graph only");
    if (BertParams.kv_capacity <= 0 || kv_len < 0 || kv_len + 1 > BertParams.kv_capacity)
      throw std::runtime_error("Bert_Model::forward_decode: kv_len + 1 exceeds the KV-cache capacity");
    if (batch_size < 1 || batch_size > BertParams.max_batch_size)
      throw std::runtime_error("Bert_Model::forward_decode: batch outside the configured maximum");
    if (slot < 0) { slot = next_slot; next_slot = (next_slot + 1) % (int)slots.size(); }
    Workspace& w = slots.at(slot);
    const Shape sh{batch_size, 1, slot};
    const int ws = SParam.world_size, L = BertParams.layer_num, M = batch_size;
    std::vector<FuncWrap> vec;
    vec.push_back(encoders[0]->ln_mha->forward(kPrologueName, input, w.normed, M));
    const void* resid = input;
    for (int l = 0; l < L; ++l) {
      const Bert_Encoder* e = encoders[l];
      const bool last = (l == L - 1);
      PostOp mha_post, mlp_post;
      mha_post.residual_in = resid; mha_post.bias = e->MHA->w_bias;
      mha_post.gamma = e->ln_mlp->gamma; mha_post.beta = e->ln_mlp->beta;
      mha_post.out = w.normed; mha_post.out_off = w.normed_off;
      mlp_post.residual_in = w.hidden; mlp_post.bias = e->MLP->down_bias;
      if (!last) {
        mlp_post.gamma = encoders[l + 1]->ln_mha->gamma; mlp_post.beta = encoders[l + 1]->ln_mha->beta;
        mlp_post.out = w.normed; mlp_post.out_off = w.normed_off;
      } else {
        mlp_post.out = w.xbuf; mlp_post.out_off = w.xbuf_off;
        if (ws == 1) mlp_post.direct_out = output;
      }
      // attention block: partials in `partial`; MLP block: partials in the receive region (unused by the one-shot path)
      Workspace wa = w, wb = w;
      if (ws > 1 && Bert_MHA::is_one_shot(M, H)) {
        wa.alternating_partials = wb.alternating_partials = true;
        wb.partial = (half_t*)((uint8_t*)liger_comm_data(SParam.comm) + w.recv_off);
        wb.partial_off = w.recv_off;
      }
      std::vector<FuncWrap> t = e->MHA->forward_decode(w.normed, wa, mha_post, sh, e->k_cache, e->v_cache, kv_len,
                                                       BertParams.kv_capacity);
      vec.insert(vec.end(), t.begin(), t.end());
      t = e->MLP->forward(w.normed, wb, mlp_post, sh);
      vec.insert(vec.end(), t.begin(), t.end());
      resid = w.hidden;
    }
    if (ws > 1) {
      const void* src = w.xbuf; const size_t bytes = (size_t)M * H * 2;
      vec.push_back(FuncWrap(kEpilogueName, 0.05f, COMPUTATION, [=](const DynamicNvInitParam& dp) {
        cudaError_t err = cudaMemcpyAsync(output, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)dp.stream);
        return err == cudaSuccess ? LIGER_OK : LIGER_ERR_CUDA;
      }));
    }
    return vec;
  }

  // Fills every layer's KV cache with the seeded N(0,1) tensors (ids 0x10001 + 2*layer for keys,
  // 0x10002 + 2*layer for values; logical layout [batch][heads][kv_capacity][head_dim], this rank
  // keeping its own heads).
  void fill_kv_cache_seeded() {
    const int cap = BertParams.kv_capacity, hl = heads_local, heads = BertParams.head_num, r = SParam.world_rank;
    if (cap <= 0) throw std::runtime_error("Bert_Model::fill_kv_cache_seeded: no KV cache configured");
    for (int l = 0; l < BertParams.layer_num; ++l)
      for (int b = 0; b < BertParams.max_batch_size; ++b) {
        // rows = this rank's heads x cap positions, D columns; logical row index = (b*heads + head)*cap + pos
        half_t* kd = encoders[l]->k_cache + (size_t)b * hl * cap * D;
        half_t* vd = encoders[l]->v_cache + (size_t)b * hl * cap * D;
        const int row0 = (b * heads + r * hl) * cap;
        fill(kd, hl * cap, D, D, row0, 0, D, 0x10001u + 2u * (uint32_t)l, 0.0f, 1.0f, 0);
        fill(vd, hl * cap, D, D, row0, 0, D, 0x10002u + 2u * (uint32_t)l, 0.0f, 1.0f, 0);
      }
    cuda_check(cudaDeviceSynchronize(), "fill_kv_cache_seeded");
  }

  // number of distinct kernel names a request can contain (profile dictionary keys 0 .. n-1)
  int kernel_names() const { return kEpilogueName + 1; }

  // attention mask [B, S, S] shared by all layers (null = all ones)
  void set_mask(const half_t* mask) { for (auto* e : encoders) e->MHA->attr_mask = mask; }

 private:
  void fill(half_t* dst, int rows, int cols, int dst_ld, int row0, int col0, int src_ld, uint32_t id, float mean,
            float std, int mode) {
    host_check(liger_fill_normal(dst, rows, cols, dst_ld, row0, col0, src_ld, BertParams.seed, id, mean, std, mode,
                                 nullptr),
               "liger_fill_normal");
  }

  // Weights are generated at their full (unsharded) logical shape W[k][n] and each rank keeps its
  // slice, so results do not depend on world_size: column-parallel layers keep columns
  // [r*n/ws, (r+1)*n/ws), row-parallel layers rows likewise (src/layer/linear.h:40,92 allocate
  // k*n/ws elements per rank the same way but never initialise them).
  void init_weights() {
    const int r = SParam.world_rank;
    const int upw = BertParams.act == ACT_GEGLU ? 2 * F : F;
    for (int l = 0; l < BertParams.layer_num; ++l) {
      const uint32_t id0 = (uint32_t)l * 32u;
      Bert_Encoder* e = encoders[l];
      const uint32_t wq[3] = {W_Q, W_K, W_V}, bq[3] = {B_Q, B_K, B_V};
      for (int t = 0; t < 3; ++t) {
        // rows [t*Hl, (t+1)*Hl) of the fused W^T hold columns [r*Hl, (r+1)*Hl) of W_t
        fill(e->MHA->linear_qkv_col->weights + (size_t)t * Hl * H, H, Hl, H, 0, r * Hl, H, id0 + wq[t], 0.0f, kWeightStd, 1);
        fill(e->MHA->qkv_bias + t * Hl, 1, Hl, Hl, 0, r * Hl, H, id0 + bq[t], 0.0f, kWeightStd, 0);
      }
      fill(e->MHA->linear_w_row->weights, Hl, H, Hl, r * Hl, 0, H, id0 + W_O, 0.0f, kWeightStd, 1);
      half_t* wup = e->MLP->linear_col->weights;
      if (BertParams.act == ACT_GEGLU) {
        fill(wup, H, Fl, H, 0, r * Fl, upw, id0 + W_UP, 0.0f, kWeightStd, 2);
        fill(wup, H, Fl, H, 0, F + r * Fl, upw, id0 + W_UP, 0.0f, kWeightStd, 3);
        // the bias in the same interleaved order: a [1, Fl] "matrix" written transposed
        fill(e->MLP->bias, 1, Fl, 1, 0, r * Fl, upw, id0 + B_UP, 0.0f, kWeightStd, 2);
        fill(e->MLP->bias, 1, Fl, 1, 0, F + r * Fl, upw, id0 + B_UP, 0.0f, kWeightStd, 3);
      } else {
        fill(wup, H, Fl, H, 0, r * Fl, upw, id0 + W_UP, 0.0f, kWeightStd, 1);
        fill(e->MLP->bias, 1, Fl, Fl, 0, r * Fl, upw, id0 + B_UP, 0.0f, kWeightStd, 0);
      }
      fill(e->MLP->linear_row->weights, Fl, H, Fl, r * Fl, 0, H, id0 + W_DOWN, 0.0f, kWeightStd, 1);
      fill(e->MHA->w_bias, 1, H, H, 0, 0, H, id0 + B_O, 0.0f, kWeightStd, 0);
      fill(e->MLP->down_bias, 1, H, H, 0, 0, H, id0 + B_DOWN, 0.0f, kWeightStd, 0);
      fill(e->ln_mha->gamma, 1, H, H, 0, 0, H, id0 + LN1_G, 1.0f, kWeightStd, 0);
      fill(e->ln_mha->beta, 1, H, H, 0, 0, H, id0 + LN1_B, 0.0f, kWeightStd, 0);
      fill(e->ln_mlp->gamma, 1, H, H, 0, 0, H, id0 + LN2_G, 1.0f, kWeightStd, 0);
      fill(e->ln_mlp->beta, 1, H, H, 0, 0, H, id0 + LN2_B, 0.0f, kWeightStd, 0);
      if (BertParams.kv_capacity > 0) {
        const size_t cnt = (size_t)BertParams.max_batch_size * heads_local * BertParams.kv_capacity * D;
        e->k_cache = device_alloc<half_t>(cnt, "k_cache");
        e->v_cache = device_alloc<half_t>(cnt, "v_cache");
      }
    }
    cuda_check(cudaDeviceSynchronize(), "init_weights");
  }

  void init_workspaces() {
    const int ws = SParam.world_size;
    const size_t M = tokens_max();
    const size_t mh = round_up((M + LIGER_COMM_MAX_RANKS) * H * 2, 256);
    const int nslots = BertParams.workspace_slots > 0 ? BertParams.workspace_slots : 1;
    uint8_t* sym = nullptr;
    if (ws > 1) {
      if (liger_comm_data_bytes(SParam.comm) < 4 * mh * nslots)
        throw std::runtime_error("Bert_Model: communicator data region smaller than comm_bytes_needed()");
      sym = (uint8_t*)liger_comm_data(SParam.comm);
    }
    for (int s = 0; s < nslots; ++s) {
      Workspace w;
      if (ws > 1) {
        w.partial_off = (size_t)s * 4 * mh; w.normed_off = w.partial_off + mh; w.xbuf_off = w.normed_off + mh;
        w.recv_off = w.xbuf_off + mh;
        w.partial = (half_t*)(sym + w.partial_off);
        w.normed = (half_t*)(sym + w.normed_off);
        w.xbuf = (half_t*)(sym + w.xbuf_off);
      } else {
        w.partial = device_alloc<half_t>(M * H, "ws.partial");
        w.normed = device_alloc<half_t>(M * H, "ws.normed");
        w.xbuf = device_alloc<half_t>(M * H, "ws.xbuf");
      }
      w.hidden = device_alloc<half_t>(M * H, "ws.hidden");
      w.q = device_alloc<half_t>(M * Hl, "ws.q");
      w.k = device_alloc<half_t>(M * Hl, "ws.k");
      w.v = device_alloc<half_t>(M * Hl, "ws.v");
      w.attn = device_alloc<half_t>(M * Hl, "ws.attn");
      w.act = device_alloc<half_t>(M * Fl, "ws.act");
      if (BertParams.kv_capacity > 0) {
        const size_t bytes = liger_attention_decode_scratch_bytes(BertParams.max_batch_size, heads_local, D,
                                                                  BertParams.kv_capacity);
        w.decode_scratch = (float*)device_alloc<uint8_t>(bytes, "ws.decode_scratch");
      }
      slots.push_back(w);
    }
  }
};

}  // namespace liger_host
