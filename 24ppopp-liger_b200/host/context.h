// Host-side types of the serving path: run-time parameters, the kernel-vector element
// (FuncWrap) and the profile-dictionary key.  Names and meaning follow the reference's
// src/context.h:14-169 so that code written against it reads the same; what a FuncWrap launches
// is this library's own kernels (include/liger_b200.h) instead of cuBLAS / NCCL calls.
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "../../include/liger_b200.h"

namespace liger_host {

// Stream (and its priority) a kernel is launched on.  The reference's DynamicNvInitParam also
// carries a cuBLAS handle (src/context.h:14-31); no library handle is needed here.
// `stream` is an opaque handle owned by the Runtime (a cudaStream_t for the CUDA runtime).
struct DynamicNvInitParam {
  void* stream = nullptr;
  int priority = 0;
  int index = 0;  // 0 = main stream, 1 = secondary stream
};

// Per-process constants: rank, world size and the communicator (src/context.h:33-56).
struct StaticNvInitParam {
  int world_size = 1;
  int world_rank = 0;
  liger_comm* comm = nullptr;
  int datatype = 1;  // 1 = fp16, the only type the kernels implement (src/main.cu:35 selects it)
  StaticNvInitParam() {}
  StaticNvInitParam(int world_rank_, int world_size_, liger_comm* comm_, int datatype_ = 1)
      : world_size(world_size_), world_rank(world_rank_), comm(comm_), datatype(datatype_) {}
};

enum graph_type {
  GRAPH_REF = 0,    // MHA -> all-reduce -> LayerNorm -> MLP -> all-reduce -> LayerNorm, no residual
                    // (the reference's Bert_Encoder::forward, src/layer/bert.h:59-79)
  GRAPH_PRELN = 1   // pre-LayerNorm with residual adds (add_bias_input_layernorm_2 semantics,
                    // src/cuda/cuda_kernels.cu:360-409)
};
enum act_type { ACT_GELU = 0, ACT_GEGLU = 1 };

// Model / serving configuration: the reference's eight integers (src/main.cu:14-21,
// src/context.h:58-85) plus the fields the reference hard-codes or lacks.
struct BertInitParam {
  int max_batch_size = 2;
  int max_seq_len = 128;
  int head_num = 128;
  int size_per_head = 96;
  int layer_num = 4;
  int kernel_num = 7;    // kernels per layer in this implementation's fused layer (see layers.h)
  int factor = 8;        // decomposition factor
  int rq_interval = 12500;  // microseconds between requests
  // ---- extensions ----
  int graph = GRAPH_REF;
  int act = ACT_GELU;
  int ffn_inner = 0;     // 0 -> 4 * hidden (src/layer/bert_layer.h:23)
  int causal = 0;        // 1 -> causal mask by construction; 0 -> mask tensor (all ones by default)
  uint32_t seed = 0;
  int num_requests = 150;   // src/schedule.h:295
  int ignore_num = 20;      // src/schedule.h:327
  int schedule_deep = 6;    // src/schedule.h:30
  float contention = 0.8f;  // src/schedule.h:249; 0 -> the two factors the profile run derived (Scheduler::calibrate_contention)
  float min_slice_efficiency = 0.0f;  // a GEMM slice is used only if it runs at this fraction of the whole kernel's rate
                                      // (0: every slice that fits, as the reference, src/init.h:226-259)
  int poisson = 0;          // 0: fixed-interval arrivals (src/schedule.h:301), 1: exponential gaps
  int min_seq_len = 16;     // src/schedule.h:298 draws rand() % (max_seq_len - 28) + 16
  int seq_round = 4;        // request lengths are rounded up to a multiple of this
  int workspace_slots = 7;  // activation workspaces (schedule_deep in flight + 1 being admitted)
  int kv_capacity = 0;      // > 0 allocates a KV cache of this many positions per sequence (decode)
  BertInitParam() {}
  BertInitParam(int max_batch_size_, int max_seq_len_, int head_num_, int size_per_head_, int layer_num_,
                int kernel_num_, int factor_, int rq_interval_)
      : max_batch_size(max_batch_size_), max_seq_len(max_seq_len_), head_num(head_num_),
        size_per_head(size_per_head_), layer_num(layer_num_), kernel_num(kernel_num_), factor(factor_),
        rq_interval(rq_interval_) {}
  int hidden() const { return head_num * size_per_head; }
  int ffn() const { return ffn_inner > 0 ? ffn_inner : 4 * hidden(); }
};

enum layer_type { COMMUNICATION, COMPUTATION, GEMM };  // src/context.h:87

// What the reference keeps as an 18-element cuBLAS argument tuple (GEMM_ARGS, src/context.h:89-92)
// is here the argument block of liger_gemm_fp16; a decomposed kernel is the same block with a
// narrower [n_begin, n_end).
typedef liger_gemm_args GEMM_ARGS;

// COMM_ARGS (src/context.h:94): the arguments of one fused all-reduce launch.
struct COMM_ARGS {
  liger_comm* comm = nullptr;
  int channel = 0;
  size_t partial_off = 0, out_off = 0;
  size_t recv_off = 0;  // receive slots of the copy-engine variant
  int copy_engine = 0;  // 1: liger_allreduce_ce instead of liger_allreduce_fused
  const void* residual_in = nullptr;
  void* hidden = nullptr;
  const void* bias = nullptr;
  const void* gamma = nullptr;
  const void* beta = nullptr;
  int m = 0, n = 0, row_begin = 0, row_end = 0, one_shot = 0;
};

// One element of the function-assembled kernel vector (src/context.h:96-153).  `callback`
// launches the kernel on the given stream and returns a LIGER_* status.
class FuncWrap {
 public:
  int name = -1;          // kernel id within a layer; key of the profile dictionaries
  float duration = 0.0f;  // profiled milliseconds (a placeholder until serve() fills it in)
  layer_type type = COMPUTATION;
  std::function<int(const DynamicNvInitParam&)> callback;
  GEMM_ARGS args_gemm_tuple{};
  COMM_ARGS args_comm_tuple{};
  int units_begin = 0, units_end = 0;  // decomposed slices: [begin, end) in units of 1/factor
  // Optional: builds the launch closure of the slice [units_begin, units_end) of this kernel.  Left
  // empty by the CUDA model (slices then re-use args_gemm_tuple / args_comm_tuple); a simulated
  // model sets it so that slices launch on the simulated device.
  std::function<std::function<int(const DynamicNvInitParam&)>(int units_begin, int units_end, int factor)> slicer;

  FuncWrap() {}
  FuncWrap(int name_, float duration_, layer_type type_, std::function<int(const DynamicNvInitParam&)> cb)
      : name(name_), duration(duration_), type(type_), callback(std::move(cb)) {}
  FuncWrap(int name_, float duration_, layer_type type_, std::function<int(const DynamicNvInitParam&)> cb,
           const GEMM_ARGS& g)
      : name(name_), duration(duration_), type(type_), callback(std::move(cb)), args_gemm_tuple(g) {}
  FuncWrap(int name_, float duration_, layer_type type_, std::function<int(const DynamicNvInitParam&)> cb,
           const COMM_ARGS& c)
      : name(name_), duration(duration_), type(type_), callback(std::move(cb)), args_comm_tuple(c) {}
  bool not_comm() const { return type != COMMUNICATION; }
};

// Key of the profile dictionaries (src/context.h:155-169).
struct kernel_info {
  int kernel_name;
  int batch_size;
  int seq_len;
  bool operator==(const kernel_info& o) const {
    return kernel_name == o.kernel_name && batch_size == o.batch_size && seq_len == o.seq_len;
  }
};
struct KeyHash {
  std::size_t operator()(const kernel_info& k) const {
    // the reference XORs the three field hashes, which collides for permuted keys; mix instead
    std::size_t h = (std::size_t)k.kernel_name * 0x9E3779B97F4A7C15ull;
    h ^= (std::size_t)k.batch_size + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= (std::size_t)k.seq_len + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    return h;
  }
};
typedef std::unordered_map<kernel_info, float, KeyHash> MainDict;
typedef std::unordered_map<kernel_info, std::vector<float>, KeyHash> SubDict;

}  // namespace liger_host
