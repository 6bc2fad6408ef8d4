// C ABI over the host-side runtime (host/*.h): model construction and forward pass, the three
// serving entry points, and the scheduler on a simulated device.
#define LIGER_HOST_WITH_CUDA 1
#include <memory>
#include <string>

#include "../host/layers.h"
#include "../host/profile_io.h"
#include "../host/runtime_iface.h"
#include "../host/sample.h"
#include "../host/scheduler.h"
#include "../host/test_schedule.h"
#include "runtime.h"

using namespace liger_host;

struct liger_model {
  BertInitParam bp;
  StaticNvInitParam sp;
  Bert_Model* model = nullptr;
  half_t* io_in = nullptr;   // device staging for the host-buffer entry point
  half_t* io_out = nullptr;
  int device = 0;
  bool timing = false;
  int micro_batches = 1;
  bool shard_output = false;  // forward_host with world_size > 1: every rank downloads its own rows
  std::vector<cudaStream_t> aux_streams;
  cudaEvent_t ev_fork = nullptr;
  std::vector<cudaEvent_t> ev_join;
  std::vector<cudaEvent_t> ev_chain;  // ring of events ordering the compute segments across streams
  size_t ev_chain_next = 0;
  std::vector<cudaEvent_t> ev_pool;                      // reusable events
  std::vector<std::pair<int, std::pair<cudaEvent_t, cudaEvent_t>>> ev_rec;  // (name, (before, after))
  cudaStream_t copy_in = nullptr, copy_out = nullptr;  // host-buffer entry point: copies overlapped with the first / last kernels
  cudaEvent_t ev_io[9] = {};
  // Pipelined micro-batches (world_size > 1): every compute kernel of every micro-batch runs on pipe_compute in
  // turn, the copy-engine all-gathers on pipe_comm underneath them.
  int overlap = 1;  // 1: that schedule; 0: one stream per micro-batch with the in-kernel collective
  cudaStream_t pipe_compute = nullptr, pipe_comm = nullptr;
  cudaEvent_t ev_pipe_fork = nullptr, ev_pipe_join = nullptr;
  std::vector<cudaEvent_t> ev_reduced, ev_gather;
  double overlap_acc[4] = {0, 0, 0, 0};  // exposed-wait ms, waits, gather ms, gathers (see liger_model_overlap_times)
  bool timeline = false;  // record per-kernel events in interleaved passes too (diagnostics)
  struct TimelineRec { int name, stream; cudaEvent_t e0, e1; };
  std::vector<TimelineRec> tl_rec;
  cudaEvent_t tl_base = nullptr;
  cudaEvent_t get_event() {
    if (!ev_pool.empty()) { cudaEvent_t e = ev_pool.back(); ev_pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
  }
};

namespace {

BertInitParam to_params(const liger_model_config& c) {
  BertInitParam bp(c.max_batch_size, c.max_seq_len, c.head_num, c.size_per_head, c.layer_num, c.kernel_num, c.factor,
                   c.rq_interval);
  bp.graph = c.graph; bp.act = c.act; bp.ffn_inner = c.ffn_inner; bp.causal = c.causal; bp.seed = c.seed;
  bp.num_requests = c.num_requests; bp.ignore_num = c.ignore_num; bp.schedule_deep = c.schedule_deep;
  bp.contention = c.contention; bp.poisson = c.poisson; bp.min_seq_len = c.min_seq_len; bp.seq_round = c.seq_round;
  bp.workspace_slots = c.workspace_slots; bp.kv_capacity = c.kv_capacity;
  bp.min_slice_efficiency = c.min_slice_efficiency;
  return bp;
}

int validate(const liger_model_config* c) {
  if (!c) return liger::set_error(LIGER_ERR_INVALID, "null configuration");
  if (c->max_batch_size < 1 || c->max_seq_len < 1 || c->head_num < 1 || c->size_per_head < 1 || c->layer_num < 1 ||
      c->factor < 1 || c->workspace_slots < 1 || c->schedule_deep < 1)
    return liger::set_error(LIGER_ERR_INVALID, "configuration: sizes must be positive");
  if (c->schedule_deep + 1 > c->workspace_slots)
    return liger::set_error(LIGER_ERR_INVALID, "configuration: workspace_slots must be at least schedule_deep + 1");
  return LIGER_OK;
}

class CallbackCoordinator : public Coordinator {
 public:
  CallbackCoordinator(int rank, int size, liger_bcast_int_fn b, liger_barrier_fn bar, void* ctx)
      : rank_(rank), size_(size), bcast_(b), barrier_(bar), ctx_(ctx) {}
  int rank() const override { return rank_; }
  int size() const override { return size_; }
  int broadcast_int(int v) override { if (bcast_) bcast_(ctx_, &v); return v; }
  void barrier() override { if (barrier_) barrier_(ctx_); }
 private:
  int rank_, size_;
  liger_bcast_int_fn bcast_;
  liger_barrier_fn barrier_;
  void* ctx_;
};

void fill_metrics(liger_serving_metrics* out, const ServingMetrics& m, long segments, long secondary, long decomp) {
  if (!out) return;
  out->records = m.records; out->launch_errors = m.launch_errors;
  out->total_duration_ms = m.total_duration_ms; out->throughput_samples_s = m.throughput_samples_s;
  out->average_latency_ms = m.average_latency_ms; out->tokens_per_s = m.tokens_per_s;
  out->p50_latency_ms = m.p50_latency_ms; out->p99_latency_ms = m.p99_latency_ms; out->mean_gpu_ms = m.mean_gpu_ms;
  out->tokens = m.tokens; out->segments = segments; out->secondary_launches = secondary; out->decompositions = decomp;
}

}  // namespace

extern "C" void liger_model_config_init(liger_model_config* c) {
  if (!c) return;
  BertInitParam d;
  c->max_batch_size = d.max_batch_size; c->max_seq_len = d.max_seq_len; c->head_num = d.head_num;
  c->size_per_head = d.size_per_head; c->layer_num = d.layer_num; c->kernel_num = d.kernel_num; c->factor = d.factor;
  c->rq_interval = d.rq_interval; c->graph = d.graph; c->act = d.act; c->ffn_inner = d.ffn_inner; c->causal = d.causal;
  c->seed = d.seed; c->num_requests = d.num_requests; c->ignore_num = d.ignore_num; c->schedule_deep = d.schedule_deep;
  c->contention = d.contention; c->poisson = d.poisson; c->min_seq_len = d.min_seq_len; c->seq_round = d.seq_round;
  c->workspace_slots = d.workspace_slots; c->kv_capacity = d.kv_capacity;
  c->min_slice_efficiency = d.min_slice_efficiency;
}

extern "C" size_t liger_model_comm_bytes(const liger_model_config* cfg, int world_size) {
  if (!cfg || world_size <= 1) return 0;
  return Bert_Model::comm_bytes_needed(to_params(*cfg));
}

extern "C" int liger_model_create(liger_model** out, const liger_model_config* cfg, int rank, int world_size,
                                  liger_comm* comm) {
  if (!out) return liger::set_error(LIGER_ERR_INVALID, "model_create: null output");
  int rc = validate(cfg);
  if (rc != LIGER_OK) return rc;
  if (world_size < 1 || rank < 0 || rank >= world_size) return liger::set_error(LIGER_ERR_INVALID, "model_create: bad rank / world_size");
  const liger::DeviceInfo* dev;
  if ((rc = liger::require_sm100(&dev)) != LIGER_OK) return rc;
  liger_model* m = new liger_model();
  m->bp = to_params(*cfg);
  m->sp = StaticNvInitParam(rank, world_size, comm, 1);
  m->device = dev->device;
  try {
    m->model = new Bert_Model(m->bp, m->sp);
    const size_t n = m->model->tokens_max() * m->model->H;
    m->io_in = device_alloc<half_t>(n, "io_in");
    m->io_out = device_alloc<half_t>(n, "io_out");
  } catch (const std::exception& e) {
    delete m;
    return liger::set_error(LIGER_ERR_CUDA, "model_create: %s", e.what());
  }
  *out = m;
  return LIGER_OK;
}

extern "C" int liger_model_destroy(liger_model* m) {
  // Unlike the reference (whose layers have no destructors and never call cudaFree), a model gives back all
  // device memory, streams and events it created.  Work it has queued is waited for first.
  if (!m) return LIGER_OK;
  cudaSetDevice(m->device);
  cudaDeviceSynchronize();
  delete m->model;
  if (m->io_in) cudaFree(m->io_in);
  if (m->io_out) cudaFree(m->io_out);
  for (cudaStream_t s : m->aux_streams) cudaStreamDestroy(s);
  for (cudaStream_t s : {m->copy_in, m->copy_out, m->pipe_compute, m->pipe_comm})
    if (s) cudaStreamDestroy(s);
  auto drop = [](cudaEvent_t e) { if (e) cudaEventDestroy(e); };
  drop(m->ev_fork); drop(m->ev_pipe_fork); drop(m->ev_pipe_join); drop(m->tl_base);
  for (auto* v : {&m->ev_join, &m->ev_chain, &m->ev_pool, &m->ev_reduced, &m->ev_gather})
    for (cudaEvent_t e : *v) drop(e);
  for (auto& r : m->ev_rec) { drop(r.second.first); drop(r.second.second); }
  for (auto& r : m->tl_rec) { drop(r.e0); drop(r.e1); }
  for (cudaEvent_t e : m->ev_io) drop(e);
  delete m;
  cudaGetLastError();
  return LIGER_OK;
}

// Workspace slot(s) of a pass: an explicit slot is checked, -1 takes the next `need` consecutive slots in
// round-robin order (wrapping to slot 0 when fewer than `need` remain).
static int pick_slots(Bert_Model& b, int slot, int need, const char* who) {
  const int size = (int)b.slots.size();
  if (need > size) return liger::set_error(LIGER_ERR_INVALID, "%s: %d micro-batches need %d workspace slots, the model has %d", who, need, need, size);
  if (slot < 0) {
    if (b.next_slot + need > size) b.next_slot = 0;
    slot = b.next_slot;
    b.next_slot = (slot + need) % size;
  }
  if (slot + need > size)
    return liger::set_error(LIGER_ERR_INVALID, "%s: %d micro-batch(es) from slot %d need %d workspace slots, the model has %d", who,
                            need, slot, slot + need, size);
  return slot;
}

// One request, kernels in order on one stream.
static int forward_sequential(liger_model* m, const void* input, void* output, int batch, int seq_len, int slot,
                              void* stream) {
  std::vector<FuncWrap> vec = m->model->forward(input, output, batch, seq_len, slot);
  DynamicNvInitParam dp;
  dp.stream = stream;
  int n = 0;
  for (auto& f : vec) {
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (m->timing) { e0 = m->get_event(); e1 = m->get_event(); cudaEventRecord(e0, (cudaStream_t)stream); }
    const int rc = f.callback(dp);
    if (m->timing) { cudaEventRecord(e1, (cudaStream_t)stream); m->ev_rec.push_back({f.name, {e0, e1}}); }
    if (rc != LIGER_OK) return rc;
    ++n;
  }
  return n;
}

// The batch split into `mb` micro-requests, each on its own stream and workspace slot, launched
// segment by segment in round-robin order: while one micro-request's all-reduce is on the wire the
// other one's GEMMs keep the tensor cores busy -- Liger's interleaving of communication with other
// requests' computation (src/schedule.h:221-278), applied statically to the halves of one batch.
static int forward_interleaved(liger_model* m, const void* input, void* output, int batch, int seq_len, int slot0, int mb,
                               void* stream) {
  cudaStream_t caller = (cudaStream_t)stream;
  while ((int)m->aux_streams.size() < mb) {
    cudaStream_t s = nullptr;
    LIGER_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    m->aux_streams.push_back(s);
    cudaEvent_t e = nullptr;
    LIGER_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    m->ev_join.push_back(e);
  }
  if (!m->ev_fork) LIGER_CUDA_TRY(cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming));
  const int sub = batch / mb;
  const size_t rows = (size_t)sub * seq_len, H = m->model->H;
  std::vector<std::vector<FuncWrap>> vecs;
  for (int i = 0; i < mb; ++i)
    vecs.push_back(m->model->forward((const half_t*)input + i * rows * H, (half_t*)output + i * rows * H, sub, seq_len,
                                     slot0 + i));
  LIGER_CUDA_TRY(cudaEventRecord(m->ev_fork, caller));
  if (m->timeline) {
    if (!m->tl_base) cudaEventCreate(&m->tl_base);
    m->tl_rec.clear();
    cudaEventRecord(m->tl_base, caller);
  }
  for (int i = 0; i < mb; ++i) LIGER_CUDA_TRY(cudaStreamWaitEvent(m->aux_streams[i], m->ev_fork, 0));
  // Compute segments of all micro-requests are chained through events in issue order (a0, a1, b0,
  // b1, ...): they could not share the SMs anyway, and the chain is what staggers the streams so that
  // the all-reduce that follows a0 runs under a1, the one after a1 under b0, and so on.  Without it
  // the streams drift into lockstep and all-reduces only overlap each other.
  while (m->ev_chain.size() < 64) {
    cudaEvent_t e = nullptr;
    LIGER_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    m->ev_chain.push_back(e);
  }
  cudaEvent_t last_compute = nullptr;
  int last_compute_stream = -1;
  std::vector<size_t> cur(mb, 0);
  int n = 0;
  bool more = true;
  while (more) {
    more = false;
    for (int i = 0; i < mb; ++i) {
      std::vector<FuncWrap>& v = vecs[i];
      if (cur[i] >= v.size()) continue;
      DynamicNvInitParam dp;
      dp.stream = m->aux_streams[i];
      dp.index = i;
      // one segment: a maximal run of kernels of the same class (communication / not)
      const bool comm = v[cur[i]].type == COMMUNICATION;
      // LIGER_STAGGER=1 chains the compute segments; measured at 8 GPUs the unchained order is faster
      // with the in-kernel collective (553k vs 524k tokens/s) and the chained one only pays off with the
      // copy-engine collective (LIGER_COMM_MODE=ce, 552k), so chaining defaults to that mode only.
      static const int stagger_env = getenv("LIGER_STAGGER") ? atoi(getenv("LIGER_STAGGER")) : -1;
      const bool stagger = stagger_env >= 0 ? stagger_env != 0 : Bert_MHA::use_copy_engines();
      if (stagger && !comm && last_compute != nullptr && last_compute_stream != i)
        LIGER_CUDA_TRY(cudaStreamWaitEvent(m->aux_streams[i], last_compute, 0));
      while (cur[i] < v.size() && (v[cur[i]].type == COMMUNICATION) == comm) {
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        if (m->timeline) { cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventRecord(e0, m->aux_streams[i]); }
        const int rc = v[cur[i]].callback(dp);
        if (m->timeline) { cudaEventRecord(e1, m->aux_streams[i]); m->tl_rec.push_back({v[cur[i]].name, i, e0, e1}); }
        if (rc != LIGER_OK) return rc;
        ++cur[i];
        ++n;
      }
      if (!comm) {
        last_compute = m->ev_chain[m->ev_chain_next++ % m->ev_chain.size()];
        last_compute_stream = i;
        LIGER_CUDA_TRY(cudaEventRecord(last_compute, m->aux_streams[i]));
      }
      if (cur[i] < v.size()) more = true;
    }
  }
  for (int i = 0; i < mb; ++i) {
    LIGER_CUDA_TRY(cudaEventRecord(m->ev_join[i], m->aux_streams[i]));
    LIGER_CUDA_TRY(cudaStreamWaitEvent(caller, m->ev_join[i], 0));
  }
  return n;
}

// Pseudo kernel names of the pipelined pass's own timing records (beyond the nine real kernel names).
constexpr int kWaitRecord = 9;    // compute stream blocked until a micro-batch's all-gather has landed
constexpr int kGatherRecord = 10; // a copy-engine all-gather, timed on the communication stream

// The batch split into `mb` micro-requests (consecutive groups of sequences, one workspace slot each) that share
// ONE compute stream: their compute segments (QKV, attention, out-proj | FFN-up, FFN-down) run back to back in
// turn, never two at a time, so no kernel ever competes for SMs.  Each all-reduce is split: its reduce-scatter
// half already rode on the row-parallel GEMM's epilogue; the reduction (+ residual + LayerNorm) of the owned rows
// runs on the compute stream as a short local kernel (all-reduce mode 5); its all-gather half goes to the copy
// engines on the communication stream, underneath the other micro-request's next compute segment, which is several
// times longer than the transfer.  The next segment of the same micro-request waits for the gather's event.
// This is the reference scheduler's idea (run one request's communication under other requests' computation,
// src/schedule.h:221-278) with the decomposition along the batch instead of the output features, and with
// communication that needs no SM, since on this GPU a persistent GEMM leaves no room for a second kernel.
static int forward_pipelined(liger_model* m, const void* input, void* output, int batch, int seq_len, int slot0, int mb,
                             void* stream) {
  cudaStream_t caller = (cudaStream_t)stream;
  Bert_Model& b = *m->model;
  if (!m->pipe_compute) {
    int least = 0, greatest = 0;
    LIGER_CUDA_TRY(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    LIGER_CUDA_TRY(cudaStreamCreateWithPriority(&m->pipe_compute, cudaStreamNonBlocking, least));
    LIGER_CUDA_TRY(cudaStreamCreateWithPriority(&m->pipe_comm, cudaStreamNonBlocking, greatest));
    LIGER_CUDA_TRY(cudaEventCreateWithFlags(&m->ev_pipe_fork, cudaEventDisableTiming));
    LIGER_CUDA_TRY(cudaEventCreateWithFlags(&m->ev_pipe_join, cudaEventDisableTiming));
  }
  while ((int)m->ev_reduced.size() < mb) {
    cudaEvent_t e = nullptr;
    LIGER_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    m->ev_reduced.push_back(e);
    LIGER_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    m->ev_gather.push_back(e);
  }
  cudaStream_t s0 = m->pipe_compute, s1 = m->pipe_comm;
  const int nslots = (int)b.slots.size();
  const int sub = batch / mb;
  const size_t rows = (size_t)sub * seq_len, H = b.H;
  std::vector<std::vector<FuncWrap>> vecs;
  for (int i = 0; i < mb; ++i)
    vecs.push_back(b.forward((const half_t*)input + i * rows * H, (half_t*)output + i * rows * H, sub, seq_len, slot0 + i));
  LIGER_CUDA_TRY(cudaEventRecord(m->ev_pipe_fork, caller));
  LIGER_CUDA_TRY(cudaStreamWaitEvent(s0, m->ev_pipe_fork, 0));
  // optional per-kernel timing: events on the stream the work is queued on
  auto begin_rec = [&](cudaStream_t s) -> cudaEvent_t {
    if (!m->timing) return nullptr;
    cudaEvent_t e = m->get_event();
    cudaEventRecord(e, s);
    return e;
  };
  auto end_rec = [&](int name, cudaEvent_t e0, cudaStream_t s) {
    if (!m->timing) return;
    cudaEvent_t e1 = m->get_event();
    cudaEventRecord(e1, s);
    m->ev_rec.push_back({name, {e0, e1}});
  };
  std::vector<size_t> cur(mb, 0);
  std::vector<char> pending(mb, 0);
  DynamicNvInitParam dp;
  dp.stream = s0;
  int n = 0;
  bool more = true;
  while (more) {
    more = false;
    for (int i = 0; i < mb; ++i) {
      std::vector<FuncWrap>& v = vecs[i];
      if (cur[i] >= v.size()) continue;
      dp.index = i;
      if (pending[i]) {  // this micro-request's previous all-gather must have landed on every rank
        cudaEvent_t e0 = begin_rec(s0);
        LIGER_CUDA_TRY(cudaStreamWaitEvent(s0, m->ev_gather[i], 0));
        end_rec(kWaitRecord, e0, s0);
        pending[i] = 0;
      }
      while (cur[i] < v.size() && v[cur[i]].type != COMMUNICATION) {
        cudaEvent_t e0 = begin_rec(s0);
        const int rc = v[cur[i]].callback(dp);
        end_rec(v[cur[i]].name, e0, s0);
        if (rc != LIGER_OK) return rc;
        ++cur[i];
        ++n;
      }
      if (cur[i] < v.size()) {
        const FuncWrap& f = v[cur[i]];
        const COMM_ARGS& c = f.args_comm_tuple;
        if (c.comm != nullptr && c.one_shot == 3 && !c.copy_engine) {
          cudaEvent_t e0 = begin_rec(s0);
          int rc = liger_allreduce_fused(c.comm, c.channel, c.partial_off, c.out_off, c.residual_in, c.hidden, c.bias, c.gamma,
                                         c.beta, c.m, c.n, c.row_begin, c.row_end, 5, s0);
          end_rec(f.name, e0, s0);
          if (rc != LIGER_OK) return rc;
          LIGER_CUDA_TRY(cudaEventRecord(m->ev_reduced[i], s0));
          LIGER_CUDA_TRY(cudaStreamWaitEvent(s1, m->ev_reduced[i], 0));
          e0 = begin_rec(s1);
          rc = liger_allgather_ce(c.comm, nslots + c.channel, c.out_off, c.m, c.n, c.row_begin, c.row_end, s1);
          end_rec(kGatherRecord, e0, s1);
          if (rc != LIGER_OK) return rc;
          LIGER_CUDA_TRY(cudaEventRecord(m->ev_gather[i], s1));
          pending[i] = 1;
          n += 2;
        } else {  // latency-bound sizes: the one-shot collective, in line
          cudaEvent_t e0 = begin_rec(s0);
          const int rc = f.callback(dp);
          end_rec(f.name, e0, s0);
          if (rc != LIGER_OK) return rc;
          ++n;
        }
        ++cur[i];
      }
      if (cur[i] < v.size()) more = true;
    }
  }
  for (int i = 0; i < mb; ++i)
    if (pending[i]) LIGER_CUDA_TRY(cudaStreamWaitEvent(s0, m->ev_gather[i], 0));
  LIGER_CUDA_TRY(cudaEventRecord(m->ev_pipe_join, s0));
  LIGER_CUDA_TRY(cudaStreamWaitEvent(caller, m->ev_pipe_join, 0));
  return n;
}

// The whole batch on the caller's stream, with every bandwidth-bound all-reduce split three ways: the
// reduce-scatter rode on the row-parallel GEMM's epilogue; the reduction (+ residual + LayerNorm) of the owned
// rows is a short local kernel; and the all-gather is liger_allgather_push on the communication stream, running
// beside the NEXT GEMM -- the column-parallel one that consumes the gathered rows -- which is launched at once
// and waits tile by tile for the row blocks it loads (liger_gemm_args.gather_comm).  No batch splitting, so the
// GEMMs keep their full-size tile counts; what stays exposed of an all-reduce is the entry barrier, the local
// reduction, and whatever the first wave of GEMM tiles waits for its rows.
static int forward_gathered(liger_model* m, const void* input, void* output, int batch, int seq_len, int slot, void* stream) {
  cudaStream_t s0 = (cudaStream_t)stream;
  Bert_Model& b = *m->model;
  if (!m->pipe_comm) {
    int least = 0, greatest = 0;
    LIGER_CUDA_TRY(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    LIGER_CUDA_TRY(cudaStreamCreateWithPriority(&m->pipe_comm, cudaStreamNonBlocking, greatest));
  }
  while (m->ev_reduced.empty()) {
    cudaEvent_t e = nullptr;
    LIGER_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    m->ev_reduced.push_back(e);
    LIGER_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    m->ev_gather.push_back(e);
  }
  cudaStream_t s1 = m->pipe_comm;
  const int nslots = (int)b.slots.size();
  const uint8_t* sym = (const uint8_t*)liger_comm_data(m->sp.comm);
  std::vector<FuncWrap> vec = b.forward(input, output, batch, seq_len, slot);
  auto begin_rec = [&](cudaStream_t s) -> cudaEvent_t {
    if (!m->timing) return nullptr;
    cudaEvent_t e = m->get_event();
    cudaEventRecord(e, s);
    return e;
  };
  auto end_rec = [&](int name, cudaEvent_t e0, cudaStream_t s) {
    if (!m->timing) return;
    cudaEvent_t e1 = m->get_event();
    cudaEventRecord(e1, s);
    m->ev_rec.push_back({name, {e0, e1}});
  };
  DynamicNvInitParam dp;
  dp.stream = stream;
  bool pending = false;  // an all-gather is in flight that nothing on s0 has waited for yet
  auto settle = [&]() -> int {
    if (!pending) return LIGER_OK;
    cudaEvent_t e0 = begin_rec(s0);
    LIGER_CUDA_TRY(cudaStreamWaitEvent(s0, m->ev_gather[0], 0));
    end_rec(kWaitRecord, e0, s0);
    pending = false;
    return LIGER_OK;
  };
  int n = 0, rc;
  for (size_t i = 0; i < vec.size(); ++i) {
    const FuncWrap& f = vec[i];
    const COMM_ARGS& c = f.args_comm_tuple;
    const bool split = f.type == COMMUNICATION && c.comm != nullptr && c.one_shot == 3 && !c.copy_engine && c.row_begin == 0 &&
                       c.row_end == c.m;
    if (!split) {
      // (a kernel that is not the consumer GEMM never reads a gathered buffer that is still in flight: the only
      // readers of the all-gather's result are the GEMM below and, after the last layer, the copy-out, for which
      // the else-branch below has already waited)
      cudaEvent_t e0 = begin_rec(s0);
      rc = f.callback(dp);
      end_rec(f.name, e0, s0);
      if (rc != LIGER_OK) return rc;
      ++n;
      continue;
    }
    // the previous gather read this rank's own rows of a buffer the reduction below may overwrite
    if ((rc = settle()) != LIGER_OK) return rc;
    cudaEvent_t e0 = begin_rec(s0);
    rc = liger_allreduce_fused(c.comm, c.channel, c.partial_off, c.out_off, c.residual_in, c.hidden, c.bias, c.gamma, c.beta, c.m,
                               c.n, 0, c.m, 5, stream);
    end_rec(f.name, e0, s0);
    if (rc != LIGER_OK) return rc;
    LIGER_CUDA_TRY(cudaEventRecord(m->ev_reduced[0], s0));
    LIGER_CUDA_TRY(cudaStreamWaitEvent(s1, m->ev_reduced[0], 0));
    const int ready_channel = 2 * nslots + c.channel;
    e0 = begin_rec(s1);
    rc = liger_allgather_push(c.comm, ready_channel, nslots + c.channel, c.out_off, c.m, c.n, s1);
    end_rec(kGatherRecord, e0, s1);
    if (rc != LIGER_OK) return rc;
    LIGER_CUDA_TRY(cudaEventRecord(m->ev_gather[0], s1));
    pending = true;
    n += 2;
    const bool consumer_is_gemm = i + 1 < vec.size() && vec[i + 1].type == GEMM &&
                                  vec[i + 1].args_gemm_tuple.a == (const void*)(sym + c.out_off) &&
                                  vec[i + 1].args_gemm_tuple.m == c.m && vec[i + 1].args_gemm_tuple.lda == c.n;
    if (consumer_is_gemm) {
      GEMM_ARGS g = vec[i + 1].args_gemm_tuple;
      g.gather_comm = c.comm;
      g.gather_channel = ready_channel;
      e0 = begin_rec(s0);
      rc = liger_gemm_fp16(&g, stream);
      end_rec(vec[i + 1].name, e0, s0);
      if (rc != LIGER_OK) return rc;
      ++n;
      ++i;
    } else if ((rc = settle()) != LIGER_OK) {
      return rc;
    }
  }
  if ((rc = settle()) != LIGER_OK) return rc;
  return n;
}

extern "C" int liger_model_forward(liger_model* m, const void* input, void* output, int batch, int seq_len, int slot,
                                   void* stream) {
  if (!m || !input || !output) return liger::set_error(LIGER_ERR_INVALID, "model_forward: null argument");
  try {
    const int mb = m->micro_batches;
    Bert_Model& b = *m->model;
    if (m->overlap == 2 && m->sp.world_size > 1 && liger_comm_channels(m->sp.comm) >= 3 * (int)b.slots.size()) {
      if ((slot = pick_slots(b, slot, 1, "model_forward")) < 0) return slot;
      return forward_gathered(m, input, output, batch, seq_len, slot, stream);
    }
    if (mb > 1 && m->sp.world_size > 1 && batch % mb == 0) {
      const bool pipelined = m->overlap == 1 && liger_comm_channels(m->sp.comm) >= 2 * (int)b.slots.size();
      if (pipelined || !m->timing) {
        if ((slot = pick_slots(b, slot, mb, "model_forward")) < 0) return slot;
        return pipelined ? forward_pipelined(m, input, output, batch, seq_len, slot, mb, stream)
                         : forward_interleaved(m, input, output, batch, seq_len, slot, mb, stream);
      }
    }
    if ((slot = pick_slots(b, slot, 1, "model_forward")) < 0) return slot;
    return forward_sequential(m, input, output, batch, seq_len, slot, stream);
  } catch (const std::exception& e) {
    return liger::set_error(LIGER_ERR_INVALID, "model_forward: %s", e.what());
  }
}

extern "C" int liger_model_timeline(liger_model* m, int enable, int capacity, int* names, int* streams, double* start_ms,
                                    double* end_ms) {
  if (!m) return liger::set_error(LIGER_ERR_INVALID, "model_timeline: null model");
  int n = 0;
  if (names && streams && start_ms && end_ms) {
    LIGER_CUDA_TRY(cudaDeviceSynchronize());
    for (auto& r : m->tl_rec) {
      if (n >= capacity) break;
      float a = 0.0f, b = 0.0f;
      cudaEventElapsedTime(&a, m->tl_base, r.e0);
      cudaEventElapsedTime(&b, m->tl_base, r.e1);
      names[n] = r.name; streams[n] = r.stream; start_ms[n] = a; end_ms[n] = b;
      ++n;
    }
  }
  m->timeline = enable != 0;
  return n;
}

extern "C" int liger_model_decode(liger_model* m, const void* input, void* output, int batch, int kv_len, int slot,
                                  void* stream) {
  if (!m || !input || !output) return liger::set_error(LIGER_ERR_INVALID, "model_decode: null argument");
  try {
    std::vector<FuncWrap> vec = m->model->forward_decode(input, output, batch, kv_len, slot);
    DynamicNvInitParam dp;
    dp.stream = stream;
    int n = 0;
    for (auto& f : vec) {
      cudaEvent_t e0 = nullptr, e1 = nullptr;
      if (m->timing) { e0 = m->get_event(); e1 = m->get_event(); cudaEventRecord(e0, (cudaStream_t)stream); }
      const int rc = f.callback(dp);
      if (m->timing) { cudaEventRecord(e1, (cudaStream_t)stream); m->ev_rec.push_back({f.name, {e0, e1}}); }
      if (rc != LIGER_OK) return rc;
      ++n;
    }
    return n;
  } catch (const std::exception& e) {
    return liger::set_error(LIGER_ERR_INVALID, "model_decode: %s", e.what());
  }
}

extern "C" int liger_model_fill_kv_cache(liger_model* m) {
  if (!m) return liger::set_error(LIGER_ERR_INVALID, "model_fill_kv_cache: null model");
  try {
    m->model->fill_kv_cache_seeded();
    return LIGER_OK;
  } catch (const std::exception& e) {
    return liger::set_error(LIGER_ERR_INVALID, "model_fill_kv_cache: %s", e.what());
  }
}

extern "C" int liger_model_set_output_sharding(liger_model* m, int sharded) {
  if (!m) return liger::set_error(LIGER_ERR_INVALID, "model_set_output_sharding: null model");
  m->shard_output = sharded != 0;
  return LIGER_OK;
}

extern "C" int liger_model_set_micro_batches(liger_model* m, int micro_batches) {
  if (!m || micro_batches < 1 || micro_batches > 8) return liger::set_error(LIGER_ERR_INVALID, "model_set_micro_batches: 1..8");
  if (micro_batches > (int)m->model->slots.size())
    return liger::set_error(LIGER_ERR_INVALID, "model_set_micro_batches: %d micro-batches need %d workspace slots, the model has %zu",
                            micro_batches, micro_batches, m->model->slots.size());
  m->micro_batches = micro_batches;
  return LIGER_OK;
}

extern "C" int liger_model_set_overlap(liger_model* m, int mode) {
  if (!m || mode < 0 || mode > 2) return liger::set_error(LIGER_ERR_INVALID, "model_set_overlap: 0, 1 or 2");
  m->overlap = mode;
  return LIGER_OK;
}

extern "C" int liger_model_overlap_times(liger_model* m, double out[4]) {
  if (!m || !out) return liger::set_error(LIGER_ERR_INVALID, "model_overlap_times: null argument");
  for (int i = 0; i < 4; ++i) { out[i] = m->overlap_acc[i]; m->overlap_acc[i] = 0.0; }
  return LIGER_OK;
}

// world_size == 1: the batch is uploaded in `parts` pieces (4, 2 or 1: the largest that divides it) one after
// the other and the first kernels (input LayerNorm, QKV GEMM) run per piece, so that every upload but the first
// hides behind the previous piece's GEMM; likewise the last GEMM runs per piece and every download but the last
// hides behind the next piece's GEMM.  Rows are independent in those kernels, so the result is bit for bit
// the one of the un-split launch.  Returns the number of launches, or 0 if this form does not apply.
static int forward_host_pipelined(liger_model* m, const void* host_input, void* host_output, int batch, int seq_len, int slot,
                                  cudaStream_t s) {
  Bert_Model& b = *m->model;
  const int parts = batch % 4 == 0 ? 4 : batch % 2 == 0 ? 2 : 1;
  if (m->timing || parts == 1 || m->sp.world_size != 1) return 0;
  std::vector<FuncWrap> vec = b.forward(m->io_in, m->io_out, batch, seq_len, slot);
  const bool ln_first = vec.size() >= 2 && vec[0].name == kPrologueName && vec[1].type == GEMM && vec[1].name == 0;
  const size_t first_gemm = ln_first ? 1 : 0;
  if (vec.size() < 4 || vec[first_gemm].type != GEMM || vec[first_gemm].name != 0 || vec.back().type != GEMM) return 0;
  const GEMM_ARGS g0 = vec[first_gemm].args_gemm_tuple, gl = vec.back().args_gemm_tuple;
  if (g0.epilogue != LIGER_EPI_QKV_SPLIT || g0.kv_stride != 0 || g0.a != (const void*)(ln_first ? b.slots[slot].normed : m->io_in) ||
      gl.c != (void*)m->io_out || (gl.epilogue != LIGER_EPI_STORE && gl.epilogue != LIGER_EPI_RESIDUAL))
    return 0;
  if (!m->copy_in) {
    LIGER_CUDA_TRY(cudaStreamCreateWithFlags(&m->copy_in, cudaStreamNonBlocking));
    LIGER_CUDA_TRY(cudaStreamCreateWithFlags(&m->copy_out, cudaStreamNonBlocking));
    for (auto& e : m->ev_io) LIGER_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  }
  const int pb = batch / parts, rows = pb * seq_len, H = b.H;
  const size_t part_bytes = (size_t)rows * H * 2;
  const char* hin = (const char*)host_input;
  char* hout = (char*)host_output;
  cudaEvent_t* ev_start = &m->ev_io[0];  // [0]: caller's position; [1..4]: piece uploaded; [5..7]: piece computed; [8]: downloads done
  // uploads: ordered after everything the caller has queued (the previous step may still read io_in)
  LIGER_CUDA_TRY(cudaEventRecord(ev_start[0], s));
  LIGER_CUDA_TRY(cudaStreamWaitEvent(m->copy_in, ev_start[0], 0));
  for (int h = 0; h < parts; ++h) {
    LIGER_CUDA_TRY(cudaMemcpyAsync((char*)m->io_in + h * part_bytes, hin + h * part_bytes, part_bytes, cudaMemcpyHostToDevice,
                                   m->copy_in));
    LIGER_CUDA_TRY(cudaEventRecord(m->ev_io[1 + h], m->copy_in));
  }
  int n = 0, rc;
  for (int h = 0; h < parts; ++h) {
    LIGER_CUDA_TRY(cudaStreamWaitEvent(s, m->ev_io[1 + h], 0));
    if (ln_first) {
      const LayerNorm* ln = b.encoders[0]->ln_mha;
      rc = liger_layernorm(m->io_in + (size_t)h * rows * H, ln->gamma, ln->beta, b.slots[slot].normed + (size_t)h * rows * H, rows,
                           H, s);
      if (rc != LIGER_OK) return rc;
      ++n;
    }
    GEMM_ARGS a = g0;
    a.m = rows;
    a.a = (const half_t*)g0.a + (size_t)h * rows * g0.lda;
    const size_t head_off = (size_t)h * pb * g0.heads * seq_len * g0.head_dim;  // [B, h, S, D]: the batch is the outer dimension
    a.q_out = (half_t*)g0.q_out + head_off;
    a.k_out = (half_t*)g0.k_out + head_off;
    a.v_out = (half_t*)g0.v_out + head_off;
    if ((rc = liger_gemm_fp16(&a, s)) != LIGER_OK) return rc;
    ++n;
  }
  DynamicNvInitParam dp;
  dp.stream = s;
  for (size_t i = first_gemm + 1; i + 1 < vec.size(); ++i) {
    if ((rc = vec[i].callback(dp)) != LIGER_OK) return rc;
    ++n;
  }
  for (int h = 0; h < parts; ++h) {
    GEMM_ARGS a = gl;
    a.m = rows;
    a.a = (const half_t*)gl.a + (size_t)h * rows * gl.lda;
    a.c = (half_t*)gl.c + (size_t)h * rows * gl.ldc;
    if (gl.residual) a.residual = (const half_t*)gl.residual + (size_t)h * rows * gl.ldr;
    if ((rc = liger_gemm_fp16(&a, s)) != LIGER_OK) return rc;
    ++n;
    if (h + 1 < parts) {
      LIGER_CUDA_TRY(cudaEventRecord(m->ev_io[5 + h], s));
      LIGER_CUDA_TRY(cudaStreamWaitEvent(m->copy_out, m->ev_io[5 + h], 0));
      LIGER_CUDA_TRY(cudaMemcpyAsync(hout + h * part_bytes, (char*)m->io_out + h * part_bytes, part_bytes, cudaMemcpyDeviceToHost,
                                     m->copy_out));
    }
  }
  LIGER_CUDA_TRY(cudaEventRecord(m->ev_io[8], m->copy_out));
  LIGER_CUDA_TRY(cudaMemcpyAsync(hout + (parts - 1) * part_bytes, (char*)m->io_out + (parts - 1) * part_bytes, part_bytes,
                                 cudaMemcpyDeviceToHost, s));
  LIGER_CUDA_TRY(cudaStreamWaitEvent(s, m->ev_io[8], 0));  // the caller's stream covers the earlier pieces' downloads too
  return n;
}

extern "C" int liger_model_forward_host(liger_model* m, const void* host_input, void* host_output, int batch, int seq_len,
                                        int slot, void* stream) {
  if (!m || !host_input || !host_output) return liger::set_error(LIGER_ERR_INVALID, "model_forward_host: null argument");
  if (batch < 1 || seq_len < 1 || (size_t)batch * seq_len > m->model->tokens_max())
    return liger::set_error(LIGER_ERR_INVALID, "model_forward_host: batch/seq outside the configured maximum");
  Bert_Model& b = *m->model;
  const int M = batch * seq_len, H = b.H, ws = m->sp.world_size, rank = m->sp.world_rank;
  const size_t bytes = (size_t)M * H * 2;
  cudaStream_t s = (cudaStream_t)stream;
  // the pass below runs `need` micro-batches on consecutive slots: choose them here, once
  const bool gathered = m->overlap == 2 && ws > 1 && liger_comm_channels(m->sp.comm) >= 3 * (int)b.slots.size();
  const int need = (!gathered && m->micro_batches > 1 && ws > 1 && batch % m->micro_batches == 0) ? m->micro_batches : 1;
  if ((slot = pick_slots(b, slot, need, "model_forward_host")) < 0) return slot;
  if (ws == 1) {
    try {
      const int np = forward_host_pipelined(m, host_input, host_output, batch, seq_len, slot, s);
      if (np != 0) return np;
    } catch (const std::exception& e) {
      return liger::set_error(LIGER_ERR_INVALID, "model_forward_host: %s", e.what());
    }
    LIGER_CUDA_TRY(cudaMemcpyAsync(m->io_in, host_input, bytes, cudaMemcpyHostToDevice, s));
    const int n = liger_model_forward(m, m->io_in, m->io_out, batch, seq_len, slot, stream);
    if (n < 0) return n;
    LIGER_CUDA_TRY(cudaMemcpyAsync(host_output, m->io_out, bytes, cudaMemcpyDeviceToHost, s));
    return n;
  }
  // upload this rank's rows only, then gather the rest over peer memory
  Workspace& w = b.slots[slot];
  const int rpr = (M + ws - 1) / ws;
  const int lo = rank * rpr < M ? rank * rpr : M, hi = (rank + 1) * rpr < M ? (rank + 1) * rpr : M;
  if (hi > lo)
    LIGER_CUDA_TRY(cudaMemcpyAsync(w.partial + (size_t)lo * H, (const half_t*)host_input + (size_t)lo * H,
                                   (size_t)(hi - lo) * H * 2, cudaMemcpyHostToDevice, s));
  int rc = liger_allreduce_fused(m->sp.comm, slot, w.partial_off, w.xbuf_off, nullptr, nullptr, nullptr, nullptr, nullptr, M,
                                 H, 0, M, 2, stream);
  if (rc != LIGER_OK) return rc;
  const int n = liger_model_forward(m, w.xbuf, m->io_out, batch, seq_len, slot, stream);
  if (n < 0) return n;
  if (m->shard_output) {
    if (hi > lo)
      LIGER_CUDA_TRY(cudaMemcpyAsync((half_t*)host_output + (size_t)lo * H, m->io_out + (size_t)lo * H, (size_t)(hi - lo) * H * 2,
                                     cudaMemcpyDeviceToHost, s));
  } else if (rank == 0) {
    LIGER_CUDA_TRY(cudaMemcpyAsync(host_output, m->io_out, bytes, cudaMemcpyDeviceToHost, s));
  }
  return n + 1;
}

extern "C" int liger_model_set_kernel_timing(liger_model* m, int enable) {
  if (!m) return liger::set_error(LIGER_ERR_INVALID, "model_set_kernel_timing: null model");
  m->timing = enable != 0;
  return LIGER_OK;
}

extern "C" int liger_model_kernel_times(liger_model* m, double ms[9], long long launches[9]) {
  if (!m || !ms || !launches) return liger::set_error(LIGER_ERR_INVALID, "model_kernel_times: null argument");
  for (auto& r : m->ev_rec) {
    float t = 0.0f;
    LIGER_CUDA_TRY(cudaEventSynchronize(r.second.second));
    LIGER_CUDA_TRY(cudaEventElapsedTime(&t, r.second.first, r.second.second));
    if (r.first >= 0 && r.first < 9) { ms[r.first] += t; launches[r.first] += 1; }
    else if (r.first == kWaitRecord) { m->overlap_acc[0] += t; m->overlap_acc[1] += 1.0; }
    else if (r.first == kGatherRecord) { m->overlap_acc[2] += t; m->overlap_acc[3] += 1.0; }
    m->ev_pool.push_back(r.second.first);
    m->ev_pool.push_back(r.second.second);
  }
  m->ev_rec.clear();
  return LIGER_OK;
}

extern "C" int liger_model_kernel_work(liger_model* m, int name, int batch, int seq_len, double* flops, double* bytes) {
  if (!m || !flops || !bytes) return liger::set_error(LIGER_ERR_INVALID, "model_kernel_work: null argument");
  const Bert_Model& b = *m->model;
  const double M = (double)batch * seq_len, H = b.H, Hl = b.Hl, Fl = b.Fl, ws = m->sp.world_size;
  const double up = m->bp.act == ACT_GEGLU ? 2.0 * Fl : Fl;
  const bool preln = m->bp.graph == GRAPH_PRELN;
  double f = 0.0, by = 0.0;
  switch (name) {
    case 0: f = 2.0 * M * H * 3.0 * Hl; by = 2.0 * (M * H + 3.0 * Hl * H + 3.0 * M * Hl); break;
    case 1: f = 4.0 * (double)batch * b.heads_local * (double)seq_len * seq_len * b.D * (m->bp.causal ? 0.5 : 1.0);
            by = 2.0 * 4.0 * M * Hl; break;
    case 2: f = 2.0 * M * Hl * H; by = 2.0 * (M * Hl + H * Hl + M * H * (ws == 1 && preln ? 2.0 : 1.0)); break;
    case 3: case 6: by = ws > 1 ? 2.0 * M * H * (1.0 + (preln ? 2.0 / ws : 0.0) + 1.0) : 2.0 * 2.0 * M * H; break;
    case 4: f = 2.0 * M * H * up; by = 2.0 * (M * H + up * H + M * Fl); break;
    case 5: f = 2.0 * M * Fl * H; by = 2.0 * (M * Fl + H * Fl + M * H * (ws == 1 && preln ? 2.0 : 1.0)); break;
    case 7: by = preln ? 2.0 * 2.0 * M * H : 0.0; break;
    case 8: by = ws > 1 ? 2.0 * 2.0 * M * H : 0.0; break;
    default: return liger::set_error(LIGER_ERR_INVALID, "model_kernel_work: kernel name %d", name);
  }
  *flops = f;
  *bytes = by;
  return LIGER_OK;
}

extern "C" int liger_model_set_mask(liger_model* m, const void* mask) {
  if (!m) return liger::set_error(LIGER_ERR_INVALID, "model_set_mask: null model");
  m->model->set_mask((const half_t*)mask);
  return LIGER_OK;
}

extern "C" int liger_serve(liger_model* m, int mode, liger_bcast_int_fn bcast, liger_barrier_fn barrier, void* ctx,
                           const char* profile_dir, int print, liger_serving_metrics* metrics) {
  if (!m) return liger::set_error(LIGER_ERR_INVALID, "serve: null model");
  if (m->sp.world_size > 1 && (!bcast || !barrier))
    return liger::set_error(LIGER_ERR_INVALID, "serve: world_size > 1 needs the broadcast and barrier callbacks");
  try {
    CudaRuntime rt;
    CallbackCoordinator coord(m->sp.world_rank, m->sp.world_size, bcast, barrier, ctx);
    const std::string dir = (profile_dir && *profile_dir) ? std::string(profile_dir) + "/" : std::string("./");
    const std::string main_f = dir + profile_file_name("Main", m->bp, m->sp.world_size).substr(2);
    const std::string sub_f = dir + profile_file_name("Sub", m->bp, m->sp.world_size).substr(2);
    const size_t n = m->model->tokens_max() * m->model->H;
    host_check(liger_fill_normal(m->io_in, (int)m->model->tokens_max(), m->model->H, m->model->H, 0, 0, m->model->H,
                                 m->bp.seed, 0x10000u, 0.0f, 1.0f, 0, nullptr), "fill input");
    (void)n;
    Scheduler<Bert_Model> scheduler(m->model, m->bp, m->sp, m->io_in, m->io_out, &rt, &coord);
    if (mode == LIGER_MODE_PROFILE) {
      const int step = m->bp.seq_round > 0 ? m->bp.seq_round : 1;
      const int wb = std::min(2, m->bp.max_batch_size);
      int wsq = std::min(64, m->bp.max_seq_len);
      wsq = std::max(step, wsq / step * step);
      if (wb != m->bp.max_batch_size) scheduler.profile(wb, wb + 1, wsq, wsq + 1, main_f, sub_f, 1);
      scheduler.profile(m->bp.max_batch_size, m->bp.max_batch_size + 1, 1, m->bp.max_seq_len + 1, main_f, sub_f, step);
      policy_trial(m->model, m->bp, m->sp, m->io_in, m->io_out, &rt, &coord, main_f, sub_f);
      return LIGER_OK;
    }
    scheduler.load_profiles(main_f, sub_f);
    scheduler.serving();
    coord.barrier();
    if (mode == LIGER_MODE_SCHEDULE) scheduler.run_stream_sync();
    else if (mode == LIGER_MODE_NO_SCHEDULE) scheduler.run_sequential();
    else return liger::set_error(LIGER_ERR_INVALID, "serve: unknown mode %d", mode);
    scheduler.run_stop();
    ServingMetrics sm = scheduler.output_recording(print != 0);
    fill_metrics(metrics, sm, scheduler.segments, scheduler.secondary_launches, scheduler.decompositions);
    unsigned int st[4];
    if (liger_device_status(st) != 0)
      return liger::set_error(LIGER_ERR_DEVICE, "serve: device status %u at %#x (%u, %u)", st[0], st[1], st[2], st[3]);
    return sm.launch_errors ? liger::set_error(LIGER_ERR_CUDA, "serve: %d kernel launches failed: %s", sm.launch_errors,
                                               liger_last_error())
                            : LIGER_OK;
  } catch (const std::exception& e) {
    return liger::set_error(LIGER_ERR_INVALID, "serve: %s", e.what());
  }
}

extern "C" int liger_profile_rewrite(const char* in_path, const char* out_path, int is_sub, int* entries, double* duration_sum) {
  if (!in_path) return liger::set_error(LIGER_ERR_INVALID, "profile_rewrite: null path");
  try {
    int n = 0;
    double sum = 0.0;
    if (is_sub) {
      SubDict d = SubFileToDict(in_path);
      for (auto& e : d) { ++n; for (float v : e.second) sum += v; }
      if (out_path) SubDictToFile(d, out_path);
    } else {
      MainDict d = MainFileToDict(in_path);
      for (auto& e : d) { ++n; sum += e.second; }
      if (out_path) MainDictToFile(d, out_path);
    }
    if (entries) *entries = n;
    if (duration_sum) *duration_sum = sum;
    return LIGER_OK;
  } catch (const std::exception& e) {
    return liger::set_error(LIGER_ERR_INVALID, "profile_rewrite: %s", e.what());
  }
}

extern "C" int liger_profile_predict(const char* main_path, int max_batch, int max_seq, int name, int batch, int seq_len,
                                     double* duration_ms) {
  if (!main_path || !duration_ms || max_batch < 1 || max_seq < 1 || batch < 1 || seq_len < 1)
    return liger::set_error(LIGER_ERR_INVALID, "profile_predict: bad argument");
  try {
    MainDict d = MainFileToDict(main_path);
    *duration_ms = predict_duration(d, name, batch, seq_len, max_batch, max_seq);
    return LIGER_OK;
  } catch (const std::exception& e) {
    return liger::set_error(LIGER_ERR_INVALID, "profile_predict: %s", e.what());
  }
}

// ---- the scheduler on a simulated device --------------------------------------------------------------
namespace {

struct SimModel {
  SimRuntime* rt;
  BertInitParam bp;
  std::vector<liger_sim_kernel> kernels;
  double slice_overhead_ms;
  int next_request = 0;
  double device_slowdown = 1.0;  // what the device really takes relative to the profiled durations

  float scaled(float base, int bs, int sq) const {
    return base * (float)((double)bs * sq / ((double)bp.max_batch_size * bp.max_seq_len));
  }
  std::vector<FuncWrap> forward(const void*, void*, int bs, int sq, int /*slot*/) {
    std::vector<FuncWrap> vec;
    const int req = next_request++;
    for (int l = 0; l < bp.layer_num; ++l)
      for (size_t k = 0; k < kernels.size(); ++k) {
        const float dur = scaled(kernels[k].duration_ms, bs, sq);
        const int tag = (req << 16) | (l << 8) | (int)k;
        SimRuntime* r = rt;
        const float real = (float)(dur * device_slowdown);
        FuncWrap f((int)k, dur, (layer_type)kernels[k].type,
                   [r, real, tag](const DynamicNvInitParam& d) { r->launch(d.stream, real, tag); return LIGER_OK; });
        if (kernels[k].type == GEMM || kernels[k].type == COMMUNICATION) {
          const double ovh = slice_overhead_ms, slow = device_slowdown;
          f.slicer = [r, dur, tag, ovh, slow](int ub, int ue, int factor) {
            const float sd = (float)((ovh + (double)dur * (ue - ub) / factor) * slow);
            const int stag = tag | (ub << 24) | (ue << 28);
            return [r, sd, stag](const DynamicNvInitParam& d) { r->launch(d.stream, sd, stag); return LIGER_OK; };
          };
        }
        vec.push_back(f);
      }
    return vec;
  }
};

}  // namespace

extern "C" int liger_sim_serve(const liger_model_config* cfg, const liger_sim_kernel* layer_kernels, int kernels_per_layer,
                               int mode, double overlap_rate, double slice_overhead_ms, liger_sim_launch* log,
                               int log_capacity, int* log_count, liger_serving_metrics* metrics) {
  return liger_sim_serve_rank(cfg, layer_kernels, kernels_per_layer, mode, overlap_rate, slice_overhead_ms, 0, 1, nullptr,
                              nullptr, nullptr, 0.0, 1.0, log, log_capacity, log_count, metrics);
}

extern "C" int liger_sim_serve_rank(const liger_model_config* cfg, const liger_sim_kernel* layer_kernels,
                                    int kernels_per_layer, int mode, double overlap_rate, double slice_overhead_ms, int rank,
                                    int world_size, liger_bcast_int_fn bcast, liger_barrier_fn barrier, void* ctx,
                                    double host_skew_ms, double device_slowdown, liger_sim_launch* log, int log_capacity,
                                    int* log_count, liger_serving_metrics* metrics) {
  int rc = validate(cfg);
  if (rc != LIGER_OK) return rc;
  if (!layer_kernels || kernels_per_layer < 1 || kernels_per_layer > 255 || cfg->factor > 15 || cfg->layer_num > 255)
    return liger::set_error(LIGER_ERR_INVALID, "sim_serve: bad kernel list (<= 255 kernels, factor <= 15)");
  try {
    if (world_size < 1 || rank < 0 || rank >= world_size || (world_size > 1 && !bcast))
      return liger::set_error(LIGER_ERR_INVALID, "sim_serve: bad rank / world_size / callbacks");
    SimRuntime rt;
    rt.overlap_rate = overlap_rate;
    rt.host_advance_ms(host_skew_ms);
    CallbackCoordinator coord(rank, world_size, bcast, barrier, ctx);
    std::vector<liger_sim_kernel> kv(layer_kernels, layer_kernels + kernels_per_layer);
    SimModel model{&rt, to_params(*cfg), kv, slice_overhead_ms};
    model.device_slowdown = device_slowdown > 0.0 ? device_slowdown : 1.0;
    StaticNvInitParam sp(rank, world_size, nullptr, 1);
    Scheduler<SimModel> scheduler(&model, model.bp, sp, nullptr, nullptr, &rt, &coord);
    // the cost model: isolated durations, as a profile run on this simulated device would measure
    const std::vector<Request> reqs = make_requests(model.bp, model.bp.num_requests, model.bp.seed);
    for (const Request& r : reqs)
      for (int k = 0; k < kernels_per_layer; ++k) {
        const float dur = model.scaled(layer_kernels[k].duration_ms, r.batch_size, r.seq_len);
        scheduler.profiling_res_dict[{k, r.batch_size, r.seq_len}] = dur;
        if (layer_kernels[k].type != COMPUTATION) {
          std::vector<float> v;
          for (int n = 1; n < cfg->factor; ++n) v.push_back((float)(slice_overhead_ms + (double)dur * n / cfg->factor));
          scheduler.profiling_decompse_res_dict[{k, r.batch_size, r.seq_len}] = v;
        }
      }
    scheduler.set_requests(reqs);
    // contention == 0: measure the two factors on the simulated device, as a profile run does on a real one
    if (cfg->contention == 0.0f && !reqs.empty()) scheduler.calibrate_contention(reqs.back().batch_size, reqs.back().seq_len);
    if (mode == LIGER_MODE_SCHEDULE) scheduler.run_stream_sync();
    else if (mode == LIGER_MODE_NO_SCHEDULE) scheduler.run_sequential();
    else return liger::set_error(LIGER_ERR_INVALID, "sim_serve: unknown mode %d", mode);
    ServingMetrics sm = scheduler.output_recording(false);
    fill_metrics(metrics, sm, scheduler.segments, scheduler.secondary_launches, scheduler.decompositions);
    int n = 0;
    for (const auto& r : rt.log) {
      if (log && n < log_capacity) {
        liger_sim_launch& o = log[n];
        o.request = (r.tag >> 16) & 0xff; o.layer = (r.tag >> 8) & 0xff; o.name = r.tag & 0xff; o.stream = r.stream;
        o.units_begin = (r.tag >> 24) & 0xf; o.units_end = (r.tag >> 28) & 0xf;
        o.duration_ms = r.duration; o.t_start_ms = r.t_start; o.t_end_ms = r.t_end;
      }
      ++n;
    }
    if (log_count) *log_count = n;
    return LIGER_OK;
  } catch (const std::exception& e) {
    return liger::set_error(LIGER_ERR_INVALID, "sim_serve: %s", e.what());
  }
}
