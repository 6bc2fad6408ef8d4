// Scheduler: profiling, request admission, the unscheduled baseline loop and Liger's interleaved
// two-stream schedule with hybrid synchronisation, contention factor and run-time kernel
// decomposition.  Follows the reference's Scheduler<T, MODELTYPE> (src/schedule.h:19-351) loop by
// loop; what is different, and why:
//   * Requests are a pre-computed, seeded arrival schedule (same on every rank) that the scheduling
//     thread polls against the clock, instead of a second thread that calls model->forward and
//     pushes into an unlocked queue (src/schedule.h:25,171,285-310).
//   * How many arrived requests enter the in-flight window is decided by rank 0 and broadcast
//     (Coordinator), so every rank plans the same segments and issues its collectives in the same
//     order; the reference leaves that to per-rank thread timing.
//   * A request whose next kernel goes to a different stream than its previous one waits for that
//     previous kernel through an event (the reference has no such dependency).
//   * Every in-flight request has its own activation workspace (slot).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <queue>
#include <string>
#include <vector>

#include "context.h"
#include "profile_io.h"
#include "runtime_iface.h"
#include "sample.h"

namespace liger_host {

// Cross-rank agreement on small integers.  world_size == 1: identity.
class Coordinator {
 public:
  virtual ~Coordinator() {}
  virtual int rank() const { return 0; }
  virtual int size() const { return 1; }
  virtual int broadcast_int(int value_on_root) { return value_on_root; }  // root = rank 0
  virtual void barrier() {}
};

struct Request {
  int batch_size;
  int seq_len;
  double arrive_s;  // seconds after serving starts
  bool warmup;
};

// Seeded request schedule.  The reference draws seq = rand() % (max_seq_len - 28) + 16 with the
// maximum batch size, one request every rq_interval microseconds, after one warm-up request of
// (2, 64) (src/schedule.h:291-301); lengths here are additionally rounded up to `seq_round` so
// that they hit profiled (batch, seq) keys, and arrivals may be Poisson (exponential gaps).
inline std::vector<Request> make_requests(const BertInitParam& bp, int count, uint32_t seed) {
  std::vector<Request> out;
  uint64_t s = 0x9E3779B97F4A7C15ull ^ ((uint64_t)seed << 17) ^ 0xD1B54A32D192ED03ull;
  auto next_u32 = [&s]() {  // splitmix64
    s += 0x9E3779B97F4A7C15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return (uint32_t)((z ^ (z >> 31)) >> 32);
  };
  const int round = bp.seq_round > 0 ? bp.seq_round : 1;
  const int lo = bp.min_seq_len, hi = bp.max_seq_len;
  double t = 0.0;
  Request w{std::min(2, bp.max_batch_size), std::min(64, hi), 0.0, true};
  w.seq_len = std::max(round, w.seq_len / round * round);
  out.push_back(w);
  t += 0.05;  // the warm-up request gets the device to itself
  for (int i = 0; i < count; ++i) {
    int span = hi - lo + 1;
    if (span < 1) span = 1;
    int sq = lo + (int)(next_u32() % (uint32_t)span);
    sq = (sq + round - 1) / round * round;
    if (sq > hi) sq = hi / round * round;
    if (sq < round) sq = round;
    out.push_back(Request{bp.max_batch_size, sq, t, false});
    double gap = (double)bp.rq_interval * 1e-6;
    if (bp.poisson) {
      double u = ((double)next_u32() + 0.5) / 4294967296.0;
      gap = -std::log(u) * gap;
    }
    t += gap;
  }
  return out;
}

struct ServingMetrics {
  int records = 0;
  double total_duration_ms = 0, throughput_samples_s = 0, average_latency_ms = 0;  // the reference's three lines
  double tokens_per_s = 0, p50_latency_ms = 0, p99_latency_ms = 0, mean_gpu_ms = 0;
  long tokens = 0;
  int launch_errors = 0;
};

template <class MODELTYPE>
class Scheduler {
 private:
  MODELTYPE* _model;
  Runtime* _rt;
  Coordinator* _coord;
  std::vector<Request> _requests;
  size_t _next_request = 0;
  double _t0 = 0.0;
  int _next_id = 0;
  std::vector<int> _free_slots;

 public:
  bool tag = false;
  std::queue<Sample*> main_q;
  std::vector<Sample*> exe_vec;
  int schedule_deep;
  StaticNvInitParam SParams;
  DynamicNvInitParam DParams0, DParams1;
  MainDict profiling_res_dict;
  SubDict profiling_decompse_res_dict;
  BertInitParam BertParams;
  std::vector<recorder> recs;
  std::vector<Sample*> finished;
  const void* input;
  void* output;
  void *Main_EVENT, *Wait_EVENT;
  int launch_errors = 0;
  long segments = 0, secondary_launches = 0, decompositions = 0;

  Scheduler(MODELTYPE* model, const BertInitParam& bp, const StaticNvInitParam& sp, const void* input_, void* output_,
            Runtime* rt, Coordinator* coord)
      : _model(model), _rt(rt), _coord(coord), schedule_deep(bp.schedule_deep), SParams(sp), BertParams(bp),
        input(input_), output(output_) {
    // main stream at higher priority than the secondary one (src/schedule.h:54-55: -4 and 0)
    DParams0.stream = rt->create_stream(-4); DParams0.priority = -4; DParams0.index = 0;
    DParams1.stream = rt->create_stream(0); DParams1.priority = 0; DParams1.index = 1;
    Main_EVENT = rt->create_event();
    Wait_EVENT = rt->create_event();
    for (int s = bp.workspace_slots - 1; s >= 0; --s) _free_slots.push_back(s);
  }

  void load_profiles(const std::string& main_filename, const std::string& sub_filename) {
    profiling_res_dict = MainFileToDict(main_filename);
    profiling_decompse_res_dict = SubFileToDict(sub_filename);
  }

  // ---- profiling (src/schedule.h:79-156) ---------------------------------------------------------
  // min over 3 trials of (2 warm-up + 20 timed launches) / 20 for every kernel name of a request of
  // shape (bs, sq); for GEMM and COMMUNICATION kernels also the first n/factor slices, n = 1 ..
  // factor-1.  sq_step > 1 profiles only multiples of sq_step (the reference profiles every integer).
  void profile(int low_bs, int high_bs, int low_sq, int high_sq, const std::string& main_filename,
               const std::string& sub_filename, int sq_step = 1, int itr = 20) {
    void* start = _rt->create_event();
    void* stop = _rt->create_event();
    int last_sq = 0;
    for (int i = low_bs; i < high_bs; ++i) {
      for (int j = low_sq; j < high_sq; ++j) {
        if (sq_step > 1 && j % sq_step != 0) continue;
        if ((i * j) % 4 != 0) continue;  // src/schedule.h:88
        last_sq = j;
        if (SParams.world_rank == 0) printf("Batch Size: %d; Seq_Len: %d; \n", i, j);
        std::vector<FuncWrap> vec = _model->forward(input, output, i, j, 0);
        std::vector<bool> seen(64, false);
        for (size_t k = 0; k < vec.size(); ++k) {
          const int name = vec[k].name;
          if (name < 0 || name >= 64 || seen[name]) continue;
          seen[name] = true;
          const kernel_info info{name, i, j};
          profiling_res_dict[info] = time_kernel(vec[k], start, stop, itr);
          if (vec[k].type == GEMM || vec[k].type == COMMUNICATION) {
            std::vector<float> tmp;
            for (int n = 1; n < BertParams.factor; ++n) {
              FuncWrap fc = vec[k].type == GEMM ? decompose_callback(vec[k], BertParams.factor, n)
                                                : decompose_comm_callback(vec[k], BertParams.factor, n);
              tmp.push_back(time_kernel(fc, start, stop, itr));
            }
            profiling_decompse_res_dict[info] = tmp;
          }
        }
      }
    }
    if (high_bs > low_bs && last_sq > 0) calibrate_contention(high_bs - 1, last_sq);
    if (SParams.world_rank == 0) {
      MainDictToFile(profiling_res_dict, main_filename);
      SubDictToFile(profiling_decompse_res_dict, sub_filename);
    }
    _coord->barrier();
  }

  // ---- contention factors from measurement ----------------------------------------------------------
  // The reference scales the time budget of a scheduling window by a constant 0.8 (src/schedule.h:249), found by
  // hand on V100.  Here the factor is measured, per direction, on the machine the profile is taken on: the longest
  // GEMM of a request and its all-reduce are run (i) alone -- the profiled durations -- and (ii) at the same
  // time on the two streams, once with the GEMM as the main segment and all-reduces as secondary work, once the
  // other way round.  A kernel that takes s times longer when overlapped consumes s times its profiled duration
  // of a window that is itself stretched by the main kernel's own slow-down, so a window of profiled length T
  // has room for secondary kernels of profiled length T * s_main / s_secondary: that ratio (clamped to
  // [0.05, 1]) is the factor.  The two factors and the four slow-downs are stored in the Main profile under
  // kernel names 100..105 with batch_size = seq_len = 0, where the reference's reader ignores them.
  static constexpr int kFactorCommUnderComp = 100, kFactorCompUnderComm = 101;
  static constexpr float kMinOverlapGain = 0.15f;
  void calibrate_contention(int bs, int sq) {
    std::vector<FuncWrap> vec = _model->forward(input, output, bs, sq, 0);
    FuncWrap *g = nullptr, *c = nullptr;
    float tg = 0.0f, tc = 0.0f;
    for (auto& f : vec) {
      const float d = lookup_duration(f.name, bs, sq);
      if (f.type == GEMM && d > tg) { g = &f; tg = d; }
      if (f.type == COMMUNICATION && c == nullptr) { c = &f; tc = d; }
    }
    if (!g || !c || tg <= 0.0f || tc <= 0.0f) return;  // one GPU: nothing to overlap
    // enough all-reduces, back to back, to outlast the GEMM however much the two slow each other down
    const int reps_c = std::min(48, std::max(2, (int)std::ceil(4.0f * tg / tc)));
    void* ev_start[2] = {_rt->create_event(), _rt->create_event()};
    void* ev_gemm = _rt->create_event();
    std::vector<void*> ev_ar(reps_c);
    for (auto& e : ev_ar) e = _rt->create_event();
    float slow[2][2];  // [experiment][0: GEMM, 1: all-reduce]
    float gain[2];     // how much more work per unit time the pair got done side by side than one after the other
    for (int exp = 0; exp < 2; ++exp) {
      // exp 0: the GEMM is the main segment (stream 0), all-reduces are secondary (stream 1); exp 1: the reverse
      const DynamicNvInitParam& dg = exp == 0 ? DParams0 : DParams1;
      const DynamicNvInitParam& dc = exp == 0 ? DParams1 : DParams0;
      float best_g = 1e30f, best_c = 1e30f;
      for (int trial = 0; trial < 3; ++trial) {
        _rt->device_synchronize();
        _coord->barrier();
        _rt->record(ev_start[0], dg.stream);
        _rt->record(ev_start[1], dc.stream);
        if (exp == 0) g->callback(dg);
        for (int r = 0; r < reps_c; ++r) {
          c->callback(dc);
          _rt->record(ev_ar[r], dc.stream);
          if (exp == 1 && r == 0) g->callback(dg);  // the secondary GEMM follows the first main all-reduce
        }
        _rt->record(ev_gemm, dg.stream);
        _rt->event_synchronize(ev_gemm);
        _rt->event_synchronize(ev_ar[reps_c - 1]);
        const float t_gemm = _rt->elapsed_ms(ev_start[0], ev_gemm);
        // all-reduces (whole and a fraction of the one in flight) finished while the GEMM was running
        float done = 0.0f, prev = 0.0f;
        for (int r = 0; r < reps_c; ++r) {
          const float t = _rt->elapsed_ms(ev_start[1], ev_ar[r]);
          if (t <= t_gemm) { done += 1.0f; prev = t; }
          else { if (t > prev) done += (t_gemm - prev) / (t - prev); break; }
        }
        if (done < 0.05f) done = 0.05f;
        best_g = std::min(best_g, t_gemm);
        best_c = std::min(best_c, t_gemm / done);
      }
      slow[exp][0] = std::max(1.0f, best_g / tg);
      slow[exp][1] = std::max(1.0f, best_c / tc);
      // work done side by side during the GEMM, in isolated-time units, against the time it took
      gain[exp] = (tg + (best_g / best_c) * tc) / best_g - 1.0f;
    }
    // A direction in which running side by side gains less than kMinOverlapGain over running one after the other
    // is switched off (factor 0: no secondary launches): the schedule's own cost -- a host synchronisation per
    // segment -- is of that order.  On B200 both directions measure that way at GLM-130B shapes: a persistent GEMM
    // leaves the all-reduce kernel no registers in two of an SM's four sub-partitions, so the pair serialises.
    auto clamp = [](float v) { return v < 0.05f ? 0.05f : v > 1.0f ? 1.0f : v; };
    profiling_res_dict[{kFactorCommUnderComp, 0, 0}] = gain[0] < kMinOverlapGain ? 0.0f : clamp(slow[0][0] / slow[0][1]);
    profiling_res_dict[{kFactorCompUnderComm, 0, 0}] = gain[1] < kMinOverlapGain ? 0.0f : clamp(slow[1][1] / slow[1][0]);
    profiling_res_dict[{106, 0, 0}] = gain[0];
    profiling_res_dict[{107, 0, 0}] = gain[1];
    profiling_res_dict[{102, 0, 0}] = slow[0][0];  // GEMM main, its own slow-down
    profiling_res_dict[{103, 0, 0}] = slow[0][1];  // ... and that of the all-reduces beside it
    profiling_res_dict[{104, 0, 0}] = slow[1][1];  // all-reduce main, its own slow-down
    profiling_res_dict[{105, 0, 0}] = slow[1][0];  // ... and that of the GEMM beside it
    if (SParams.world_rank == 0)
      printf("Contention factors from measurement (batch %d, seq %d): all-reduce under GEMM %.3f (GEMM x%.2f, all-reduce x%.2f, "
             "gain %.0f %%); GEMM under all-reduce %.3f (all-reduce x%.2f, GEMM x%.2f, gain %.0f %%). \n", bs, sq,
             profiling_res_dict[{kFactorCommUnderComp, 0, 0}], slow[0][0], slow[0][1], 100.0f * gain[0],
             profiling_res_dict[{kFactorCompUnderComm, 0, 0}], slow[1][1], slow[1][0], 100.0f * gain[1]);
  }
  // The factor of a window whose main segment is of class `main_type`: the configured constant, or, with
  // BertInitParam::contention == 0, the measured one (0.8 where the profile holds none).
  float contention_factor(layer_type main_type) const {
    if (BertParams.contention > 0.0f) return BertParams.contention;
    auto it = profiling_res_dict.find({main_type == COMMUNICATION ? kFactorCompUnderComm : kFactorCommUnderComp, 0, 0});
    return it != profiling_res_dict.end() ? it->second : 0.8f;
  }

  float time_kernel(FuncWrap& f, void* start, void* stop, int itr) {
    float time_min = 100000.0f;
    for (int test = 0; test < 3; ++test) {
      f.callback(DParams0);
      f.callback(DParams0);
      _rt->device_synchronize();
      _rt->record(start, DParams0.stream);
      for (int m = 0; m < itr; ++m) f.callback(DParams0);
      _rt->record(stop, DParams0.stream);
      _rt->event_synchronize(stop);
      const float elapsed = _rt->elapsed_ms(start, stop);
      if (elapsed < time_min) time_min = elapsed;
    }
    return time_min / (float)itr;
  }

  // Cost model: profiled duration of kernel `name` for (bs, sq).  The reference looks the exact key up and gets 0 for
  // anything it did not profile (operator[] default, src/schedule.h:166), which is why it profiles every integer
  // length (src/test_schedule.h:103).  Here a profile taken at a few lengths serves all of them: between two profiled
  // lengths of the same batch size the duration is interpolated linearly, beyond the last one it is extrapolated in
  // proportion to the length, and a batch size that was not profiled borrows the nearest profiled one scaled by the
  // token count.
  float lookup_duration(int name, int bs, int sq) const {
    return predict_duration(profiling_res_dict, name, bs, sq, BertParams.max_batch_size, BertParams.max_seq_len);
  }

  // ---- admission (src/schedule.h:159-202) --------------------------------------------------------
  // Build the kernel vector of one request, stamp the profiled durations and queue it.
  void serve(int batch_size, int seq_len, double arrive_s = -1.0) {
    int slot = 0;
    if (!_free_slots.empty()) { slot = _free_slots.back(); _free_slots.pop_back(); }
    std::vector<FuncWrap> vec = _model->forward(input, output, batch_size, seq_len, slot);
    for (auto& f : vec) f.duration = lookup_duration(f.name, batch_size, seq_len);
    Sample* sample = new Sample(std::move(vec), &profiling_decompse_res_dict, batch_size, seq_len, BertParams.factor, _rt);
    sample->id = _next_id++;
    sample->slot = slot;
    sample->min_slice_efficiency = BertParams.min_slice_efficiency;
    if (arrive_s >= 0.0) sample->sample_arrive = arrive_s;
    main_q.push(sample);
  }

  void set_requests(const std::vector<Request>& reqs) { _requests = reqs; _next_request = 0; }

  // Generates the request schedule (the reference spawns a thread that sleeps between requests,
  // src/schedule.h:312-321; here arrivals are time stamps that update_vec() polls).
  void serving() {
    set_requests(make_requests(BertParams, BertParams.num_requests, BertParams.seed));
    if (SParams.world_rank == 0) printf("Request schedule ready: %zu requests. \n", _requests.size());
  }

  void update_vec() {
    if (!exe_vec.empty() && exe_vec[0]->empty()) {  // retire the head (src/schedule.h:176-187)
      Sample* tmp = exe_vec[0];
      recs.push_back(tmp->get_recording());
      launch_errors += tmp->launch_errors;
      exe_vec.erase(exe_vec.begin());
      _free_slots.push_back(tmp->slot);
      finished.push_back(tmp);
    }
    // rank 0 decides how many arrived requests enter the window; everyone follows
    int admit = 0;
    if (_coord->rank() == 0) {
      const double now = _rt->wall_seconds() - _t0;
      size_t arrived = _next_request;
      while (arrived < _requests.size() && _requests[arrived].arrive_s <= now) ++arrived;
      const size_t space = exe_vec.size() < (size_t)schedule_deep ? (size_t)schedule_deep - exe_vec.size() : 0;
      const size_t fresh = std::min(arrived - _next_request, _free_slots.size());  // each needs a workspace
      admit = (int)std::min(space, main_q.size() + fresh);
    }
    if (_coord->size() > 1) admit = _coord->broadcast_int(admit);
    for (int a = 0; a < admit; ++a) {
      if (main_q.empty()) {
        if (_next_request >= _requests.size()) break;
        const Request& r = _requests[_next_request++];
        serve(r.batch_size, r.seq_len, _t0 + r.arrive_s);
      }
      exe_vec.push_back(main_q.front());
      main_q.pop();
    }
    if (exe_vec.empty()) {
      if (_next_request >= _requests.size() && main_q.empty()) tag = false;  // schedule exhausted
      else _rt->sleep_us(100);
    }
  }

  // ---- the unscheduled tensor-parallel baseline (src/schedule.h:204-219) ------------------------------
  void run_sequential() {
    tag = true;
    _t0 = _rt->wall_seconds();
    _rt->record(Wait_EVENT, DParams0.stream);
    while (tag) {
      update_vec();
      if (!exe_vec.empty()) {
        _rt->event_synchronize(Wait_EVENT);
        while (!exe_vec.at(0)->empty()) exe_vec.at(0)->dequeue(DParams0, 1, 0.0f);
        _rt->record(Wait_EVENT, DParams0.stream);
        ++segments;
      }
    }
    _rt->device_synchronize();
  }

  // ---- Liger: interleaved two-stream schedule (src/schedule.h:221-278) ---------------------------------
  // With measured constants (contention == 0) the profile also holds the outcome of a trial that test_profile runs on
  // the machine: a saturated burst of requests through this loop and through run_sequential (kernel name
  // kTrialRatio: tokens/s of the interleaved loop over tokens/s of the unscheduled one).  Where interleaving did not
  // win that trial -- or both measured factors are 0 -- the derived schedule IS the unscheduled one.
  static constexpr int kTrialRatio = 108;
  bool force_interleave = false;  // set by the trial itself
  bool interleaving_pays() const {
    if (BertParams.contention > 0.0f || force_interleave) return true;
    if (contention_factor(COMMUNICATION) <= 0.0f && contention_factor(GEMM) <= 0.0f) return false;
    auto it = profiling_res_dict.find({kTrialRatio, 0, 0});
    return it == profiling_res_dict.end() || it->second > 1.02f;
  }

  void run_stream_sync() {
    if (!interleaving_pays()) {
      if (SParams.world_rank == 0) printf("Interleaving did not pay in the profile's trial on this machine: unscheduled loop. \n");
      run_sequential();
      return;
    }
    tag = true;
    _t0 = _rt->wall_seconds();
    float time_planned = 0.0f;
    layer_type main_type = COMPUTATION;
    _rt->record(Wait_EVENT, DParams0.stream);
    while (tag) {
      update_vec();
      if (exe_vec.empty()) continue;
      // hybrid synchronisation: the host waits for the event recorded just before the last kernel of
      // the previous main segment (one kernel of lead time to prepare launches), the secondary
      // stream waits on the device for the end of that segment.
      _rt->event_synchronize(Wait_EVENT);
      _rt->stream_wait_event(DParams1.stream, Main_EVENT);
      Sample* head = exe_vec.at(0);
      while (!head->empty()) {
        main_type = head->type();
        if (head->is_switch()) {
          _rt->record(Wait_EVENT, DParams0.stream);
          time_planned += head->dequeue(DParams0, 1, time_planned);
          _rt->record(Main_EVENT, DParams0.stream);
          break;
        }
        time_planned += head->dequeue(DParams0, 1, time_planned);
      }
      ++segments;
      time_planned *= contention_factor(main_type);  // the contention factor
      // fill the window with kernels of the other class from the other in-flight requests
      for (size_t sub = 1; sub < exe_vec.size(); ++sub) {
        Sample* s = exe_vec.at(sub);
        while (time_planned > 0.0f) {
          if (s->empty()) break;
          if (s->is_same_type(main_type)) break;
          if (s->duration(0, time_planned) > time_planned) {
            if (s->type() == GEMM) {
              if (!s->possible_duration(time_planned)) time_planned = 0.0f;
              else ++decompositions;
            } else {
              time_planned = 0.0f;
            }
          } else {
            time_planned -= s->dequeue(DParams1, 0, time_planned);
            ++secondary_launches;
          }
        }
      }
      time_planned = 0.0f;
    }
    _rt->device_synchronize();
  }

  void run_stop() { tag = false; }

  // ---- metrics (src/schedule.h:325-350) -----------------------------------------------------------
  // Prints the reference's lines (first `ignore_num` requests dropped; CPU_Time relative to the
  // first kept request's queue wait; throughput in samples/s) and returns them together with
  // tokens/s and latency percentiles (queue wait + device time per request).
  ServingMetrics output_recording(bool print = true) {
    ServingMetrics m;
    m.launch_errors = launch_errors;
    const size_t ignore = (size_t)BertParams.ignore_num < recs.size() ? (size_t)BertParams.ignore_num : 0;
    if (recs.size() <= ignore) return m;
    std::vector<double> lat;
    double total_avg = 0.0, gpu_sum = 0.0;
    int times = 0;
    for (size_t i = ignore; i < recs.size(); ++i) {
      const float cuda_time = _rt->elapsed_ms(recs[i].start, recs[i].stop);
      const float cpu_time = (float)((recs[i].cpu_time - recs[ignore].cpu_time) * 1000.0);
      if (print && SParams.world_rank == 0)
        printf("request: %d, CPU_Time: %f ms, CUDA_Time: %f ms. \n", times, cpu_time, cuda_time);
      total_avg += cpu_time + cuda_time;
      gpu_sum += cuda_time;
      lat.push_back(recs[i].cpu_time * 1000.0 + cuda_time);
      m.tokens += (long)recs[i].batch_size * recs[i].seq_len;
      ++times;
    }
    const float total = _rt->elapsed_ms(recs[ignore].start, recs.back().stop);
    m.records = times;
    m.total_duration_ms = total;
    m.throughput_samples_s = 1000.0 * times / total;
    m.average_latency_ms = total_avg / times;
    m.tokens_per_s = 1000.0 * (double)m.tokens / total;
    m.mean_gpu_ms = gpu_sum / times;
    std::sort(lat.begin(), lat.end());
    m.p50_latency_ms = lat[lat.size() / 2];
    m.p99_latency_ms = lat[std::min(lat.size() - 1, (size_t)(lat.size() * 99 / 100))];
    if (print && SParams.world_rank == 0) {
      printf("Total_Duration: %f ms. \n", m.total_duration_ms);
      printf("Throughput: %f samples/s. \n", m.throughput_samples_s);
      printf("Average Latency: %f ms. \n", m.average_latency_ms);
      printf("Total %d records. \n", times);
      printf("Tokens/s: %f ; p50 latency: %f ms ; p99 latency: %f ms ; segments: %ld ; secondary launches: %ld ; "
             "decompositions: %ld. \n",
             m.tokens_per_s, m.p50_latency_ms, m.p99_latency_ms, segments, secondary_launches, decompositions);
    }
    return m;
  }
};

}  // namespace liger_host
