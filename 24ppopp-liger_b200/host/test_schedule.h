// The three entry points of the serving path (src/test_schedule.h:19-104): profile the kernels,
// serve with Liger's interleaved schedule, serve with the unscheduled tensor-parallel baseline.
// Each allocates the request input / output buffers, builds the model and the scheduler, and names
// the profile files ./Main_<ws>_<size_per_head>_<head_num>_<max_batch>_<max_seq>.json / ./Sub_...
#pragma once
#include <cmath>
#include <string>

#include "layers.h"
#include "profile_io.h"
#include "runtime_iface.h"
#include "scheduler.h"

namespace liger_host {

struct EntryContext {
  Runtime* rt;
  Coordinator* coord;
  Bert_Model* model = nullptr;  // built on first use and shared by the three entry points
  half_t* input = nullptr;
  half_t* output = nullptr;
};

inline void ensure_model(EntryContext& ctx, const BertInitParam& bp, const StaticNvInitParam& sp) {
  if (ctx.model) return;
  cuda_check(cudaSetDevice(sp.world_rank % std::max(1, device_count())), "cudaSetDevice");
  const size_t m = (size_t)bp.max_seq_len * bp.max_batch_size, k = (size_t)bp.hidden();
  ctx.input = device_alloc<half_t>(m * k, "input");
  ctx.output = device_alloc<half_t>(m * k, "output");
  // seeded activations ~ N(0,1) (the reference's input is uninitialised memory, src/test_schedule.h:29)
  host_check(liger_fill_normal(ctx.input, (int)m, (int)k, (int)k, 0, 0, (int)k, bp.seed, 0x10000u, 0.0f, 1.0f, 0, nullptr),
             "fill input");
  ctx.model = new Bert_Model(bp, sp);
}

inline ServingMetrics test_schedule(EntryContext& ctx, const BertInitParam& bp, const StaticNvInitParam& sp) {
  ensure_model(ctx, bp, sp);
  Scheduler<Bert_Model> scheduler(ctx.model, bp, sp, ctx.input, ctx.output, ctx.rt, ctx.coord);
  scheduler.load_profiles(profile_file_name("Main", bp, sp.world_size), profile_file_name("Sub", bp, sp.world_size));
  scheduler.serving();
  scheduler.run_stream_sync();
  scheduler.run_stop();
  return scheduler.output_recording();
}

inline ServingMetrics test_no_schedule(EntryContext& ctx, const BertInitParam& bp, const StaticNvInitParam& sp) {
  ensure_model(ctx, bp, sp);
  Scheduler<Bert_Model> scheduler(ctx.model, bp, sp, ctx.input, ctx.output, ctx.rt, ctx.coord);
  scheduler.load_profiles(profile_file_name("Main", bp, sp.world_size), profile_file_name("Sub", bp, sp.world_size));
  scheduler.serving();
  scheduler.run_sequential();
  scheduler.run_stop();
  return scheduler.output_recording();
}

// The trial behind `--contention auto`: does the interleaved loop, with the constants just measured, beat the
// unscheduled loop on this machine?  Ten full-size requests that all arrive at once go through each loop; the
// ratio of tokens/s is stored in the Main profile (Scheduler::kTrialRatio), where run_stream_sync finds it.
template <class MODELTYPE>
inline void policy_trial(MODELTYPE* model, const BertInitParam& bp, const StaticNvInitParam& sp, const void* input, void* output,
                         Runtime* rt, Coordinator* coord, const std::string& main_filename, const std::string& sub_filename) {
  if (sp.world_size < 2) return;
  BertInitParam trial = bp;
  trial.num_requests = 10; trial.ignore_num = 2; trial.rq_interval = 1; trial.poisson = 0;
  trial.min_seq_len = trial.max_seq_len; trial.contention = 0.0f;
  double tps[2] = {0.0, 0.0};
  for (int loop = 0; loop < 2; ++loop) {
    Scheduler<MODELTYPE> t(model, trial, sp, input, output, rt, coord);
    t.load_profiles(main_filename, sub_filename);
    t.serving();
    coord->barrier();
    if (loop == 0) t.run_sequential();
    else { t.force_interleave = true; t.run_stream_sync(); }
    t.run_stop();
    tps[loop] = t.output_recording(false).tokens_per_s;
  }
  const float ratio = tps[0] > 0.0 ? (float)(tps[1] / tps[0]) : 1.0f;
  // every rank timed its own copy of the same lock-step run; rank 0's figure is the one that is stored
  const int stored = coord->broadcast_int((int)std::lround(ratio * 1000.0f));
  if (sp.world_rank == 0) {
    MainDict d = MainFileToDict(main_filename);
    d[{Scheduler<MODELTYPE>::kTrialRatio, 0, 0}] = (float)stored / 1000.0f;
    MainDictToFile(d, main_filename);
    printf("Trial on this machine: interleaved loop %.0f tokens/s, unscheduled loop %.0f tokens/s (ratio %.3f). \n", tps[1], tps[0],
           (float)stored / 1000.0f);
  }
  coord->barrier();
}

// sq_step: profile only sequence lengths that are multiples of it (the reference profiles every
// integer length, src/test_schedule.h:103, which takes hours at this model size)
inline void test_profile(EntryContext& ctx, const BertInitParam& bp, const StaticNvInitParam& sp, int sq_step = 0) {
  ensure_model(ctx, bp, sp);
  Scheduler<Bert_Model> scheduler(ctx.model, bp, sp, ctx.input, ctx.output, ctx.rt, ctx.coord);
  const std::string main_filename = profile_file_name("Main", bp, sp.world_size);
  const std::string sub_filename = profile_file_name("Sub", bp, sp.world_size);
  if (sq_step <= 0) sq_step = bp.seq_round > 0 ? bp.seq_round : 1;
  // the warm-up request's shape, then every served shape
  const int wb = std::min(2, bp.max_batch_size);
  int wsq = std::min(64, bp.max_seq_len);
  wsq = std::max(sq_step, wsq / sq_step * sq_step);
  if (wb != bp.max_batch_size) scheduler.profile(wb, wb + 1, wsq, wsq + 1, main_filename, sub_filename, 1);
  scheduler.profile(bp.max_batch_size, bp.max_batch_size + 1, 1, bp.max_seq_len + 1, main_filename, sub_filename, sq_step);
  policy_trial(ctx.model, bp, sp, ctx.input, ctx.output, ctx.rt, ctx.coord, main_filename, sub_filename);
}

}  // namespace liger_host
