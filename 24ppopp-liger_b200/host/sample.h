// Sample: one in-flight request -- its kernel vector, a cursor, and the run-time decomposition of
// the GEMM (or all-reduce) at the cursor into slices that fit a scheduling window.  Follows the
// reference's Sample (src/init.h:22-283) and decompose_callback / decompose_comm_callback
// (src/utils.h:218-281) predicate by predicate; the differences are deliberate and listed here:
//   * slices tile the kernel exactly: a slice covers output features (GEMM) or rows (all-reduce)
//     [N*b/factor, N*e/factor); the reference restarts every slice at column 0 and rescales an
//     already scaled size when it re-splits a remainder (src/init.h:245-254), so its decomposed
//     results are not those of the whole kernel;
//   * a re-split slice of n units gets the profiled duration of n units (the reference uses vec[1]);
//   * the decomposition dictionary is shared, not copied into every request (src/init.h:51-53);
//   * timestamps and events come from a Runtime, so the same code runs on a simulated device.
#pragma once
#include <memory>
#include <stdexcept>
#include <vector>

#include "context.h"
#include "runtime_iface.h"

namespace liger_host {

struct recorder {  // src/init.h:16-20
  double cpu_time;   // queue wait: start - arrival, seconds
  void* start;
  void* stop;
  double arrive_s, start_s;
  int batch_size, seq_len;
};

inline int slice_bound(int total, int unit, int factor, int align) {
  if (unit >= factor) return total;
  long b = (long)total * unit / factor;
  return (int)(b / align * align);
}

// A slice of `n` units of a GEMM starting where `old_func` starts (src/utils.h:218-260).
inline FuncWrap decompose_callback(const FuncWrap& old_func, int factor, int n, float duration = 0.0f) {
  const int ub = old_func.units_end > old_func.units_begin ? old_func.units_begin : 0;
  GEMM_ARGS a = old_func.args_gemm_tuple;
  // the whole kernel's feature range is recorded in the un-decomposed FuncWrap; a slice keeps it in n
  const int align = a.epilogue == LIGER_EPI_GEGLU ? 64 : 8;
  const int total = a.n;
  a.n_begin = slice_bound(total, ub, factor, align);
  a.n_end = slice_bound(total, ub + n, factor, align);
  FuncWrap f(old_func.name, duration, GEMM,
             [a](const DynamicNvInitParam& d) { return a.n_end > a.n_begin ? liger_gemm_fp16(&a, d.stream) : LIGER_OK; }, a);
  if (old_func.slicer) { f.callback = old_func.slicer(ub, ub + n, factor); f.slicer = old_func.slicer; }
  f.units_begin = ub;
  f.units_end = ub + n;
  return f;
}

// A slice of `n` units of an all-reduce: rows [M*b/factor, M*e/factor) (src/utils.h:262-281).
inline FuncWrap decompose_comm_callback(const FuncWrap& old_func, int factor, int n, float duration = 0.0f) {
  const int ub = old_func.units_end > old_func.units_begin ? old_func.units_begin : 0;
  COMM_ARGS c = old_func.args_comm_tuple;
  c.row_begin = slice_bound(c.m, ub, factor, 1);
  c.row_end = slice_bound(c.m, ub + n, factor, 1);
  FuncWrap f(old_func.name, duration, COMMUNICATION,
             [c](const DynamicNvInitParam& d) {
               if (c.copy_engine)
                 return liger_allreduce_ce(c.comm, c.channel, c.partial_off, c.recv_off, c.out_off, c.residual_in, c.hidden,
                                           c.bias, c.gamma, c.beta, c.m, c.n, c.row_begin, c.row_end, d.stream);
               return liger_allreduce_fused(c.comm, c.channel, c.partial_off, c.out_off, c.residual_in, c.hidden, c.bias,
                                            c.gamma, c.beta, c.m, c.n, c.row_begin, c.row_end, c.one_shot, d.stream);
             },
             c);
  if (old_func.slicer) { f.callback = old_func.slicer(ub, ub + n, factor); f.slicer = old_func.slicer; }
  f.units_begin = ub;
  f.units_end = ub + n;
  return f;
}

// The rest of a kernel after its first `n` units.
template <typename Decompose>
inline FuncWrap remainder_of(const FuncWrap& old_func, int factor, int n, float duration, Decompose dec) {
  FuncWrap shifted = old_func;
  const int ub = old_func.units_end > old_func.units_begin ? old_func.units_begin : 0;
  const int ue = old_func.units_end > old_func.units_begin ? old_func.units_end : factor;
  shifted.units_begin = ub + n;
  shifted.units_end = ue;
  return dec(shifted, factor, ue - ub - n, duration);
}

class Sample {
 private:
  std::vector<FuncWrap> _SubFuncWrapVec;  // empty, or [slice that fits, remainder]
  int _factor = 0;
  int _remain = 0;  // units of the current GEMM not yet issued
  float _whole_duration = 0.0f;  // profiled duration of the GEMM being decomposed
  size_t _sub_exe_num = 0;
  Runtime* _rt;

  bool _sub_empty() const { return _SubFuncWrapVec.size() == _sub_exe_num; }
  void _sub_clear() { _SubFuncWrapVec.clear(); _sub_exe_num = 0; }

 public:
  std::vector<FuncWrap> FuncWrapVec;
  const SubDict* profiling_decompse_res_dict;
  double sample_arrive = 0.0, sample_start = 0.0;  // seconds (src/init.h:45: struct timeval)
  size_t exe_num = 0;
  void *start, *stop;  // device events
  int batch_size, seq_len;
  int id = 0;
  int slot = 0;  // activation workspace of this request
  int launch_errors = 0;
  float min_slice_efficiency = 0.0f;  // see BertInitParam::min_slice_efficiency

  Sample(std::vector<FuncWrap> vec, const SubDict* dict, int batch_size_, int seq_len_, int factor, Runtime* rt)
      : _factor(factor), _rt(rt), FuncWrapVec(std::move(vec)), profiling_decompse_res_dict(dict),
        batch_size(batch_size_), seq_len(seq_len_) {
    start = rt->create_event();
    stop = rt->create_event();
    record_arrival();
  }

  bool main_empty() const { return FuncWrapVec.size() == exe_num; }
  bool empty() const { return main_empty() && _sub_empty(); }

  // "the next dequeue is the last one" (src/init.h:85-95)
  bool next_empty() const {
    if (_sub_empty()) return FuncWrapVec.size() - 1 == exe_num;
    if (main_empty()) return _SubFuncWrapVec.size() - 1 == _sub_exe_num;
    return false;
  }
  size_t size() const { return FuncWrapVec.size() - exe_num + _SubFuncWrapVec.size() - _sub_exe_num; }

  bool is_switch_from_comp_to_comm() const {  // src/init.h:101-110
    if (_sub_empty()) {
      if (exe_num + 1 >= FuncWrapVec.size()) return false;
      return COMMUNICATION == FuncWrapVec[exe_num + 1].type && COMMUNICATION != FuncWrapVec[exe_num].type;
    } else if (_SubFuncWrapVec.size() - 1 == _sub_exe_num) {
      // on the last slice the main cursor already points at the kernel after the GEMM
      return exe_num < FuncWrapVec.size() && COMMUNICATION == FuncWrapVec[exe_num].type;
    }
    return false;
  }
  bool is_switch_from_comm_to_comp() const {  // src/init.h:112-119
    if (_sub_empty()) {
      if (exe_num + 1 >= FuncWrapVec.size()) return false;
      return COMMUNICATION == FuncWrapVec[exe_num].type && COMMUNICATION != FuncWrapVec[exe_num + 1].type;
    }
    return false;
  }
  // "this dequeue ends a segment" (src/init.h:121-129)
  bool is_switch() const { return next_empty() || is_switch_from_comp_to_comm() || is_switch_from_comm_to_comp(); }

  // is the next kernel of the same class (communication / not) as `type` (src/init.h:131-149)
  bool is_same_type(layer_type type) const {
    if (_sub_empty()) return (type == COMMUNICATION) == (FuncWrapVec.at(exe_num).type == COMMUNICATION);
    return type != COMMUNICATION;
  }
  layer_type type() const { return _sub_empty() ? FuncWrapVec.at(exe_num).type : GEMM; }  // src/init.h:151-157

  // launch the next kernel (or slice) and return its planned duration (src/init.h:160-194)
  float dequeue(const DynamicNvInitParam& DParams, int is_main, float time_planned) {
    float duration = 0.0f;
    if (!_started) {
      _started = true;
      record_start();
      record_gpu_start(DParams);
    }
    // A request's kernels are ordered only within one stream: when the next kernel goes to the other
    // stream, make that stream wait for the request's previous kernel.
    if (_has_last && _last_dp.stream != DParams.stream) {
      if (_xs_event == nullptr) _xs_event = _rt->create_event();
      _rt->record(_xs_event, _last_dp.stream);
      _rt->stream_wait_event(DParams.stream, _xs_event);
    }
    _last_dp = DParams;
    _has_last = true;
    // The reference records the stop event *before* launching the last kernel (src/init.h:168-170),
    // so its CUDA_Time leaves the final kernel out; here the event goes after the last launch.
    const bool last = next_empty();
    if (!_sub_empty()) {
      // the whole GEMM is consumed when its first slice is issued; a re-split of the remainder must
      // not advance the cursor again (the reference does, src/init.h:172-175 after :249, and skips
      // the kernel that follows the GEMM)
      if (!_gemm_consumed) { exe_num++; _gemm_consumed = true; }
      FuncWrap& f = _SubFuncWrapVec.at(_sub_exe_num);
      if (f.callback(DParams) != LIGER_OK) launch_errors++;
      duration = f.duration;
      _sub_exe_num++;
      if (_sub_empty()) { _sub_clear(); _gemm_consumed = false; }
    } else if (!empty()) {
      FuncWrap& f = FuncWrapVec.at(exe_num);
      if (f.callback(DParams) != LIGER_OK) launch_errors++;
      duration = f.duration;
      if (is_main == 0 && f.type == COMMUNICATION) duration = time_planned;
      exe_num++;
    }
    if (last) record_gpu_stop(DParams);
    return duration;
  }

  recorder get_recording() const {
    return recorder{time_cpu_elapsed(), start, stop, sample_arrive, sample_start, batch_size, seq_len};
  }

  // planned duration of the next kernel on the given stream (src/init.h:201-216)
  float duration(int is_main, float time_planned) const {
    if (_sub_empty()) {
      if (is_main == 0 && FuncWrapVec.at(exe_num).type == COMMUNICATION) return time_planned;
      return FuncWrapVec.at(exe_num).duration;
    }
    return _SubFuncWrapVec.at(_sub_exe_num).duration;
  }

  // Try to split the GEMM at the cursor so that its first part fits `time_planned`
  // (src/init.h:226-259): the largest i+1 of `factor` slices whose profiled time vec[i] fits.
  // Slice durations of kernel `name` at this request's shape: the profiled vector, or, for a length between
  // profiled ones, the vector of the next profiled length of the same batch size scaled by the ratio of the whole
  // kernel's (interpolated) duration to the largest profiled slice.
  bool slice_durations(int name, float whole_duration, std::vector<float>& out) const {
    auto it = profiling_decompse_res_dict->find({name, batch_size, seq_len});
    if (it != profiling_decompse_res_dict->end()) { out = it->second; return (int)out.size() >= _factor - 1; }
    for (int s = seq_len + 1; s <= seq_len + 4096; ++s) {
      it = profiling_decompse_res_dict->find({name, batch_size, s});
      if (it == profiling_decompse_res_dict->end()) continue;
      if ((int)it->second.size() < _factor - 1 || it->second.back() <= 0.0f) return false;
      out = it->second;
      // the (factor-1)/factor slice of the borrowed shape against the same share of this shape's whole kernel
      const float scale = whole_duration > 0.0f ? whole_duration * (float)(_factor - 1) / (float)_factor / out.back() : 1.0f;
      if (scale < 1.0f) for (float& v : out) v *= scale;
      return true;
    }
    return false;
  }

  bool possible_duration(float time_planned) {
    if (_factor < 2 || profiling_decompse_res_dict == nullptr) return false;
    if (_sub_empty()) {
      const FuncWrap& whole = FuncWrapVec.at(exe_num);
      std::vector<float> vec;
      if (!slice_durations(whole.name, whole.duration, vec)) return false;
      _whole_duration = whole.duration;
      for (int i = _factor - 2; i >= 0; --i) {
        if (time_planned >= vec[i] && slice_pays(i + 1, vec[i])) {
          _sub_clear();
          const int n_run = i + 1;
          _remain = _factor - n_run;
          _SubFuncWrapVec.push_back(decompose_callback(whole, _factor, n_run, vec[i]));
          _SubFuncWrapVec.push_back(remainder_of(whole, _factor, n_run, vec[_remain - 1], decompose_callback));
          return true;
        }
      }
      return false;
    }
    // a remainder is pending: split it again
    const FuncWrap pending = _SubFuncWrapVec.at(_sub_exe_num);
    if (_sub_exe_num + 1 != _SubFuncWrapVec.size()) return false;  // only the trailing remainder re-splits
    std::vector<float> vec;
    if (!slice_durations(pending.name, _whole_duration, vec)) return false;
    for (int i = _remain - 2; i >= 0; --i) {
      if (time_planned >= vec[i] && slice_pays(i + 1, vec[i])) {
        const int n_run = i + 1;
        _remain -= n_run;
        _sub_clear();
        _SubFuncWrapVec.push_back(decompose_callback(pending, _factor, n_run, vec[n_run - 1]));
        _SubFuncWrapVec.push_back(remainder_of(pending, _factor, n_run, vec[_remain - 1], decompose_callback));
        return true;
      }
    }
    return false;
  }

  // A slice of n of the kernel's `factor` units that was profiled at slice_ms: worth launching only if it runs at
  // min_slice_efficiency of the whole kernel's rate or better.  On a GPU whose GEMM tiles are 256 columns wide and
  // whose persistent grid wants a multiple of 74 tile pairs, a narrow slice can cost several times its share.
  bool slice_pays(int n, float slice_ms) const {
    if (min_slice_efficiency <= 0.0f || _whole_duration <= 0.0f || slice_ms <= 0.0f) return true;
    return _whole_duration * (float)n / (float)_factor >= min_slice_efficiency * slice_ms;
  }

  void record_arrival() { sample_arrive = _rt->wall_seconds(); }
  void record_start() { sample_start = _rt->wall_seconds(); }
  void record_gpu_start(const DynamicNvInitParam& d) { _rt->record(start, d.stream); }
  void record_gpu_stop(const DynamicNvInitParam& d) { _rt->record(stop, d.stream); }
  double time_cpu_elapsed() const { return sample_start - sample_arrive; }

 private:
  bool _started = false;
  bool _gemm_consumed = false;
  bool _has_last = false;
  DynamicNvInitParam _last_dp;
  void* _xs_event = nullptr;
};

}  // namespace liger_host
