// The few device-runtime operations the scheduler needs (streams, events, clocks), behind an
// interface so that the scheduling logic can run against a simulated device on a machine without
// a GPU.  CudaRuntime maps one to one onto the CUDA calls the reference's scheduler makes
// (src/schedule.h:54-55,204-278, src/init.h:160-170,261-275); SimRuntime is a discrete-event
// model of two streams sharing one device.
#pragma once
#include <sys/time.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <deque>
#include <string>
#include <vector>

namespace liger_host {

class Runtime {
 public:
  virtual ~Runtime() {}
  virtual void* create_stream(int priority) = 0;
  virtual void* create_event() = 0;
  virtual void record(void* event, void* stream) = 0;
  virtual void event_synchronize(void* event) = 0;           // host blocks until the event completed
  virtual void stream_wait_event(void* stream, void* event) = 0;
  virtual float elapsed_ms(void* start, void* stop) = 0;
  virtual void device_synchronize() = 0;
  virtual double wall_seconds() = 0;
  virtual void sleep_us(long us) = 0;
};

#if defined(LIGER_HOST_WITH_CUDA)
}  // namespace liger_host
#include <cuda_runtime.h>
namespace liger_host {
class CudaRuntime : public Runtime {
 public:
  void* create_stream(int priority) override {
    cudaStream_t s = nullptr;
    // non-blocking streams, as cudaStreamCreateWithPriority(&s, 1, prio) at src/context.h:26-30
    cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, priority);
    return (void*)s;
  }
  void* create_event() override {
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return (void*)e;
  }
  void record(void* event, void* stream) override { cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream); }
  void event_synchronize(void* event) override { cudaEventSynchronize((cudaEvent_t)event); }
  void stream_wait_event(void* stream, void* event) override {
    cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0);
  }
  float elapsed_ms(void* start, void* stop) override {
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, (cudaEvent_t)start, (cudaEvent_t)stop);
    return ms;
  }
  void device_synchronize() override { cudaDeviceSynchronize(); }
  double wall_seconds() override {
    struct timeval tv;
    gettimeofday(&tv, 0);
    return (double)tv.tv_sec + 1e-6 * (double)tv.tv_usec;
  }
  void sleep_us(long us) override { usleep((useconds_t)us); }
};
#endif

// ---------------------------------------------------------------------------------------------
// Simulated device.  Each stream is a FIFO of items (kernel of a given duration, event record,
// wait-for-event).  At most one kernel per stream runs at a time; when both streams run kernels
// concurrently each progresses at `overlap_rate` of its isolated speed (1.0 = perfect overlap).
// The host clock only moves when the host blocks (event_synchronize, device_synchronize, sleep_us).
// Every kernel launch is logged with its start and end time.
// ---------------------------------------------------------------------------------------------
class SimRuntime : public Runtime {
 public:
  struct LaunchRecord {
    int stream;
    int tag;        // caller-defined: (request id << 16) | kernel name, etc.
    float duration; // isolated duration in ms
    double t_start, t_end;  // simulated ms
  };
  struct SimEvent { bool recorded = false; bool done = false; double t_done = 0.0; };

  double overlap_rate = 1.0;
  std::vector<LaunchRecord> log;

  ~SimRuntime() override {
    for (auto* s : streams_) delete s;
    for (auto* e : events_) delete e;
  }
  void* create_stream(int priority) override {
    Stream* s = new Stream();
    s->id = (int)streams_.size();
    s->priority = priority;
    streams_.push_back(s);
    return s;
  }
  void* create_event() override {
    SimEvent* e = new SimEvent();
    events_.push_back(e);
    return e;
  }
  // enqueue a kernel (called from FuncWrap callbacks of simulated models)
  void launch(void* stream, float duration_ms, int tag) {
    Item it; it.kind = Item::KERNEL; it.remaining = duration_ms; it.duration = duration_ms; it.tag = tag;
    it.t_enqueue = host_ms_;
    ((Stream*)stream)->q.push_back(it);
  }
  void record(void* event, void* stream) override {
    SimEvent* e = (SimEvent*)event;
    e->recorded = true; e->done = false;
    Item it; it.kind = Item::RECORD; it.ev = e; it.t_enqueue = host_ms_;
    ((Stream*)stream)->q.push_back(it);
    settle();
  }
  void stream_wait_event(void* stream, void* event) override {
    SimEvent* e = (SimEvent*)event;
    if (!e->recorded) return;  // waiting on a never-recorded event is a no-op, as in CUDA
    if (e->done) return;
    Item it; it.kind = Item::WAIT; it.ev = e; it.t_enqueue = host_ms_;
    ((Stream*)stream)->q.push_back(it);
  }
  void event_synchronize(void* event) override {
    SimEvent* e = (SimEvent*)event;
    if (!e->recorded) return;
    while (!e->done) { if (!step(1e300)) break; }
    if (e->done && e->t_done > host_ms_) host_ms_ = e->t_done;
  }
  float elapsed_ms(void* start, void* stop) override {
    event_synchronize(stop);
    return (float)(((SimEvent*)stop)->t_done - ((SimEvent*)start)->t_done);
  }
  void device_synchronize() override {
    while (step(1e300)) {}
    if (dev_ms_ > host_ms_) host_ms_ = dev_ms_;
  }
  double wall_seconds() override { return host_ms_ * 1e-3; }
  void sleep_us(long us) override { host_ms_ += (double)us * 1e-3; }
  // host-side cost of issuing work (lets tests model launch overhead)
  void host_advance_ms(double ms) { host_ms_ += ms; }
  double host_ms() const { return host_ms_; }
  double event_time_ms(void* event) const { return ((SimEvent*)event)->t_done; }

 private:
  struct Item {
    enum Kind { KERNEL, RECORD, WAIT } kind = KERNEL;
    double remaining = 0.0; float duration = 0.0f; int tag = 0; SimEvent* ev = nullptr;
    bool started = false; double t_start = 0.0; double t_enqueue = 0.0;
  };
  struct Stream { int id = 0; int priority = 0; std::deque<Item> q; };
  std::vector<Stream*> streams_;
  std::vector<SimEvent*> events_;
  double dev_ms_ = 0.0;   // device time up to which the simulation has been resolved
  double host_ms_ = 0.0;

  // resolve zero-time items (records, satisfied waits) at the heads of all streams
  void settle() {
    bool again = true;
    while (again) {
      again = false;
      for (auto* s : streams_) {
        while (!s->q.empty()) {
          Item& it = s->q.front();
          if (it.kind == Item::RECORD) {
            it.ev->done = true;
            it.ev->t_done = std::max(dev_ms_, it.t_enqueue);
            s->q.pop_front(); again = true;
          } else if (it.kind == Item::WAIT && it.ev->done) {
            s->q.pop_front(); again = true;
          } else break;
        }
      }
    }
  }
  // advance the device to the next kernel start or completion, but not past `limit_ms`;
  // false when nothing can make progress before the limit
  bool step(double limit_ms) {
    settle();
    std::vector<Stream*> heads, running;
    for (auto* s : streams_)
      if (!s->q.empty() && s->q.front().kind == Item::KERNEL) heads.push_back(s);
    if (heads.empty()) return false;
    double next_enq = 1e300;
    for (auto* s : heads) {
      Item& it = s->q.front();
      if (it.started || it.t_enqueue <= dev_ms_) running.push_back(s);
      else next_enq = std::min(next_enq, it.t_enqueue);
    }
    if (running.empty()) {  // device idle until the next kernel was submitted
      if (next_enq > limit_ms) { dev_ms_ = std::max(dev_ms_, limit_ms); return false; }
      dev_ms_ = next_enq;
      return true;
    }
    const double rate = running.size() > 1 ? overlap_rate : 1.0;
    double dt = next_enq - dev_ms_;
    for (auto* s : running) {
      Item& it = s->q.front();
      if (!it.started) { it.started = true; it.t_start = dev_ms_; }
      dt = std::min(dt, it.remaining / rate);
    }
    bool capped = false;
    if (dev_ms_ + dt > limit_ms) { dt = limit_ms - dev_ms_; capped = true; }
    if (dt < 0) dt = 0;
    for (auto* s : running) s->q.front().remaining -= dt * rate;
    dev_ms_ += dt;
    for (auto* s : running) {
      Item& it = s->q.front();
      if (it.remaining <= 1e-9) {
        LaunchRecord r{s->id, it.tag, it.duration, it.t_start, dev_ms_};
        log.push_back(r);
        s->q.pop_front();
      }
    }
    settle();
    return !capped;
  }
};

}  // namespace liger_host
