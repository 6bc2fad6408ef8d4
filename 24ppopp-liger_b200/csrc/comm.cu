// Tensor-parallel communication over NVLink / NVSwitch peer memory.
//
// Replaces the reference's NCCL communicator and ncclAllReduce (src/communicator.h:9-41,
// src/layer/func_wrapper.h:40-43): each rank owns a symmetric segment that every peer maps
// (CUDA IPC between processes, peer access inside one process), and the all-reduce is a kernel
// that reads peers' partial sums directly (plain peer loads), reduces in fp32, applies the
// residual add and LayerNorm that follow the all-reduce in the layer, and stores the finished
// rows into every peer's segment (plain peer stores).  No NCCL, no multicast objects.
//
// Cross-rank synchronisation: per channel, rank r has flags[p] written by peer p.  A barrier with
// epoch e = "write e into my slot on every peer, then wait until all my slots are >= e".  Epochs
// are handed out by the host per launch.  Every wait is bounded (common.cuh).
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "comm_internal.h"
#include "runtime.h"

LIGER_REGISTER_WAIT_BUDGET()

namespace liger {

constexpr int kArThreads = 256;
constexpr int kArMaxVec = 8;

struct CommDev {
  uint8_t* base[kMaxRanks];
  int rank, ws;
};

struct HandleBlob {
  uint32_t magic;
  int32_t rank;
  int32_t device;
  int32_t pad;
  int64_t pid;
  uint64_t ptr;
  uint64_t seg_bytes;
  cudaIpcMemHandle_t ipc;
};
static_assert(sizeof(HandleBlob) <= LIGER_COMM_HANDLE_BYTES, "handle blob too large");
constexpr uint32_t kHandleMagic = 0x4c474843u;

}  // namespace liger

namespace liger {

__device__ __forceinline__ uint32_t* flag_ptr(uint8_t* seg_base, int channel, int slot) {
  return reinterpret_cast<uint32_t*>(seg_base) + ((size_t)channel * kMaxRanks + slot) * kFlagStrideWords;
}

// threads 0..ws-1: publish `epoch` into my slot on every rank (including myself)
__device__ __forceinline__ void barrier_signal(const CommDev& c, int channel, uint32_t epoch) {
  if ((int)threadIdx.x < c.ws) st_release_sys(flag_ptr(c.base[threadIdx.x], channel, c.rank), epoch);
}
// threads 0..ws-1 poll the local slots; returns false (for the whole CTA) on timeout
__device__ __forceinline__ bool barrier_wait(const CommDev& c, int channel, uint32_t epoch, int* s_fail,
                                             DeviceStatus* st, unsigned int where) {
  if ((int)threadIdx.x < c.ws) {
    const uint32_t* f = flag_ptr(c.base[c.rank], channel, threadIdx.x);
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
      if ((++spins & 0xffu) == 0 && globaltimer_ns() - t0 > g_wait_budget_ns) {
        *s_fail = 1;
        report_failure(st, LIGER_DEV_TIMEOUT, where, (unsigned)threadIdx.x, epoch);
        break;
      }
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

// Entry barrier of a fused all-reduce as a kernel of its own (one warp): "every rank's partial is
// complete and visible".  Keeping the wait out of the data kernel means that no more than one tiny
// CTA per collective ever spins on a peer, so a collective that is ahead of its peers cannot
// occupy the SMs that the peers' (or this rank's other streams') GEMMs need in order to catch up.
__global__ void allreduce_entry_barrier_kernel(CommDev c, int channel, uint32_t epoch_in, unsigned long long* stamps,
                                               DeviceStatus* st) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const unsigned long long t_enter = globaltimer_ns();
  barrier_signal(c, channel, epoch_in);
  barrier_wait(c, channel, epoch_in, &s_fail, st, 0x200u);
  if (threadIdx.x == 0) { stamps[0] = t_enter; stamps[1] = globaltimer_ns(); stamps[4] += stamps[1] - t_enter; }
}

// VEC = 16-byte vectors per thread a row needs (n <= 256 * VEC * 8 columns); the row lives in registers.
template <int VEC>
__global__ void __launch_bounds__(kArThreads, 2)
allreduce_fused_kernel(CommDev c, int channel, size_t partial_off, size_t recv_off, size_t out_off,
                       const __half* residual_in, __half* hidden,
                       const __half* __restrict__ bias, const __half* __restrict__ gamma,
                       const __half* __restrict__ beta, int n, int row_lo, int row_hi, int one_shot, int rows_per_rank,
                       uint32_t epoch_in,
                       uint32_t epoch_out, unsigned int* done_counter, unsigned long long* stamps, DeviceStatus* st,
                       int barrier_mode) {  // 0: exit barrier only (entry ran as its own kernel); 1: no exit barrier; 2: entry barrier here too; 3: entry here, no exit
  __shared__ float red[32];
  __shared__ int s_fail;
  __shared__ int s_last;
  if (threadIdx.x == 0) { s_fail = 0; s_last = 0; }
  __syncthreads();

  // The entry barrier normally ran as allreduce_entry_barrier_kernel, earlier on this stream.  The latency-bound
  // one-shot form (barrier_mode == 2) does it here instead and saves a launch: block 0 publishes this rank's
  // arrival, every block waits for all ranks' arrivals on its own (nothing else is running beside a decode step, so
  // blocks that spin take nothing from anyone).
  if (barrier_mode >= 2) {
    const unsigned long long t_enter = globaltimer_ns();
    if (blockIdx.x == 0) barrier_signal(c, channel, epoch_in);
    barrier_wait(c, channel, epoch_in, &s_fail, st, 0x200u);
    if (blockIdx.x == 0 && threadIdx.x == 0) { stamps[0] = t_enter; stamps[1] = globaltimer_ns(); stamps[4] += stamps[1] - t_enter; }
  }

  const int nvec = n >> 3;
  for (int row = row_lo + blockIdx.x; row < row_hi; row += gridDim.x) {
    const size_t roff = (size_t)row * n;
    float v[VEC][8];
#pragma unroll
    for (int i = 0; i < VEC; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
    // Summation order: starts at rank (row mod ws) and continues cyclically.  It depends only on the
    // row, not on which rank owns it or on how a batch was split, so results are reproducible across
    // one-shot / two-shot and across micro-batching, and different rows start at different peers,
    // which spreads the reads over all links.  Gather mode reads only this rank's own rows.
    const int nsum = one_shot == 2 ? 1 : c.ws;
    const int first = one_shot == 2 ? c.rank : row % c.ws;
    // where rank p's contribution to this row lives
    // mode 3: the producing GEMMs already stored every rank's rows for this owner into local slots
    // mode 5: the same input, but the finished rows are stored locally only (a copy-engine all-gather follows)
    // mode 4: peers' rows were copied into local receive slots by the copy engines; own rows are
    // read from the own partial in place
    auto source = [&](int p) -> const __half* {
      return (one_shot == 3 || one_shot == 5) ? reinterpret_cast<const __half*>(c.base[c.rank] + partial_off) +
                              ((size_t)p * rows_per_rank + (row - c.rank * rows_per_rank)) * n
          : one_shot == 4
              ? (p == c.rank ? reinterpret_cast<const __half*>(c.base[c.rank] + partial_off) + roff
                             : reinterpret_cast<const __half*>(c.base[c.rank] + recv_off) +
                                   ((size_t)p * rows_per_rank + (row - c.rank * rows_per_rank)) * n)
              : reinterpret_cast<const __half*>(c.base[p] + partial_off) + roff;
    };
    auto accumulate = [&](float (&acc)[8], const uint4& u) {
      const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __half22float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    };
    // The loads of two ranks are in flight together (where the registers allow: VEC <= 6), which halves the number
    // of dependent round trips over NVLink; the additions still happen in the order first, first + 1, ...
    constexpr bool kPair = VEC <= 6;
    for (int kx = 0; kx < nsum; kx += kPair ? 2 : 1) {
      int p0 = first + kx;
      if (p0 >= c.ws) p0 -= c.ws;
      const __half* s0 = source(p0);
      uint4 u0[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int idx = threadIdx.x + i * kArThreads;
        if (idx < nvec) u0[i] = __ldcg(reinterpret_cast<const uint4*>(s0 + (size_t)idx * 8));
      }
      if constexpr (kPair) {
        const bool two = kx + 1 < nsum;
        int p1 = first + kx + 1;
        if (p1 >= c.ws) p1 -= c.ws;
        const __half* s1 = two ? source(p1) : s0;
        uint4 u1[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const int idx = threadIdx.x + i * kArThreads;
          if (two && idx < nvec) u1[i] = __ldcg(reinterpret_cast<const uint4*>(s1 + (size_t)idx * 8));
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const int idx = threadIdx.x + i * kArThreads;
          if (idx < nvec) {
            accumulate(v[i], u0[i]);
            if (two) accumulate(v[i], u1[i]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const int idx = threadIdx.x + i * kArThreads;
          if (idx < nvec) accumulate(v[i], u0[i]);
        }
      }
    }
    // residual + bias; round to fp16 (the value every later consumer sees)
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int idx = threadIdx.x + i * kArThreads;
      if (idx < nvec) {
        if (hidden != nullptr) {
          uint4 r = *reinterpret_cast<const uint4*>(residual_in + roff + (size_t)idx * 8);
          const __half2* rh = reinterpret_cast<const __half2*>(&r);
          uint4 bu = bias ? __ldg(reinterpret_cast<const uint4*>(bias + (size_t)idx * 8)) : make_uint4(0, 0, 0, 0);
          const __half2* bh = reinterpret_cast<const __half2*>(&bu);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __half22float2(rh[j]);
            float2 b = __half22float2(bh[j]);
            v[i][2 * j] += f.x + b.x;
            v[i][2 * j + 1] += f.y + b.y;
          }
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sum += v[i][2 * j] + v[i][2 * j + 1];
          __half2 hh = __floats2half2_rn(v[i][2 * j], v[i][2 * j + 1]);
          ow[j] = *reinterpret_cast<uint32_t*>(&hh);
          float2 back = __half22float2(hh);
          v[i][2 * j] = back.x;
          v[i][2 * j + 1] = back.y;
        }
        if (hidden != nullptr) *reinterpret_cast<uint4*>(hidden + roff + (size_t)idx * 8) = o;
      }
    }
    float mean = 0.0f, rstd = 1.0f;
    if (gamma != nullptr) {
      // two-pass statistics as in the reference's LayerNorm (src/cuda/cuda_kernels.cu:463-508)
      sum = warp_sum(sum);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
      __syncthreads();
      float t = (threadIdx.x & 31) < (kArThreads >> 5) ? red[threadIdx.x & 31] : 0.0f;
      mean = warp_sum(t) / (float)n;
      float vs = 0.0f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int idx = threadIdx.x + i * kArThreads;
        if (idx < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; vs += d * d; }
        }
      }
      vs = warp_sum(vs);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = vs;
      __syncthreads();
      t = (threadIdx.x & 31) < (kArThreads >> 5) ? red[threadIdx.x & 31] : 0.0f;
      rstd = rsqrtf(warp_sum(t) / (float)n + 1e-6f);
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int idx = threadIdx.x + i * kArThreads;
      if (idx < nvec) {
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
        if (gamma != nullptr) {
          uint4 gu = __ldg(reinterpret_cast<const uint4*>(gamma + (size_t)idx * 8));
          uint4 bu = __ldg(reinterpret_cast<const uint4*>(beta + (size_t)idx * 8));
          const __half2* gh = reinterpret_cast<const __half2*>(&gu);
          const __half2* bh = reinterpret_cast<const __half2*>(&bu);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 g = __half22float2(gh[j]);
            float2 b = __half22float2(bh[j]);
            ow[j] = pack_half2((v[i][2 * j] - mean) * rstd * g.x + b.x, (v[i][2 * j + 1] - mean) * rstd * g.y + b.y);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) ow[j] = pack_half2(v[i][2 * j], v[i][2 * j + 1]);
        }
        if (one_shot == 1 || one_shot == 4 || one_shot == 5) {
          *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(c.base[c.rank] + out_off) + roff + (size_t)idx * 8) = o;
        } else {
          for (int kx = 0; kx < c.ws; ++kx) {
            int p = c.rank + kx;
            if (p >= c.ws) p -= c.ws;
            *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(c.base[p] + out_off) + roff + (size_t)idx * 8) = o;
          }
        }
      }
    }
  }

  // ---- exit barrier: all of this rank's stores are visible before any rank moves on ----
  // One system-scope fence per CTA, by the thread that counts the CTA in, after the CTA barrier: fences are
  // cumulative, so it covers the stores of all 256 threads (a fence per thread serialises in the memory pipeline).
  // Without an exit barrier nothing is signalled and the end of the kernel publishes the (local) stores.
  const bool exit_barrier = !(barrier_mode == 1 || barrier_mode == 3);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (exit_barrier) __threadfence_system();
    const unsigned int ticket = atomicAdd(done_counter, 1u);
    if (ticket == gridDim.x - 1) {
      *done_counter = 0u;
      s_last = 1;
      if (exit_barrier) __threadfence_system();  // the other CTAs' stores, seen through the counter, before the signal
    }
  }
  __syncthreads();
  if (s_last && !exit_barrier) {
    if (threadIdx.x == 0) { stamps[2] = globaltimer_ns(); stamps[5] += stamps[2] - stamps[1]; stamps[7] += 1ull; }
  } else if (s_last) {
    const unsigned long long t_work = globaltimer_ns();
    if ((int)threadIdx.x < c.ws) __threadfence_system();
    barrier_signal(c, channel, epoch_out);
    barrier_wait(c, channel, epoch_out, &s_fail, st, 0x201u);
    if (threadIdx.x == 0) {
      // stamps of the last CTA to finish: wait for peers at entry / own work / wait for peers at exit
      const unsigned long long t_exit = globaltimer_ns();
      stamps[2] = t_work; stamps[3] = t_exit;
      stamps[5] += t_work - stamps[1]; stamps[6] += t_exit - t_work; stamps[7] += 1ull;
    }
  }
}


// ---- all-gather whose consumer is the next GEMM (liger_allgather_push) ---------------------------------------
__global__ void set_word_kernel(uint32_t* word, uint32_t value) { *word = value; }

}  // namespace liger

using namespace liger;

namespace liger {
__global__ void comm_barrier_kernel(CommDev c, int channel, uint32_t epoch, unsigned long long* stamps, int stamp_slot,
                                    DeviceStatus* st, unsigned int where);
}

// Launches the instance whose per-thread row buffer just fits n columns.
template <typename... Args>
static void launch_allreduce_kernel(int grid, cudaStream_t stream, int n, Args... args) {
  const int vec = (n / 8 + kArThreads - 1) / kArThreads;
  if (vec <= 2) allreduce_fused_kernel<2><<<grid, kArThreads, 0, stream>>>(args...);
  else if (vec <= 4) allreduce_fused_kernel<4><<<grid, kArThreads, 0, stream>>>(args...);
  else if (vec <= 6) allreduce_fused_kernel<6><<<grid, kArThreads, 0, stream>>>(args...);
  else allreduce_fused_kernel<8><<<grid, kArThreads, 0, stream>>>(args...);
}

extern "C" int liger_comm_create(liger_comm** out, int rank, int world_size, size_t data_bytes, int channels) {
  if (!out || world_size < 1 || world_size > kMaxRanks || rank < 0 || rank >= world_size || channels < 1 ||
      (size_t)channels * kMaxRanks * kFlagStrideWords * 4 > kFlagRegionBytes)
    return set_error(LIGER_ERR_INVALID, "comm_create: bad argument (world_size <= %d, channels <= %d)", kMaxRanks,
                     (int)(kFlagRegionBytes / (kMaxRanks * kFlagStrideWords * 4)));
  const DeviceInfo* dev = current_device();
  if (!dev) return LIGER_ERR_CUDA;
  liger_comm* c = new liger_comm();
  c->rank = rank; c->ws = world_size; c->channels = channels; c->device = dev->device;
  c->data_bytes = (data_bytes + 255) & ~(size_t)255;
  c->seg_bytes = kFlagRegionBytes + c->data_bytes;
  cudaError_t e = cudaMalloc((void**)&c->local, c->seg_bytes);
  if (e == cudaSuccess) e = cudaMemset(c->local, 0, kFlagRegionBytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&c->done, sizeof(unsigned int) * channels);
  if (e == cudaSuccess) e = cudaMemset(c->done, 0, sizeof(unsigned int) * channels);
  if (e == cudaSuccess) e = cudaMalloc((void**)&c->stamps, sizeof(unsigned long long) * 8 * channels);
  if (e == cudaSuccess) e = cudaMemset(c->stamps, 0, sizeof(unsigned long long) * 8 * channels);
  if (e == cudaSuccess) e = cudaMalloc((void**)&c->ready_src, sizeof(uint32_t) * channels);
  if (e == cudaSuccess) e = cudaMemset(c->ready_src, 0, sizeof(uint32_t) * channels);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (c->local) cudaFree(c->local);
    if (c->done) cudaFree(c->done);
    if (c->stamps) cudaFree(c->stamps);
    if (c->ready_src) cudaFree(c->ready_src);
    delete c;
    return set_error(LIGER_ERR_CUDA, "comm_create: allocating %zu bytes failed: %s", data_bytes, cudaGetErrorString(e));
  }
  c->epoch.assign(channels, 0u);
  c->ready_block_rows.assign(channels, 0);
  c->peer[rank] = c->local;
  if (world_size == 1) c->connected = true;
  *out = c;
  return LIGER_OK;
}

extern "C" int liger_comm_export(liger_comm* c, void* handle_out) {
  if (!c || !handle_out) return set_error(LIGER_ERR_INVALID, "comm_export: null argument");
  HandleBlob b;
  memset(&b, 0, sizeof(b));
  b.magic = kHandleMagic; b.rank = c->rank; b.device = c->device; b.pid = (int64_t)getpid();
  b.ptr = (uint64_t)(uintptr_t)c->local; b.seg_bytes = c->seg_bytes;
  if (c->ws > 1) {
    cudaError_t e = cudaIpcGetMemHandle(&b.ipc, c->local);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return set_error(LIGER_ERR_COMM, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    }
  }
  memset(handle_out, 0, LIGER_COMM_HANDLE_BYTES);
  memcpy(handle_out, &b, sizeof(b));
  return LIGER_OK;
}

extern "C" int liger_comm_connect(liger_comm* c, const void* all_handles) {
  if (!c || !all_handles) return set_error(LIGER_ERR_INVALID, "comm_connect: null argument");
  LIGER_CUDA_TRY(cudaSetDevice(c->device));
  for (int p = 0; p < c->ws; ++p) {
    HandleBlob b;
    memcpy(&b, (const uint8_t*)all_handles + (size_t)p * LIGER_COMM_HANDLE_BYTES, sizeof(b));
    if (b.magic != kHandleMagic || b.rank != p)
      return set_error(LIGER_ERR_COMM, "comm_connect: handle %d is malformed (magic %08x, rank %d)", p, b.magic, b.rank);
    if (b.seg_bytes != c->seg_bytes)
      return set_error(LIGER_ERR_COMM, "comm_connect: rank %d segment is %llu bytes, mine is %zu", p,
                       (unsigned long long)b.seg_bytes, c->seg_bytes);
    if (p == c->rank) continue;
    if (b.pid == (int64_t)getpid()) {
      if (b.device != c->device) {
        int can = 0;
        LIGER_CUDA_TRY(cudaDeviceCanAccessPeer(&can, c->device, b.device));
        if (!can) return set_error(LIGER_ERR_COMM, "comm_connect: device %d cannot access device %d", c->device, b.device);
        cudaError_t e = cudaDeviceEnablePeerAccess(b.device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
          return set_error(LIGER_ERR_COMM, "cudaDeviceEnablePeerAccess(%d): %s", b.device, cudaGetErrorString(e));
        cudaGetLastError();
      }
      c->peer[p] = (uint8_t*)(uintptr_t)b.ptr;
    } else {
      void* ptr = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&ptr, b.ipc, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error(LIGER_ERR_COMM, "cudaIpcOpenMemHandle(rank %d): %s", p, cudaGetErrorString(e));
      }
      c->peer[p] = (uint8_t*)ptr;
      c->ipc_open[p] = true;
    }
  }
  c->connected = true;
  return LIGER_OK;
}

extern "C" int liger_comm_destroy(liger_comm* c) {
  if (!c) return LIGER_OK;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int p = 0; p < c->ws; ++p)
    if (c->ipc_open[p]) cudaIpcCloseMemHandle(c->peer[p]);
  if (c->local) cudaFree(c->local);
  if (c->done) cudaFree(c->done);
  if (c->stamps) cudaFree(c->stamps);
  if (c->ready_src) cudaFree(c->ready_src);
  for (cudaStream_t hs : c->gather_streams) cudaStreamDestroy(hs);
  for (cudaEvent_t he : c->gather_events) cudaEventDestroy(he);
  if (c->gather_fork) cudaEventDestroy(c->gather_fork);
  delete c;
  cudaGetLastError();
  return LIGER_OK;
}

extern "C" int liger_comm_timing(liger_comm* c, int channel, int reset, double out_us[4]) {
  if (!c || !out_us || channel < 0 || channel >= c->channels) return set_error(LIGER_ERR_INVALID, "comm_timing: bad argument");
  unsigned long long h[8];
  LIGER_CUDA_TRY(cudaMemcpy(h, c->stamps + 8 * channel, sizeof(h), cudaMemcpyDeviceToHost));
  out_us[0] = (double)h[4] * 1e-3; out_us[1] = (double)h[5] * 1e-3; out_us[2] = (double)h[6] * 1e-3; out_us[3] = (double)h[7];
  if (reset) LIGER_CUDA_TRY(cudaMemset(c->stamps + 8 * channel, 0, sizeof(h)));
  return LIGER_OK;
}

extern "C" void* liger_comm_data(liger_comm* c) { return c ? c->local + kFlagRegionBytes : nullptr; }
extern "C" size_t liger_comm_data_bytes(liger_comm* c) { return c ? c->data_bytes : 0; }
extern "C" int liger_comm_rank(liger_comm* c) { return c ? c->rank : -1; }
extern "C" int liger_comm_world_size(liger_comm* c) { return c ? c->ws : 0; }

extern "C" int liger_allreduce_fused(liger_comm* c, int channel, size_t partial_off, size_t out_off,
                                     const void* residual_in, void* hidden, const void* bias, const void* gamma, const void* beta, int m, int n, int row_begin,
                                     int row_end, int one_shot, void* stream) {
  if (!c) return set_error(LIGER_ERR_INVALID, "allreduce_fused: null communicator");
  if (!c->connected) return set_error(LIGER_ERR_COMM, "allreduce_fused: communicator is not connected");
  if (channel < 0 || channel >= c->channels) return set_error(LIGER_ERR_INVALID, "allreduce_fused: channel %d of %d", channel, c->channels);
  if (m <= 0 || n <= 0 || n % 8 || n > kArThreads * kArMaxVec * 8)
    return set_error(LIGER_ERR_UNSUPPORTED, "allreduce_fused: n = %d must be a multiple of 8 and <= %d", n,
                     kArThreads * kArMaxVec * 8);
  if (row_begin < 0 || row_end > m || row_begin > row_end) return set_error(LIGER_ERR_INVALID, "allreduce_fused: bad row range");
  const size_t bytes = (size_t)m * n * 2;
  const int rpr_all = (m + c->ws - 1) / c->ws;
  const size_t in_bytes = (one_shot == 3 || one_shot == 5) ? (size_t)c->ws * rpr_all * n * 2 : bytes;
  if (partial_off % 16 || out_off % 16 || partial_off + in_bytes > c->data_bytes || out_off + bytes > c->data_bytes)
    return set_error(LIGER_ERR_INVALID, "allreduce_fused: offsets must be 16-byte aligned and inside the %zu-byte data region",
                     c->data_bytes);
  if ((gamma == nullptr) != (beta == nullptr)) return set_error(LIGER_ERR_INVALID, "allreduce_fused: gamma and beta go together");
  if (hidden && !residual_in) residual_in = hidden;
  if (((uintptr_t)hidden | (uintptr_t)residual_in | (uintptr_t)bias | (uintptr_t)gamma | (uintptr_t)beta) & 15u)
    return set_error(LIGER_ERR_INVALID, "allreduce_fused: pointers must be 16-byte aligned");
  const DeviceInfo* dev = current_device();
  if (!dev) return LIGER_ERR_CUDA;
  CommDev cd;
  for (int p = 0; p < kMaxRanks; ++p) cd.base[p] = p < c->ws ? c->peer[p] : nullptr;
  cd.rank = c->rank; cd.ws = c->ws;
  if (one_shot < 0 || one_shot > 6 || one_shot == 4)
    return set_error(LIGER_ERR_INVALID, "allreduce_fused: one_shot must be 0, 1, 2, 3, 5 or 6");
  // 6 = one-shot without the exit barrier: the caller alternates between two partial buffers, so the barrier at the
  // entry of the next call on this channel is what tells it that every rank has finished reading this one's input
  const int barrier_mode = one_shot == 5 ? 1 : one_shot == 1 ? 2 : one_shot == 6 ? 3 : 0;
  if (one_shot == 6) one_shot = 1;
  int lo = row_begin, hi = row_end;
  if (one_shot != 1) {
    const int rpr = (m + c->ws - 1) / c->ws;
    lo = row_begin > c->rank * rpr ? row_begin : c->rank * rpr;
    const int own_hi = (c->rank + 1) * rpr < m ? (c->rank + 1) * rpr : m;
    hi = row_end < own_hi ? row_end : own_hi;
    if (hi < lo) hi = lo;
  }
  int grid = hi - lo;
  // The collective is bandwidth bound (NVLink for the stores to peers, HBM for the local reads); a
  // fraction of the SMs saturates both, and every CTA beyond that only takes registers and issue
  // slots away from the GEMMs and attention kernels of other requests running next to it.
  // Measured at 8 GPUs (GLM-130B shape): 64 CTAs move the data as fast as 592 do when the kernel runs
  // alone (251 vs 215 us) and cost the neighbouring GEMMs much less; with fewer ranks each rank owns
  // more rows, so the cap scales with 8 / world_size.  LIGER_AR_MAX_CTAS overrides it.
  static int max_ctas = -1;
  if (max_ctas < 0) {
    const char* e = getenv("LIGER_AR_MAX_CTAS");
    max_ctas = (e && atoi(e) > 0) ? atoi(e) : 0;
  }
  // Mode 5 touches local memory only and is meant to run with the SMs to itself: no cap below the machine.
  const int cap = one_shot == 5 ? dev->sm_count * 4
                  : max_ctas > 0 ? max_ctas
                                 : (64 * kMaxRanks / c->ws < dev->sm_count * 4 ? 64 * kMaxRanks / c->ws : dev->sm_count * 4);
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  const uint32_t e_in = ++c->epoch[channel];
  const uint32_t e_out = (barrier_mode == 1 || barrier_mode == 3) ? e_in : ++c->epoch[channel];  // no exit barrier: no second epoch
  int rc;
  if (one_shot != 1) {
    allreduce_entry_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(cd, channel, e_in, c->stamps + 8 * channel,
                                                                       dev->status_dev);
    if ((rc = check_launch("allreduce_entry_barrier_kernel")) != LIGER_OK) return rc;
  }
  launch_allreduce_kernel(
      grid, (cudaStream_t)stream, n, cd, channel, kFlagRegionBytes + partial_off, (size_t)0, kFlagRegionBytes + out_off, (const __half*)residual_in, (__half*)hidden, (const __half*)bias,
      (const __half*)gamma, (const __half*)beta, n, lo, hi, one_shot, rpr_all, e_in, e_out, c->done + channel,
      c->stamps + 8 * channel, dev->status_dev, barrier_mode);
  return check_launch("allreduce_fused_kernel");
}

extern "C" int liger_comm_channels(liger_comm* c) { return c ? c->channels : 0; }

// All-gather of finished rows by the copy engines: this rank's own rows of the [m, n] tensor at out_off go to the
// same place in every peer's segment, then a one-warp barrier kernel on `channel` tells every rank that all rows
// have landed.  No SM takes part in the transfer, so it runs under whatever kernels another stream has in flight.
extern "C" int liger_allgather_ce(liger_comm* c, int channel, size_t out_off, int m, int n, int row_begin, int row_end,
                                  void* stream) {
  if (!c) return set_error(LIGER_ERR_INVALID, "allgather_ce: null communicator");
  if (!c->connected) return set_error(LIGER_ERR_COMM, "allgather_ce: communicator is not connected");
  if (channel < 0 || channel >= c->channels) return set_error(LIGER_ERR_INVALID, "allgather_ce: channel %d of %d", channel, c->channels);
  if (m <= 0 || n <= 0 || n % 8) return set_error(LIGER_ERR_INVALID, "allgather_ce: n = %d must be a positive multiple of 8", n);
  if (row_begin < 0 || row_end > m || row_begin > row_end) return set_error(LIGER_ERR_INVALID, "allgather_ce: bad row range");
  if (out_off % 16 || out_off + (size_t)m * n * 2 > c->data_bytes)
    return set_error(LIGER_ERR_INVALID, "allgather_ce: region must be 16-byte aligned and inside the %zu-byte data region", c->data_bytes);
  const DeviceInfo* dev = current_device();
  if (!dev) return LIGER_ERR_CUDA;
  cudaStream_t s = (cudaStream_t)stream;
  const int ws = c->ws, rank = c->rank, rpr = (m + ws - 1) / ws;
  int lo = rank * rpr > row_begin ? rank * rpr : row_begin;
  const int own_hi = (rank + 1) * rpr < m ? (rank + 1) * rpr : m;
  int hi = own_hi < row_end ? own_hi : row_end;
  if (hi < lo) hi = lo;
  for (int k = 1; k < ws && hi > lo; ++k) {
    const int p = (rank + k) % ws;
    LIGER_CUDA_TRY(cudaMemcpyAsync(c->peer[p] + kFlagRegionBytes + out_off + (size_t)lo * n * 2,
                                   c->local + kFlagRegionBytes + out_off + (size_t)lo * n * 2, (size_t)(hi - lo) * n * 2,
                                   cudaMemcpyDefault, s));
  }
  CommDev cd;
  for (int p = 0; p < kMaxRanks; ++p) cd.base[p] = p < ws ? c->peer[p] : nullptr;
  cd.rank = rank; cd.ws = ws;
  const uint32_t e = ++c->epoch[channel];
  comm_barrier_kernel<<<1, 32, 0, s>>>(cd, channel, e, c->stamps + 8 * channel, 6, dev->status_dev, 0x212u);
  return check_launch("comm_barrier_kernel");
}

// ---- the same collective with the data movement on the copy engines ------------------------------------
// A stand-alone barrier (one warp): used after copy-engine transfers, which cannot signal by themselves.
namespace liger {
__global__ void comm_barrier_kernel(CommDev c, int channel, uint32_t epoch, unsigned long long* stamps, int stamp_slot,
                                    DeviceStatus* st, unsigned int where) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const unsigned long long t0 = globaltimer_ns();
  __threadfence_system();
  barrier_signal(c, channel, epoch);
  barrier_wait(c, channel, epoch, &s_fail, st, where);
  if (threadIdx.x == 0) {
    const unsigned long long t1 = globaltimer_ns();
    if (stamp_slot == 4) { stamps[0] = t0; stamps[1] = t1; }
    stamps[stamp_slot] += t1 - t0;
  }
}
}  // namespace liger

extern "C" int liger_allreduce_ce(liger_comm* c, int channel, size_t partial_off, size_t recv_off, size_t out_off,
                                  const void* residual_in, void* hidden, const void* bias, const void* gamma,
                                  const void* beta, int m, int n, int row_begin, int row_end, void* stream) {
  if (!c) return set_error(LIGER_ERR_INVALID, "allreduce_ce: null communicator");
  if (!c->connected) return set_error(LIGER_ERR_COMM, "allreduce_ce: communicator is not connected");
  if (channel < 0 || channel >= c->channels) return set_error(LIGER_ERR_INVALID, "allreduce_ce: channel %d of %d", channel, c->channels);
  if (m <= 0 || n <= 0 || n % 8 || n > kArThreads * kArMaxVec * 8)
    return set_error(LIGER_ERR_UNSUPPORTED, "allreduce_ce: n = %d must be a multiple of 8 and <= %d", n, kArThreads * kArMaxVec * 8);
  if (row_begin < 0 || row_end > m || row_begin > row_end) return set_error(LIGER_ERR_INVALID, "allreduce_ce: bad row range");
  const int ws = c->ws, rank = c->rank;
  const int rpr = (m + ws - 1) / ws;
  const size_t bytes = (size_t)m * n * 2, recv_bytes = (size_t)ws * rpr * n * 2;
  if (partial_off % 16 || out_off % 16 || recv_off % 16 || partial_off + bytes > c->data_bytes ||
      out_off + bytes > c->data_bytes || recv_off + recv_bytes > c->data_bytes)
    return set_error(LIGER_ERR_INVALID, "allreduce_ce: regions must be 16-byte aligned and inside the %zu-byte data region", c->data_bytes);
  if ((gamma == nullptr) != (beta == nullptr)) return set_error(LIGER_ERR_INVALID, "allreduce_ce: gamma and beta go together");
  if (hidden && !residual_in) residual_in = hidden;
  if (((uintptr_t)hidden | (uintptr_t)residual_in | (uintptr_t)bias | (uintptr_t)gamma | (uintptr_t)beta) & 15u)
    return set_error(LIGER_ERR_INVALID, "allreduce_ce: pointers must be 16-byte aligned");
  const DeviceInfo* dev = current_device();
  if (!dev) return LIGER_ERR_CUDA;
  cudaStream_t s = (cudaStream_t)stream;
  CommDev cd;
  for (int p = 0; p < kMaxRanks; ++p) cd.base[p] = p < ws ? c->peer[p] : nullptr;
  cd.rank = rank; cd.ws = ws;
  auto clip = [&](int owner, int& lo, int& hi) {
    lo = owner * rpr > row_begin ? owner * rpr : row_begin;
    const int oh = (owner + 1) * rpr < m ? (owner + 1) * rpr : m;
    hi = oh < row_end ? oh : row_end;
    if (hi < lo) hi = lo;
  };
  // 1. reduce-scatter: my rows of every peer's slice go to that peer's receive slot for me
  for (int k = 1; k < ws; ++k) {
    const int p = (rank + k) % ws;
    int lo, hi;
    clip(p, lo, hi);
    if (hi > lo)
      LIGER_CUDA_TRY(cudaMemcpyAsync(c->peer[p] + kFlagRegionBytes + recv_off + ((size_t)rank * rpr + (lo - p * rpr)) * n * 2,
                                     c->local + kFlagRegionBytes + partial_off + (size_t)lo * n * 2, (size_t)(hi - lo) * n * 2,
                                     cudaMemcpyDefault, s));
  }
  const uint32_t e_in = ++c->epoch[channel];
  const uint32_t e_out = ++c->epoch[channel];
  comm_barrier_kernel<<<1, 32, 0, s>>>(cd, channel, e_in, c->stamps + 8 * channel, 4, dev->status_dev, 0x210u);
  int rc = check_launch("comm_barrier_kernel");
  if (rc != LIGER_OK) return rc;
  // 2. local reduction (+ residual + LayerNorm) of the rows this rank owns, result stored locally
  int lo, hi;
  clip(rank, lo, hi);
  int grid = hi - lo;
  static int max_ctas = -1;
  if (max_ctas < 0) {
    const char* e = getenv("LIGER_AR_MAX_CTAS");
    max_ctas = (e && atoi(e) > 0) ? atoi(e) : dev->sm_count * 4;
  }
  if (grid > max_ctas) grid = max_ctas;
  if (grid < 1) grid = 1;
  launch_allreduce_kernel(
      grid, s, n, cd, channel, kFlagRegionBytes + partial_off, kFlagRegionBytes + recv_off, kFlagRegionBytes + out_off,
      (const __half*)residual_in, (__half*)hidden, (const __half*)bias, (const __half*)gamma, (const __half*)beta, n, lo, hi, 4,
      rpr, e_in, e_out, c->done + channel, c->stamps + 8 * channel, dev->status_dev, 1);
  if ((rc = check_launch("allreduce_fused_kernel")) != LIGER_OK) return rc;
  // 3. all-gather of the finished rows
  for (int k = 1; k < ws; ++k) {
    const int p = (rank + k) % ws;
    if (hi > lo)
      LIGER_CUDA_TRY(cudaMemcpyAsync(c->peer[p] + kFlagRegionBytes + out_off + (size_t)lo * n * 2,
                                     c->local + kFlagRegionBytes + out_off + (size_t)lo * n * 2, (size_t)(hi - lo) * n * 2,
                                     cudaMemcpyDefault, s));
  }
  comm_barrier_kernel<<<1, 32, 0, s>>>(cd, channel, e_out, c->stamps + 8 * channel, 6, dev->status_dev, 0x211u);
  return check_launch("comm_barrier_kernel");
}


// All-gather whose consumer is the next GEMM (liger_gemm_args.gather_comm): see allgather_push_kernel.  The push
// is followed by a one-warp barrier kernel on barrier_channel, so that work ordered after this call on `stream`
// (or after an event recorded there) sees every rank's rows, flags or no flags.
extern "C" int liger_allgather_push(liger_comm* c, int ready_channel, int barrier_channel, size_t out_off, int m, int n,
                                    void* stream) {
  if (!c) return set_error(LIGER_ERR_INVALID, "allgather_push: null communicator");
  if (!c->connected) return set_error(LIGER_ERR_COMM, "allgather_push: communicator is not connected");
  if (ready_channel < 0 || ready_channel >= c->channels || barrier_channel < 0 || barrier_channel >= c->channels ||
      ready_channel == barrier_channel)
    return set_error(LIGER_ERR_INVALID, "allgather_push: channels %d, %d of %d (two different ones)", ready_channel, barrier_channel,
                     c->channels);
  if (m <= 0 || n <= 0 || n % 8) return set_error(LIGER_ERR_INVALID, "allgather_push: n = %d must be a positive multiple of 8", n);
  if (out_off % 16 || out_off + (size_t)m * n * 2 > c->data_bytes)
    return set_error(LIGER_ERR_INVALID, "allgather_push: region must be 16-byte aligned and inside the %zu-byte data region", c->data_bytes);
  const DeviceInfo* dev = current_device();
  if (!dev) return LIGER_ERR_CUDA;
  cudaStream_t s = (cudaStream_t)stream;
  const int ws = c->ws, rank = c->rank, rpr = (m + ws - 1) / ws;
  const int lo = rank * rpr < m ? rank * rpr : m, hi = (rank + 1) * rpr < m ? (rank + 1) * rpr : m;
  // row blocks of 256 rows (a GEMM tile), more when a rank owns more than 32 of them
  int block_rows = 256;
  while ((rpr + block_rows - 1) / block_rows > kReadyBlocksMax) block_rows *= 2;
  CommDev cd;
  for (int p = 0; p < kMaxRanks; ++p) cd.base[p] = p < ws ? c->peer[p] : nullptr;
  cd.rank = rank; cd.ws = ws;
  const uint32_t e_ready = ++c->epoch[ready_channel];
  c->ready_block_rows[ready_channel] = block_rows;
  // The copy engines move the data: per (row block, peer) one peer copy of the rows and one 4-byte peer copy that
  // publishes the epoch, in stream order.  No SM is involved, so the transfer is indifferent to what the GEMM
  // beside it occupies.  (A copy kernel on the SMs was tried and dropped: a 10-warp 256x512 GEMM CTA, or a
  // 6-warp one at 255 registers per thread, leaves two of an SM's four sub-partitions without registers for even
  // one more warp, so the copy kernel was never scheduled while the GEMM waited for its data.)
  // The steps are dealt round-robin to a few internal streams so that more than one copy engine works at a time.
  if (hi > lo && ws > 1) {
    static int nstreams = -1;
    if (nstreams < 0) { const char* e = getenv("LIGER_GATHER_STREAMS"); nstreams = (e && atoi(e) >= 1 && atoi(e) <= 4) ? atoi(e) : 2; }
    while ((int)c->gather_streams.size() < nstreams) {
      cudaStream_t hs = nullptr;
      cudaEvent_t he = nullptr;
      LIGER_CUDA_TRY(cudaStreamCreateWithFlags(&hs, cudaStreamNonBlocking));
      LIGER_CUDA_TRY(cudaEventCreateWithFlags(&he, cudaEventDisableTiming));
      c->gather_streams.push_back(hs);
      c->gather_events.push_back(he);
    }
    if (!c->gather_fork) LIGER_CUDA_TRY(cudaEventCreateWithFlags(&c->gather_fork, cudaEventDisableTiming));
    uint32_t* word = c->ready_src + ready_channel;  // epoch source for the flag copies
    set_word_kernel<<<1, 1, 0, s>>>(word, e_ready);
    int rc = check_launch("set_word_kernel");
    if (rc != LIGER_OK) return rc;
    LIGER_CUDA_TRY(cudaEventRecord(c->gather_fork, s));
    for (int h = 0; h < nstreams; ++h) LIGER_CUDA_TRY(cudaStreamWaitEvent(c->gather_streams[h], c->gather_fork, 0));
    const int nblk = (hi - lo + block_rows - 1) / block_rows;
    int step = 0;
    for (int blk = 0; blk < nblk; ++blk) {
      const int r0 = lo + blk * block_rows, r1 = r0 + block_rows < hi ? r0 + block_rows : hi;
      const size_t off = kFlagRegionBytes + out_off + (size_t)r0 * n * 2, bytes = (size_t)(r1 - r0) * n * 2;
      for (int k = 1; k < ws; ++k, ++step) {
        const int p = (rank - k + ws) % ws;
        cudaStream_t hs = c->gather_streams[step % nstreams];
        LIGER_CUDA_TRY(cudaMemcpyAsync(c->peer[p] + off, c->local + off, bytes, cudaMemcpyDefault, hs));
        uint32_t* flag = reinterpret_cast<uint32_t*>(c->peer[p]) + ((size_t)ready_channel * kMaxRanks + rank) * kFlagStrideWords + blk;
        LIGER_CUDA_TRY(cudaMemcpyAsync(flag, word, sizeof(uint32_t), cudaMemcpyDefault, hs));
      }
    }
    for (int h = 0; h < nstreams; ++h) {
      LIGER_CUDA_TRY(cudaEventRecord(c->gather_events[h], c->gather_streams[h]));
      LIGER_CUDA_TRY(cudaStreamWaitEvent(s, c->gather_events[h], 0));
    }
  }
  const uint32_t e_bar = ++c->epoch[barrier_channel];
  comm_barrier_kernel<<<1, 32, 0, s>>>(cd, barrier_channel, e_bar, c->stamps + 8 * barrier_channel, 6, dev->status_dev, 0x213u);
  return check_launch("comm_barrier_kernel");
}
