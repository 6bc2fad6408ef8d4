// Internal view of a communicator shared by the collective kernels (comm.cu) and the GEMM that
// scatters its result tiles straight into the peers' segments (gemm_sm100.cu).
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/liger_b200.h"

namespace liger {
constexpr int kMaxRanks = LIGER_COMM_MAX_RANKS;
constexpr size_t kFlagRegionBytes = 65536;  // flags live in front of the data region
constexpr int kFlagStrideWords = 32;        // one 128-byte line per (channel, peer): flag word(s) written by that peer
constexpr int kReadyBlocksMax = 32;         // row blocks per rank an all-gather can announce (words of one flag line)
}  // namespace liger

struct liger_comm {
  int rank = 0, ws = 1, channels = 1, device = 0;
  size_t data_bytes = 0, seg_bytes = 0;
  uint8_t* local = nullptr;
  uint8_t* peer[liger::kMaxRanks] = {};
  bool ipc_open[liger::kMaxRanks] = {};
  bool connected = false;
  std::vector<uint32_t> epoch;   // per channel, host side
  unsigned int* done = nullptr;  // per channel CTA-completion counters (device)
  unsigned long long* stamps = nullptr;  // per channel: 4 globaltimer stamps of the last launch + 4 running sums
  uint32_t* ready_src = nullptr;         // per channel: device word holding the epoch that flag copies publish
  std::vector<cudaStream_t> gather_streams;  // internal streams the copies of liger_allgather_push are dealt to
  std::vector<cudaEvent_t> gather_events;
  cudaEvent_t gather_fork = nullptr;
  std::vector<int> ready_block_rows;     // per channel: row-block size of the most recent liger_allgather_push
};

