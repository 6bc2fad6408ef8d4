// Internal view of a communicator shared by the collective kernels (comm.cu) and the GEMM that
// scatters its result tiles straight into the peers' segments (gemm_sm100.cu).
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

#include "../../include/liger_b200.h"

namespace liger {
constexpr int kMaxRanks = LIGER_COMM_MAX_RANKS;
constexpr size_t kFlagRegionBytes = 65536;  // flags live in front of the data region
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
};

