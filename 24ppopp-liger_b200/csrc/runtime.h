// Host-side runtime shared by the launchers: error reporting, per-device state, tensor maps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace liger {

// Records a message for liger_last_error() and returns `code`.
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

#define LIGER_CUDA_TRY(expr)                                                                               \
  do {                                                                                                     \
    cudaError_t _e = (expr);                                                                               \
    if (_e != cudaSuccess)                                                                                 \
      return ::liger::set_error(LIGER_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                                __FILE__, __LINE__);                                                       \
  } while (0)

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t smem_optin = 0;
  DeviceStatus* status_host = nullptr;  // pinned, mapped
  DeviceStatus* status_dev = nullptr;   // device alias of status_host
};

// State of the current CUDA device (created on first use); nullptr + error set on failure.
const DeviceInfo* current_device();

// Checks that the current device can run the sm_100a kernels.
int require_sm100(const DeviceInfo** out);

// 2-D fp16 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch `ld`
// elements; box = box_inner x box_outer elements; 128-byte swizzle when box_inner*2 == 128.
int make_tmap_2d_f16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_inner, uint32_t box_outer);

// 3-D fp16 tensor map over a contiguous [n2][n1][inner] array; box = box_inner x box_n1 x 1.
int make_tmap_3d_f16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t n1, uint64_t n2, uint32_t box_inner,
                     uint32_t box_n1);

// Launch-error check after a <<<>>> launch.
int check_launch(const char* what);

// Every translation unit whose kernels make bounded waits owns a copy of g_wait_budget_ns (common.cuh) and
// registers a function that sets it on the current device.
typedef cudaError_t (*WaitBudgetSetter)(unsigned long long ns);
void register_wait_budget_setter(WaitBudgetSetter fn);
#define LIGER_REGISTER_WAIT_BUDGET()                                                                  \
  namespace {                                                                                         \
  cudaError_t liger_tu_set_wait_budget(unsigned long long ns) {                                       \
    return cudaMemcpyToSymbol(::liger::g_wait_budget_ns, &ns, sizeof(ns));                            \
  }                                                                                                   \
  struct LigerTuWaitBudgetRegistration {                                                              \
    LigerTuWaitBudgetRegistration() { ::liger::register_wait_budget_setter(&liger_tu_set_wait_budget); } \
  } liger_tu_wait_budget_registration;                                                                \
  }

}  // namespace liger
