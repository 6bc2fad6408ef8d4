// Host-side runtime: thread-local error text, per-device state (SM count, sticky status word),
// tensor-map encoding through the driver entry point (no link-time dependency on libcuda).
#include "runtime.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <mutex>
#include <vector>

namespace liger {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static const int kMaxDevices = 64;
static DeviceInfo g_dev[kMaxDevices];
static std::mutex g_dev_mu;

static std::vector<WaitBudgetSetter>& wait_budget_setters() {
  static std::vector<WaitBudgetSetter> v;
  return v;
}
void register_wait_budget_setter(WaitBudgetSetter fn) { wait_budget_setters().push_back(fn); }
static unsigned long long g_wait_budget_ms[kMaxDevices];  // 0 = the built-in default

// Sets the budget of every translation unit's copy on the current device.
static int apply_wait_budget(int dev, unsigned long long ms) {
  const unsigned long long ns = ms * 1000000ull;
  for (WaitBudgetSetter fn : wait_budget_setters()) {
    cudaError_t e = fn(ns);
    if (e != cudaSuccess) return set_error(LIGER_ERR_CUDA, "setting the wait budget failed: %s", cudaGetErrorString(e));
  }
  g_wait_budget_ms[dev] = ms;
  return LIGER_OK;
}

const DeviceInfo* current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error(LIGER_ERR_CUDA, "no usable CUDA device: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DeviceInfo& d = g_dev[dev];
  if (d.device == dev) return &d;
  cudaDeviceProp p;
  if ((e = cudaGetDeviceProperties(&p, dev)) != cudaSuccess) {
    set_error(LIGER_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    return nullptr;
  }
  void* h = nullptr;
  if ((e = cudaHostAlloc(&h, sizeof(DeviceStatus), cudaHostAllocMapped)) != cudaSuccess) {
    set_error(LIGER_ERR_CUDA, "cudaHostAlloc(status): %s", cudaGetErrorString(e));
    return nullptr;
  }
  memset(h, 0, sizeof(DeviceStatus));
  void* dptr = nullptr;
  if ((e = cudaHostGetDevicePointer(&dptr, h, 0)) != cudaSuccess) {
    set_error(LIGER_ERR_CUDA, "cudaHostGetDevicePointer: %s", cudaGetErrorString(e));
    cudaFreeHost(h);
    return nullptr;
  }
  d.sm_count = p.multiProcessorCount;
  d.cc_major = p.major;
  d.cc_minor = p.minor;
  d.smem_optin = p.sharedMemPerBlockOptin;
  d.status_host = (DeviceStatus*)h;
  d.status_dev = (DeviceStatus*)dptr;
  d.device = dev;
  // LIGER_WAIT_BUDGET_MS: budget of the bounded device-side waits on every device this process uses
  if (const char* env = getenv("LIGER_WAIT_BUDGET_MS")) {
    const long ms = atol(env);
    if (ms > 0 && apply_wait_budget(dev, (unsigned long long)ms) != LIGER_OK) return nullptr;
  }
  return &d;
}

int require_sm100(const DeviceInfo** out) {
  const DeviceInfo* d = current_device();
  if (!d) return LIGER_ERR_CUDA;
  if (d->cc_major != 10)
    return set_error(LIGER_ERR_UNSUPPORTED, "device compute capability %d.%d: this library is built for sm_100a only",
                     d->cc_major, d->cc_minor);
  *out = d;
  return LIGER_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

int make_tmap_2d_f16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                     uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return set_error(LIGER_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if (((uintptr_t)base & 15u) != 0 || (ld * 2) % 16 != 0)
    return set_error(LIGER_ERR_INVALID, "tensor map: base %p / pitch %llu B must be 16-byte aligned", base,
                     (unsigned long long)(ld * 2));
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = (box_inner * 2 == 128) ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (box_inner * 2 == 64) ? CU_TENSOR_MAP_SWIZZLE_64B
                                                  : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LIGER_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return LIGER_OK;
}

int make_tmap_3d_f16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t n1, uint64_t n2, uint32_t box_inner,
                     uint32_t box_n1) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return set_error(LIGER_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  if (((uintptr_t)base & 15u) != 0 || (inner * 2) % 16 != 0)
    return set_error(LIGER_ERR_INVALID, "tensor map: base %p / row %llu B must be 16-byte aligned", base,
                     (unsigned long long)(inner * 2));
  cuuint64_t dims[3] = {inner, n1, n2};
  cuuint64_t strides[2] = {inner * 2, inner * n1 * 2};
  cuuint32_t box[3] = {box_inner, box_n1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = (box_inner * 2 == 128) ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (box_inner * 2 == 64) ? CU_TENSOR_MAP_SWIZZLE_64B
                                                  : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LIGER_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with CUresult %d", (int)r);
  return LIGER_OK;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(LIGER_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  return LIGER_OK;
}

}  // namespace liger

extern "C" {

const char* liger_last_error(void) { return liger::g_err; }
const char* liger_version(void) { return "liger-b200 0.1 (sm_100a)"; }

int liger_device_status(unsigned int out[4]) {
  const liger::DeviceInfo* d = liger::current_device();
  if (!d) return LIGER_ERR_CUDA;
  volatile liger::DeviceStatus* s = d->status_host;
  unsigned int code = s->code;
  if (out) { out[0] = code; out[1] = s->where; out[2] = s->detail0; out[3] = s->detail1; }
  return (int)code;
}

int liger_set_wait_budget_ms(int milliseconds) {
  if (milliseconds < 1 || milliseconds > 600000)
    return liger::set_error(LIGER_ERR_INVALID, "set_wait_budget_ms: 1 .. 600000 ms");
  const liger::DeviceInfo* d = liger::current_device();
  if (!d) return LIGER_ERR_CUDA;
  std::lock_guard<std::mutex> lk(liger::g_dev_mu);
  return liger::apply_wait_budget(d->device, (unsigned long long)milliseconds);
}

int liger_device_status_clear(void) {
  const liger::DeviceInfo* d = liger::current_device();
  if (!d) return LIGER_ERR_CUDA;
  memset((void*)d->status_host, 0, sizeof(liger::DeviceStatus));
  return LIGER_OK;
}

}  // extern "C"
