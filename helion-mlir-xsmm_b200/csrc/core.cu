// Process-wide state of the launcher: counters, enable switch, device
// properties, the kernel status word, error text.
#include <mutex>

#include "common.cuh"

namespace b200 {

namespace {
std::atomic<int> g_enabled{1};
constexpr int kMaxDevices = 64;
DeviceInfo g_devices[kMaxDevices];
std::atomic<int> g_device_ready[kMaxDevices];
std::mutex g_device_mutex;
DeviceInfo g_no_device;

// One status word per device, in device memory of the library's own module.
__device__ int32_t g_kernel_status;
int32_t* g_status_ptr[kMaxDevices];
}  // namespace

Counters& counters() {
  static Counters c;
  return c;
}

bool enabled() { return g_enabled.load(std::memory_order_relaxed) != 0; }

int finish(int code) {
  Counters& c = counters();
  if (code == 0) {
    c.calls.fetch_add(1, std::memory_order_relaxed);
  } else if (code > 0) {
    c.refusals.fetch_add(1, std::memory_order_relaxed);
    c.last_refusal.store(code, std::memory_order_relaxed);
  } else {
    c.cuda_errors.fetch_add(1, std::memory_order_relaxed);
  }
  return code;
}

int check_launch(int kernels) {
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return -static_cast<int>(err);
  counters().launches.fetch_add(static_cast<uint64_t>(kernels), std::memory_order_relaxed);
  return 0;
}

int launched(int kernels) { return finish(check_launch(kernels)); }

const DeviceInfo& device_info() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return g_no_device;
  }
  if (g_device_ready[dev].load(std::memory_order_acquire)) return g_devices[dev];
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (g_device_ready[dev].load(std::memory_order_acquire)) return g_devices[dev];
  DeviceInfo info;
  info.device = dev;
  int value = 0;
  if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) info.sm_count = value;
  if (cudaDeviceGetAttribute(&value, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess) info.cc_major = value;
  if (cudaDeviceGetAttribute(&value, cudaDevAttrComputeCapabilityMinor, dev) == cudaSuccess) info.cc_minor = value;
  if (cudaDeviceGetAttribute(&value, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess)
    info.smem_optin = static_cast<size_t>(value);
  // The cubins in this library are sm_100a only.
  if (info.cc_major != 10) info.sm_count = 0;
  void* status = nullptr;
  if (info.sm_count > 0 && cudaGetSymbolAddress(&status, g_kernel_status) == cudaSuccess)
    g_status_ptr[dev] = static_cast<int32_t*>(status);
  cudaGetLastError();
  g_devices[dev] = info;
  g_device_ready[dev].store(1, std::memory_order_release);
  return g_devices[dev];
}

int32_t* kernel_status_word() {
  const DeviceInfo& info = device_info();
  if (info.device < 0) return nullptr;
  return g_status_ptr[info.device];
}

}  // namespace b200

using namespace b200;

extern "C" int b200_get_counters(b200_counters_t* out) {
  if (!out) return B200_E_NULL;
  Counters& c = counters();
  out->launches = c.launches.load();
  out->calls = c.calls.load();
  out->refusals = c.refusals.load();
  out->cuda_errors = c.cuda_errors.load();
  out->last_refusal = c.last_refusal.load();
  out->reserved_ = 0;
  return 0;
}

extern "C" int b200_reset_counters(void) {
  Counters& c = counters();
  c.launches = 0;
  c.calls = 0;
  c.refusals = 0;
  c.cuda_errors = 0;
  c.last_refusal = 0;
  return 0;
}

extern "C" int b200_read_kernel_status(void* stream, int32_t* out_status) {
  if (!out_status) return B200_E_NULL;
  int32_t* word = kernel_status_word();
  if (!word) return B200_E_DEVICE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemcpyAsync(out_status, word, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) return -static_cast<int>(err);
  if (*out_status != 0) {
    err = cudaMemsetAsync(word, 0, sizeof(int32_t), s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (err != cudaSuccess) return -static_cast<int>(err);
  }
  return 0;
}

extern "C" const char* b200_strerror(int code) {
  if (code < 0) return cudaGetErrorString(static_cast<cudaError_t>(-code));
  switch (code) {
    case B200_OK:
      return "ok";
    case B200_E_DTYPE:
      return "unsupported or mismatched element type";
    case B200_E_SHAPE:
      return "sizes do not fit the operator";
    case B200_E_STRIDE:
      return "unsupported strides";
    case B200_E_ALIGN:
      return "pointer alignment too small";
    case B200_E_ALIAS:
      return "output overlaps an input";
    case B200_E_NULL:
      return "required pointer is NULL";
    case B200_E_ARG:
      return "option value out of range";
    case B200_E_WORKSPACE:
      return "workspace missing or too small";
    case B200_E_DEVICE:
      return "no sm_100 device is current";
    case B200_E_DISABLED:
      return "native calls are disabled";
    case B200_E_TOO_LARGE:
      return "size beyond the entry point's fixed capacity";
    default:
      return "unknown b200ops code";
  }
}

extern "C" int b200_abi_version(void) { return B200OPS_ABI_VERSION; }

extern "C" int b200_set_enabled(int enabled_flag) {
  g_enabled.store(enabled_flag ? 1 : 0, std::memory_order_relaxed);
  return 0;
}

extern "C" int b200_sm_count(void) { return device_info().sm_count; }
