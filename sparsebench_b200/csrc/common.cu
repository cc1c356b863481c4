// Status strings, per-thread error text, per-device caches and the arch probe.

#include <mutex>

#include "sb_common.cuh"

namespace sb {
namespace {

thread_local char g_error[512] = "";

std::mutex g_device_mutex;
DeviceInfo g_device_info[kMaxDevices];
bool g_device_known[kMaxDevices] = {};

__global__ void arch_probe_kernel(int32_t* __restrict__ out, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
#ifdef __CUDA_ARCH__
    out[i] = __CUDA_ARCH__;
#endif
  }
}

}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

void clear_error() { g_error[0] = '\0'; }

int check_launch(const char* what) {
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(SB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
  return SB_OK;
}

const DeviceInfo* current_device_info(int* device_out) {
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) {
    fail(SB_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(err));
    return nullptr;
  }
  if (device < 0 || device >= kMaxDevices) {
    fail(SB_ERR_CUDA, "device ordinal %d outside [0, %d)", device, kMaxDevices);
    return nullptr;
  }
  if (device_out != nullptr) *device_out = device;
  std::lock_guard<std::mutex> lock(g_device_mutex);
  if (!g_device_known[device]) {
    DeviceInfo info;
    err = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device);
    if (err == cudaSuccess)
      err = cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (err != cudaSuccess) {
      fail(SB_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(err));
      return nullptr;
    }
    g_device_info[device] = info;
    g_device_known[device] = true;
  }
  return &g_device_info[device];
}

}  // namespace sb

extern "C" {

const char* sb_last_error(void) { return sb::g_error; }

const char* sb_status_string(int code) {
  switch (code) {
    case SB_OK: return "ok";
    case SB_ERR_INVALID_ARGUMENT: return "invalid argument";
    case SB_ERR_UNSUPPORTED: return "unsupported";
    case SB_ERR_CUDA: return "CUDA error";
    case SB_ERR_TENSOR_MAP: return "tensor map encode failed";
    default: return "unknown status";
  }
}

const char* sb_version(void) { return "0.1.0"; }

int sb_arch_probe(int32_t* out, int64_t n, sb_stream_t stream) {
  sb::clear_error();
  if (n <= 0) return sb::fail(SB_ERR_INVALID_ARGUMENT, "arch_probe: n must be positive, got %lld", (long long)n);
  if (out == nullptr) return sb::fail(SB_ERR_INVALID_ARGUMENT, "arch_probe: out is NULL");
  constexpr int kThreads = 256;
  int64_t blocks = (n + kThreads - 1) / kThreads;
  if (blocks > 4096) blocks = 4096;  // grid-stride loop covers the rest
  sb::arch_probe_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, sb::as_stream(stream)>>>(out, n);
  return sb::check_launch("arch_probe");
}

}  // extern "C"
