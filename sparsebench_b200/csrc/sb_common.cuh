// Shared host-side helpers: status codes, per-thread error text, per-device caches.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/sparsebench_b200.h"

namespace sb {

// Writes the calling thread's error text (printf style) and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

inline cudaStream_t as_stream(sb_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Returns SB_OK or records the CUDA error text. Used after launches (cudaGetLastError is not a sync).
int check_launch(const char* what);

// Cached per-device properties. Looked up once per device; later calls are a table read.
struct DeviceInfo {
  int sm_count = 0;
  int max_smem_optin = 0;
};
// Info of the calling thread's current device, or nullptr after recording an error.
const DeviceInfo* current_device_info(int* device_out = nullptr);

constexpr int kMaxDevices = 64;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace sb
