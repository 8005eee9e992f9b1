// Host-side glue shared by the translation units of libbdfp4.so.
#pragma once

#include <cuda_runtime.h>

#include <atomic>

#include "../../include/bdfp4.h"

namespace bdfp4 {

// Records a failed CUDA call for bdfp4_last_cuda_error and maps it to a status code.
int cuda_status(cudaError_t error);

// Per-device once-flags for settings CUDA keeps per device (a kernel's dynamic shared-memory limit):
// `done` is indexed by the current device, since a process may drive several GPUs. Two threads
// racing on a slot both set the attribute, which is harmless; the flag itself is atomic.
constexpr int kDeviceSlots = 64;
struct PerDeviceOnce {
  std::atomic<bool> done[kDeviceSlots] = {};
};
// Index of the current device, or -1 when it cannot be read or is past kDeviceSlots (the caller
// then sets the attribute on every call).
inline int current_device_slot() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kDeviceSlots) return -1;
  return device;
}

}  // namespace bdfp4
