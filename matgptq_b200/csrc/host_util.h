// Host-side state shared by the launchers: per-device caches that are safe to use from several host
// threads and on machines whose GPUs differ (each device has its own entry).
#pragma once
#include <cuda_runtime.h>

#include <atomic>

#include "kernels.h"

namespace mg {

constexpr int kMaxDevices = 64;

// Index of the current device, checked against the size of the per-device tables.
inline int current_device(int *dev_out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MG_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return MG_ERR_BAD_ARG;
  *dev_out = dev;
  return MG_OK;
}

// Number of SMs of the current device.  Queried once per device; two threads that race on the first call
// both store the same value.
inline int current_device_sm_count(int *sm_out) {
  static std::atomic<int> cache[kMaxDevices];
  int dev = 0;
  const int st = current_device(&dev);
  if (st != MG_OK) return st;
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return MG_ERR_CUDA;
    cache[dev].store(v, std::memory_order_relaxed);
  }
  *sm_out = v;
  return MG_OK;
}

// One per kernel instantiation (a function-local static of the launcher): raises the kernel's dynamic
// shared-memory limit once per device.  Setting the attribute twice from two racing threads is harmless.
struct SharedMemoryOptIn {
  std::atomic<bool> done[kMaxDevices];
  template <typename Kernel> int ensure(Kernel kernel, int bytes) {
    int dev = 0;
    const int st = current_device(&dev);
    if (st != MG_OK) return st;
    if (!done[dev].load(std::memory_order_acquire)) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return MG_ERR_CUDA;
      done[dev].store(true, std::memory_order_release);
    }
    return MG_OK;
  }
};

}  // namespace mg
