// Per-device host-side caches.  cudaFuncSetAttribute and the SM count are facts of one device, and one
// process may drive several devices through this library (threads, one module per GPU), so nothing here is
// cached per process.
#pragma once
#include <cuda_runtime.h>

#include <atomic>

namespace smoe {

constexpr int kMaxDevices = 64;

// The calling thread's current device, or -1.
inline int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// One flag per device: "this kernel's launch attributes have been set on that device".  Two threads racing on
// the first call both set the attribute, which is harmless.
struct PerDeviceFlag {
  std::atomic<bool> done[kMaxDevices] = {};
  bool test(int dev) const { return done[dev].load(std::memory_order_acquire); }
  void set(int dev) { done[dev].store(true, std::memory_order_release); }
};

// Multiprocessor count of the current device (0 on failure).
inline int num_sms() {
  static std::atomic<int> sms[kMaxDevices] = {};
  const int dev = current_device();
  if (dev < 0) return 0;
  int v = sms[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    sms[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

}  // namespace smoe
