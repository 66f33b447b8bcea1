// Once-per-device host-side set-up (kernel attributes such as the dynamic shared-memory opt-in are per device, not
// per process: a process that drives several GPUs has to apply them on each one before its first launch there).
#pragma once
#include <atomic>
#include <cstdint>
#include <cuda_runtime.h>

namespace b200 {

// One bit per device ordinal (0..63). `pending()` is true until `done()` was called with the same device current.
// Two host threads that make the first call on a device at the same time both run the set-up; every set-up guarded
// by this class is idempotent, so that is harmless.
class PerDeviceOnce {
 public:
  bool pending(int* dev_out = nullptr) const {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (dev_out) *dev_out = dev;
    return (mask_.load(std::memory_order_acquire) & (1ull << dev)) == 0;
  }
  void done(int dev) { mask_.fetch_or(1ull << dev, std::memory_order_release); }

 private:
  std::atomic<uint64_t> mask_{0};
};

}  // namespace b200
