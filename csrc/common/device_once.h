// One-time set-up that CUDA keeps per device (cudaFuncSetAttribute, symbol addresses) needs a
// per-device "done" mark: a process-wide flag would leave every device after the first unconfigured.
#pragma once
#include <cuda_runtime.h>

namespace zx {

struct PerDeviceOnce {
  static constexpr int kMaxDevices = 64;
  bool done[kMaxDevices] = {false};
  // The mark of the device that is current on the calling thread.
  bool& current() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
    return done[dev];
  }
};

}  // namespace zx
