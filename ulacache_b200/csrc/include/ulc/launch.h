// Host-side launch helpers shared by the kernels' entry points.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <stdint.h>

namespace ulc {

// "Done once per device" flag set.  A function attribute such as the dynamic shared-memory
// opt-in belongs to the function IN ONE CONTEXT: a process that drives several GPUs has to set it
// on each of them, so a process-wide boolean is not enough.
struct PerDeviceOnce {
  std::atomic<uint64_t> done{0};
};

// Opt `kernel` into `bytes` of dynamic shared memory on the current device, the first time it is
// launched there.  Returns 0 or a cudaError_t.  Safe to call from several host threads.
inline int ensure_dynamic_smem(const void* kernel, int bytes, PerDeviceOnce& once) {
  int dev = -1;
  const bool known = cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64;
  if (known && (once.done.load(std::memory_order_acquire) >> dev & 1ull)) return 0;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (known) once.done.fetch_or(1ull << dev, std::memory_order_release);
  return 0;
}

}  // namespace ulc
