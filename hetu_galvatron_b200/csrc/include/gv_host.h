// Host-side helpers shared by the launchers of the kernel library.
#pragma once
#include <cuda_runtime.h>

#include <atomic>

namespace gv {

// A function attribute (here: the opt-in dynamic shared-memory limit) belongs to the device that was current
// when it was set. One process can drive several devices, so "already set" is tracked per device; the flags are
// atomic because launchers may be called from several host threads (setting the attribute twice is harmless).
struct PerDeviceOnce {
  static constexpr int kMaxDevices = 64;
  std::atomic<bool> done[kMaxDevices];
};

template <class Kernel>
inline cudaError_t ensure_max_dynamic_smem(PerDeviceOnce& once, Kernel kern, int bytes) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool tracked = dev >= 0 && dev < PerDeviceOnce::kMaxDevices;
  if (tracked && once.done[dev].load(std::memory_order_acquire)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && tracked) once.done[dev].store(true, std::memory_order_release);
  return e;
}

}  // namespace gv
