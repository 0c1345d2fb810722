// Allocation-free attention backward: see include/gv_no_alloc.h for who needs it and for the limits.
//
// The scratch lives in a file-scope __device__ array. Host code must not pass the array's name to a kernel:
// on the host that name is only a stand-in symbol, not a device address. The address is fetched once per
// device with cudaGetSymbolAddress (with that device current) and cached; the existing gv_attn_bwd is then
// called with its two scratch pointers aimed into the array.
#include "include/gv_no_alloc.h"

#include <cuda_runtime.h>

#include <atomic>

namespace {

constexpr long long kDqElems = GV_NOALLOC_ATTN_MAX_DQ_ELEMS;
constexpr long long kRows = GV_NOALLOC_ATTN_MAX_ROWS;
constexpr int kMaxDevices = 64;

// [ dQ accumulator : kDqElems floats | delta : kRows floats ]
static __device__ __align__(256) float g_attn_scratch[kDqElems + kRows];

// Per-device cache of the resolved address. Atomic because two host threads may make their first call together;
// both then resolve the same value, and either store is fine.
std::atomic<float*> g_scratch_addr[kMaxDevices];

// One-time set-up for the current device: resolve the device address of the scratch array.
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return GV_NOALLOC_ERR_DEVICE;
  float* ptr = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_attn_scratch);
    if (e != cudaSuccess || ptr == nullptr) return GV_NOALLOC_ERR_SYMBOL;
    g_scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return 0;
}

}  // namespace

extern "C" int gv_attn_bwd_noalloc(const gv_attn_args* args, gv_stream_t stream) {
  if (args == nullptr) return GV_NOALLOC_ERR_ARGS;
  if (args->b <= 0 || args->sq <= 0 || args->sk <= 0) return 0;
  if (args->hq <= 0 || args->hk <= 0 || args->dh <= 0 || args->hq % args->hk != 0) return GV_NOALLOC_ERR_ARGS;
  const long long dq_elems = static_cast<long long>(args->b) * args->sq * args->hq * args->dh;
  const long long rows = static_cast<long long>(args->b) * args->hq * args->sq;
  if (dq_elems > kDqElems || rows > kRows) return GV_NOALLOC_ERR_TOO_LARGE;
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  gv_attn_args a = *args;
  a.dq_accum = scratch;            // cleared by gv_attn_bwd (cudaMemsetAsync on `stream`) before it is used
  a.delta = scratch + kDqElems;    // fully overwritten before it is read
  return gv_attn_bwd(&a, stream);
}

extern "C" const char* gv_attn_bwd_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case GV_NOALLOC_ERR_TOO_LARGE:
      return "gv_attn_bwd_noalloc: problem too large for the built-in scratch "
             "(need b*sq*hq*dh <= 4194304 and b*hq*sq <= 65536); use gv_attn_bwd with caller-provided scratch";
    case GV_NOALLOC_ERR_ARGS:
      return "gv_attn_bwd_noalloc: bad arguments (NULL argument block, or head counts / head size not positive, "
             "or hq not a multiple of hk)";
    case GV_NOALLOC_ERR_SYMBOL: return "gv_attn_bwd_noalloc: could not resolve the device address of the scratch array";
    case GV_NOALLOC_ERR_DEVICE: return "gv_attn_bwd_noalloc: could not query the current CUDA device";
    default: return "gv_attn_bwd_noalloc: error reported by gv_attn_bwd (argument check or launch failure)";
  }
}
