// Peer-memory signalling for kernels that fuse a collective with their compute.
//
// Every rank owns one symmetric workspace (same layout on all ranks, each mapped into every peer's address
// space). Its first GV_FLAG_BYTES bytes are a flag area: flags[slot * GV_MAX_RANKS + src_rank] holds the last
// epoch that `src_rank` announced on `slot`. A producer announces with a system-scope release store into the
// consumer's flag area; the consumer polls its own copy with acquire loads. All waits are bounded: when the
// budget runs out the kernel records an error word and carries on to its exit, so the GPU is never left spinning.
#pragma once
#include "gv_ptx.cuh"

#define GV_MAX_RANKS 8
#define GV_FLAG_SLOTS 16
#define GV_FLAG_BYTES (GV_MAX_RANKS * GV_FLAG_SLOTS * 4)

namespace gv {

struct PeerTable {
  void* base[GV_MAX_RANKS];   // workspace base address of every rank, as mapped in THIS process
  int world;
  int rank;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t* flag_ptr(void* ws_base, int slot, int src_rank) {
  return reinterpret_cast<uint32_t*>(ws_base) + slot * GV_MAX_RANKS + src_rank;
}

// Announce `epoch` on `slot` to every rank (own copy included). Call from ONE thread after the data it guards
// has been written by this kernel (the caller orders its own writes with __syncthreads / __threadfence_system).
__device__ __forceinline__ void signal_all(const PeerTable& pt, int slot, uint32_t epoch) {
  __threadfence_system();
  for (int p = 0; p < pt.world; ++p) st_release_sys(flag_ptr(pt.base[p], slot, pt.rank), epoch);
}

// Wait until rank `src` has announced at least `epoch` on `slot`. Returns false (after recording an error) when
// the time budget runs out. Epochs are compared as a signed distance so a 32-bit wrap is harmless.
__device__ __forceinline__ bool wait_flag(const PeerTable& pt, int slot, int src, uint32_t epoch, unsigned int site,
                                          uint64_t budget_ns = GV_WAIT_NS) {
  const uint32_t* f = flag_ptr(pt.base[pt.rank], slot, src);
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (static_cast<int32_t>(ld_acquire_sys(f) - epoch) >= 0) return true;
    if ((spin & 0x3f) == 0x3f) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > budget_ns) {
        record_error((site << 16) | 2u, static_cast<unsigned>(src), epoch);
        return false;
      }
      __nanosleep(64);
    }
  }
}

__device__ __forceinline__ bool wait_all(const PeerTable& pt, int slot, uint32_t epoch, unsigned int site,
                                         uint64_t budget_ns = GV_WAIT_NS) {
  bool ok = true;
  for (int p = 0; p < pt.world; ++p) ok = wait_flag(pt, slot, p, epoch, site, budget_ns) && ok;
  return ok;
}

}  // namespace gv
