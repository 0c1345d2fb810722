// NVLink-5 / NVSwitch collectives as plain kernels over peer-mapped memory, used by the hardware profiler to
// measure what the fabric gives this package's own kernels (point-to-point pull, all-to-all, two-shot all-reduce,
// in-switch multimem all-reduce) next to the NCCL figures. The reference measures the fabric with the vendored
// nccl-tests binaries driven over mpirun (galvatron/core/profiler/hardware_profiler.py:184-315,
// galvatron/site_package/nccl-tests/src/*.cu); here the measurement kernels are part of the kernel library, run
// inside the already initialised job and are timed with CUDA events. They are also usable as collectives in their
// own right (same flag protocol as csrc/comm_kernels.cu; every wait is bounded).
#include "include/gv_kernels.h"
#include "include/gv_comm.cuh"

namespace gv {
int num_sms();
typedef __nv_bfloat16 bf16;

static PeerTable table_of(const gv_peers* p) {
  PeerTable t;
  for (int i = 0; i < GV_MAX_RANKS; ++i) t.base[i] = i < p->world ? p->bases[i] : nullptr;
  t.world = p->world;
  t.rank = p->rank;
  return t;
}

__device__ __forceinline__ bool block_wait_flag(const PeerTable& pt, int slot, int src, uint32_t epoch, unsigned site) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = wait_flag(pt, slot, src, epoch, site) ? 1 : 0;
  __syncthreads();
  const bool ok = ok_s != 0;
  __syncthreads();
  return ok;
}

// 8 independent 16-byte transfers in flight per thread
__device__ __forceinline__ void copy_vec(uint4* __restrict__ dst, const uint4* __restrict__ src, long long nvec) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += stride * 8) {
    uint4 tmp[8];
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (i0 + q * stride < nvec) tmp[q] = src[i0 + q * stride];
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (i0 + q * stride < nvec) dst[i0 + q * stride] = tmp[q];
  }
}

// ---------------------------------------------------------------- point to point (send/recv as a pull)
__global__ void p2p_pull_kernel(PeerTable pt, int src, long long src_off, uint4* __restrict__ out, long long nvec, int slot,
                                uint32_t epoch) {
  if (!block_wait_flag(pt, slot, src, epoch, 0x51)) return;
  copy_vec(out, reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(pt.base[src]) + src_off), nvec);
}

// ---------------------------------------------------------------- all-to-all: out[s] = peer s's block for me
__global__ void alltoall_pull_kernel(PeerTable pt, long long src_off, uint4* __restrict__ out, long long nvec, int slot,
                                     uint32_t epoch) {
  for (int k = 0; k < pt.world; ++k) {
    const int src = (pt.rank + k) % pt.world;
    if (!block_wait_flag(pt, slot, src, epoch, 0x52)) return;
    const uint4* in = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(pt.base[src]) + src_off) +
                      static_cast<long long>(pt.rank) * nvec;
    copy_vec(out + static_cast<long long>(src) * nvec, in, nvec);
  }
}

// ---------------------------------------------------------------- two-shot all-reduce, first shot:
// this rank owns shard `rank` of the buffer: sum it over all peers (fp32) and write the result back into every
// peer's buffer. Only the owner touches its shard, so the exchange is in place. The caller then announces a second
// epoch and waits for everybody's.
__global__ void allreduce_shard_kernel(PeerTable pt, long long off, long long shard_vec, int slot, uint32_t epoch) {
  for (int p = 0; p < pt.world; ++p)
    if (!block_wait_flag(pt, slot, p, epoch, 0x53)) return;
  const long long first = static_cast<long long>(pt.rank) * shard_vec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < shard_vec; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < pt.world; ++k) {
      const int r = (pt.rank + k) % pt.world;
      const uint4 u = (reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(pt.base[r]) + off))[first + i];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    for (int k = 0; k < pt.world; ++k) {
      const int r = (pt.rank + k) % pt.world;
      (reinterpret_cast<uint4*>(reinterpret_cast<char*>(pt.base[r]) + off))[first + i] = o;
    }
  }
}

// ---------------------------------------------------------------- in-switch all-reduce through the multicast mapping:
// multimem.ld_reduce sums the shard over every replica inside NVSwitch, multimem.st broadcasts the result.
__global__ void allreduce_multimem_kernel(PeerTable pt, char* mc_base, long long off, long long shard_vec, int slot,
                                          uint32_t epoch) {
  for (int p = 0; p < pt.world; ++p)
    if (!block_wait_flag(pt, slot, p, epoch, 0x54)) return;
  const long long first = static_cast<long long>(pt.rank) * shard_vec;
  uint4* mc = reinterpret_cast<uint4*>(mc_base + off) + first;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < shard_vec; i += stride) {
    uint32_t x, y, z, w;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(x), "=r"(y), "=r"(z), "=r"(w)
                 : "l"(mc + i)
                 : "memory");
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc + i), "r"(x), "r"(y), "r"(z), "r"(w)
                 : "memory");
  }
}

static int grid_for(long long nvec, int per_sm) {
  long long grid = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * per_sm;
  if (grid > cap) grid = cap;
  return grid < 1 ? 1 : static_cast<int>(grid);
}

}  // namespace gv

using namespace gv;

extern "C" int gv_p2p_pull(const gv_peers* peers, int src, long long src_off, void* out, long long nbytes, int slot,
                           unsigned int epoch, gv_stream_t s) {
  if (nbytes <= 0) return 0;
  if (src < 0 || src >= peers->world || nbytes % 16 || src_off % 16 || (reinterpret_cast<uintptr_t>(out) & 15)) return 2701;
  const long long nvec = nbytes / 16;
  p2p_pull_kernel<<<grid_for(nvec, 4), 256, 0, (cudaStream_t)s>>>(table_of(peers), src, src_off, (uint4*)out, nvec, slot, epoch);
  return (int)cudaGetLastError();
}

// Same pull with a caller-chosen number of CTAs: a transfer that runs next to a compute kernel (the K/V fetch of
// ring attention) should leave the SMs to that kernel; a few dozen CTAs keep NVLink busy.
extern "C" int gv_p2p_pull_ex(const gv_peers* peers, int src, long long src_off, void* out, long long nbytes, int slot,
                              unsigned int epoch, int max_blocks, gv_stream_t s) {
  if (nbytes <= 0) return 0;
  if (src < 0 || src >= peers->world || nbytes % 16 || src_off % 16 || (reinterpret_cast<uintptr_t>(out) & 15)) return 2701;
  const long long nvec = nbytes / 16;
  int grid = grid_for(nvec, 4);
  if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
  p2p_pull_kernel<<<grid, 256, 0, (cudaStream_t)s>>>(table_of(peers), src, src_off, (uint4*)out, nvec, slot, epoch);
  return (int)cudaGetLastError();
}

extern "C" int gv_alltoall_pull(const gv_peers* peers, long long src_off, void* out, long long bytes_per_rank, int slot,
                                unsigned int epoch, gv_stream_t s) {
  if (bytes_per_rank <= 0) return 0;
  if (bytes_per_rank % 16 || src_off % 16 || (reinterpret_cast<uintptr_t>(out) & 15)) return 2702;
  const long long nvec = bytes_per_rank / 16;
  alltoall_pull_kernel<<<grid_for(nvec, 4), 256, 0, (cudaStream_t)s>>>(table_of(peers), src_off, (uint4*)out, nvec, slot, epoch);
  return (int)cudaGetLastError();
}

// First shot of the two-shot all-reduce over the bf16 buffer at byte offset `off` (n_elems elements, a multiple of
// 8 * world). mc_base != NULL selects the in-switch (multimem) form on the multicast mapping of the same workspace.
extern "C" int gv_allreduce_shard(const gv_peers* peers, void* mc_base, long long off, long long n_elems, int slot,
                                  unsigned int epoch, gv_stream_t s) {
  if (n_elems <= 0) return 0;
  if (n_elems % (8LL * peers->world) || off % 16) return 2703;
  const long long shard_vec = n_elems / 8 / peers->world;
  if (mc_base != nullptr)
    allreduce_multimem_kernel<<<grid_for(shard_vec, 4), 256, 0, (cudaStream_t)s>>>(table_of(peers), (char*)mc_base, off, shard_vec,
                                                                                   slot, epoch);
  else
    allreduce_shard_kernel<<<grid_for(shard_vec, 8), 256, 0, (cudaStream_t)s>>>(table_of(peers), off, shard_vec, slot, epoch);
  return (int)cudaGetLastError();
}

GV_DEFINE_ERROR_READER(gv_read_error_nvl)
