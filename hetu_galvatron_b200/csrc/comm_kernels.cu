// Collectives written as kernels over NVSwitch peer memory (plain peer loads / stores + flag signalling):
// barrier, pull all-gather (ZeRO-3 parameter gather), slot reduction (the tail of GEMM -> reduce-scatter),
// gradient reduce-scatter fused with AdamW and the parameter all-gather (ZeRO-1/2/3 step), and the inter-layer
// reshard gather. The reference reaches all of these through NCCL via torch.distributed / FSDP1
// (galvatron/core/runtime/pipeline/sp_grad_reduce.py:93-132; galvatron/core/runtime/redistribute.py:269-350).
// Every wait is bounded (include/gv_comm.cuh).
#include "include/gv_kernels.h"
#include "include/gv_comm.cuh"

namespace gv {
int num_sms();
typedef __nv_bfloat16 bf16;

static PeerTable make_table(const gv_peers* p) {
  PeerTable t;
  for (int i = 0; i < GV_MAX_RANKS; ++i) t.base[i] = i < p->world ? p->bases[i] : nullptr;
  t.world = p->world;
  t.rank = p->rank;
  return t;
}

static uint64_t budget_ns(int timeout_ms) { return timeout_ms > 0 ? static_cast<uint64_t>(timeout_ms) * 1000000ull : GV_WAIT_NS; }

__global__ void barrier_kernel(PeerTable pt, int slot, uint32_t epoch, uint64_t budget) {
  if (threadIdx.x == 0) signal_all(pt, slot, epoch);
  if (threadIdx.x < pt.world) wait_flag(pt, slot, threadIdx.x, epoch, 0x31, budget);
}

__global__ void signal_kernel(PeerTable pt, int slot, uint32_t epoch) {
  if (threadIdx.x == 0) signal_all(pt, slot, epoch);
}

__global__ void wait_kernel(PeerTable pt, int slot, int src, uint32_t epoch, uint64_t budget) {
  if (threadIdx.x == 0) wait_flag(pt, slot, src, epoch, 0x32, budget);
}

// Block-wide wait for one source's flag: thread 0 polls, everybody learns the outcome.
__device__ __forceinline__ bool block_wait(const PeerTable& pt, int slot, int src, uint32_t epoch, unsigned site,
                                           uint64_t budget = GV_WAIT_NS) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = wait_flag(pt, slot, src, epoch, site, budget) ? 1 : 0;
  __syncthreads();
  const bool ok = ok_s != 0;
  __syncthreads();
  return ok;
}

// ---------------------------------------------------------------- pull all-gather
__global__ void allgather_pull_kernel(PeerTable pt, long long src_off, uint4* __restrict__ out, long long nvec, int slot,
                                      uint32_t epoch, uint64_t budget = GV_WAIT_NS) {
  // sources in the order rank, rank+1, ...: the local shard first, every rank starts on a different peer
  for (int k = 0; k < pt.world; ++k) {
    const int src = (pt.rank + k) % pt.world;
    if (!block_wait(pt, slot, src, epoch, 0x33, budget)) return;
    const uint4* in = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(pt.base[src]) + src_off);
    uint4* dst = out + static_cast<long long>(src) * nvec;
    // 8 independent 16-byte loads in flight per thread: the link needs a few MB outstanding to run at full rate
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += stride * 8) {
      uint4 tmp[8];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (i0 + q * stride < nvec) tmp[q] = in[i0 + q * stride];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (i0 + q * stride < nvec) dst[i0 + q * stride] = tmp[q];
    }
  }
}

// ---------------------------------------------------------------- slot reduction
__global__ void reduce_slots_kernel(PeerTable pt, long long slots_off, bf16* __restrict__ out,
                                    const bf16* __restrict__ residual, const bf16* __restrict__ bias, long long rows,
                                    int cols, int slot, uint32_t epoch) {
  for (int p = 0; p < pt.world; ++p)
    if (!block_wait(pt, slot, p, epoch, 0x34)) return;
  const long long nvec = rows * cols / 8;
  const int cvec = cols / 8;
  const uint4* base = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(pt.base[pt.rank]) + slots_off);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < pt.world; ++r) {
      const uint4 u = base[static_cast<long long>(r) * nvec + i];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    if (residual) {
      const uint4 u = reinterpret_cast<const uint4*>(residual)[i];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    if (bias) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(bias) + (i % cvec));
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// ---------------------------------------------------------------- reduce-scatter + AdamW (+ parameter all-gather)
template <bool GRAD_BF16>
__global__ void rs_adamw_kernel(PeerTable pt, long long grad_off, long long lo, long long n, float* __restrict__ master,
                                float* __restrict__ m, float* __restrict__ v, long long param_off, int push_params, float lr,
                                float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
                                const float* __restrict__ clip_coef, float* __restrict__ sumsq_out, int slot,
                                uint32_t epoch) {
  for (int p = 0; p < pt.world; ++p)
    if (!block_wait(pt, slot, p, epoch, 0x35)) return;
  const float gs = grad_scale * (clip_coef ? *clip_coef : 1.f);
  const long long nvec = n >> 2;
  float local_sq = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < pt.world; ++k) {
      const int r = (pt.rank + k) % pt.world;
      const char* gb = reinterpret_cast<const char*>(pt.base[r]) + grad_off;
      if (GRAD_BF16) {
        const uint2 u = reinterpret_cast<const uint2*>(gb)[(lo >> 2) + i];
        float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
        g[0] += a.x; g[1] += a.y; g[2] += b.x; g[3] += b.y;
      } else {
        const float4 a = reinterpret_cast<const float4*>(gb)[(lo >> 2) + i];
        g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
      }
    }
    float4 w4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float w[4] = {w4.x, w4.y, w4.z, w4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float raw = g[e] * grad_scale;
      local_sq += raw * raw;
      const float ge = g[e] * gs;
      mm[e] = b1 * mm[e] + (1.f - b1) * ge;
      vv[e] = b2 * vv[e] + (1.f - b2) * ge * ge;
      w[e] = w[e] - lr * ((mm[e] / bc1) / (sqrtf(vv[e] / bc2) + eps) + wd * w[e]);
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    uint2 o;
    o.x = pack_bf16x2(w[0], w[1]);
    o.y = pack_bf16x2(w[2], w[3]);
    if (push_params) {
      for (int k = 0; k < pt.world; ++k) {
        const int r = (pt.rank + k) % pt.world;
        reinterpret_cast<uint2*>(reinterpret_cast<char*>(pt.base[r]) + param_off)[(lo >> 2) + i] = o;
      }
    } else {
      reinterpret_cast<uint2*>(reinterpret_cast<char*>(pt.base[pt.rank]) + param_off)[(lo >> 2) + i] = o;
    }
  }
  if (sumsq_out) {
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) local_sq += __shfl_xor_sync(0xffffffffu, local_sq, o2);
    if ((threadIdx.x & 31) == 0) atomicAdd(sumsq_out, local_sq);
  }
}

// ---------------------------------------------------------------- ZeRO gradient path, phase A: reduce-scatter
// Grid-wide completion: the last CTA to arrive resets the counter and returns true (its thread 0 only).
__device__ __forceinline__ bool last_block_done(unsigned int* ctr) {
  __shared__ int last_s;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(ctr, 1u);
    last_s = (old == gridDim.x - 1) ? 1 : 0;
    if (last_s) *ctr = 0u;
  }
  __syncthreads();
  return last_s != 0 && threadIdx.x == 0;
}

// Every rank keeps its whole gradient bucket in the symmetric region at `grad_off`. This kernel, launched by every
// rank when the block's backward is complete, (1) announces "my bucket is final" (READY, CTA 0), (2) waits for the
// peers' announcements, (3) sums this rank's slice [lo, lo + n) over all ranks in fp32 into `out` (+= when
// `accumulate`), optionally writing the sum back into every rank's bucket (all-reduce for unsharded optimizers),
// (4) adds the slice's sum of squares into `sumsq_out`, (5) announces DONE once all its peer reads (and writes)
// have completed, which is what a peer waits for before it clears or overwrites its bucket.
template <bool GRAD_BF16, bool WRITE_BACK>
__global__ void grad_reduce_kernel(PeerTable pt, long long grad_off, long long lo, long long n, float* __restrict__ out,
                                   int accumulate, float* __restrict__ sumsq_out, unsigned int* __restrict__ ctr,
                                   int slot_ready, int slot_done, uint32_t epoch, uint64_t budget) {
  if (blockIdx.x == 0 && threadIdx.x == 0) signal_all(pt, slot_ready, epoch);
  {
    __shared__ int ok_s;
    if (threadIdx.x == 0) {
      bool ok = true;
      for (int k = 1; k < pt.world && ok; ++k) ok = wait_flag(pt, slot_ready, (pt.rank + k) % pt.world, epoch, 0x37, budget);
      ok_s = ok ? 1 : 0;
    }
    __syncthreads();
    if (!ok_s) return;
  }
  const long long nvec = n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float local_sq = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
    float g[4] = {0.f, 0.f, 0.f, 0.f};
    if (GRAD_BF16) {
      uint2 u[GV_MAX_RANKS];
#pragma unroll
      for (int k = 0; k < GV_MAX_RANKS; ++k)
        if (k < pt.world) {
          const int r = (pt.rank + k) % pt.world;
          u[k] = reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(pt.base[r]) + grad_off)[(lo >> 2) + i];
        }
#pragma unroll
      for (int k = 0; k < GV_MAX_RANKS; ++k)
        if (k < pt.world) {
          float2 a = unpack_bf16x2(u[k].x), b = unpack_bf16x2(u[k].y);
          g[0] += a.x; g[1] += a.y; g[2] += b.x; g[3] += b.y;
        }
    } else {
      float4 u[GV_MAX_RANKS];
#pragma unroll
      for (int k = 0; k < GV_MAX_RANKS; ++k)
        if (k < pt.world) {
          const int r = (pt.rank + k) % pt.world;
          u[k] = reinterpret_cast<const float4*>(reinterpret_cast<const char*>(pt.base[r]) + grad_off)[(lo >> 2) + i];
        }
#pragma unroll
      for (int k = 0; k < GV_MAX_RANKS; ++k)
        if (k < pt.world) { g[0] += u[k].x; g[1] += u[k].y; g[2] += u[k].z; g[3] += u[k].w; }
    }
    local_sq += g[0] * g[0] + g[1] * g[1] + g[2] * g[2] + g[3] * g[3];
    if (out) {
      float4 o = make_float4(g[0], g[1], g[2], g[3]);
      if (accumulate) {
        const float4 p = reinterpret_cast<const float4*>(out)[i];
        o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
      }
      reinterpret_cast<float4*>(out)[i] = o;
    }
    if (WRITE_BACK) {
      for (int k = 0; k < pt.world; ++k) {
        const int r = (pt.rank + k) % pt.world;
        char* gb = reinterpret_cast<char*>(pt.base[r]) + grad_off;
        if (GRAD_BF16) {
          uint2 o2;
          o2.x = pack_bf16x2(g[0], g[1]);
          o2.y = pack_bf16x2(g[2], g[3]);
          reinterpret_cast<uint2*>(gb)[(lo >> 2) + i] = o2;
        } else {
          reinterpret_cast<float4*>(gb)[(lo >> 2) + i] = make_float4(g[0], g[1], g[2], g[3]);
        }
      }
    }
  }
  if (sumsq_out) {
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) local_sq += __shfl_xor_sync(0xffffffffu, local_sq, o2);
    if ((threadIdx.x & 31) == 0) atomicAdd(sumsq_out, local_sq);
  }
  if (last_block_done(ctr)) signal_all(pt, slot_done, epoch);
}

// ---------------------------------------------------------------- ZeRO gradient path, phase B: AdamW + parameter push
// AdamW on this rank's fp32 shard; the new bf16 values go straight into the parameter buffer of every rank
// (push_all) or of this rank only (a ZeRO-3 shard that peers pull later). The last CTA announces PARAM = epoch,
// which the next reader of these parameters (a forward pass, a pull all-gather) waits for.
__global__ void adamw_push_kernel(PeerTable pt, long long param_off, long long lo, long long n, float* __restrict__ master,
                                  float* __restrict__ m, float* __restrict__ v, const float* __restrict__ grad,
                                  int push_all, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                                  float grad_scale, const float* __restrict__ clip_coef, unsigned int* __restrict__ ctr,
                                  int slot_param, uint32_t epoch) {
  const float gs = grad_scale * (clip_coef ? *clip_coef : 1.f);
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float4 w4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float g[4] = {g4.x, g4.y, g4.z, g4.w};
    float w[4] = {w4.x, w4.y, w4.z, w4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float ge = g[e] * gs;
      mm[e] = b1 * mm[e] + (1.f - b1) * ge;
      vv[e] = b2 * vv[e] + (1.f - b2) * ge * ge;
      w[e] = w[e] - lr * ((mm[e] / bc1) / (sqrtf(vv[e] / bc2) + eps) + wd * w[e]);
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    uint2 o;
    o.x = pack_bf16x2(w[0], w[1]);
    o.y = pack_bf16x2(w[2], w[3]);
    if (push_all) {
      for (int k = 0; k < pt.world; ++k) {
        const int r = (pt.rank + k) % pt.world;
        reinterpret_cast<uint2*>(reinterpret_cast<char*>(pt.base[r]) + param_off)[(lo >> 2) + i] = o;
      }
    } else {
      reinterpret_cast<uint2*>(reinterpret_cast<char*>(pt.base[pt.rank]) + param_off)[(lo >> 2) + i] = o;
    }
  }
  if (last_block_done(ctr)) signal_all(pt, slot_param, epoch);
}

// Wait until every peer (not this rank: its own work is ordered by the stream) announced `epoch` on `slot`.
__global__ void wait_peers_kernel(PeerTable pt, int slot, uint32_t epoch, uint64_t budget) {
  if (threadIdx.x < pt.world && static_cast<int>(threadIdx.x) != pt.rank) wait_flag(pt, slot, threadIdx.x, epoch, 0x38, budget);
}

// Clear a buffer once every peer announced `epoch` on `slot` (they are done reading it).
__global__ void wait_zero_kernel(PeerTable pt, int slot, uint32_t epoch, uint4* __restrict__ ptr, long long nvec, uint64_t budget) {
  {
    __shared__ int ok_s;
    if (threadIdx.x == 0) {
      bool ok = true;
      for (int k = 1; k < pt.world && ok; ++k) ok = wait_flag(pt, slot, (pt.rank + k) % pt.world, epoch, 0x39, budget);
      ok_s = ok ? 1 : 0;
    }
    __syncthreads();
    if (!ok_s) return;
  }
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    ptr[i] = z;
}

// ---------------------------------------------------------------- reshard gather
__global__ void reshard_gather_kernel(PeerTable pt, long long src_off, uint4* __restrict__ out,
                                      const int* __restrict__ src_rank, const int* __restrict__ src_row,
                                      const int* __restrict__ src_col, int s_new, int b_new, int b_old, int hvec, int slot,
                                      uint32_t epoch) {
  for (int p = 0; p < pt.world; ++p)
    if (!block_wait(pt, slot, p, epoch, 0x36)) return;
  const long long rows = static_cast<long long>(s_new) * b_new;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const int s = static_cast<int>(row / b_new), b = static_cast<int>(row % b_new);
    const int r = src_rank[row];
    const long long srow = static_cast<long long>(src_row[s]) * b_old + src_col[b];
    const uint4* in = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(pt.base[r]) + src_off) + srow * hvec;
    uint4* dst = out + row * hvec;
    for (int i = threadIdx.x; i < hvec; i += blockDim.x) dst[i] = in[i];
  }
}

}  // namespace gv

using namespace gv;

extern "C" int gv_comm_barrier(const gv_peers* peers, int slot, unsigned int epoch, int timeout_ms, gv_stream_t s) {
  if (peers->world > GV_MAX_RANKS || slot < 0 || slot >= GV_FLAG_SLOTS) return 2501;
  barrier_kernel<<<1, 32, 0, (cudaStream_t)s>>>(make_table(peers), slot, epoch, budget_ns(timeout_ms));
  return (int)cudaGetLastError();
}
extern "C" int gv_comm_signal(const gv_peers* peers, int slot, unsigned int epoch, gv_stream_t s) {
  if (peers->world > GV_MAX_RANKS || slot < 0 || slot >= GV_FLAG_SLOTS) return 2501;
  signal_kernel<<<1, 32, 0, (cudaStream_t)s>>>(make_table(peers), slot, epoch);
  return (int)cudaGetLastError();
}
extern "C" int gv_comm_wait(const gv_peers* peers, int slot, int src, unsigned int epoch, int timeout_ms, gv_stream_t s) {
  if (peers->world > GV_MAX_RANKS || slot < 0 || slot >= GV_FLAG_SLOTS || src < 0 || src >= peers->world) return 2501;
  wait_kernel<<<1, 32, 0, (cudaStream_t)s>>>(make_table(peers), slot, src, epoch, budget_ns(timeout_ms));
  return (int)cudaGetLastError();
}

extern "C" int gv_allgather_pull(const gv_peers* peers, long long src_off, void* out, long long n_elems, int slot,
                                 unsigned int epoch, gv_stream_t s) {
  if (n_elems <= 0) return 0;
  if (n_elems % 8 || src_off % 16 || (reinterpret_cast<uintptr_t>(out) & 15)) return 2502;
  const long long nvec = n_elems / 8;
  long long grid = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 4;
  if (grid > cap) grid = cap;
  allgather_pull_kernel<<<(int)grid, 256, 0, (cudaStream_t)s>>>(make_table(peers), src_off, (uint4*)out, nvec, slot, epoch,
                                                               GV_WAIT_NS);
  return (int)cudaGetLastError();
}

extern "C" int gv_reduce_slots(const gv_peers* peers, long long slots_off, void* out, const void* residual, const void* bias,
                               long long rows, int cols, int slot, unsigned int epoch, gv_stream_t s) {
  if (rows <= 0) return 0;
  if (cols % 8 || slots_off % 16) return 2503;
  long long grid = (rows * cols / 8 + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (grid > cap) grid = cap;
  reduce_slots_kernel<<<(int)grid, 256, 0, (cudaStream_t)s>>>(make_table(peers), slots_off, (bf16*)out, (const bf16*)residual,
                                                             (const bf16*)bias, rows, cols, slot, epoch);
  return (int)cudaGetLastError();
}

extern "C" int gv_rs_adamw(const gv_peers* peers, long long grad_off, int grad_is_bf16, long long lo, long long n,
                           float* master, float* m, float* v, long long param_off, int push_params, float lr, float beta1,
                           float beta2, float eps, float weight_decay, float bias_corr1, float bias_corr2, float grad_scale,
                           const float* clip_coef, float* sumsq_out, int slot, unsigned int epoch, gv_stream_t s) {
  if (n <= 0) return 0;
  if (n % 4 || lo % 4 || grad_off % 16 || param_off % 16) return 2504;
  long long grid = (n / 4 + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (grid > cap) grid = cap;
  PeerTable pt = make_table(peers);
  if (grad_is_bf16)
    rs_adamw_kernel<true><<<(int)grid, 256, 0, (cudaStream_t)s>>>(pt, grad_off, lo, n, master, m, v, param_off, push_params, lr,
                                                                 beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2,
                                                                 grad_scale, clip_coef, sumsq_out, slot, epoch);
  else
    rs_adamw_kernel<false><<<(int)grid, 256, 0, (cudaStream_t)s>>>(pt, grad_off, lo, n, master, m, v, param_off, push_params, lr,
                                                                  beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2,
                                                                  grad_scale, clip_coef, sumsq_out, slot, epoch);
  return (int)cudaGetLastError();
}

extern "C" int gv_reshard_gather(const gv_peers* peers, long long src_off, void* out, const int* src_rank, const int* src_row,
                                 const int* src_col, int s_new, int b_new, int b_old, int hidden, int slot,
                                 unsigned int epoch, gv_stream_t s) {
  if (s_new <= 0 || b_new <= 0) return 0;
  if (hidden % 8 || src_off % 16) return 2505;
  long long rows = static_cast<long long>(s_new) * b_new;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (rows > cap) rows = cap;
  reshard_gather_kernel<<<(int)rows, 128, 0, (cudaStream_t)s>>>(make_table(peers), src_off, (uint4*)out, src_rank, src_row,
                                                               src_col, s_new, b_new, b_old, hidden / 8, slot, epoch);
  return (int)cudaGetLastError();
}

extern "C" int gv_grad_reduce(const gv_peers* peers, long long grad_off, int grad_is_bf16, long long lo, long long n,
                              float* out, int accumulate, int write_back, float* sumsq_out, long long ctr_off,
                              int slot_ready, int slot_done, unsigned int epoch, int timeout_ms, int max_blocks,
                              gv_stream_t s) {
  if (n <= 0) return 0;
  if (peers->world > GV_MAX_RANKS || n % 4 || lo % 4 || grad_off % 16 || ctr_off % 4 || (reinterpret_cast<uintptr_t>(out) & 15))
    return 2506;
  long long grid = (n / 4 + 255) / 256;
  long long cap = max_blocks > 0 ? max_blocks : 64;
  if (grid > cap) grid = cap;
  PeerTable pt = make_table(peers);
  unsigned int* ctr = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(peers->bases[peers->rank]) + ctr_off);
  const uint64_t b = budget_ns(timeout_ms);
#define GV_LAUNCH_GR(BF, WB)                                                                                          \
  grad_reduce_kernel<BF, WB><<<(int)grid, 256, 0, (cudaStream_t)s>>>(pt, grad_off, lo, n, out, accumulate, sumsq_out, \
                                                                    ctr, slot_ready, slot_done, epoch, b)
  if (grad_is_bf16) {
    if (write_back) GV_LAUNCH_GR(true, true); else GV_LAUNCH_GR(true, false);
  } else {
    if (write_back) GV_LAUNCH_GR(false, true); else GV_LAUNCH_GR(false, false);
  }
#undef GV_LAUNCH_GR
  return (int)cudaGetLastError();
}

extern "C" int gv_adamw_push(const gv_peers* peers, long long param_off, long long lo, long long n, float* master, float* m,
                             float* v, const float* grad, int push_all, float lr, float beta1, float beta2, float eps,
                             float weight_decay, float bias_corr1, float bias_corr2, float grad_scale,
                             const float* clip_coef, long long ctr_off, int slot_param, unsigned int epoch, gv_stream_t s) {
  if (n <= 0) return 0;
  if (peers->world > GV_MAX_RANKS || n % 4 || lo % 4 || param_off % 16 || ctr_off % 4) return 2507;
  long long grid = (n / 4 + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 4;
  if (grid > cap) grid = cap;
  unsigned int* ctr = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(peers->bases[peers->rank]) + ctr_off);
  adamw_push_kernel<<<(int)grid, 256, 0, (cudaStream_t)s>>>(make_table(peers), param_off, lo, n, master, m, v, grad, push_all,
                                                           lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2,
                                                           grad_scale, clip_coef, ctr, slot_param, epoch);
  return (int)cudaGetLastError();
}

extern "C" int gv_comm_wait_peers(const gv_peers* peers, int slot, unsigned int epoch, int timeout_ms, gv_stream_t s) {
  if (peers->world > GV_MAX_RANKS || slot < 0 || slot >= GV_FLAG_SLOTS) return 2501;
  wait_peers_kernel<<<1, 32, 0, (cudaStream_t)s>>>(make_table(peers), slot, epoch, budget_ns(timeout_ms));
  return (int)cudaGetLastError();
}

extern "C" int gv_wait_zero(const gv_peers* peers, int slot, unsigned int epoch, void* ptr, long long nbytes, int timeout_ms,
                            gv_stream_t s) {
  if (nbytes <= 0) return 0;
  if (peers->world > GV_MAX_RANKS || slot < 0 || slot >= GV_FLAG_SLOTS || nbytes % 16 || (reinterpret_cast<uintptr_t>(ptr) & 15))
    return 2508;
  const long long nvec = nbytes / 16;
  long long grid = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (grid > cap) grid = cap;
  wait_zero_kernel<<<(int)grid, 256, 0, (cudaStream_t)s>>>(make_table(peers), slot, epoch, (uint4*)ptr, nvec, budget_ns(timeout_ms));
  return (int)cudaGetLastError();
}

// Pull all-gather with a caller-chosen wait budget (parameter gathers may wait for a peer that is a step behind).
extern "C" int gv_allgather_pull_ex(const gv_peers* peers, long long src_off, void* out, long long n_elems, int slot,
                                    unsigned int epoch, int timeout_ms, gv_stream_t s) {
  if (n_elems <= 0) return 0;
  if (n_elems % 8 || src_off % 16 || (reinterpret_cast<uintptr_t>(out) & 15)) return 2502;
  const long long nvec = n_elems / 8;
  long long grid = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 2;
  if (grid > cap) grid = cap;
  allgather_pull_kernel<<<(int)grid, 256, 0, (cudaStream_t)s>>>(make_table(peers), src_off, (uint4*)out, nvec, slot, epoch,
                                                               budget_ns(timeout_ms));
  return (int)cudaGetLastError();
}

GV_DEFINE_ERROR_READER(gv_read_error_comm)
