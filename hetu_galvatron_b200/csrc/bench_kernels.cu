// Tensor-pipe characterisation kernel used by `python -m hetu_galvatron_b200.ops.kernel_bench --op mma_issue`:
// cycles per tcgen05.mma instruction (bf16, K = 16) issued back to back by one thread, for several M / N, in the
// single-CTA form and in the cta_group::2 pair form. Operands sit in (zeroed) shared memory, the accumulator in
// tensor memory; nothing else runs, so the figure is the tensor pipe's cost of one instruction. The attention and
// GEMM tile shapes were chosen from this table (an N = 64 instruction costs 48 cycles, not 32).
// The reference has no GPU code of its own and therefore no counterpart of this file.
#include "include/gv_kernels.h"
#include "include/gv_host.h"
#include "include/gv_ptx.cuh"
#include <cuda_runtime.h>

namespace gv {
template <int N, int M>
__global__ void __launch_bounds__(128, 1) probe_single(long long* out, int reps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag_s;
  volatile uint32_t* abort_flag = &abort_flag_s;
  for (int i = threadIdx.x; i < 64 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag_s = 0; mbar_fence_init(); }
  fence_async_smem();
  if (threadIdx.x < 32) { tmem_alloc<1>(&tmem_slot, 512); tmem_relinquish<1>(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = make_idesc_bf16(M, N, 0, 0);
    const uint64_t da0 = make_smem_desc_sw128(smem_u32(smem), 0, 1024);
    const uint64_t db0 = make_smem_desc_sw128(smem_u32(smem) + 16384, 0, 1024);
    long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) umma_f16_ss<1>(tmem_base, da0 + kk * 2, db0 + kk * 2, idesc, 1u);
    }
    umma_commit<1>(&bar);
    long long t_issue = clock64();
    bool ok = mbar_wait(&bar, 0, abort_flag, 0x99);
    long long t1 = clock64();
    out[0] = t1 - t0; out[1] = t_issue - t0; out[2] = ok;
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc<1>(tmem_base, 512); }
}

template <int N, int M>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) probe_pair(long long* out, int reps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag_s;
  volatile uint32_t* abort_flag = &abort_flag_s;
  const uint32_t cta = cluster_ctarank();
  for (int i = threadIdx.x; i < 64 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag_s = 0; mbar_fence_init(); }
  fence_async_smem();
  if (threadIdx.x < 32) { tmem_alloc<2>(&tmem_slot, 512); tmem_relinquish<2>(); }
  tc_fence_before(); __syncthreads(); cluster_sync_all(); tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (threadIdx.x == 0 && cta == 0) {
    constexpr uint32_t idesc = make_idesc_bf16(M, N, 0, 0);
    const uint64_t da0 = make_smem_desc_sw128(smem_u32(smem), 0, 1024);
    const uint64_t db0 = make_smem_desc_sw128(smem_u32(smem) + 16384, 0, 1024);
    long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) umma_f16_ss<2>(tmem_base, da0 + kk * 2, db0 + kk * 2, idesc, 1u);
    }
    umma_commit<2>(&bar);
    bool ok = mbar_wait(&bar, 0, abort_flag, 0x99);
    long long t1 = clock64();
    out[0] = t1 - t0; out[2] = ok;
  }
  tc_fence_before(); __syncthreads(); cluster_sync_all();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc<2>(tmem_base, 512); }
}


template <int N, int M>
static int launch_single(long long* out, int reps, cudaStream_t s) {
  auto k = probe_single<N, M>;
  static PerDeviceOnce once;
  cudaError_t e = ensure_max_dynamic_smem(once, k, 70 * 1024);
  if (e != cudaSuccess) return static_cast<int>(e);
  k<<<1, 128, 70 * 1024, s>>>(out, reps);
  return static_cast<int>(cudaGetLastError());
}
template <int N, int M>
static int launch_pair(long long* out, int reps, cudaStream_t s) {
  auto k = probe_pair<N, M>;
  static PerDeviceOnce once;
  cudaError_t e = ensure_max_dynamic_smem(once, k, 70 * 1024);
  if (e != cudaSuccess) return static_cast<int>(e);
  k<<<2, 128, 70 * 1024, s>>>(out, reps);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gv

using namespace gv;

// out_dev[0] = cycles from the first issue to the completion of the last instruction, out_dev[1] = cycles spent
// issuing (single form only), out_dev[2] = 1 when the completion wait did not expire. 4 * reps instructions run.
extern "C" int gv_bench_mma_issue(int pair, int m, int n, int reps, long long* out_dev, gv_stream_t stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (reps <= 0 || out_dev == nullptr) return 2601;
  if (!pair) {
    if (m == 128 && n == 256) return launch_single<256, 128>(out_dev, reps, s);
    if (m == 128 && n == 128) return launch_single<128, 128>(out_dev, reps, s);
    if (m == 128 && n == 64) return launch_single<64, 128>(out_dev, reps, s);
    if (m == 128 && n == 32) return launch_single<32, 128>(out_dev, reps, s);
    if (m == 64 && n == 256) return launch_single<256, 64>(out_dev, reps, s);
    if (m == 64 && n == 128) return launch_single<128, 64>(out_dev, reps, s);
  } else {
    if (m == 256 && n == 256) return launch_pair<256, 256>(out_dev, reps, s);
    if (m == 256 && n == 128) return launch_pair<128, 256>(out_dev, reps, s);
    if (m == 128 && n == 256) return launch_pair<256, 128>(out_dev, reps, s);
  }
  return 2602;
}

GV_DEFINE_ERROR_READER(gv_read_error_bench)
