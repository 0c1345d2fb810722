// Microbenchmark: cycles per tcgen05.mma instruction (bf16, K = 16) issued back to back by one thread, for several
// M / N, in the single-CTA form and in the cta_group::2 pair form. Operands sit in (zeroed) shared memory, the
// accumulator in tensor memory; nothing else runs, so the figure is the tensor pipe's cost of one instruction.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr \
//        -o mma_issue_cost hetu_galvatron_b200/csrc/bench/mma_issue_cost.cu -lcuda && ./mma_issue_cost
//
// Measured on B200: M128 N256 / N128 / N64 / N32 = 128 / 64 / 48 / 44.6 cycles; M64 costs the same as M128;
// pair M256 N256 = 128 cycles. So N = 64 tiles (attention with 64-wide KV blocks) run the pipe at 67 % at best.
#include <cstdio>
#include <cuda_runtime.h>
#include <cuda.h>
#include "../include/gv_ptx.cuh"
using namespace gv;
GV_DEFINE_ERROR_READER(probe_read_error)
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
void run_single(const char* name) {
  long long* d; cudaMalloc(&d, 32);
  auto k = probe_single<N, M>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 70 * 1024);
  const int reps = 2000;
  k<<<1, 128, 70 * 1024>>>(d, 10); cudaDeviceSynchronize();
  k<<<1, 128, 70 * 1024>>>(d, reps); cudaError_t e = cudaDeviceSynchronize();
  long long h[3]; cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost);
  printf("%s: err=%d ok=%lld total=%lld cycles, issue=%lld, per-MMA total=%.1f issue=%.1f\n", name, (int)e, h[2], h[0], h[1],
         (double)h[0] / (reps * 4), (double)h[1] / (reps * 4));
  cudaFree(d);
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
void run_pair(const char* name) {
  long long* d; cudaMalloc(&d, 32);
  auto k = probe_pair<N, M>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 70 * 1024);
  const int reps = 2000;
  k<<<2, 128, 70 * 1024>>>(d, 10); cudaDeviceSynchronize();
  k<<<2, 128, 70 * 1024>>>(d, reps); cudaError_t e = cudaDeviceSynchronize();
  long long h[3]; cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost);
  printf("%s: err=%d ok=%lld total=%lld cycles, per-MMA=%.1f\n", name, (int)e, h[2], h[0], (double)h[0] / (reps * 4));
  cudaFree(d);
}
int main() {
  run_single<256, 128>("M128 N256"); run_single<128, 128>("M128 N128"); run_single<64, 128>("M128 N64");
  run_single<32, 128>("M128 N32"); run_single<256, 64>("M64 N256"); run_single<128, 64>("M64 N128");
  run_pair<256, 256>("pair M256 N256"); run_pair<128, 256>("pair M256 N128"); run_pair<256, 128>("pair M128 N256");
  unsigned int err[4];
  printf("error word: %d\n", probe_read_error(err));
  return 0;
}
