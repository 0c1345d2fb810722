// Host-side glue of the kernel library: aggregated error read-back and device queries.
#include "include/gv_kernels.h"
#include <cuda_runtime.h>

extern "C" int gv_read_error_gemm(unsigned int out[4]);
extern "C" int gv_read_error_attn(unsigned int out[4]);
extern "C" int gv_read_error_comm(unsigned int out[4]);
extern "C" int gv_read_error_fgemm(unsigned int out[4]);
extern "C" int gv_read_error_nvl(unsigned int out[4]);
extern "C" int gv_read_error_bench(unsigned int out[4]);

// Polls every translation unit that contains bounded waits. Returns 1 and fills `out`
// with the first record found (and clears it), 0 if no kernel reported an error.
extern "C" int gv_read_error(unsigned int out[4]) {
  int r = gv_read_error_gemm(out);
  if (r != 0) return r;
  r = gv_read_error_attn(out);
  if (r != 0) return r;
  r = gv_read_error_comm(out);
  if (r != 0) return r;
  r = gv_read_error_fgemm(out);
  if (r != 0) return r;
  r = gv_read_error_nvl(out);
  if (r != 0) return r;
  return gv_read_error_bench(out);
}

extern "C" int gv_device_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}
