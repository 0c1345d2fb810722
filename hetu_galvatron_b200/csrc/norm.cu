// RMSNorm / LayerNorm forward and backward for sm_100a (HBM-bound: 16-byte vector
// accesses, the row kept in registers between the statistics pass and the output pass).
//
// Replaces flash-attn's dropout_layer_norm extension used by the reference's Llama blocks
// (galvatron/models/llama_hf/LlamaModel_tensor_parallel.py:2,48,90) and torch.nn.LayerNorm in the
// GPT / ViT / BERT blocks (galvatron/models/gpt_hf/GPTModel_tensor_parallel.py:5,30,50).
// The optional residual input fuses the pre-norm residual add (reference: plain adds at
// LlamaModel_tensor_parallel.py:81,96).
#include "include/gv_kernels.h"
#include "include/gv_ptx.cuh"

namespace gv {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;  // 16-byte vectors per thread held in registers -> cols <= 8192

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide sum of up to two values; every thread gets the result.
__device__ __forceinline__ float2 block_sum2(float a, float b, float2* scratch) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = make_float2(a, b);
  __syncthreads();
  float2 t = (lane < (blockDim.x >> 5)) ? scratch[lane] : make_float2(0.f, 0.f);
  t.x = warp_sum(t.x);
  t.y = warp_sum(t.y);
  return t;
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// LAYER = false: RMSNorm; LAYER = true: LayerNorm (mean subtracted, bias added).
template <bool LAYER>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out, float* __restrict__ mean_out,
                float* __restrict__ rstd_out, int rows, int cols, float eps) {
  __shared__ float2 scratch[NORM_THREADS / 32];
  const int nvec = cols >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * cols);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + static_cast<size_t>(row) * cols) : nullptr;
    float v[NORM_MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_MAXV; ++j) {
      const int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        unpack8(xr[i], v[j]);
        if (rr) {
          float t[8];
          unpack8(rr[i], t);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[j][e] += t[e];
          if (h_out) {
            // the residual stream is carried in bf16; normalise what is actually stored
            uint4 hv = pack8(v[j]);
            reinterpret_cast<uint4*>(h_out + static_cast<size_t>(row) * cols)[i] = hv;
            unpack8(hv, v[j]);
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) { s1 += v[j][e]; s2 += v[j][e] * v[j][e]; }
      }
    }
    float2 tot = block_sum2(s1, s2, scratch);
    float mean = 0.f, rstd;
    if (LAYER) {
      mean = tot.x / cols;
      float var = fmaxf(tot.y / cols - mean * mean, 0.f);
      rstd = rsqrtf(var + eps);
    } else {
      rstd = rsqrtf(tot.y / cols + eps);
    }
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (LAYER) mean_out[row] = mean;
    }
#pragma unroll
    for (int j = 0; j < NORM_MAXV; ++j) {
      const int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float wv[8], o[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(w) + i), wv);
        if (LAYER) {
          float bv[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(b) + i), bv);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = (v[j][e] - mean) * rstd * wv[e] + bv[e];
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = v[j][e] * rstd * wv[e];
        }
        reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * cols)[i] = pack8(o);
      }
    }
  }
}

// Backward. Each CTA walks rows with a grid stride and keeps the weight (and bias) gradient of the columns its threads
// own in registers. The loads of the CTA's next row are issued before the block-wide reduction of the current one, so
// the memory latency hides behind the two barriers of that reduction. At the end every CTA stores its partial
// weight / bias gradient to its own row of `partial` ([gridDim.x, cols], then [gridDim.x, cols] for the bias); a
// second, tiny kernel adds the rows up in a fixed order: the weight gradient is bitwise repeatable and no atomic is
// issued. V = 16-byte vectors per thread (cols <= 2048 * V).
template <bool LAYER, int V>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int cols) {
  __shared__ float2 scratch[NORM_THREADS / 32];
  const int nvec = cols >> 3;
  float dw[V][8], db[V][8], wv[V][8];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int i = threadIdx.x + j * NORM_THREADS;
#pragma unroll
    for (int e = 0; e < 8; ++e) { dw[j][e] = 0.f; db[j][e] = 0.f; wv[j][e] = 0.f; }
    if (i < nvec) unpack8(__ldg(reinterpret_cast<const uint4*>(w) + i), wv[j]);
  }
  uint4 nx[V], ndy[V];
  {
    const int row = blockIdx.x;
    if (row < rows) {
      const size_t off = static_cast<size_t>(row) * cols;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const int i = threadIdx.x + j * NORM_THREADS;
        if (i < nvec) {
          nx[j] = reinterpret_cast<const uint4*>(x + off)[i];
          ndy[j] = reinterpret_cast<const uint4*>(dy + off)[i];
        }
      }
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * cols;
    const float rstd = rstd_in[row];
    const float mean = LAYER ? mean_in[row] : 0.f;
    uint4 cx[V], cdy[V];
#pragma unroll
    for (int j = 0; j < V; ++j) { cx[j] = nx[j]; cdy[j] = ndy[j]; }
    const int nrow = row + gridDim.x;
    if (nrow < rows) {
      const size_t noff = static_cast<size_t>(nrow) * cols;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const int i = threadIdx.x + j * NORM_THREADS;
        if (i < nvec) {
          nx[j] = reinterpret_cast<const uint4*>(x + noff)[i];
          ndy[j] = reinterpret_cast<const uint4*>(dy + noff)[i];
        }
      }
    }
    float xh[V][8], g[V][8];
    float s1 = 0.f, s2 = 0.f;  // sum(g), sum(g * xhat) with g = dy * w
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float xv[8], dyv[8];
        unpack8(cx[j], xv);
        unpack8(cdy[j], dyv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[j][e] = (xv[e] - mean) * rstd;
          g[j][e] = dyv[e] * wv[j][e];
          dw[j][e] += dyv[e] * xh[j][e];
          if (LAYER) db[j][e] += dyv[e];
          s1 += g[j][e];
          s2 += g[j][e] * xh[j][e];
        }
      }
    }
    float2 tot = block_sum2(s1, s2, scratch);
    const float m1 = LAYER ? tot.x / cols : 0.f;
    const float m2 = tot.y / cols;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rstd * (g[j][e] - m1 - xh[j][e] * m2);
        if (dres) {
          float t[8];
          unpack8(reinterpret_cast<const uint4*>(dres + off)[i], t);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += t[e];
        }
        reinterpret_cast<uint4*>(dx + off)[i] = pack8(o);
      }
    }
  }
  float* pw = partial + static_cast<size_t>(blockIdx.x) * cols;
  float* pb = partial + (static_cast<size_t>(gridDim.x) + blockIdx.x) * cols;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int i = threadIdx.x + j * NORM_THREADS;
    if (i < nvec) {
      reinterpret_cast<float4*>(pw + i * 8)[0] = make_float4(dw[j][0], dw[j][1], dw[j][2], dw[j][3]);
      reinterpret_cast<float4*>(pw + i * 8)[1] = make_float4(dw[j][4], dw[j][5], dw[j][6], dw[j][7]);
      if (LAYER) {
        reinterpret_cast<float4*>(pb + i * 8)[0] = make_float4(db[j][0], db[j][1], db[j][2], db[j][3]);
        reinterpret_cast<float4*>(pb + i * 8)[1] = make_float4(db[j][4], db[j][5], db[j][6], db[j][7]);
      }
    }
  }
}

// Second stage: out[c] += sum over parts (in order) of partial[part, c]; one thread per column, 4 independent chains.
__global__ void norm_partial_reduce_kernel(const float* __restrict__ partial, int parts, int cols, float* __restrict__ dw_accum,
                                           float* __restrict__ db_accum) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const float* src = blockIdx.y == 0 ? partial : partial + static_cast<size_t>(parts) * cols;
  float* dst = blockIdx.y == 0 ? dw_accum : db_accum;
  if (dst == nullptr) return;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int p = 0;
  for (; p + 4 <= parts; p += 4) {
    a0 += src[static_cast<size_t>(p) * cols + c];
    a1 += src[static_cast<size_t>(p + 1) * cols + c];
    a2 += src[static_cast<size_t>(p + 2) * cols + c];
    a3 += src[static_cast<size_t>(p + 3) * cols + c];
  }
  for (; p < parts; ++p) a0 += src[static_cast<size_t>(p) * cols + c];
  dst[c] += (a0 + a1) + (a2 + a3);
}

int num_sms();

static int check_norm(int rows, int cols) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8 != 0 || cols > 8 * NORM_THREADS * NORM_MAXV) return 2101;
  return -1;
}

}  // namespace gv

using namespace gv;
typedef __nv_bfloat16 bf16;

extern "C" int gv_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                              int rows, int cols, float eps, gv_stream_t s) {
  int c = check_norm(rows, cols);
  if (c >= 0) return c;
  int grid = rows < num_sms() * 8 ? rows : num_sms() * 8;
  norm_fwd_kernel<false><<<grid, NORM_THREADS, 0, (cudaStream_t)s>>>((const bf16*)x, (const bf16*)res, (const bf16*)w,
                                                                    nullptr, (bf16*)y, (bf16*)h_out, nullptr, rstd,
                                                                    rows, cols, eps);
  return (int)cudaGetLastError();
}

static int bwd_grid(int rows, int cols, bool layer) {
  const int v = (cols / 8 + NORM_THREADS - 1) / NORM_THREADS;
  const int per_sm = layer ? (v <= 1 ? 3 : (v == 2 ? 2 : 1)) : (v <= 1 ? 4 : (v == 2 ? 2 : 1));
  return rows < num_sms() * per_sm ? rows : num_sms() * per_sm;
}

// Number of fp32 elements of scratch the backward kernels need for [rows, cols]: one row of partial weight gradients
// (and one of partial bias gradients) per CTA.
extern "C" long long gv_norm_bwd_scratch_elems(int rows, int cols, int layer) {
  if (rows <= 0 || cols <= 0) return 0;
  return 2ll * bwd_grid(rows, cols, layer != 0) * cols;
}

extern "C" int gv_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in,
                              void* dx, float* dw_accum, float* scratch, long long scratch_elems, int rows, int cols,
                              gv_stream_t s) {
  int c = check_norm(rows, cols);
  if (c >= 0) return c;
  if (scratch == nullptr || scratch_elems < gv_norm_bwd_scratch_elems(rows, cols, 0)) return 2102;
  const int v = (cols / 8 + NORM_THREADS - 1) / NORM_THREADS;
  const int grid = bwd_grid(rows, cols, false);
#define GV_LAUNCH_RMS_BWD(VV)                                                                                          \
  norm_bwd_kernel<false, VV><<<grid, NORM_THREADS, 0, (cudaStream_t)s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, \
                                                                        nullptr, rstd, (const bf16*)dres_in, (bf16*)dx,  \
                                                                        scratch, rows, cols)
  if (v <= 1) GV_LAUNCH_RMS_BWD(1);
  else if (v == 2) GV_LAUNCH_RMS_BWD(2);
  else GV_LAUNCH_RMS_BWD(4);
#undef GV_LAUNCH_RMS_BWD
  norm_partial_reduce_kernel<<<dim3((cols + 255) / 256, 1), 256, 0, (cudaStream_t)s>>>(scratch, grid, cols, dw_accum, nullptr);
  return (int)cudaGetLastError();
}

extern "C" int gv_layernorm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* h_out,
                                float* mean, float* rstd, int rows, int cols, float eps, gv_stream_t s) {
  int c = check_norm(rows, cols);
  if (c >= 0) return c;
  int grid = rows < num_sms() * 8 ? rows : num_sms() * 8;
  norm_fwd_kernel<true><<<grid, NORM_THREADS, 0, (cudaStream_t)s>>>((const bf16*)x, (const bf16*)res, (const bf16*)w,
                                                                   (const bf16*)b, (bf16*)y, (bf16*)h_out, mean, rstd,
                                                                   rows, cols, eps);
  return (int)cudaGetLastError();
}

extern "C" int gv_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                const void* dres_in, void* dx, float* dw_accum, float* db_accum, float* scratch,
                                long long scratch_elems, int rows, int cols, gv_stream_t s) {
  int c = check_norm(rows, cols);
  if (c >= 0) return c;
  if (scratch == nullptr || scratch_elems < gv_norm_bwd_scratch_elems(rows, cols, 1)) return 2102;
  const int v = (cols / 8 + NORM_THREADS - 1) / NORM_THREADS;
  const int grid = bwd_grid(rows, cols, true);
#define GV_LAUNCH_LN_BWD(VV)                                                                                          \
  norm_bwd_kernel<true, VV><<<grid, NORM_THREADS, 0, (cudaStream_t)s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, \
                                                                       mean, rstd, (const bf16*)dres_in, (bf16*)dx,    \
                                                                       scratch, rows, cols)
  if (v <= 1) GV_LAUNCH_LN_BWD(1);
  else if (v == 2) GV_LAUNCH_LN_BWD(2);
  else GV_LAUNCH_LN_BWD(4);
#undef GV_LAUNCH_LN_BWD
  norm_partial_reduce_kernel<<<dim3((cols + 255) / 256, db_accum ? 2 : 1), 256, 0, (cudaStream_t)s>>>(scratch, grid, cols, dw_accum,
                                                                                                    db_accum);
  return (int)cudaGetLastError();
}
