// HBM-bound sm_100a kernels: RoPE, SwiGLU / GELU, bias-gradient column sums, embedding
// gather / scatter-add, vocab-shard cross-entropy, fused AdamW, gradient sum of squares, casts.
// All use 16-byte vector accesses and grid-stride loops sized from the SM count.
//
// Reference call sites these replace:
//   RoPE          megatron/core/models/common/embeddings/rotary_pos_embedding.py:185-227
//   SwiGLU/GELU   galvatron/core/runtime/tensor_parallel/transformer.py:122-135
//   embedding     megatron/core/tensor_parallel/layers.py:243-256
//   cross entropy megatron/core/tensor_parallel/cross_entropy.py:16-152
//   Adam          galvatron/core/runtime/utils.py:137-149 (apex FusedAdam)
//   grad norm     megatron/core/optimizer/clip_grads.py:80-107 (amp_C multi_tensor_l2norm / scale)
#include "include/gv_kernels.h"
#include "include/gv_ptx.cuh"

namespace gv {
int num_sms();
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void unpack8e(const uint4& u, float* f) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8e(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}
__device__ __forceinline__ float warp_sum_e(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_e(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

static inline int grid_for(long long work_items, int threads, int ctas_per_sm = 8) {
  long long g = (work_items + threads - 1) / threads;
  long long cap = static_cast<long long>(num_sms()) * ctas_per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

// ------------------------------------------------------------------ RoPE
// One thread rotates 8 consecutive pairs (i, i + dh/2) of one (token, head).
__global__ void rope_kernel(bf16* __restrict__ x, const int* __restrict__ pos, const float* __restrict__ inv_freq,
                            long long tokens, int heads, int dh, long long ld, int pos_div, int pos_mod,
                            int pos_offset, int inverse) {
  const int half = dh >> 1;
  const int vec_per_head = half >> 3;
  const long long total = tokens * heads * vec_per_head;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int vi = static_cast<int>(idx % vec_per_head);
    const long long th = idx / vec_per_head;
    const int h = static_cast<int>(th % heads);
    const long long t = th / heads;
    const float p = pos ? static_cast<float>(pos[t])
                        : static_cast<float>(static_cast<int>((t / pos_div) % pos_mod) + pos_offset);
    bf16* base = x + t * ld + static_cast<long long>(h) * dh + vi * 8;
    uint4 u1 = *reinterpret_cast<uint4*>(base);
    uint4 u2 = *reinterpret_cast<uint4*>(base + half);
    float a[8], b[8], oa[8], ob[8];
    unpack8e(u1, a);
    unpack8e(u2, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float s, c;
      sincosf(p * __ldg(inv_freq + vi * 8 + e), &s, &c);
      if (inverse) s = -s;
      oa[e] = a[e] * c - b[e] * s;
      ob[e] = b[e] * c + a[e] * s;
    }
    *reinterpret_cast<uint4*>(base) = pack8e(oa);
    *reinterpret_cast<uint4*>(base + half) = pack8e(ob);
  }
}

// ------------------------------------------------------------------ SwiGLU / GELU
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long long rows, int f) {
  const int vec = f >> 3;
  const long long total = rows * vec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / vec;
    const int c = static_cast<int>(idx % vec) * 8;
    const bf16* g = gu + r * 2 * f + c;
    float a[8], b[8], o[8];
    unpack8e(*reinterpret_cast<const uint4*>(g), a);
    unpack8e(*reinterpret_cast<const uint4*>(g + f), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = a[e] / (1.f + __expf(-a[e])) * b[e];
    *reinterpret_cast<uint4*>(out + r * f + c) = pack8e(o);
  }
}

__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ gu, bf16* __restrict__ dgu,
                                  long long rows, int f) {
  const int vec = f >> 3;
  const long long total = rows * vec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / vec;
    const int c = static_cast<int>(idx % vec) * 8;
    const bf16* g = gu + r * 2 * f + c;
    float a[8], b[8], d[8], da[8], db[8];
    unpack8e(*reinterpret_cast<const uint4*>(g), a);
    unpack8e(*reinterpret_cast<const uint4*>(g + f), b);
    unpack8e(*reinterpret_cast<const uint4*>(dout + r * f + c), d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.f / (1.f + __expf(-a[e]));
      const float silu = a[e] * sg;
      da[e] = d[e] * b[e] * (sg + silu * (1.f - sg));
      db[e] = d[e] * silu;
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * f + c) = pack8e(da);
    *reinterpret_cast<uint4*>(dgu + r * 2 * f + f + c) = pack8e(db);
  }
}

__device__ __forceinline__ float gelu_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (x + k1 * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
}

__global__ void gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long nvec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a[8], o[8];
    unpack8e(reinterpret_cast<const uint4*>(x)[i], a);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = gelu_f(a[e]);
    reinterpret_cast<uint4*>(y)[i] = pack8e(o);
  }
}
__global__ void gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, bf16* __restrict__ dx,
                                long long nvec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a[8], d[8], o[8];
    unpack8e(reinterpret_cast<const uint4*>(x)[i], a);
    unpack8e(reinterpret_cast<const uint4*>(dy)[i], d);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = d[e] * gelu_grad_f(a[e]);
    reinterpret_cast<uint4*>(dx)[i] = pack8e(o);
  }
}

// db[c] += sum_r dy[r, c]. CTA = 32 x 8 threads; each thread owns 8 columns of a 256-column
// strip and walks rows with stride 8 * gridDim.y; partial sums meet in shared memory.
__global__ void colsum_kernel(const bf16* __restrict__ dy, float* __restrict__ out, long long rows, int cols) {
  __shared__ float sm[8][256];
  const int c0 = blockIdx.x * 256 + threadIdx.x * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < cols) {
    for (long long r = blockIdx.y * 8 + threadIdx.y; r < rows; r += static_cast<long long>(gridDim.y) * 8) {
      float v[8];
      unpack8e(*reinterpret_cast<const uint4*>(dy + r * cols + c0), v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) sm[threadIdx.y][threadIdx.x * 8 + e] = acc[e];
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) s += sm[j][t];
  const int c = blockIdx.x * 256 + t;
  if (c < cols) atomicAdd(out + c, s);
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ table,
                                     const int* __restrict__ pos_ids, const bf16* __restrict__ pos_table,
                                     bf16* __restrict__ out, long long tokens, int hidden, long long vocab_start,
                                     long long vocab_rows) {
  const int vec = hidden >> 3;
  for (long long t = blockIdx.x; t < tokens; t += gridDim.x) {
    const long long id = ids[t] - vocab_start;
    const bool in = id >= 0 && id < vocab_rows;
    const uint4* src = in ? reinterpret_cast<const uint4*>(table + id * hidden) : nullptr;
    const uint4* psrc = pos_table ? reinterpret_cast<const uint4*>(pos_table + static_cast<long long>(pos_ids[t]) * hidden) : nullptr;
    uint4* dst = reinterpret_cast<uint4*>(out + t * hidden);
    for (int i = threadIdx.x; i < vec; i += blockDim.x) {
      uint4 v = in ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
      if (psrc) {
        float a[8], b[8];
        unpack8e(v, a);
        unpack8e(__ldg(psrc + i), b);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] += b[e];
        v = pack8e(a);
      }
      dst[i] = v;
    }
  }
}

__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ dout,
                                     float* __restrict__ dtable, long long tokens, int hidden, long long vocab_start,
                                     long long vocab_rows) {
  const int vec = hidden >> 3;
  for (long long t = blockIdx.x; t < tokens; t += gridDim.x) {
    const long long id = ids[t] - vocab_start;
    if (id < 0 || id >= vocab_rows) continue;
    float* dst = dtable + id * hidden;
    for (int i = threadIdx.x; i < vec; i += blockDim.x) {
      float a[8];
      unpack8e(reinterpret_cast<const uint4*>(dout + t * hidden)[i], a);
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(dst + i * 8 + e, a[e]);
    }
  }
}

// ------------------------------------------------------------------ cross entropy
constexpr int XENT_THREADS = 512;

__global__ void __launch_bounds__(XENT_THREADS)
xent_stats_kernel(const bf16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ row_max,
                  float* __restrict__ row_sum, float* __restrict__ tgt, long long rows, int vocab, long long ld,
                  long long vocab_start) {
  __shared__ float sm_a[XENT_THREADS / 32], sm_b[XENT_THREADS / 32];
  const int vec = vocab >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const bf16* lp = logits + r * ld;
    // online (max, sumexp) per thread, merged across the block afterwards
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < vec; i += XENT_THREADS) {
      float a[8];
      unpack8e(reinterpret_cast<const uint4*>(lp)[i], a);
      float lm = a[0];
#pragma unroll
      for (int e = 1; e < 8; ++e) lm = fmaxf(lm, a[e]);
      const float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += __expf(a[e] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    for (int i = vec * 8 + threadIdx.x; i < vocab; i += XENT_THREADS) {
      const float a = __bfloat162float(lp[i]);
      const float nm = fmaxf(m, a);
      s = s * __expf(m - nm) + __expf(a - nm);
      m = nm;
    }
    const float wm = warp_max_e(m);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - wm);
    s = warp_sum_e(s);
    __syncthreads();
    if (lane == 0) { sm_a[warp] = wm; sm_b[warp] = s; }
    __syncthreads();
    if (warp == 0) {
      float m2 = lane < XENT_THREADS / 32 ? sm_a[lane] : -INFINITY;
      float s2 = lane < XENT_THREADS / 32 ? sm_b[lane] : 0.f;
      const float bm = warp_max_e(m2);
      s2 = (m2 == -INFINITY) ? 0.f : s2 * __expf(m2 - bm);
      s2 = warp_sum_e(s2);
      if (lane == 0) {
        row_max[r] = bm;
        row_sum[r] = s2;
        const long long lab = labels[r] - vocab_start;
        tgt[r] = (lab >= 0 && lab < vocab) ? __bfloat162float(lp[lab]) : 0.f;
      }
    }
  }
}

__global__ void __launch_bounds__(XENT_THREADS)
xent_loss_grad_kernel(bf16* __restrict__ logits, const long long* __restrict__ labels,
                      const float* __restrict__ row_max, const float* __restrict__ row_sum,
                      const float* __restrict__ tgt, float* __restrict__ loss, float grad_scale,
                      const float* __restrict__ grad_scale_ptr, long long rows, int vocab, long long ld,
                      long long vocab_start, long long ignore_index) {
  const int vec = vocab >> 3;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    bf16* lp = logits + r * ld;
    const long long label = labels[r];
    const bool ignored = label == ignore_index;
    const float m = row_max[r];
    const float inv = 1.f / row_sum[r];
    const float gs = ignored ? 0.f : grad_scale * (grad_scale_ptr ? grad_scale_ptr[r] : 1.f);
    const long long lab = label - vocab_start;
    if (threadIdx.x == 0 && loss) loss[r] = ignored ? 0.f : (__logf(row_sum[r]) + m - tgt[r]);
    for (int i = threadIdx.x; i < vec; i += XENT_THREADS) {
      float a[8];
      unpack8e(reinterpret_cast<const uint4*>(lp)[i], a);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float pr = __expf(a[e] - m) * inv;
        if (static_cast<long long>(i) * 8 + e == lab) pr -= 1.f;
        a[e] = pr * gs;
      }
      reinterpret_cast<uint4*>(lp)[i] = pack8e(a);
    }
    for (int i = vec * 8 + threadIdx.x; i < vocab; i += XENT_THREADS) {
      float pr = __expf(__bfloat162float(lp[i]) - m) * inv;
      if (i == lab) pr -= 1.f;
      lp[i] = __float2bfloat16(pr * gs);
    }
  }
}

// ------------------------------------------------------------------ log-sum-exp merge of attention partials
// Ring / blockwise attention: `acc` (fp32 [b, s, h, dh], contiguous) and `lse_acc` (fp32 [b, h, s]) hold the
// attention of the key blocks seen so far; a new partial (o_blk bf16 [b, sb, h, dh] with strides, lse_blk fp32
// [b, h, sb] contiguous) over rows [s_off, s_off + sb) is folded in:
//   lse' = log(exp(lse) + exp(lse_blk));  acc' = acc * exp(lse - lse') + o_blk * exp(lse_blk - lse')
// One warp per (b, row, head); lse_acc rows that are still -inf take the partial as is.
__global__ void lse_merge_kernel(float* __restrict__ acc, float* __restrict__ lse_acc, const bf16* __restrict__ o_blk,
                                 const float* __restrict__ lse_blk, int b, int s, int sb, int s_off, int h, int dh,
                                 long long o_sb, long long o_ss, long long o_sh, int update_lse) {
  const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(b) * sb * h;
  if (warp >= total) return;
  const int hd = static_cast<int>(warp % h);
  const int r = static_cast<int>((warp / h) % sb);
  const int bi = static_cast<int>(warp / (static_cast<long long>(h) * sb));
  const long long li = (static_cast<long long>(bi) * h + hd) * s + s_off + r;
  const float la = lse_acc[li];
  const float lb = lse_blk[(static_cast<long long>(bi) * h + hd) * sb + r];
  const float m = fmaxf(la, lb);
  float wa, wb, ln;
  if (m == -INFINITY) {
    wa = 0.f; wb = 0.f; ln = -INFINITY;
  } else {
    const float ea = __expf(la - m), eb = __expf(lb - m);
    const float sum = ea + eb;
    wa = ea / sum; wb = eb / sum;
    ln = m + __logf(sum);
  }
  float* a = acc + ((static_cast<long long>(bi) * s + s_off + r) * h + hd) * dh;
  const bf16* o = o_blk + bi * o_sb + r * o_ss + hd * o_sh;
  for (int c = lane; c < dh; c += 32) a[c] = a[c] * wa + __bfloat162float(o[c]) * wb;
  __syncwarp();
  if (update_lse && lane == 0) lse_acc[li] = ln;
}

// ------------------------------------------------------------------ optimizer
template <bool GRAD_BF16>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const void* __restrict__ grad, bf16* __restrict__ param, long long n, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
                             const float* __restrict__ clip_coef) {
  const float gs = grad_scale * (clip_coef ? *clip_coef : 1.f);
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 w4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float g[4];
    if (GRAD_BF16) {
      uint2 u = reinterpret_cast<const uint2*>(grad)[i];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    } else {
      float4 g4 = reinterpret_cast<const float4*>(grad)[i];
      g[0] = g4.x; g[1] = g4.y; g[2] = g4.z; g[3] = g4.w;
    }
    float w[4] = {w4.x, w4.y, w4.z, w4.w};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float ge = g[e] * gs;
      mm[e] = b1 * mm[e] + (1.f - b1) * ge;
      vv[e] = b2 * vv[e] + (1.f - b2) * ge * ge;
      const float mh = mm[e] / bc1;
      const float vh = vv[e] / bc2;
      w[e] = w[e] - lr * (mh / (sqrtf(vh) + eps) + wd * w[e]);
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (param) {
      uint2 o;
      o.x = pack_bf16x2(w[0], w[1]);
      o.y = pack_bf16x2(w[2], w[3]);
      reinterpret_cast<uint2*>(param)[i] = o;
    }
  }
  // tail (n not a multiple of 4)
  const long long tail0 = nvec << 2;
  const long long ti = tail0 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (ti < n) {
    float ge = (GRAD_BF16 ? __bfloat162float(reinterpret_cast<const bf16*>(grad)[ti])
                          : reinterpret_cast<const float*>(grad)[ti]) * gs;
    float mm = b1 * m[ti] + (1.f - b1) * ge;
    float vv = b2 * v[ti] + (1.f - b2) * ge * ge;
    float w = master[ti];
    w = w - lr * ((mm / bc1) / (sqrtf(vv / bc2) + eps) + wd * w);
    master[ti] = w; m[ti] = mm; v[ti] = vv;
    if (param) param[ti] = __float2bfloat16(w);
  }
}

template <bool IS_BF16>
__global__ void sumsq_kernel(const void* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float sm[32];
  float acc = 0.f;
  if (IS_BF16) {
    const long long nvec = n >> 3;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float a[8];
      unpack8e(reinterpret_cast<const uint4*>(x)[i], a);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += a[e] * a[e];
    }
    for (long long i = (nvec << 3) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float a = __bfloat162float(reinterpret_cast<const bf16*>(x)[i]);
      acc += a * a;
    }
  } else {
    const long long nvec = n >> 2;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float4 a = reinterpret_cast<const float4*>(x)[i];
      acc += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
    for (long long i = (nvec << 2) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float a = reinterpret_cast<const float*>(x)[i];
      acc += a * a;
    }
  }
  acc = warp_sum_e(acc);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sm[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? sm[lane] : 0.f;
    t = warp_sum_e(t);
    if (lane == 0) atomicAdd(out, t);
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out, long long n, float scale) {
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 a = reinterpret_cast<const float4*>(in)[i];
    uint2 o;
    o.x = pack_bf16x2(a.x * scale, a.y * scale);
    o.y = pack_bf16x2(a.z * scale, a.w * scale);
    reinterpret_cast<uint2*>(out)[i] = o;
  }
  const long long ti = (nvec << 2) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (ti < n) out[ti] = __float2bfloat16(in[ti] * scale);
}

__global__ void cast_bf16_f32_kernel(const bf16* __restrict__ in, float* __restrict__ out, long long n, float scale,
                                     int accumulate) {
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint2 u = reinterpret_cast<const uint2*>(in)[i];
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    float4 o = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
    if (accumulate) {
      float4 old = reinterpret_cast<float4*>(out)[i];
      o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
    }
    reinterpret_cast<float4*>(out)[i] = o;
  }
  const long long ti = (nvec << 2) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (ti < n) {
    float o = __bfloat162float(in[ti]) * scale;
    out[ti] = accumulate ? out[ti] + o : o;
  }
}

}  // namespace gv

using namespace gv;

extern "C" int gv_rope(void* x, const int* pos, const float* inv_freq, long long tokens, int heads, int dh,
                       long long ld, int pos_div, int pos_mod, int pos_offset, int inverse, gv_stream_t s) {
  if (tokens <= 0) return 0;
  if (dh % 16 != 0 || ld % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return 2201;
  const long long total = tokens * heads * (dh / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)s>>>((bf16*)x, pos, inv_freq, tokens, heads, dh, ld,
                                                                 pos_div > 0 ? pos_div : 1,
                                                                 pos_mod > 0 ? pos_mod : 0x7fffffff, pos_offset,
                                                                 inverse);
  return (int)cudaGetLastError();
}

extern "C" int gv_swiglu_fwd(const void* gu, void* out, long long rows, int f, gv_stream_t s) {
  if (rows <= 0) return 0;
  if (f % 8) return 2202;
  swiglu_fwd_kernel<<<grid_for(rows * (f / 8), 256), 256, 0, (cudaStream_t)s>>>((const bf16*)gu, (bf16*)out, rows, f);
  return (int)cudaGetLastError();
}
extern "C" int gv_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long rows, int f, gv_stream_t s) {
  if (rows <= 0) return 0;
  if (f % 8) return 2202;
  swiglu_bwd_kernel<<<grid_for(rows * (f / 8), 256), 256, 0, (cudaStream_t)s>>>((const bf16*)dout, (const bf16*)gu,
                                                                                (bf16*)dgu, rows, f);
  return (int)cudaGetLastError();
}
extern "C" int gv_gelu_fwd(const void* x, void* y, long long n, gv_stream_t s) {
  if (n <= 0) return 0;
  if (n % 8) return 2203;
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)s>>>((const bf16*)x, (bf16*)y, n / 8);
  return (int)cudaGetLastError();
}
extern "C" int gv_gelu_bwd(const void* dy, const void* x, void* dx, long long n, gv_stream_t s) {
  if (n <= 0) return 0;
  if (n % 8) return 2203;
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)s>>>((const bf16*)dy, (const bf16*)x, (bf16*)dx, n / 8);
  return (int)cudaGetLastError();
}
extern "C" int gv_colsum_accum(const void* dy, float* out, long long rows, int cols, gv_stream_t s) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8) return 2204;
  dim3 block(32, 8);
  const int gx = (cols + 255) / 256;
  long long gy = (rows + 63) / 64;
  const long long cap = (static_cast<long long>(num_sms()) * 4 + gx - 1) / gx;
  if (gy > cap) gy = cap;
  if (gy < 1) gy = 1;
  colsum_kernel<<<dim3(gx, (unsigned)gy), block, 0, (cudaStream_t)s>>>((const bf16*)dy, out, rows, cols);
  return (int)cudaGetLastError();
}

extern "C" int gv_embedding_fwd(const long long* ids, const void* table, const int* pos_ids, const void* pos_table,
                                void* out, long long tokens, int hidden, long long vocab_start, long long vocab_rows,
                                gv_stream_t s) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return 2205;
  int grid = (int)(tokens < (long long)num_sms() * 16 ? tokens : (long long)num_sms() * 16);
  embedding_fwd_kernel<<<grid, 128, 0, (cudaStream_t)s>>>(ids, (const bf16*)table, pos_ids, (const bf16*)pos_table,
                                                          (bf16*)out, tokens, hidden, vocab_start, vocab_rows);
  return (int)cudaGetLastError();
}
extern "C" int gv_embedding_bwd(const long long* ids, const void* dout, float* dtable, long long tokens, int hidden,
                                long long vocab_start, long long vocab_rows, gv_stream_t s) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return 2205;
  int grid = (int)(tokens < (long long)num_sms() * 16 ? tokens : (long long)num_sms() * 16);
  embedding_bwd_kernel<<<grid, 128, 0, (cudaStream_t)s>>>(ids, (const bf16*)dout, dtable, tokens, hidden, vocab_start,
                                                          vocab_rows);
  return (int)cudaGetLastError();
}

extern "C" int gv_xent_stats(const void* logits, const long long* labels, float* row_max, float* row_sumexp,
                             float* tgt_logit, long long rows, int vocab_local, long long ld, long long vocab_start,
                             gv_stream_t s) {
  if (rows <= 0) return 0;
  if (ld % 8 || (reinterpret_cast<uintptr_t>(logits) & 15)) return 2206;
  int grid = (int)(rows < (long long)num_sms() * 4 ? rows : (long long)num_sms() * 4);
  xent_stats_kernel<<<grid, XENT_THREADS, 0, (cudaStream_t)s>>>((const bf16*)logits, labels, row_max, row_sumexp,
                                                               tgt_logit, rows, vocab_local, ld, vocab_start);
  return (int)cudaGetLastError();
}
extern "C" int gv_xent_loss_grad(void* logits, const long long* labels, const float* row_max, const float* row_sumexp,
                                 const float* tgt_logit, float* loss, float grad_scale,
                                 const float* grad_scale_ptr, long long rows, int vocab_local, long long ld,
                                 long long vocab_start, long long ignore_index, gv_stream_t s) {
  if (rows <= 0) return 0;
  if (ld % 8 || (reinterpret_cast<uintptr_t>(logits) & 15)) return 2206;
  int grid = (int)(rows < (long long)num_sms() * 4 ? rows : (long long)num_sms() * 4);
  xent_loss_grad_kernel<<<grid, XENT_THREADS, 0, (cudaStream_t)s>>>((bf16*)logits, labels, row_max, row_sumexp,
                                                                   tgt_logit, loss, grad_scale, grad_scale_ptr, rows,
                                                                   vocab_local, ld, vocab_start, ignore_index);
  return (int)cudaGetLastError();
}

extern "C" int gv_adamw(float* master, float* m, float* v, const void* grad, int grad_is_bf16, void* param_bf16,
                        long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                        float bias_corr1, float bias_corr2, float grad_scale, const float* clip_coef, gv_stream_t s) {
  if (n <= 0) return 0;
  const int grid = grid_for((n + 3) / 4 + 4, 256);
  if (grad_is_bf16)
    adamw_kernel<true><<<grid, 256, 0, (cudaStream_t)s>>>(master, m, v, grad, (bf16*)param_bf16, n, lr, beta1, beta2,
                                                          eps, weight_decay, bias_corr1, bias_corr2, grad_scale,
                                                          clip_coef);
  else
    adamw_kernel<false><<<grid, 256, 0, (cudaStream_t)s>>>(master, m, v, grad, (bf16*)param_bf16, n, lr, beta1, beta2,
                                                           eps, weight_decay, bias_corr1, bias_corr2, grad_scale,
                                                           clip_coef);
  return (int)cudaGetLastError();
}

extern "C" int gv_sumsq_accum(const void* x, int is_bf16, long long n, float* out, gv_stream_t s) {
  if (n <= 0) return 0;
  const int grid = grid_for(n / 8 + 1, 256, 4);
  if (is_bf16)
    sumsq_kernel<true><<<grid, 256, 0, (cudaStream_t)s>>>(x, n, out);
  else
    sumsq_kernel<false><<<grid, 256, 0, (cudaStream_t)s>>>(x, n, out);
  return (int)cudaGetLastError();
}

extern "C" int gv_cast_f32_to_bf16(const float* in, void* out, long long n, float scale, gv_stream_t s) {
  if (n <= 0) return 0;
  cast_f32_bf16_kernel<<<grid_for(n / 4 + 4, 256), 256, 0, (cudaStream_t)s>>>(in, (bf16*)out, n, scale);
  return (int)cudaGetLastError();
}
extern "C" int gv_cast_bf16_to_f32(const void* in, float* out, long long n, float scale, int accumulate,
                                   gv_stream_t s) {
  if (n <= 0) return 0;
  cast_bf16_f32_kernel<<<grid_for(n / 4 + 4, 256), 256, 0, (cudaStream_t)s>>>((const bf16*)in, out, n, scale,
                                                                              accumulate);
  return (int)cudaGetLastError();
}

extern "C" int gv_lse_merge(float* acc, float* lse_acc, const void* o_blk, const float* lse_blk, int b, int s, int sb, int s_off,
                            int h, int dh, long long o_sb, long long o_ss, long long o_sh, gv_stream_t st) {
  const long long warps = static_cast<long long>(b) * sb * h;
  if (warps <= 0) return 0;
  if (s_off < 0 || s_off + sb > s) return 2301;
  const long long blocks = (warps * 32 + 255) / 256;
  lse_merge_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)st>>>(acc, lse_acc, (const bf16*)o_blk, lse_blk, b, s, sb, s_off, h, dh,
                                                                  o_sb, o_ss, o_sh, 1);
  return (int)cudaGetLastError();
}
