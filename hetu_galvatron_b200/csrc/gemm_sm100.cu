// bf16 GEMM for sm_100a: TMA-fed shared-memory ring -> tcgen05.mma (one issuing thread)
// -> fp32 accumulators in tensor memory (double buffered) -> epilogue warps.
//
// Replaces the library GEMMs reached through torch.matmul in the reference's
// column/row-parallel linears (megatron/core/tensor_parallel/layers.py:417 forward,
// :462 input gradient, :534 weight gradient and the fused accumulate variant :498-509).
//
// One persistent CTA per SM, 6 warps:
//   warp 0      : TMA producer (one elected lane)
//   warp 1      : TMEM allocator + MMA issuer (one elected lane)
//   warps 2..5  : epilogue; warp w owns TMEM lanes 32*(w%4)..+31
// Tile 128 x BN x 64 (BN = 256 or 128), 128-byte swizzled operands, both operand majors
// supported through the shared-memory descriptors, so forward, dgrad and wgrad GEMMs all read
// the tensors in the layout they already have (no transposes are materialised).
#include <cstdlib>
#include "include/gv_kernels.h"
#include "include/gv_host.h"
#include "include/gv_ptx.cuh"

namespace gv {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 8;

struct GemmDev {
  void* C;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int M, N, K;
  int ldc, ldr;
  int c_f32, accumulate, act;
  float alpha;
  // cross-entropy epilogues of the language-model head (xent_mode 0 = off)
  int xent_mode;               // 1: per-tile (max, sum exp) + target logit, nothing stored to C; 2: C = (softmax - onehot) * gscale
  const long long* labels;     // [M] global label ids
  long long vocab_start, ignore_index;
  float* stats;                // mode 1: [M, stat_tiles, 2]
  float* target;               // mode 1: [M]
  const float* lse;            // mode 2: [M]
  const float* gscale;         // mode 2: [M]
  int stat_tiles;
  // rotary embedding applied to the leading rope_cols columns of the output (the q and k heads of a packed QKV
  // projection) while the accumulators are still in registers; 0 = off
  // gated activation in the epilogue of the MLP up-projection (0 = off): B = [gate rows (f) | up rows (f)], one tile
  // holds 128 gate columns and the 128 up columns of the same units; besides C = [gate | up] (kept for the backward
  // pass) the epilogue stores act = silu(gate) * up
  int swiglu_f;
  __nv_bfloat16* act_out;
  int ld_act;
  int rope_cols, rope_dh;
  const float* rope_inv_freq;  // [rope_dh / 2]
  const int* rope_pos;         // [M] explicit positions, or NULL: position = (row / div) % mod + offset
  int rope_pos_div, rope_pos_mod, rope_pos_offset;
};

template <int BN>
struct GemmSmem {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& tm, int& tn) {
  const int group_span = GROUP_M * num_n;
  const int group = tile / group_span;
  const int first_m = group * GROUP_M;
  const int gsize = min(num_m - first_m, GROUP_M);
  const int in_group = tile - group * group_span;
  tm = first_m + in_group % gsize;
  tn = in_group / gsize;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}

// Epilogue of one 32-column chunk of one output row: alpha, bias, GELU, residual, accumulate, store (bf16 or fp32).
__device__ __forceinline__ void epilogue_chunk(const GemmDev& p, const uint32_t (&r)[32], int row, int col0) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
        const bool full = col0 + 32 <= p.N;
        if (p.bias != nullptr) {
          if (full) {
            const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 b = __ldg(bp + j);
              float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
              v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
              v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
            }
          } else {
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
          }
        }
        if (p.xent_mode == 2) {
          // gradient of the cross entropy w.r.t. the logits, straight from the recomputed fp32 logits
          const float l = p.lse[row], g = p.gscale[row];
          const long long lab = p.labels[row];
          const long long tcol = (lab == p.ignore_index) ? -1 : lab - p.vocab_start - col0;
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = (__expf(v[i] - l) - (tcol == i ? 1.f : 0.f)) * g;
        }
        if (p.act == 1) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
        }
        if (p.residual != nullptr) {
          const __nv_bfloat16* rp = p.residual + static_cast<size_t>(row) * p.ldr + col0;
          if (full) {
            const uint4* rp4 = reinterpret_cast<const uint4*>(rp);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 b = rp4[j];
              float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
              v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
              v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
            }
          } else {
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += __bfloat162float(rp[i]);
          }
        }
        if (p.c_f32) {
          float* cp = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
          if (full) {
            float4* cp4 = reinterpret_cast<float4*>(cp);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 o = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
              if (p.accumulate) {
                float4 old = cp4[j];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              cp4[j] = o;
            }
          } else {
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) cp[i] = p.accumulate ? cp[i] + v[i] : v[i];
          }
        } else {
          __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
          if (full) {
            uint4* cp4 = reinterpret_cast<uint4*>(cp);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (p.accumulate) {
                uint4 b = cp4[j];
                float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
                v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
                v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
              }
              uint4 o;
              o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
              o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
              o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
              o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
              cp4[j] = o;
            }
          } else {
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) {
                float o = v[i];
                if (p.accumulate) o += __bfloat162float(cp[i]);
                cp[i] = __float2bfloat16(o);
              }
          }
        }
}

// Rotary embedding (non-interleaved halves) on two 32-column chunks of one output row that sit half a head apart:
// r1 holds columns [c, c + 32) of the head's first half, r2 the same columns of its second half
// (reference: megatron/core/models/common/embeddings/rotary_pos_embedding.py:204-227 as a separate pass over q and k).
__device__ __forceinline__ void rope_rotate_chunks(const GemmDev& p, uint32_t (&r1)[32], uint32_t (&r2)[32], int row, int freq0) {
  const float pos = p.rope_pos ? static_cast<float>(p.rope_pos[row])
                               : static_cast<float>((row / p.rope_pos_div) % p.rope_pos_mod + p.rope_pos_offset);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float sn, cs;
    sincosf(pos * __ldg(p.rope_inv_freq + freq0 + i), &sn, &cs);
    const float a = __uint_as_float(r1[i]), b = __uint_as_float(r2[i]);
    r1[i] = __float_as_uint(a * cs - b * sn);
    r2[i] = __float_as_uint(b * cs + a * sn);
  }
}

// SwiGLU on two accumulator chunks of one row: rg = gate pre-activations, ru = up values of the same 32 hidden units.
// Stores both (bf16) into C = [gate | up] and silu(gate) * up into the activation output
// (reference: chunk + silu * mul as separate passes, galvatron/core/runtime/tensor_parallel/transformer.py:122-124).
__device__ __forceinline__ void swiglu_chunks(const GemmDev& p, const uint32_t (&rg)[32], const uint32_t (&ru)[32], int row,
                                              int unit0) {
  epilogue_chunk(p, rg, row, unit0);
  epilogue_chunk(p, ru, row, p.swiglu_f + unit0);
  __nv_bfloat16* ap = p.act_out + static_cast<size_t>(row) * p.ld_act + unit0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      // on the bf16-rounded values, like the stand-alone kernel that reads the stored projection
      const float g = __bfloat162float(__float2bfloat16(__uint_as_float(rg[j * 8 + e]) * p.alpha));
      const float u = __bfloat162float(__float2bfloat16(__uint_as_float(ru[j * 8 + e]) * p.alpha));
      o[e] = g / (1.f + __expf(-g)) * u;
    }
    uint4 w;
    w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]); w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
    reinterpret_cast<uint4*>(ap)[j] = w;
  }
}

// Cross-entropy statistics of one 32-column chunk of one row of logits (fp32, straight from the accumulator): the
// running (max, sum exp(x - max)) of the row over the current tile, and the target logit when the label's column is
// in this chunk. Replaces the passes over materialised logits of the reference's vocab-parallel cross entropy
// (megatron/core/tensor_parallel/cross_entropy.py:16-152).
__device__ __forceinline__ void xent_stats_chunk(const GemmDev& p, const uint32_t (&r)[32], int row, int col0, float& xm,
                                                 float& xl) {
  float v[32];
  const int valid = min(32, p.N - col0);
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = i < valid ? __uint_as_float(r[i]) * p.alpha : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  const float m_new = fmaxf(xm, mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) sum += __expf(v[i] - m_new);
  xl = xl * __expf(xm - m_new) + sum;
  xm = m_new;
  const long long lab = p.labels[row];
  if (lab != p.ignore_index) {
    const long long t = lab - p.vocab_start - col0;
    if (t >= 0 && t < valid) {
      float tv = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) tv = (t == i) ? v[i] : tv;
      p.target[row] = tv;
    }
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmDev p) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = p.swiglu_f > 0 ? p.swiglu_f / 128 : (p.N + BN - 1) / BN;   // gated: a tile = 128 hidden units
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulator buffers (512 or 256 columns)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, num_m, num_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, 1)) { ok = false; break; }
          uint8_t* sA = smem + stage * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int q = 0; q < BM / 64; ++q) tma_load_2d(sA + q * (BK * 128), &tmA, &full_bar[stage], m0 + q * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            if (p.swiglu_f > 0) {
              // 128 gate rows and the 128 up rows of the same hidden units (the map's box is 128 rows in this mode)
              tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, tn * 128);
              tma_load_2d(sB + 128 * 128, &tmB, &full_bar[stage], kb * BK, p.swiglu_f + tn * 128);
            } else {
              tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, n0);
            }
          } else {
#pragma unroll
            for (int q = 0; q < BN / 64; ++q) tma_load_2d(sB + q * (BK * 128), &tmB, &full_bar[stage], n0 + q * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // K-major: step 16 elements = 32 B inside the 128-B swizzle row.
            // MN-major: step 16 K-rows = two 8-row atoms = 2048 B; 64-wide panels are BK*128 B apart.
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_addr + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(a_addr + k * 32, 0, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_addr + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(b_addr + k * 32, 0, 1024);
            umma_f16_ss<1>(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit<1>(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit<1>(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;  // TMEM lane group this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, num_m, num_n, tm, tn);
      const int row = tm * BM + quarter * 32 + lane;
      const int n0 = tn * BN;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, 4)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool row_ok = row < p.M;
      float xm = -INFINITY, xl = 0.f;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (p.swiglu_f > 0) {
          // columns [0, 128) of the tile are gate, [128, 256) up, of hidden units tn * 128 ...
          if (c >= 4) continue;
          uint32_t r2[32];
          tmem_ld_32x32b_x32(t_addr + (c + 4) * 32, r2);
          tmem_ld_wait();
          if (row_ok) swiglu_chunks(p, r, r2, row, tn * 128 + c * 32);
          continue;
        }
        if (p.rope_cols > 0 && col0 < p.rope_cols) {
          // q / k heads: the chunk and its partner half a head further right are rotated together
          const int hc = p.rope_dh >> 6;                      // chunks per half head
          const int in_head = (col0 % p.rope_dh) >> 5;
          if (in_head >= hc) continue;                        // second halves were stored with their partners
          uint32_t r2[32];
          tmem_ld_32x32b_x32(t_addr + (c + hc) * 32, r2);
          tmem_ld_wait();
          if (row_ok) {
            rope_rotate_chunks(p, r, r2, row, in_head * 32);
            epilogue_chunk(p, r, row, col0);
            epilogue_chunk(p, r2, row, col0 + hc * 32);
          }
          continue;
        }
        if (row_ok && col0 < p.N) {
          if (p.xent_mode == 1) xent_stats_chunk(p, r, row, col0, xm, xl);
          else epilogue_chunk(p, r, row, col0);
        }
      }
      if (p.xent_mode == 1 && row_ok) {
        float* st = p.stats + (static_cast<size_t>(row) * p.stat_tiles + tn) * 2;
        st[0] = xm;
        st[1] = xl;
      }
      __syncwarp();
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------------
// Pair kernel: two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 tile with tcgen05.mma.cta_group::2.
// Each CTA stages its own 128 rows of A and its own 128 of the 256 B rows per k-block (32 KB instead of 48 KB per
// 128 x 256 x 64 of work), so the same tensor-core work needs a third less L2 -> shared-memory traffic and the ring
// is six stages deep. The even CTA of the pair issues every MMA; accumulators live in both CTAs' TMEM (each its own
// 128 rows x 256 columns, double buffered). No load is multicast: the odd CTA's TMA loads simply complete on the even
// CTA's barrier. All four operand layouts (forward, dgrad, wgrad) like the single-CTA kernel above.
// Measured 1.63-1.72 PFLOP/s on the Llama-7B forward shapes (0.98-1.04 of the measured cuBLAS burst peak) against
// 1.41-1.50 for the single-CTA kernel; used whenever every CTA pair gets a 256 x 256 tile (GV_GEMM_PAIR=0 turns it off).
// ----------------------------------------------------------------------------------
constexpr int P_STAGES = 6;
constexpr int P_HALF_BYTES = BM * BK * 2;                  // 16 KB: A half or B half of one k-block
constexpr int P_STAGE_BYTES = 2 * P_HALF_BYTES;
constexpr int P_BAR_OFFSET = P_STAGES * P_STAGE_BYTES;
constexpr int P_SMEM_TOTAL = P_BAR_OFFSET + 256 + 1024;

// TMA tile load of this CTA's shared memory whose completion is counted on CTA 0's barrier (pair form of the load)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* desc, uint64_t* bar, int32_t c0, int32_t c1) {
  uint32_t leader_bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(leader_bar) : "r"(smem_u32(bar)), "r"(0));
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(leader_bar), "r"(c0), "r"(c1)
      : "memory");
}
// commit of the pair's MMAs: arrives on the same barrier in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + P_BAR_OFFSET);   // used in CTA 0 only
  uint64_t* empty_bar = full_bar + P_STAGES;                                // one set per CTA
  uint64_t* acc_full = empty_bar + P_STAGES;                                // [2], one set per CTA
  uint64_t* acc_empty = acc_full + 2;                                       // [2], used in CTA 0 only (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();               // 0: issues the MMAs; 1: peer
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  constexpr int TM = 2 * BM, TN = 256;
  const int num_m = (p.M + TM - 1) / TM, num_n = p.swiglu_f > 0 ? p.swiglu_f / 128 : (p.N + TN - 1) / TN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 2 * TN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);       // CTA 0 arms it for the bytes of both CTAs
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 256);    // the epilogue threads of both CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, TMEM_COLS);
    tmem_relinquish<2>();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                   // the peer's barriers exist before anything arrives on them remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        tile_coords(tile, num_m, num_n, tm, tn);
        const int m0 = tm * TM + static_cast<int>(cta) * BM;      // this CTA's rows of A and of the output
        // this CTA's 128 rows of B (columns of the output); gated mode: CTA 0 stages the gate rows, CTA 1 the up rows
        const int nb0 = p.swiglu_f > 0 ? tn * 128 + static_cast<int>(cta) * p.swiglu_f : tn * TN + static_cast<int>(cta) * BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, 5)) { ok = false; break; }
          uint8_t* sA = smem + stage * P_STAGE_BYTES;
          uint8_t* sB = sA + P_HALF_BYTES;
          // CTA 0 arms its barrier for the bytes of BOTH CTAs; the peer only issues its loads (their completions may
          // land before the arming: the phase still cannot complete before CTA 0's arrival). A remote arrive per
          // stage from the peer would put a cluster round trip into its producer loop.
          if (cta == 0) mbar_expect_tx(&full_bar[stage], 2 * P_STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d_pair(sA, &tmA, &full_bar[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int q = 0; q < BM / 64; ++q) tma_load_2d_pair(sA + q * (BK * 128), &tmA, &full_bar[stage], m0 + q * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sB, &tmB, &full_bar[stage], kb * BK, nb0);
          } else {
#pragma unroll
            for (int q = 0; q < BM / 64; ++q) tma_load_2d_pair(sB + q * (BK * 128), &tmB, &full_bar[stage], nb0 + q * 64, kb * BK);
          }
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (CTA 0 only) --------------------------------
    if (cta == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(TM, TN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      // K-major: 16 elements along K = 32 B inside the swizzle row; MN-major: 16 K-rows = 2048 B, 64-wide panels BK*128 B apart
      const uint64_t a_desc0 = A_MN ? make_smem_desc_sw128(smem_u32(smem), BK * 128, 1024) : make_smem_desc_sw128(smem_u32(smem), 0, 1024);
      const uint64_t b_desc0 = B_MN ? make_smem_desc_sw128(smem_u32(smem) + P_HALF_BYTES, BK * 128, 1024)
                                    : make_smem_desc_sw128(smem_u32(smem) + P_HALF_BYTES, 0, 1024);
      constexpr uint64_t A_STEP = A_MN ? (2048 >> 4) : (32 >> 4), B_STEP = B_MN ? (2048 >> 4) : (32 >> 4);
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, 6)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, 7)) { ok = false; break; }
          tc_fence_after();
          const uint64_t so = static_cast<uint64_t>(stage) * (P_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16_ss<2>(d_tmem, a_desc0 + so + k * A_STEP, b_desc0 + so + k * B_STEP, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage]);   // frees this stage in both CTAs once these MMAs retire
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs, own 128 rows) ----------------------------------
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int tm, tn;
      tile_coords(tile, num_m, num_n, tm, tn);
      const int row = tm * TM + static_cast<int>(cta) * BM + quarter * 32 + lane;
      const int n0 = tn * TN;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, 8)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * TN + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool row_ok = row < p.M;
      float xm = -INFINITY, xl = 0.f;
#pragma unroll 1
      for (int c = 0; c < TN / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (p.swiglu_f > 0) {
          // columns [0, 128) of the tile are gate, [128, 256) up, of hidden units tn * 128 ...
          if (c >= 4) continue;
          uint32_t r2[32];
          tmem_ld_32x32b_x32(t_addr + (c + 4) * 32, r2);
          tmem_ld_wait();
          if (row_ok) swiglu_chunks(p, r, r2, row, tn * 128 + c * 32);
          continue;
        }
        if (p.rope_cols > 0 && col0 < p.rope_cols) {
          // q / k heads: the chunk and its partner half a head further right are rotated together
          const int hc = p.rope_dh >> 6;                      // chunks per half head
          const int in_head = (col0 % p.rope_dh) >> 5;
          if (in_head >= hc) continue;                        // second halves were stored with their partners
          uint32_t r2[32];
          tmem_ld_32x32b_x32(t_addr + (c + hc) * 32, r2);
          tmem_ld_wait();
          if (row_ok) {
            rope_rotate_chunks(p, r, r2, row, in_head * 32);
            epilogue_chunk(p, r, row, col0);
            epilogue_chunk(p, r2, row, col0 + hc * 32);
          }
          continue;
        }
        if (row_ok && col0 < p.N) {
          if (p.xent_mode == 1) xent_stats_chunk(p, r, row, col0, xm, xl);
          else epilogue_chunk(p, r, row, col0);
        }
      }
      if (p.xent_mode == 1 && row_ok) {
        float* st = p.stats + (static_cast<size_t>(row) * p.stat_tiles + tn) * 2;
        st[0] = xm;
        st[1] = xl;
      }
      __syncwarp();
      tc_fence_before();
      mbar_arrive_cluster(&acc_empty[acc], 0);   // both CTAs report to the issuing CTA
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                   // nobody frees tensor memory while the pair's MMAs could still write it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2>(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, ld] buffer with `cols` valid columns,
// box = [box_rows, 64 columns] with 128-byte swizzle.
// Makes the primary context of the device that owns `ptr` current on the calling thread (a thread that has made no
// runtime call yet, e.g. an autograd worker, has none, and driver entry points then fail with INVALID_CONTEXT).
void bind_context_of(const void* ptr) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, ptr) == cudaSuccess && attr.type == cudaMemoryTypeDevice) {
    cudaSetDevice(attr.device);
  } else {
    cudaGetLastError();
  }
  cudaFree(nullptr);
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return 1001;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // a thread that has made no runtime call yet (an autograd worker) has no current context: bind the primary one
    bind_context_of(base);
    r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? 0 : 1000 + static_cast<int>(r);
}

static int g_num_sms = 0;
int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

static void fill_xent(GemmDev& p, const gv_xent_args* x, int tile_n) {
  p.xent_mode = 0;
  p.labels = nullptr; p.vocab_start = 0; p.ignore_index = -100;
  p.stats = nullptr; p.target = nullptr; p.lse = nullptr; p.gscale = nullptr; p.stat_tiles = 0;
  if (x == nullptr) return;
  p.xent_mode = x->mode;
  p.labels = x->labels; p.vocab_start = x->vocab_start; p.ignore_index = x->ignore_index;
  p.stats = x->stats; p.target = x->target; p.lse = x->lse; p.gscale = x->gscale;
  p.stat_tiles = (p.N + tile_n - 1) / tile_n;
}

static void fill_swiglu(GemmDev& p, const gv_gemm_args* a) {
  p.swiglu_f = a->swiglu_out ? a->N / 2 : 0;
  p.act_out = reinterpret_cast<__nv_bfloat16*>(a->swiglu_out);
  p.ld_act = a->swiglu_ld;
}

static void fill_rope(GemmDev& p, const gv_gemm_args* a) {
  p.rope_cols = a->rope_cols; p.rope_dh = a->rope_dh;
  p.rope_inv_freq = a->rope_inv_freq; p.rope_pos = a->rope_pos;
  p.rope_pos_div = a->rope_pos_div > 0 ? a->rope_pos_div : 1;
  p.rope_pos_mod = a->rope_pos_mod > 0 ? a->rope_pos_mod : 0x7fffffff;
  p.rope_pos_offset = a->rope_pos_offset;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const gv_gemm_args* a, cudaStream_t stream, const gv_xent_args* x = nullptr) {
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN)
    rc = make_tmap_bf16_2d(&tmA, a->A, a->M, a->K, a->lda, 64, BM);
  else
    rc = make_tmap_bf16_2d(&tmA, a->A, a->K, a->M, a->lda, 64, BK);
  if (rc) return rc;
  if (!B_MN)
    rc = make_tmap_bf16_2d(&tmB, a->B, a->N, a->K, a->ldb, 64, a->swiglu_out ? 128 : BN);
  else
    rc = make_tmap_bf16_2d(&tmB, a->B, a->K, a->N, a->ldb, 64, BK);
  if (rc) return rc;
  GemmDev p;
  p.C = a->C;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.ldc = a->ldc; p.ldr = a->ldr;
  p.c_f32 = a->c_f32; p.accumulate = a->accumulate; p.act = a->act;
  p.alpha = a->alpha;
  fill_xent(p, x, BN);
  fill_rope(p, a);
  fill_swiglu(p, a);
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  constexpr int smem = GemmSmem<BN>::TOTAL;
  static PerDeviceOnce smem_once;
  {
    cudaError_t e = ensure_max_dynamic_smem(smem_once, kern, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int tiles = ((a->M + BM - 1) / BM) * (a->swiglu_out ? a->N / 256 : (a->N + BN - 1) / BN);
  const int grid = tiles < num_sms() ? tiles : num_sms();
  kern<<<grid, GEMM_THREADS, smem, stream>>>(tmA, tmB, p);
  return static_cast<int>(cudaGetLastError());
}

template <bool A_MN, bool B_MN>
static int launch_gemm_pair(const gv_gemm_args* a, cudaStream_t stream, const gv_xent_args* x = nullptr) {
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN)
    rc = make_tmap_bf16_2d(&tmA, a->A, a->M, a->K, a->lda, 64, BM);
  else
    rc = make_tmap_bf16_2d(&tmA, a->A, a->K, a->M, a->lda, 64, BK);
  if (rc) return rc;
  if (!B_MN)
    rc = make_tmap_bf16_2d(&tmB, a->B, a->N, a->K, a->ldb, 64, BM);   // each CTA of the pair loads 128 of the 256 B rows
  else
    rc = make_tmap_bf16_2d(&tmB, a->B, a->K, a->N, a->ldb, 64, BK);
  if (rc) return rc;
  GemmDev p;
  p.C = a->C;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.ldc = a->ldc; p.ldr = a->ldr;
  p.c_f32 = a->c_f32; p.accumulate = a->accumulate; p.act = a->act;
  p.alpha = a->alpha;
  fill_xent(p, x, 256);
  fill_rope(p, a);
  fill_swiglu(p, a);
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN>;
  static PerDeviceOnce smem_once;
  {
    cudaError_t e = ensure_max_dynamic_smem(smem_once, kern, P_SMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int tiles = ((a->M + 2 * BM - 1) / (2 * BM)) * ((a->N + 255) / 256);
  // A persistent grid must not exceed the number of CTA pairs the device can hold at once (a part with an odd number
  // of SMs enabled in some TPCs holds fewer than num_sms / 2): the pairs left over would run as a second wave.
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(num_sms() / 2 * 2));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = P_SMEM_TOTAL;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = num_sms() / 2;
    }
    max_pairs = n;
  }
  int pairs = max_pairs;
  if (tiles < pairs) pairs = tiles;
  kern<<<2 * pairs, GEMM_THREADS, P_SMEM_TOTAL, stream>>>(tmA, tmB, p);
  return static_cast<int>(cudaGetLastError());
}

// GV_GEMM_PAIR: 0 never, 1 (default) when there is a 256 x 256 tile for every SM pair, 2 always (used by the
// numerics tests on small shapes).
static int pair_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("GV_GEMM_PAIR");
    mode = e ? (e[0] - '0') : 1;
    if (mode < 0 || mode > 2) mode = 1;
  }
  return mode;
}

}  // namespace gv

GV_DEFINE_ERROR_READER(gv_read_error_gemm)

extern "C" int gv_gemm_bf16(const gv_gemm_args* a, gv_stream_t s) {
  using namespace gv;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(s);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  if ((a->K % 8) || (a->lda % 8) || (a->ldb % 8) || (a->ldc % (a->c_f32 ? 4 : 8))) return 2001;
  if ((reinterpret_cast<uintptr_t>(a->A) | reinterpret_cast<uintptr_t>(a->B) | reinterpret_cast<uintptr_t>(a->C)) & 15)
    return 2002;
  if (a->a_mn_major && (a->M % 8)) return 2003;
  if (a->b_mn_major && (a->N % 8)) return 2004;
  if (a->residual && ((a->ldr % 8) || (reinterpret_cast<uintptr_t>(a->residual) & 15))) return 2005;
  if (a->rope_cols > 0 && ((a->rope_dh != 64 && a->rope_dh != 128) || a->rope_cols % a->rope_dh || a->rope_cols > a->N ||
                           a->rope_inv_freq == nullptr || a->bias || a->residual || a->act || a->accumulate || a->alpha != 1.f))
    return 2006;
  if (a->swiglu_out) {
    // gated up-projection: K-major operands, N = 2 f with f a multiple of 128, plain store of C
    if (a->a_mn_major || a->b_mn_major || a->bias || a->residual || a->act || a->accumulate || a->c_f32 || a->rope_cols ||
        (a->N % 256) || (a->swiglu_ld % 8) || (reinterpret_cast<uintptr_t>(a->swiglu_out) & 15))
      return 2007;
    const long pair_tiles = static_cast<long>((a->M + 255) / 256) * (a->N / 256);
    if (pair_mode() != 0 && (pair_mode() == 2 || pair_tiles >= num_sms() / 2)) return launch_gemm_pair<false, false>(a, stream);
    return launch_gemm<256, false, false>(a, stream);
  }
  // Narrow tiles when wide ones would leave most SMs idle.
  const long tiles256 = static_cast<long>((a->M + BM - 1) / BM) * ((a->N + 255) / 256);
  const bool narrow = (a->N <= 128) || (tiles256 < num_sms());
  const int key = (a->a_mn_major ? 2 : 0) | (a->b_mn_major ? 1 : 0);
  // K-major operands and enough 256 x 256 tiles for every SM pair: the two-CTA kernel
  if (pair_mode() != 0) {
    const long pair_tiles = static_cast<long>((a->M + 255) / 256) * ((a->N + 255) / 256);
    if (pair_mode() == 2 || (!narrow && pair_tiles >= num_sms() / 2)) {
      switch (key) {
        case 0: return launch_gemm_pair<false, false>(a, stream);
        case 1: return launch_gemm_pair<false, true>(a, stream);
        case 2: return launch_gemm_pair<true, false>(a, stream);
        default: return launch_gemm_pair<true, true>(a, stream);
      }
    }
  }
  if (!narrow) {
    switch (key) {
      case 0: return launch_gemm<256, false, false>(a, stream);
      case 1: return launch_gemm<256, false, true>(a, stream);
      case 2: return launch_gemm<256, true, false>(a, stream);
      default: return launch_gemm<256, true, true>(a, stream);
    }
  } else {
    switch (key) {
      case 0: return launch_gemm<128, false, false>(a, stream);
      case 1: return launch_gemm<128, false, true>(a, stream);
      case 2: return launch_gemm<128, true, false>(a, stream);
      default: return launch_gemm<128, true, true>(a, stream);
    }
  }
}

// Language-model head with the cross entropy in the GEMM epilogue. Always runs the 256-column-wide tiles, so the
// statistics buffer of mode 1 has ceil(N / 256) entries per row.
extern "C" int gv_gemm_xent(const gv_gemm_args* a, const gv_xent_args* x, gv_stream_t s) {
  using namespace gv;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(s);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  if (x == nullptr || (x->mode != 1 && x->mode != 2) || x->labels == nullptr) return 2011;
  if (x->mode == 1 && (x->stats == nullptr || x->target == nullptr)) return 2012;
  if (x->mode == 2 && (x->lse == nullptr || x->gscale == nullptr || a->C == nullptr || a->c_f32 || a->accumulate)) return 2013;
  if (a->a_mn_major || a->b_mn_major || a->bias || a->residual || a->act) return 2014;
  if ((a->K % 8) || (a->lda % 8) || (a->ldb % 8) || (x->mode == 2 && (a->ldc % 8))) return 2001;
  if ((reinterpret_cast<uintptr_t>(a->A) | reinterpret_cast<uintptr_t>(a->B) | reinterpret_cast<uintptr_t>(a->C)) & 15) return 2002;
  const long pair_tiles = static_cast<long>((a->M + 255) / 256) * ((a->N + 255) / 256);
  if (pair_mode() != 0 && (pair_mode() == 2 || pair_tiles >= num_sms() / 2)) return launch_gemm_pair<false, false>(a, stream, x);
  return launch_gemm<256, false, false>(a, stream, x);
}
