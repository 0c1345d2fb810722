// Flash attention forward / backward for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// Replaces the FlashAttention-2 library calls of the reference
// (galvatron/core/runtime/tensor_parallel/transformer.py:495-506 flash_attn_varlen_func, and the private
// forward/backward with log-sum-exp used by ring attention, :2359-2387 and :2467-2498).
//
// Forward: one CTA = 128 query rows of one (batch, head); KV blocks of 64 rows stream through a 2-stage TMA
// ring. S = Q K^T lands in TMEM (double buffered), four softmax warps (one row per thread) turn it into
// bf16 P in swizzled shared memory, O += P V accumulates in TMEM with lazy rescaling (O is only rescaled
// when the running row maximum grew by more than 2^8). Two CTAs fit per SM so one CTA's softmax overlaps
// the other's MMAs.
//
// Backward: one CTA = 128 KV rows of one (batch, kv head); it loops over the query heads of its group and
// over 64-row query blocks, holding dK and dV in TMEM. Per block: S^T = K Q^T, dP^T = V dO^T (TMEM),
// P^T and dS^T are written to shared memory by two epilogue warpgroups, dV += P^T dO, dK += dS^T Q,
// dQ^T = K^T dS^T is read back from TMEM and added into an fp32 dQ buffer with coalesced reductions.
// Every operand is consumed in the layout it has in shared memory (K-major or MN-major descriptors).
#include "include/gv_kernels.h"
#include "include/gv_host.h"
#include "include/gv_ptx.cuh"

namespace gv {

int num_sms();
typedef __nv_bfloat16 bf16;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn attn_encode_fn() {
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

// 4-D bf16 map over [b, s, h, dh] with element strides; box = [1, rows, 1, 64] (128-byte swizzle).
void bind_context_of(const void* ptr);

static int make_tmap_bshd(CUtensorMap* out, const void* base, int b, int s, int h, int dh, long long sb, long long ss,
                          long long sh, int box_rows) {
  EncodeTiledFn fn = attn_encode_fn();
  if (fn == nullptr) return 1001;
  cuuint64_t dims[4] = {(cuuint64_t)dh, (cuuint64_t)h, (cuuint64_t)s, (cuuint64_t)b};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // a thread that has made no runtime call yet (an autograd worker) has no current context: bind the primary one
    bind_context_of(base);
    r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? 0 : 1000 + static_cast<int>(r);
}

// Counter-based dropout of attention probabilities: whether entry (q, k) of head h of batch element b is kept is a
// pure function of (seed, b, h, q, k), so the forward and the backward kernel (and a recomputed forward under
// activation checkpointing) draw the same mask without storing it. `bh_key` folds seed, batch and global head index.
__device__ __forceinline__ uint32_t drop_key(unsigned long long seed, int batch, int head) {
  uint32_t x = static_cast<uint32_t>(seed) ^ (static_cast<uint32_t>(seed >> 32) * 0x9E3779B1u);
  x ^= static_cast<uint32_t>(batch) * 0x85EBCA77u + 0x165667B1u;
  x ^= x >> 15; x *= 0x2C1B3C6Du;
  x ^= static_cast<uint32_t>(head) * 0xC2B2AE3Du + 0x27D4EB2Fu;
  x ^= x >> 13; x *= 0x297A2D39u; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ bool drop_keep(uint32_t bh_key, int q, int k, uint32_t threshold) {
  uint32_t x = bh_key ^ (static_cast<uint32_t>(q) * 0x9E3779B1u) ^ (static_cast<uint32_t>(k) * 0x85EBCA77u);
  x ^= x >> 15; x *= 0x2C1B3C6Du; x ^= x >> 12; x *= 0x297A2D39u; x ^= x >> 15;
  return x >= threshold;     // threshold = p * 2^32: dropped with probability p
}

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// =====================================================================================
// Forward
// =====================================================================================
constexpr int FWD_BM = 128;
constexpr int FWD_BN = 64;
constexpr int FWD_THREADS = 192;

template <int DH>
struct FwdSmem {
  static constexpr int PANELS = DH / 64;
  static constexpr int Q_BYTES = FWD_BM * DH * 2;
  static constexpr int KV_BYTES = FWD_BN * DH * 2;
  static constexpr int P_BYTES = FWD_BM * FWD_BN * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 768;
};

struct FwdParams {
  bf16* o;
  float* lse;
  const int* kv_lens;  // optional [b]: keys at or beyond kv_lens[batch] are padding (masked out)
  uint32_t drop_threshold;          // 0 = no dropout; else p * 2^32
  float drop_scale;                 // 1 / (1 - p)
  unsigned long long drop_seed;
  int drop_head_offset;
  int b, sq, sk, hq, hk, dh;
  long long o_sb, o_ss, o_sh;
  int causal;
  float scale_log2;
  // BIAS instantiation only (each may be null): bias bf16 [hq, sq, bias_ld], additive mask fp32 [mask_n, sq, bias_ld],
  // group ids int32 [mask_n, bias_ld]
  const bf16* bias;
  const float* mask;
  const int* ids;
  int mask_n, bias_ld;
};

// Kernel variants (template parameter MODE), so that the plain kernels carry none of the optional code:
// MODE_BIAS: the scaled scores take an additive bias (per head), an additive mask and / or group ids (per batch element
// modulo mask_n) before the softmax -- windowed attention with a relative-position bias and a shifted-window mask.
// MODE_DROP: counter-based dropout of the probabilities.
constexpr int MODE_PLAIN = 0, MODE_BIAS = 1, MODE_DROP = 2;

template <int DH, int MODE>
__global__ void __launch_bounds__(FWD_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, FwdParams p) {
  using S = FwdSmem<DH>;
  constexpr bool BIAS = MODE == MODE_BIAS, DROP = MODE == MODE_DROP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* kv_empty = bars + 5;  // [2]
  uint64_t* s_full = bars + 7;    // [2]
  uint64_t* s_empty = bars + 9;   // [2]
  uint64_t* p_full = bars + 11;
  uint64_t* pv_done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  if (static_cast<int>(smem - smem_raw) + S::OFF_BAR + 128 > S::TOTAL) {  // dynamic smem base less aligned than assumed
    if (threadIdx.x == 0) record_error((0x10u << 16) | 2u, static_cast<unsigned>(smem - smem_raw));
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (p.sq + FWD_BM - 1) / FWD_BM;
  const int q_tile = num_q_tiles - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.hq / p.hk);
  const int q0 = q_tile * FWD_BM;
  const int shift = p.sk - p.sq;  // causal: query i sees keys <= i + shift
  const int sk_eff = p.kv_lens ? max(0, min(p.sk, p.kv_lens[batch])) : p.sk;   // keys that are not padding
  int kv_end = sk_eff;
  if (p.causal) kv_end = min(sk_eff, min(p.sq, q0 + FWD_BM) + shift);
  const int n_blocks = kv_end > 0 ? (kv_end + FWD_BN - 1) / FWD_BN : 0;
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t TM_S = 0, TM_O = 2 * FWD_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
    if (elect_one() && n_blocks > 0) {
      mbar_expect_tx(q_full, S::Q_BYTES);
#pragma unroll
      for (int c = 0; c < S::PANELS; ++c)
        tma_load_4d(smem + S::OFF_Q + c * (FWD_BM * 128), &tmQ, q_full, c * 64, head, q0, batch);
      for (int j = 0; j < n_blocks; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1, abort_flag, 0x11)) break;
        mbar_expect_tx(&k_full[st], S::KV_BYTES);
#pragma unroll
        for (int c = 0; c < S::PANELS; ++c)
          tma_load_4d(smem + S::OFF_K + st * S::KV_BYTES + c * (FWD_BN * 128), &tmK, &k_full[st], c * 64, kv_head,
                      j * FWD_BN, batch);
        mbar_expect_tx(&v_full[st], S::KV_BYTES);
#pragma unroll
        for (int c = 0; c < S::PANELS; ++c)
          tma_load_4d(smem + S::OFF_V + st * S::KV_BYTES + c * (FWD_BN * 128), &tmV, &v_full[st], c * 64, kv_head,
                      j * FWD_BN, batch);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_blocks > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(FWD_BM, FWD_BN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(FWD_BM, DH, 0, 1);
      const uint32_t q_addr = smem_u32(smem + S::OFF_Q);
      const uint32_t p_addr = smem_u32(smem + S::OFF_P);
      // Descriptors are built once; inside the loops an operand advances by adding (bytes >> 4) to its descriptor, so
      // the single issuing thread spends one add per operand per MMA instead of rebuilding 64-bit descriptors.
      const uint64_t q_desc = make_smem_desc_sw128(q_addr, 0, 1024);
      const uint64_t p_desc = make_smem_desc_sw128(p_addr, 0, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem + S::OFF_K), 0, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem + S::OFF_V), FWD_BN * 128, 1024);
      auto issue_s = [&](int j) {
        const uint64_t k_desc = k_desc0 + static_cast<uint64_t>((j & 1) * (S::KV_BYTES >> 4));
        const uint32_t d_tmem = tmem_base + TM_S + (j & 1) * FWD_BN;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint64_t da = q_desc + static_cast<uint64_t>(((kk >> 2) * (FWD_BM * 128) + (kk & 3) * 32) >> 4);
          const uint64_t db = k_desc + static_cast<uint64_t>(((kk >> 2) * (FWD_BN * 128) + (kk & 3) * 32) >> 4);
          umma_f16_ss<1>(d_tmem, da, db, idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit<1>(&s_full[j & 1]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, 0x12) && mbar_wait(&k_full[0], 0, abort_flag, 0x13);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks) {
          const int jn = j + 1;
          if (!mbar_wait(&k_full[jn & 1], (jn >> 1) & 1, abort_flag, 0x14)) { ok = false; break; }
          if (!mbar_wait(&s_empty[jn & 1], ((jn >> 1) & 1) ^ 1, abort_flag, 0x15)) { ok = false; break; }
          tc_fence_after();
          issue_s(jn);
        }
        if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1, abort_flag, 0x16)) { ok = false; break; }
        if (!mbar_wait(p_full, j & 1, abort_flag, 0x17)) { ok = false; break; }
        tc_fence_after();
        const uint64_t v_desc = v_desc0 + static_cast<uint64_t>((j & 1) * (S::KV_BYTES >> 4));
#pragma unroll
        for (int kk = 0; kk < FWD_BN / 16; ++kk) {
          const uint64_t da = p_desc + static_cast<uint64_t>((kk * 32) >> 4);
          const uint64_t db = v_desc + static_cast<uint64_t>((kk * 2048) >> 4);
          umma_f16_ss<1>(tmem_base + TM_O, da, db, idesc_pv, (j | kk) != 0 ? 1u : 0u);
        }
        umma_commit<1>(&kv_empty[j & 1]);
        umma_commit<1>(pv_done);
      }
    }
  } else {
    // ---------------- softmax / correction / epilogue: one query row per thread ----------------
    const int quarter = warp & 3;
    const int rloc = quarter * 32 + lane;
    const int qrow = q0 + rloc;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    uint8_t* p_row = smem + S::OFF_P + rloc * 128;
    const uint32_t bh_key = DROP ? drop_key(p.drop_seed, batch, head + p.drop_head_offset) : 0u;
    for (int j = 0; j < n_blocks && ok; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag, 0x18)) { ok = false; break; }
      tc_fence_after();
      uint32_t r[64];
      __syncwarp();
      tmem_ld_32x32b_x32(tmem_base + lane_off + TM_S + (j & 1) * FWD_BN, r);
      tmem_ld_32x32b_x32(tmem_base + lane_off + TM_S + (j & 1) * FWD_BN + 32, r + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_empty[j & 1]);
      const int kv0 = j * FWD_BN;
      const bool boundary = (kv0 + FWD_BN > sk_eff) || (p.causal && (kv0 + FWD_BN - 1 > q0 + shift));
      float sl2 = p.scale_log2;
      if constexpr (BIAS) {
        // the scores leave this block in the log2 domain with the additive terms folded in:
        // r = s * scale * log2(e) + (bias + mask) * log2(e); rows are bias_ld elements apart (a multiple of 64, so the 64
        // columns of this block are in range and 16-byte aligned whatever sk is)
        const int brow = min(qrow, p.sq - 1);       // padded query rows read a valid row; their output is never stored
        const uint4* b8 = p.bias ? reinterpret_cast<const uint4*>(
            p.bias + (static_cast<long long>(head) * p.sq + brow) * p.bias_ld + kv0) : nullptr;
        const float4* m4 = p.mask ? reinterpret_cast<const float4*>(
            p.mask + (static_cast<long long>(batch % p.mask_n) * p.sq + brow) * p.bias_ld + kv0) : nullptr;
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
          float add[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (b8) {
            const uint4 u = __ldg(b8 + c8);
            const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
            add[0] = f0.x; add[1] = f0.y; add[2] = f1.x; add[3] = f1.y; add[4] = f2.x; add[5] = f2.y; add[6] = f3.x; add[7] = f3.y;
          }
          if (m4) {
            const float4 ma = __ldg(m4 + 2 * c8), mb = __ldg(m4 + 2 * c8 + 1);
            add[0] += ma.x; add[1] += ma.y; add[2] += ma.z; add[3] += ma.w;
            add[4] += mb.x; add[5] += mb.y; add[6] += mb.z; add[7] += mb.w;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i)
            r[c8 * 8 + i] = __float_as_uint(fmaf(__uint_as_float(r[c8 * 8 + i]), p.scale_log2, add[i] * LOG2E));
        }
        sl2 = 1.f;
        if (p.ids) {
          // group ids: a key of another group is invisible; every thread of the CTA reads the same 64 key ids (broadcast)
          const int* idw = p.ids + static_cast<long long>(batch % p.mask_n) * p.bias_ld;
          const int rid = __ldg(idw + brow);
          const int4* k4 = reinterpret_cast<const int4*>(idw + kv0);
#pragma unroll
          for (int c4 = 0; c4 < 16; ++c4) {
            const int4 kk = __ldg(k4 + c4);
            if (kk.x != rid) r[c4 * 4 + 0] = __float_as_uint(-INFINITY);
            if (kk.y != rid) r[c4 * 4 + 1] = __float_as_uint(-INFINITY);
            if (kk.z != rid) r[c4 * 4 + 2] = __float_as_uint(-INFINITY);
            if (kk.w != rid) r[c4 * 4 + 3] = __float_as_uint(-INFINITY);
          }
        }
      }
      // row maximum on the RAW scores (scale > 0 commutes with max); masked entries become -inf first
      float mx = -INFINITY;
      if (boundary) {
        const int limit = p.causal ? min(sk_eff - 1, qrow + shift) : sk_eff - 1;
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          if (kv0 + c > limit) r[c] = __float_as_uint(-INFINITY);
        }
      }
#pragma unroll
      for (int c = 0; c < 64; c += 2) mx = fmax3(mx, __uint_as_float(r[c]), __uint_as_float(r[c + 1]));
      mx *= sl2;
      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1, abort_flag, 0x19)) { ok = false; break; }
        tc_fence_after();
      }
      if (j == 0) {
        m_used = (mx == -INFINITY) ? 0.f : mx;
      } else {
        const bool need = mx > m_used + 8.f;
        if (__any_sync(0xffffffffu, need)) {
          const float m_new = fmaxf(m_used, mx);
          const float alpha = fast_exp2(m_used - m_new);
          l *= alpha;
          m_used = m_new;
#pragma unroll 1
          for (int c = 0; c < DH / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(tmem_base + lane_off + TM_O + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(tmem_base + lane_off + TM_O + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      // p = exp2(s * scale_log2 - m): one packed FMA per two scores, two exp2, one packed add into the row sum
      {
        const uint64_t sc2 = f2_pack(sl2, sl2), nm2 = f2_pack(-m_used, -m_used);
        uint64_t l2 = f2_pack(l, 0.f);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint64_t a2 = f2_fma(f2_pack(__uint_as_float(r[ch * 8 + 2 * e]), __uint_as_float(r[ch * 8 + 2 * e + 1])), sc2, nm2);
            float a0, a1;
            f2_unpack(a2, a0, a1);
            float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
            l2 = f2_add(l2, f2_pack(p0, p1));          // the normaliser counts every probability, dropped or not
            if constexpr (DROP) {
              const int kc = kv0 + ch * 8 + 2 * e;
              p0 = drop_keep(bh_key, qrow, kc, p.drop_threshold) ? p0 * p.drop_scale : 0.f;
              p1 = drop_keep(bh_key, qrow, kc + 1, p.drop_threshold) ? p1 * p.drop_scale : 0.f;
            }
            pk[e] = pack_bf16x2(p0, p1);
          }
          uint4 u;
          u.x = pk[0]; u.y = pk[1]; u.z = pk[2]; u.w = pk[3];
          *reinterpret_cast<uint4*>(p_row + ((ch ^ (rloc & 7)) << 4)) = u;
        }
        float la, lb;
        f2_unpack(l2, la, lb);
        l = la + lb;
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    // epilogue
    if (ok && n_blocks > 0) ok = mbar_wait(pv_done, (n_blocks - 1) & 1, abort_flag, 0x1a);
    tc_fence_after();
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    if (qrow < p.sq && ok) {
      p.lse[(static_cast<long long>(batch) * p.hq + head) * p.sq + qrow] =
          (l > 0.f) ? (m_used + log2f(l)) * LN2 : -INFINITY;
    }
    bf16* o_row = p.o + batch * p.o_sb + static_cast<long long>(qrow) * p.o_ss + head * p.o_sh;
#pragma unroll 1
    for (int c = 0; c < DH / 32; ++c) {
      uint32_t o[32];
      __syncwarp();
      if (n_blocks > 0) {
        tmem_ld_32x32b_x32(tmem_base + lane_off + TM_O + c * 32, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0u;
      }
      if (qrow < p.sq && ok) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int col = c * 32 + g * 8;
          if (col < p.dh) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(o[g * 8 + 0]) * inv_l, __uint_as_float(o[g * 8 + 1]) * inv_l);
            u.y = pack_bf16x2(__uint_as_float(o[g * 8 + 2]) * inv_l, __uint_as_float(o[g * 8 + 3]) * inv_l);
            u.z = pack_bf16x2(__uint_as_float(o[g * 8 + 4]) * inv_l, __uint_as_float(o[g * 8 + 5]) * inv_l);
            u.w = pack_bf16x2(__uint_as_float(o[g * 8 + 6]) * inv_l, __uint_as_float(o[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(o_row + col) = u;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

// =====================================================================================
// Backward
// =====================================================================================
constexpr int BWD_BKV = 128;  // KV rows per CTA
constexpr int BWD_BQ = 64;    // query rows per inner block
constexpr int BWD_DH = 128;   // head dim is padded to 128 inside the kernel
constexpr int BWD_THREADS = 64 + 256;
constexpr int BWD_QSTAGES = 3;

// Two (kv tile, q block) iterations are in flight per CTA: epilogue group 0 (warps 2-5) owns the even iterations,
// group 1 (warps 6-9) the odd ones, each with its own S / dP accumulators in TMEM and its own P^T / dS^T tile in
// shared memory, so the tensor cores work for one group while the other does its exponentials.
// TMEM (512 columns): group g: S^T at g*128 (reused for dQ^T once P^T has been extracted), dP^T at g*128 + 64;
// dV at 256, dK at 384.
struct BwdSmem {
  static constexpr int K_BYTES = BWD_BKV * BWD_DH * 2;   // 32 KB, 2 panels of [128 x 128 B]
  static constexpr int Q_BYTES = BWD_BQ * BWD_DH * 2;    // 16 KB, 2 panels of [64 x 128 B]
  static constexpr int PT_BYTES = BWD_BKV * BWD_BQ * 2;  // 16 KB, 1 panel of [128 x 128 B]
  static constexpr int R_BYTES = 2 * PT_BYTES;           // per group: P^T | dS^T, later the dQ block [64][dh] fp32
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = K_BYTES;
  static constexpr int OFF_Q = 2 * K_BYTES;                       // [BWD_QSTAGES]
  static constexpr int OFF_DO = OFF_Q + BWD_QSTAGES * Q_BYTES;    // [BWD_QSTAGES]
  static constexpr int OFF_R = OFF_DO + BWD_QSTAGES * Q_BYTES;    // [2]
  static constexpr int OFF_STAT = OFF_R + 2 * R_BYTES;            // lse[3][64], delta[3][64] floats
  static constexpr int OFF_BAR = OFF_STAT + 2 * BWD_QSTAGES * 64 * 4;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};
static_assert(BwdSmem::TOTAL <= 232448, "attention backward shared memory budget");
static_assert(BWD_BQ * BWD_DH * 4 <= BwdSmem::R_BYTES, "dQ staging fits the group region");

struct BwdParams {
  const float* lse;
  const float* delta;
  const int* kv_lens;  // optional [b], as in the forward pass
  uint32_t drop_threshold;
  float drop_scale;
  unsigned long long drop_seed;
  int drop_head_offset;
  float* dq_accum;  // fp32 [b, sq, hq, dh] contiguous
  bf16* dk;
  bf16* dv;
  int b, sq, sk, hq, hk, dh;
  long long dk_sb, dk_ss, dk_sh;
  long long dv_sb, dv_ss, dv_sh;
  int causal;
  float scale;
  float scale_log2;
  // BIAS instantiation only (each may be null): transposed bias bf16 [hq, sk, bias_ld], additive mask fp32
  // [mask_n, sq, bias_ld], group ids int32 [mask_n, bias_ld], bias gradient fp32 [hq, sq, bias_ld]
  const bf16* bias_t;
  const float* mask;
  const int* ids;
  float* dbias;
  int mask_n, bias_ld;
};

template <int MODE>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmDQ, BwdParams p) {
  using S = BwdSmem;
  constexpr bool BIAS = MODE == MODE_BIAS, DROP = MODE == MODE_DROP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_lse = reinterpret_cast<float*>(smem + S::OFF_STAT);  // [3][64]
  float* s_delta = s_lse + BWD_QSTAGES * 64;                     // [3][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;    // [3]
  uint64_t* qdo_empty = bars + 4;   // [3]
  uint64_t* stat_full = bars + 7;   // [3]
  // per group g (7 barriers each, starting at 10 + 7 g)
  auto gbar = [&](int g, int which) { return bars + 10 + 7 * g + which; };
  enum { B_S_FULL = 0, B_DP_FULL, B_PT_FULL, B_DS_FULL, B_DQ_FULL, B_S_FREE, B_DP_FREE };
  uint64_t* all_done = bars + 24;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, kv_head = blockIdx.y, batch = blockIdx.z;
  const int kv0 = kv_tile * BWD_BKV;
  const int rep = p.hq / p.hk;
  const int shift = p.sk - p.sq;
  const int sk_eff = p.kv_lens ? max(0, min(p.sk, p.kv_lens[batch])) : p.sk;   // keys that are not padding
  // first query block that can see this KV tile (causal): q + shift >= kv0
  int q_start = 0;
  if (p.causal) q_start = max(0, kv0 - shift) / BWD_BQ;
  const int n_qblocks_total = (p.sq + BWD_BQ - 1) / BWD_BQ;
  // a tile made of padding keys only receives no gradient: no iterations, zeros are written
  const int n_q = kv0 >= sk_eff ? 0 : max(0, n_qblocks_total - q_start);
  const int n_iter = n_q * rep;  // iterations: (head in group, q block)
  const int panels = p.dh <= 64 ? 1 : 2;     // 64-wide head-dim panels that hold data
  const int ksteps = panels * 4;             // 16-wide contraction steps over the head dim (S^T, dP^T)
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t TM_DV = 256, TM_DK = 384;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < BWD_QSTAGES; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
      mbar_init(&stat_full[i], 32);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(gbar(g, B_S_FULL), 1);
      mbar_init(gbar(g, B_DP_FULL), 1);
      mbar_init(gbar(g, B_PT_FULL), 128);
      mbar_init(gbar(g, B_DS_FULL), 128);
      mbar_init(gbar(g, B_DQ_FULL), 1);
      mbar_init(gbar(g, B_S_FREE), 128);
      mbar_init(gbar(g, B_DP_FREE), 128);
    }
    mbar_init(all_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQ);
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
    // ---------------- producer: K, V once; then (Q, dO, lse, delta) per iteration into a 3-deep ring ----------------
    bool ok = true;
    if (lane == 0 && n_iter > 0) {
      // head sizes up to 64 fill one 64-wide panel of every operand: the second panel is neither loaded nor multiplied
      mbar_expect_tx(kv_full, 2 * panels * (BWD_BKV * 128));
      for (int c = 0; c < panels; ++c) {
        tma_load_4d(smem + S::OFF_K + c * (BWD_BKV * 128), &tmK, kv_full, c * 64, kv_head, kv0, batch);
        tma_load_4d(smem + S::OFF_V + c * (BWD_BKV * 128), &tmV, kv_full, c * 64, kv_head, kv0, batch);
      }
    }
    for (int it = 0; it < n_iter && ok; ++it) {
      const int st = it % BWD_QSTAGES, use = it / BWD_QSTAGES;
      const int head = kv_head * rep + it / n_q;
      const int qb = q_start + it % n_q;
      if (!mbar_wait(&qdo_empty[st], (use & 1) ^ 1, abort_flag, 0x21)) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(&qdo_full[st], 2 * panels * (BWD_BQ * 128));
        for (int c = 0; c < panels; ++c) {
          tma_load_4d(smem + S::OFF_Q + st * S::Q_BYTES + c * (BWD_BQ * 128), &tmQ, &qdo_full[st], c * 64, head,
                      qb * BWD_BQ, batch);
          tma_load_4d(smem + S::OFF_DO + st * S::Q_BYTES + c * (BWD_BQ * 128), &tmDO, &qdo_full[st], c * 64, head,
                      qb * BWD_BQ, batch);
        }
      }
      // per-row statistics of the block (plain loads: tiny)
      const long long base = (static_cast<long long>(batch) * p.hq + head) * p.sq + qb * BWD_BQ;
      for (int i = lane; i < BWD_BQ; i += 32) {
        const bool in = qb * BWD_BQ + i < p.sq;
        s_lse[st * 64 + i] = in ? p.lse[base + i] * LOG2E : INFINITY;  // +inf -> P = 0 for padded rows
        s_delta[st * 64 + i] = in ? p.delta[base + i] : 0.f;
      }
      mbar_arrive(&stat_full[st]);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one thread multiplexing the two groups' pipelines ----------------
    if (elect_one()) {
      constexpr uint32_t idesc_st = make_idesc_bf16(BWD_BKV, BWD_BQ, 0, 0);   // S^T, dP^T: A=K/V (K-major), B=Q/dO (K-major)
      // dV, dK: A=P^T/dS^T (K-major), B=dO/Q (MN-major); 64 output columns are enough for head sizes up to 64
      const uint32_t idesc_dv = panels == 1 ? make_idesc_bf16(BWD_BKV, 64, 0, 1) : make_idesc_bf16(BWD_BKV, BWD_DH, 0, 1);
      constexpr uint32_t idesc_dq = make_idesc_bf16(BWD_DH, BWD_BQ, 1, 1);    // dQ^T: A=K (MN-major), B=dS^T (MN-major)
      // Base descriptors, built once (an operand advances by adding (bytes >> 4)): K and V as K-major A operands, K
      // again as the MN-major A operand of dQ^T; Q / dO per ring stage as K-major B (S^T, dP^T) and MN-major B (dK, dV);
      // P^T / dS^T per group as K-major A (dV, dK) and dS^T as MN-major B (dQ^T).
      const uint64_t k_kmaj = make_smem_desc_sw128(smem_u32(smem + S::OFF_K), 0, 1024);
      const uint64_t v_kmaj = make_smem_desc_sw128(smem_u32(smem + S::OFF_V), 0, 1024);
      const uint64_t k_mnmaj = make_smem_desc_sw128(smem_u32(smem + S::OFF_K), BWD_BKV * 128, 1024);
      const uint64_t q_kmaj0 = make_smem_desc_sw128(smem_u32(smem + S::OFF_Q), 0, 1024);
      const uint64_t do_kmaj0 = make_smem_desc_sw128(smem_u32(smem + S::OFF_DO), 0, 1024);
      const uint64_t q_mnmaj0 = make_smem_desc_sw128(smem_u32(smem + S::OFF_Q), BWD_BQ * 128, 1024);
      const uint64_t do_mnmaj0 = make_smem_desc_sw128(smem_u32(smem + S::OFF_DO), BWD_BQ * 128, 1024);
      const uint64_t pt_kmaj0 = make_smem_desc_sw128(smem_u32(smem + S::OFF_R), 0, 1024);
      const uint64_t dst_kmaj0 = make_smem_desc_sw128(smem_u32(smem + S::OFF_R + S::PT_BYTES), 0, 1024);
      const uint64_t dst_mnmaj0 = make_smem_desc_sw128(smem_u32(smem + S::OFF_R + S::PT_BYTES), BWD_BKV * 128, 1024);
      constexpr uint64_t Q_STEP = S::Q_BYTES >> 4, R_STEP = S::R_BYTES >> 4;
      bool dv_started = false, dk_started = false;
      // A(it): S^T = K Q^T and dP^T = V dO^T of iteration `it` into its group's accumulators
      auto issue_a = [&](int it) {
        const int g = it & 1, st = it % BWD_QSTAGES;
        const uint64_t qd = q_kmaj0 + st * Q_STEP, dod = do_kmaj0 + st * Q_STEP;
        const uint32_t d_s = tmem_base + g * 128;
#pragma unroll
        for (int kk = 0; kk < BWD_DH / 16; ++kk) {
          if (kk >= ksteps) break;
          const uint64_t da = k_kmaj + static_cast<uint64_t>(((kk >> 2) * (BWD_BKV * 128) + (kk & 3) * 32) >> 4);
          const uint64_t db = qd + static_cast<uint64_t>(((kk >> 2) * (BWD_BQ * 128) + (kk & 3) * 32) >> 4);
          umma_f16_ss<1>(d_s, da, db, idesc_st, kk != 0 ? 1u : 0u);
        }
        umma_commit<1>(gbar(g, B_S_FULL));
#pragma unroll
        for (int kk = 0; kk < BWD_DH / 16; ++kk) {
          if (kk >= ksteps) break;
          const uint64_t da = v_kmaj + static_cast<uint64_t>(((kk >> 2) * (BWD_BKV * 128) + (kk & 3) * 32) >> 4);
          const uint64_t db = dod + static_cast<uint64_t>(((kk >> 2) * (BWD_BQ * 128) + (kk & 3) * 32) >> 4);
          umma_f16_ss<1>(d_s + 64, da, db, idesc_st, kk != 0 ? 1u : 0u);
        }
        umma_commit<1>(gbar(g, B_DP_FULL));
      };
      // B(it): dV += P^T dO (reduction over the 64 query rows)
      auto issue_b = [&](int it) {
        const int g = it & 1, st = it % BWD_QSTAGES;
        const uint64_t ptd = pt_kmaj0 + g * R_STEP, dod = do_mnmaj0 + st * Q_STEP;
#pragma unroll
        for (int kk = 0; kk < BWD_BQ / 16; ++kk) {
          const uint64_t da = ptd + static_cast<uint64_t>((kk * 32) >> 4);
          const uint64_t db = dod + static_cast<uint64_t>((kk * 2048) >> 4);
          umma_f16_ss<1>(tmem_base + TM_DV, da, db, idesc_dv, (dv_started || kk != 0) ? 1u : 0u);
        }
        dv_started = true;
      };
      // C(it): dK += dS^T Q ; dQ^T = K^T dS^T into the group's S columns (P^T has been extracted by then)
      auto issue_c = [&](int it) {
        const int g = it & 1, st = it % BWD_QSTAGES;
        const uint64_t dsd = dst_kmaj0 + g * R_STEP, dsd_mn = dst_mnmaj0 + g * R_STEP, qd = q_mnmaj0 + st * Q_STEP;
#pragma unroll
        for (int kk = 0; kk < BWD_BQ / 16; ++kk) {
          const uint64_t da = dsd + static_cast<uint64_t>((kk * 32) >> 4);
          const uint64_t db = qd + static_cast<uint64_t>((kk * 2048) >> 4);
          umma_f16_ss<1>(tmem_base + TM_DK, da, db, idesc_dv, (dk_started || kk != 0) ? 1u : 0u);
        }
        dk_started = true;
#pragma unroll
        for (int kk = 0; kk < BWD_BKV / 16; ++kk) {
          // A = K as [M = dh, K = kv]: MN-major, dh panels 128 rows * 128 B apart, 16 kv rows per step;
          // B = dS^T as [N = q, K = kv]: MN-major, a single 64-wide panel
          const uint64_t da = k_mnmaj + static_cast<uint64_t>((kk * 2048) >> 4);
          const uint64_t db = dsd_mn + static_cast<uint64_t>((kk * 2048) >> 4);
          umma_f16_ss<1>(tmem_base + g * 128, da, db, idesc_dq, kk != 0 ? 1u : 0u);
        }
        umma_commit<1>(gbar(g, B_DQ_FULL));
        umma_commit<1>(&qdo_empty[st]);
      };
      bool ok = n_iter == 0 || mbar_wait(kv_full, 0, abort_flag, 0x22);
      // next iteration to issue per kind: A in global order (a ring stage must not be probed two uses ahead),
      // B and C in order within each group
      int next_a = 0, next_b[2] = {0, 1}, next_c[2] = {0, 1};
      uint32_t idle = 0;
      uint64_t t0 = 0;
      while (ok && (next_c[0] < n_iter || next_c[1] < n_iter)) {
        bool progress = false;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          int it = next_c[g];
          if (it < n_iter && next_b[g] > it && mbar_test(gbar(g, B_DS_FULL), (it >> 1) & 1)) {
            tc_fence_after();
            issue_c(it);
            next_c[g] += 2;
            progress = true;
          }
          it = next_b[g];
          if (it < n_iter && next_a > it && mbar_test(gbar(g, B_PT_FULL), (it >> 1) & 1)) {
            tc_fence_after();
            issue_b(it);
            next_b[g] += 2;
            progress = true;
          }
        }
        if (next_a < n_iter) {
          const int it = next_a, g = it & 1, j = it >> 1, st = it % BWD_QSTAGES;
          bool ready = mbar_test(&qdo_full[st], (it / BWD_QSTAGES) & 1);
          if (ready && j > 0)
            ready = mbar_test(gbar(g, B_S_FREE), (j - 1) & 1) && mbar_test(gbar(g, B_DP_FREE), (j - 1) & 1);
          if (ready) {
            tc_fence_after();
            issue_a(it);
            ++next_a;
            progress = true;
          }
        }
        if (progress) {
          idle = 0;
          t0 = 0;
        } else if ((++idle & 0x3ff) == 0) {
          if (*abort_flag) { ok = false; break; }
          const uint64_t now = global_timer_ns();
          if (t0 == 0) {
            t0 = now;
          } else if (now - t0 > GV_WAIT_NS) {
            *abort_flag = 1;
            record_error((0x30u << 16) | 1u, static_cast<unsigned>(next_a), static_cast<unsigned>(next_c[0]));
            ok = false;
            break;
          }
        }
      }
      umma_commit<1>(all_done);
    }
  } else {
    // ---------------- two epilogue groups: thread = one KV row (TMEM lane), all 64 query columns of its block ----------------
    const int g = (warp - 2) >> 2;      // group 0: warps 2-5, group 1: warps 6-9
    const int quarter = warp & 3;       // TMEM lane group
    const int rloc = quarter * 32 + lane;
    const int kvrow = kv0 + rloc;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tm_s = tmem_base + lane_off + g * 128, tm_dp = tm_s + 64;
    uint8_t* region = smem + S::OFF_R + g * S::R_BYTES;
    uint8_t* pt_row = region + rloc * 128;
    uint8_t* dst_row = region + S::PT_BYTES + rloc * 128;
    float* dq_stage = reinterpret_cast<float*>(region);
    const bool issuer = (threadIdx.x == 64 + g * 128);   // first thread of the group issues its dQ bulk reductions
    bool ok = true;
    for (int it = g; it < n_iter; it += 2) {
      const int j = it >> 1, st = it % BWD_QSTAGES;
      const int head = kv_head * rep + it / n_q;
      const int qb = q_start + it % n_q;
      const int qbase = qb * BWD_BQ;
      const uint32_t bh_key = DROP ? drop_key(p.drop_seed, batch, head + p.drop_head_offset) : 0u;
      // `good` stays warp-uniform (voted) so the .sync.aligned TMEM loads never diverge; every barrier of the group is
      // a vote that all 128 threads reach, and the loop is only left right after a vote.
      bool good = mbar_wait(gbar(g, B_S_FULL), j & 1, abort_flag, 0x2b);
      good = good && mbar_wait(&stat_full[st], (it / BWD_QSTAGES) & 1, abort_flag, 0x2a);
      good = good && mbar_wait(gbar(g, B_DP_FULL), j & 1, abort_flag, 0x2d);
      // the group's region still holds the dQ block of its previous iteration until that bulk reduction has read it
      if (issuer) tma_store_wait_read<0>();
      const bool v1 = g == 0 ? named_bar_all<2, 128>(good) : named_bar_all<3, 128>(good);
      if (!v1) { ok = false; break; }
      tc_fence_after();
      const bool boundary = (kv0 + BWD_BKV > sk_eff) || (p.causal && (kv0 + BWD_BKV - 1 > qbase + shift));
      // P^T = exp2(S^T * scale - lse), dS^T = P^T * (dP^T - delta) * scale; S and dP of a 32-column half are loaded
      // together so one TMEM round trip covers both
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(tm_s + h * 32, rs);
        tmem_ld_32x32b_x32(tm_dp + h * 32, rd);
        tmem_ld_wait();
        // per-row statistics of these 32 query columns: the same for every thread -> broadcast 16-byte loads
        const float4* lse4 = reinterpret_cast<const float4*>(s_lse + st * 64 + h * 32);
        const float4* del4 = reinterpret_cast<const float4*>(s_delta + st * 64 + h * 32);
        const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2), ps2 = f2_pack(p.scale, p.scale);
        // BIAS: this thread's key in the bias / mask / gradient matrices and in the group ids, at the 32 query columns of this half
        const int kr = min(kvrow, p.sk - 1);
        const bf16* bt_row = nullptr;
        uint4 bt4[4];
        const int* qid_row = nullptr;
        const float* mask_col = nullptr;     // entry (first query column of this half, this thread's key) of the additive mask
        float* dbias_col = nullptr;          // ... and of the bias gradient; column c of the half is c * bias_ld further
        const int qlim = p.sq - (qbase + h * 32);      // columns of this half that are real queries
        int kid = 0;
        if constexpr (BIAS) {
          if (kvrow < p.sk) {
            const long long col0 = static_cast<long long>(qbase + h * 32) * p.bias_ld + kvrow;
            if (p.mask) mask_col = p.mask + static_cast<long long>(batch % p.mask_n) * p.sq * p.bias_ld + col0;
            if (p.dbias) dbias_col = p.dbias + static_cast<long long>(head) * p.sq * p.bias_ld + col0;
          }
          // this thread's key row of the transposed bias at the 32 query columns of this half: four 16-byte loads up front
          if (p.bias_t) {
            bt_row = p.bias_t + (static_cast<long long>(head) * p.sk + kr) * p.bias_ld + qbase + h * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) bt4[i] = __ldg(reinterpret_cast<const uint4*>(bt_row) + i);
          }
          if (p.ids) {
            const int* idw = p.ids + static_cast<long long>(batch % p.mask_n) * p.bias_ld;
            kid = __ldg(idw + kr);
            qid_row = idw + qbase + h * 32;
          }
        }
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 ls = lse4[c4], dl = del4[c4];
          const uint64_t nl2[2] = {f2_pack(-ls.x, -ls.y), f2_pack(-ls.z, -ls.w)};
          const uint64_t nd2[2] = {f2_pack(-dl.x, -dl.y), f2_pack(-dl.z, -dl.w)};
          float badd[4] = {0.f, 0.f, 0.f, 0.f};
          int qid[4] = {0, 0, 0, 0};
          if constexpr (BIAS) {
            if (bt_row) {
              const uint4 u = bt4[c4 >> 1];
              const float2 f0 = unpack_bf16x2((c4 & 1) ? u.z : u.x), f1 = unpack_bf16x2((c4 & 1) ? u.w : u.y);
              badd[0] = f0.x; badd[1] = f0.y; badd[2] = f1.x; badd[3] = f1.y;
            }
            if (qid_row) {
              const int4 q4 = __ldg(reinterpret_cast<const int4*>(qid_row + c4 * 4));     // the same for every thread
              qid[0] = q4.x; qid[1] = q4.y; qid[2] = q4.z; qid[3] = q4.w;
            }
          }
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = c4 * 4 + 2 * e;
            // P = exp2(S * scale_log2 - lse); dS = P * scale * (dP - delta): packed pairs, two exp2
            float a0, a1;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(rs[c]), __uint_as_float(rs[c + 1])), sc2, nl2[e]), a0, a1);
            if constexpr (BIAS) {
              float add0 = badd[2 * e], add1 = badd[2 * e + 1];
              if (mask_col) {          // general additive mask: entry (q, kvrow); a warp's loads cover one line per column
                add0 += (c < qlim) ? __ldg(mask_col + static_cast<long long>(c) * p.bias_ld) : 0.f;
                add1 += (c + 1 < qlim) ? __ldg(mask_col + static_cast<long long>(c + 1) * p.bias_ld) : 0.f;
              }
              a0 = fmaf(add0, LOG2E, a0);
              a1 = fmaf(add1, LOG2E, a1);
              if (qid_row) {           // keys of another group than the query's carry no probability
                if (qid[2 * e] != kid) a0 = -INFINITY;
                if (qid[2 * e + 1] != kid) a1 = -INFINITY;
              }
            }
            float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
            if (boundary) {
              const int q = qbase + h * 32 + c;
              if (kvrow >= sk_eff || (p.causal && kvrow > q + shift)) p0 = 0.f;
              if (kvrow >= sk_eff || (p.causal && kvrow > q + 1 + shift)) p1 = 0.f;
            }
            const uint64_t p2 = f2_pack(p0, p1);
            float dp0 = __uint_as_float(rd[c]), dp1 = __uint_as_float(rd[c + 1]);
            if constexpr (DROP) {
              // O = (D * P / (1 - p)) V: dV takes the dropped probabilities, dP the dropped upstream gradient
              const int q = qbase + h * 32 + c;
              const bool k0 = drop_keep(bh_key, q, kvrow, p.drop_threshold), k1 = drop_keep(bh_key, q + 1, kvrow, p.drop_threshold);
              dp0 = k0 ? dp0 * p.drop_scale : 0.f;
              dp1 = k1 ? dp1 * p.drop_scale : 0.f;
              p0 = k0 ? p0 * p.drop_scale : 0.f;
              p1 = k1 ? p1 * p.drop_scale : 0.f;
            }
            const uint64_t t2 = f2_add(f2_pack(dp0, dp1), nd2[e]);
            float d0, d1;
            f2_unpack(f2_mul(f2_mul(p2, ps2), t2), d0, d1);
            if constexpr (BIAS) {
              // gradient of the additive term = P * (dP - delta) (dS without the score scale), summed over the batch:
              // consecutive lanes hold consecutive keys, so each atomic add covers one 128-byte line per warp
              if (dbias_col) {
                float g0, g1;
                f2_unpack(f2_mul(p2, t2), g0, g1);
                if (c < qlim) atomicAdd(dbias_col + static_cast<long long>(c) * p.bias_ld, g0);
                if (c + 1 < qlim) atomicAdd(dbias_col + static_cast<long long>(c + 1) * p.bias_ld, g1);
              }
            }
            rs[c] = __float_as_uint(p0); rs[c + 1] = __float_as_uint(p1);
            rd[c] = __float_as_uint(d0); rd[c + 1] = __float_as_uint(d1);
          }
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4 u, w;
          u.x = pack_bf16x2(__uint_as_float(rs[ch * 8 + 0]), __uint_as_float(rs[ch * 8 + 1]));
          u.y = pack_bf16x2(__uint_as_float(rs[ch * 8 + 2]), __uint_as_float(rs[ch * 8 + 3]));
          u.z = pack_bf16x2(__uint_as_float(rs[ch * 8 + 4]), __uint_as_float(rs[ch * 8 + 5]));
          u.w = pack_bf16x2(__uint_as_float(rs[ch * 8 + 6]), __uint_as_float(rs[ch * 8 + 7]));
          w.x = pack_bf16x2(__uint_as_float(rd[ch * 8 + 0]), __uint_as_float(rd[ch * 8 + 1]));
          w.y = pack_bf16x2(__uint_as_float(rd[ch * 8 + 2]), __uint_as_float(rd[ch * 8 + 3]));
          w.z = pack_bf16x2(__uint_as_float(rd[ch * 8 + 4]), __uint_as_float(rd[ch * 8 + 5]));
          w.w = pack_bf16x2(__uint_as_float(rd[ch * 8 + 6]), __uint_as_float(rd[ch * 8 + 7]));
          const int piece = ((h * 4 + ch) ^ (rloc & 7)) << 4;
          *reinterpret_cast<uint4*>(pt_row + piece) = u;
          *reinterpret_cast<uint4*>(dst_row + piece) = w;
        }
      }
      tc_fence_before();
      mbar_arrive(gbar(g, B_DP_FREE));
      fence_async_smem();
      mbar_arrive(gbar(g, B_PT_FULL));
      mbar_arrive(gbar(g, B_DS_FULL));
      // dQ^T [lane = head-dim index, columns = query rows] comes back in the S columns once dK / dQ MMAs are done; by
      // then nothing reads P^T / dS^T any more, so the region is reused to stage the block as [query row][head dim] fp32,
      // which ONE bulk tensor reduction adds into dq_accum (the adds happen at L2).
      good = mbar_wait(gbar(g, B_DQ_FULL), j & 1, abort_flag, 0x2e);
      const bool v2 = g == 0 ? named_bar_all<2, 128>(good) : named_bar_all<3, 128>(good);
      if (!v2) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32b_x32(tm_s, r0);
        tmem_ld_32x32b_x32(tm_s + 32, r1);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(gbar(g, B_S_FREE));
        if (rloc < p.dh) {
          float* dst = dq_stage + rloc;
#pragma unroll
          for (int c = 0; c < 32; ++c) dst[c * p.dh] = __uint_as_float(r0[c]);
#pragma unroll
          for (int c = 0; c < 32; ++c) dst[(32 + c) * p.dh] = __uint_as_float(r1[c]);
        }
      }
      fence_async_smem();
      if (g == 0) named_bar_sync<2, 128>(); else named_bar_sync<3, 128>();
      if (issuer) {
        tma_reduce_add_4d(&tmDQ, dq_stage, 0, head, qbase, batch);
        tma_store_commit();
      }
    }
    if (issuer) tma_store_wait<0>();                  // every reduction of this group has been performed
    // final: dK, dV from TMEM (group g takes 64 of the 128 head-dim columns)
    if (ok && n_iter > 0) ok = mbar_wait(all_done, 0, abort_flag, 0x2f);
    tc_fence_after();
    if (ok) {
      bf16* dk_row = p.dk + batch * p.dk_sb + static_cast<long long>(kvrow) * p.dk_ss + kv_head * p.dk_sh;
      bf16* dv_row = p.dv + batch * p.dv_sb + static_cast<long long>(kvrow) * p.dv_ss + kv_head * p.dv_sh;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        const int colbase = g * 64 + c * 32;
        uint32_t a[32], bq[32];
        __syncwarp();
        if (n_iter > 0) {
          tmem_ld_32x32b_x32(tmem_base + lane_off + TM_DK + colbase, a);
          tmem_ld_32x32b_x32(tmem_base + lane_off + TM_DV + colbase, bq);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { a[i] = 0u; bq[i] = 0u; }
        }
        if (kvrow < p.sk) {
#pragma unroll
          for (int gg = 0; gg < 4; ++gg) {
            const int col = colbase + gg * 8;
            if (col < p.dh) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(a[gg * 8 + 0]), __uint_as_float(a[gg * 8 + 1]));
              u.y = pack_bf16x2(__uint_as_float(a[gg * 8 + 2]), __uint_as_float(a[gg * 8 + 3]));
              u.z = pack_bf16x2(__uint_as_float(a[gg * 8 + 4]), __uint_as_float(a[gg * 8 + 5]));
              u.w = pack_bf16x2(__uint_as_float(a[gg * 8 + 6]), __uint_as_float(a[gg * 8 + 7]));
              *reinterpret_cast<uint4*>(dk_row + col) = u;
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(bq[gg * 8 + 0]), __uint_as_float(bq[gg * 8 + 1]));
              w.y = pack_bf16x2(__uint_as_float(bq[gg * 8 + 2]), __uint_as_float(bq[gg * 8 + 3]));
              w.z = pack_bf16x2(__uint_as_float(bq[gg * 8 + 4]), __uint_as_float(bq[gg * 8 + 5]));
              w.w = pack_bf16x2(__uint_as_float(bq[gg * 8 + 6]), __uint_as_float(bq[gg * 8 + 7]));
              *reinterpret_cast<uint4*>(dv_row + col) = w;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

// delta[b, h, s] = sum_d dO * O: LPR lanes per row (8 head-dim elements per lane and pass), 32 / LPR rows per warp
template <int LPR>
__global__ void attn_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout, float* __restrict__ delta,
                                  int b, int sq, int hq, int dh, long long o_sb, long long o_ss, long long o_sh,
                                  long long do_sb, long long do_ss, long long do_sh) {
  const long long total = static_cast<long long>(b) * hq * sq;
  const int sub = threadIdx.x % LPR;
  // whole warps stay in the loop together (the shuffles below are warp-wide): rows are padded up to a multiple of 32 / LPR
  const long long rows_padded = (total + (32 / LPR) - 1) / (32 / LPR) * (32 / LPR);
  for (long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) / LPR; row < rows_padded;
       row += (static_cast<long long>(gridDim.x) * blockDim.x) / LPR) {
    float acc = 0.f;
    if (row < total) {
      const int s = static_cast<int>(row % sq);
      const int h = static_cast<int>((row / sq) % hq);
      const int bb = static_cast<int>(row / (static_cast<long long>(sq) * hq));
      const bf16* op = o + bb * o_sb + s * o_ss + h * o_sh;
      const bf16* dp = dout + bb * do_sb + s * do_ss + h * do_sh;
      for (int i = sub * 8; i < dh; i += LPR * 8) {
        uint4 a = *reinterpret_cast<const uint4*>(op + i);
        uint4 d = *reinterpret_cast<const uint4*>(dp + i);
        float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
        float2 d0 = unpack_bf16x2(d.x), d1 = unpack_bf16x2(d.y), d2 = unpack_bf16x2(d.z), d3 = unpack_bf16x2(d.w);
        acc += a0.x * d0.x + a0.y * d0.y + a1.x * d1.x + a1.y * d1.y + a2.x * d2.x + a2.y * d2.y + a3.x * d3.x + a3.y * d3.y;
      }
    }
#pragma unroll
    for (int o2 = LPR / 2; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
    if (sub == 0 && row < total) delta[row] = acc;
  }
}

// dq (bf16, strided) = dq_accum (fp32 [b, sq, hq, dh])
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, int b, int sq, int hq,
                                       int dh, long long sb, long long ss, long long sh) {
  const int vec = dh >> 3;
  const long long total = static_cast<long long>(b) * sq * hq * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vec);
    const long long row = i / vec;  // (b, s, h)
    const int h = static_cast<int>(row % hq);
    const int s = static_cast<int>((row / hq) % sq);
    const int bb = static_cast<int>(row / (static_cast<long long>(hq) * sq));
    const float4 x = *reinterpret_cast<const float4*>(acc + row * dh + v * 8);
    const float4 y = *reinterpret_cast<const float4*>(acc + row * dh + v * 8 + 4);
    uint4 u;
    u.x = pack_bf16x2(x.x, x.y); u.y = pack_bf16x2(x.z, x.w);
    u.z = pack_bf16x2(y.x, y.y); u.w = pack_bf16x2(y.z, y.w);
    *reinterpret_cast<uint4*>(dq + bb * sb + s * ss + h * sh + v * 8) = u;
  }
}

// dq (bf16, strided) = R^T(dq_accum): the fp32 -> bf16 conversion with the inverse rotary rotation of the query
// gradient folded in (the forward pass rotated q; the gradient w.r.t. the un-rotated projection is the transposed
// rotation of dq). One thread converts 8 columns of the first half of a head and their partners in the second half.
__global__ void attn_dq_convert_rope_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, int b, int sq, int hq,
                                            int dh, long long sb, long long ss, long long sh,
                                            const float* __restrict__ inv_freq, const int* __restrict__ pos, int pos_offset) {
  const int half = dh >> 1;
  const int vec = half >> 3;
  const long long total = static_cast<long long>(b) * sq * hq * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vec);
    const long long row = i / vec;  // (b, s, h)
    const int h = static_cast<int>(row % hq);
    const int s = static_cast<int>((row / hq) % sq);
    const int bb = static_cast<int>(row / (static_cast<long long>(hq) * sq));
    const float p = pos ? static_cast<float>(pos[static_cast<long long>(s) * b + bb]) : static_cast<float>(s + pos_offset);
    const float* src = acc + row * dh + v * 8;
    float x1[8], x2[8], o1[8], o2[8];
    *reinterpret_cast<float4*>(x1) = *reinterpret_cast<const float4*>(src);
    *reinterpret_cast<float4*>(x1 + 4) = *reinterpret_cast<const float4*>(src + 4);
    *reinterpret_cast<float4*>(x2) = *reinterpret_cast<const float4*>(src + half);
    *reinterpret_cast<float4*>(x2 + 4) = *reinterpret_cast<const float4*>(src + half + 4);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float sn, cs;
      sincosf(p * __ldg(inv_freq + v * 8 + e), &sn, &cs);
      o1[e] = x1[e] * cs + x2[e] * sn;      // transposed rotation: sin -> -sin
      o2[e] = x2[e] * cs - x1[e] * sn;
    }
    uint4 u, w;
    u.x = pack_bf16x2(o1[0], o1[1]); u.y = pack_bf16x2(o1[2], o1[3]); u.z = pack_bf16x2(o1[4], o1[5]); u.w = pack_bf16x2(o1[6], o1[7]);
    w.x = pack_bf16x2(o2[0], o2[1]); w.y = pack_bf16x2(o2[2], o2[3]); w.z = pack_bf16x2(o2[4], o2[5]); w.w = pack_bf16x2(o2[6], o2[7]);
    bf16* dst = dq + bb * sb + s * ss + h * sh + v * 8;
    *reinterpret_cast<uint4*>(dst) = u;
    *reinterpret_cast<uint4*>(dst + half) = w;
  }
}

template <class P>
static void fill_dropout(P& p, const gv_attn_args* a) {
  const float dp = a->dropout_p;
  if (dp > 0.f && dp < 1.f) {
    const double t = static_cast<double>(dp) * 4294967296.0;
    p.drop_threshold = t >= 4294967295.0 ? 4294967295u : static_cast<uint32_t>(t);
    if (p.drop_threshold == 0) p.drop_threshold = 1;
    p.drop_scale = 1.f / (1.f - dp);
  } else {
    p.drop_threshold = 0;
    p.drop_scale = 1.f;
  }
  p.drop_seed = a->dropout_seed;
  p.drop_head_offset = a->dropout_head_offset;
}

static int check_attn(const gv_attn_args* a) {
  if (a->dh % 8 != 0 || a->dh > 128 || a->dh <= 0) return 2301;
  if (a->hq <= 0 || a->hk <= 0 || a->hq % a->hk != 0) return 2302;
  if (a->causal && a->sq > a->sk) return 2303;
  const long long strides[] = {a->q_stride_b, a->q_stride_s, a->q_stride_h, a->k_stride_b, a->k_stride_s,
                               a->k_stride_h, a->v_stride_b, a->v_stride_s, a->v_stride_h, a->o_stride_b,
                               a->o_stride_s, a->o_stride_h};
  for (long long s : strides)
    if (s % 8 != 0) return 2304;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
       reinterpret_cast<uintptr_t>(a->o)) & 15)
    return 2305;
  return 0;
}

static bool has_additive(const gv_attn_args* a) { return a->bias != nullptr || a->mask != nullptr || a->ids != nullptr; }

// bias / mask / group ids: row stride a multiple of 64 that covers both sequence lengths, 16-byte aligned bases
static int check_bias(const gv_attn_args* a, bool backward) {
  if (a->bias_ld < a->sk || a->bias_ld < a->sq || a->bias_ld % 64 != 0) return 2310;
  if ((reinterpret_cast<uintptr_t>(a->bias) | reinterpret_cast<uintptr_t>(a->bias_t) | reinterpret_cast<uintptr_t>(a->mask) |
       reinterpret_cast<uintptr_t>(a->ids) | reinterpret_cast<uintptr_t>(a->dbias)) & 15)
    return 2311;
  if ((a->mask != nullptr || a->ids != nullptr) && a->mask_n <= 0) return 2312;
  if (a->dropout_p > 0.f || a->causal) return 2313;     // not combined with dropout of the probabilities or the causal mask
  if (a->ids != nullptr && a->sq != a->sk) return 2315;
  if (backward && a->bias != nullptr && a->bias_t == nullptr) return 2316;
  if (a->dbias != nullptr && a->bias == nullptr) return 2314;
  return 0;
}

template <int DH, int MODE>
static int launch_fwd(const gv_attn_args* a, cudaStream_t stream) {
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_bshd(&tmQ, a->q, a->b, a->sq, a->hq, a->dh, a->q_stride_b, a->q_stride_s, a->q_stride_h, FWD_BM);
  if (rc) return rc;
  rc = make_tmap_bshd(&tmK, a->k, a->b, a->sk, a->hk, a->dh, a->k_stride_b, a->k_stride_s, a->k_stride_h, FWD_BN);
  if (rc) return rc;
  rc = make_tmap_bshd(&tmV, a->v, a->b, a->sk, a->hk, a->dh, a->v_stride_b, a->v_stride_s, a->v_stride_h, FWD_BN);
  if (rc) return rc;
  FwdParams p;
  p.o = reinterpret_cast<bf16*>(a->o);
  p.lse = a->lse;
  p.b = a->b; p.sq = a->sq; p.sk = a->sk; p.hq = a->hq; p.hk = a->hk; p.dh = a->dh;
  p.o_sb = a->o_stride_b; p.o_ss = a->o_stride_s; p.o_sh = a->o_stride_h;
  p.causal = a->causal;
  p.scale_log2 = a->scale * LOG2E;
  p.kv_lens = a->kv_lens;
  p.bias = reinterpret_cast<const bf16*>(a->bias); p.mask = a->mask; p.ids = a->ids;
  p.mask_n = a->mask_n > 0 ? a->mask_n : 1; p.bias_ld = a->bias_ld;
  fill_dropout(p, a);
  auto kern = attn_fwd_kernel<DH, MODE>;
  constexpr int smem = FwdSmem<DH>::TOTAL;
  static PerDeviceOnce smem_once;
  {
    cudaError_t e = ensure_max_dynamic_smem(smem_once, kern, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid((a->sq + FWD_BM - 1) / FWD_BM, a->hq, a->b);
  kern<<<grid, FWD_THREADS, smem, stream>>>(tmQ, tmK, tmV, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gv

GV_DEFINE_ERROR_READER(gv_read_error_attn)

extern "C" int gv_attn_fwd(const gv_attn_args* a, gv_stream_t s) {
  using namespace gv;
  if (a->b <= 0 || a->sq <= 0 || a->sk <= 0) return 0;
  int rc = check_attn(a);
  if (rc) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(s);
  if (has_additive(a)) {
    rc = check_bias(a, false);
    if (rc) return rc;
    return a->dh <= 64 ? launch_fwd<64, MODE_BIAS>(a, stream) : launch_fwd<128, MODE_BIAS>(a, stream);
  }
  if (a->dropout_p > 0.f && a->dropout_p < 1.f)
    return a->dh <= 64 ? launch_fwd<64, MODE_DROP>(a, stream) : launch_fwd<128, MODE_DROP>(a, stream);
  return a->dh <= 64 ? launch_fwd<64, MODE_PLAIN>(a, stream) : launch_fwd<128, MODE_PLAIN>(a, stream);
}

extern "C" int gv_attn_bwd(const gv_attn_args* a, gv_stream_t s) {
  using namespace gv;
  if (a->b <= 0 || a->sq <= 0 || a->sk <= 0) return 0;
  int rc = check_attn(a);
  if (rc) return rc;
  const long long strides[] = {a->do_stride_b, a->do_stride_s, a->do_stride_h, a->dq_stride_b, a->dq_stride_s,
                               a->dq_stride_h, a->dk_stride_b, a->dk_stride_s, a->dk_stride_h, a->dv_stride_b,
                               a->dv_stride_s, a->dv_stride_h};
  for (long long st : strides)
    if (st % 8 != 0) return 2306;
  if (has_additive(a)) {
    rc = check_bias(a, true);
    if (rc) return rc;
  } else if (a->dbias != nullptr) {
    return 2314;                                  // a bias gradient without a bias
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(s);
  // delta = rowsum(dO * O); dq_accum = 0
  {
    const long long rows = static_cast<long long>(a->b) * a->hq * a->sq;
    const int lpr = a->dh <= 32 ? 4 : (a->dh <= 64 ? 8 : 16);
    long long blocks = (rows * lpr + 255) / 256;
    const long long cap = static_cast<long long>(num_sms()) * 8;
    if (blocks > cap) blocks = cap;
    auto delta_kern = lpr == 4 ? attn_delta_kernel<4> : (lpr == 8 ? attn_delta_kernel<8> : attn_delta_kernel<16>);
    delta_kern<<<static_cast<int>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const bf16*>(a->o), reinterpret_cast<const bf16*>(a->dout), a->delta, a->b, a->sq, a->hq,
        a->dh, a->o_stride_b, a->o_stride_s, a->o_stride_h, a->do_stride_b, a->do_stride_s, a->do_stride_h);
    cudaError_t e = cudaMemsetAsync(a->dq_accum, 0, sizeof(float) * static_cast<size_t>(a->b) * a->sq * a->hq * a->dh,
                                    stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  CUtensorMap tmQ, tmK, tmV, tmDO;
  rc = make_tmap_bshd(&tmQ, a->q, a->b, a->sq, a->hq, a->dh, a->q_stride_b, a->q_stride_s, a->q_stride_h, BWD_BQ);
  if (rc) return rc;
  rc = make_tmap_bshd(&tmDO, a->dout, a->b, a->sq, a->hq, a->dh, a->do_stride_b, a->do_stride_s, a->do_stride_h, BWD_BQ);
  if (rc) return rc;
  rc = make_tmap_bshd(&tmK, a->k, a->b, a->sk, a->hk, a->dh, a->k_stride_b, a->k_stride_s, a->k_stride_h, BWD_BKV);
  if (rc) return rc;
  rc = make_tmap_bshd(&tmV, a->v, a->b, a->sk, a->hk, a->dh, a->v_stride_b, a->v_stride_s, a->v_stride_h, BWD_BKV);
  if (rc) return rc;
  CUtensorMap tmDQ;
  {
    // fp32 accumulator [b, sq, hq, dh] contiguous; one reduction covers 64 query rows of one head
    EncodeTiledFn fn = attn_encode_fn();
    if (fn == nullptr) return 1001;
    if (reinterpret_cast<uintptr_t>(a->dq_accum) & 15) return 2307;
    cuuint64_t dims[4] = {(cuuint64_t)a->dh, (cuuint64_t)a->hq, (cuuint64_t)a->sq, (cuuint64_t)a->b};
    cuuint64_t strides[3] = {(cuuint64_t)a->dh * 4, (cuuint64_t)a->hq * a->dh * 4, (cuuint64_t)a->sq * a->hq * a->dh * 4};
    cuuint32_t box[4] = {(cuuint32_t)a->dh, 1, (cuuint32_t)BWD_BQ, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(&tmDQ, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a->dq_accum, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_ERROR_INVALID_CONTEXT) {   // see make_tmap_bshd
      bind_context_of(a->dq_accum);
      r = fn(&tmDQ, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a->dq_accum, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return 1000 + static_cast<int>(r);
  }
  BwdParams p;
  p.lse = a->lse; p.delta = a->delta; p.dq_accum = a->dq_accum;
  p.dk = reinterpret_cast<bf16*>(a->dk); p.dv = reinterpret_cast<bf16*>(a->dv);
  p.b = a->b; p.sq = a->sq; p.sk = a->sk; p.hq = a->hq; p.hk = a->hk; p.dh = a->dh;
  p.dk_sb = a->dk_stride_b; p.dk_ss = a->dk_stride_s; p.dk_sh = a->dk_stride_h;
  p.dv_sb = a->dv_stride_b; p.dv_ss = a->dv_stride_s; p.dv_sh = a->dv_stride_h;
  p.causal = a->causal; p.scale = a->scale; p.scale_log2 = a->scale * LOG2E;
  p.kv_lens = a->kv_lens;
  p.bias_t = reinterpret_cast<const bf16*>(a->bias_t); p.mask = a->mask; p.ids = a->ids; p.dbias = a->dbias;
  p.mask_n = a->mask_n > 0 ? a->mask_n : 1; p.bias_ld = a->bias_ld;
  fill_dropout(p, a);
  dim3 grid((a->sk + BWD_BKV - 1) / BWD_BKV, a->hk, a->b);
  auto launch = [&](auto kern, PerDeviceOnce& once) -> cudaError_t {
    cudaError_t e = ensure_max_dynamic_smem(once, kern, BwdSmem::TOTAL);
    if (e != cudaSuccess) return e;
    kern<<<grid, BWD_THREADS, BwdSmem::TOTAL, stream>>>(tmQ, tmK, tmV, tmDO, tmDQ, p);
    return cudaSuccess;
  };
  static PerDeviceOnce once_plain, once_bias, once_drop;
  cudaError_t le;
  if (has_additive(a)) le = launch(attn_bwd_kernel<MODE_BIAS>, once_bias);
  else if (p.drop_threshold != 0) le = launch(attn_bwd_kernel<MODE_DROP>, once_drop);
  else le = launch(attn_bwd_kernel<MODE_PLAIN>, once_plain);
  if (le != cudaSuccess) return static_cast<int>(le);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  {
    const long long total = static_cast<long long>(a->b) * a->sq * a->hq * (a->dh / 8);
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(num_sms()) * 8;
    if (blocks > cap) blocks = cap;
    if (a->dq_rope_inv_freq != nullptr && a->dh % 16 == 0)
      attn_dq_convert_rope_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
          a->dq_accum, reinterpret_cast<bf16*>(a->dq), a->b, a->sq, a->hq, a->dh, a->dq_stride_b, a->dq_stride_s,
          a->dq_stride_h, a->dq_rope_inv_freq, a->dq_rope_pos, a->dq_rope_pos_offset);
    else
      attn_dq_convert_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
          a->dq_accum, reinterpret_cast<bf16*>(a->dq), a->b, a->sq, a->hq, a->dh, a->dq_stride_b, a->dq_stride_s,
          a->dq_stride_h);
  }
  return static_cast<int>(cudaGetLastError());
}
