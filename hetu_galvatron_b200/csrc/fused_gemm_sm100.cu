// GEMM fused with the collective that precedes or follows it, over NVSwitch peer memory.
//
//   all-gather -> GEMM   (Megatron-SP column-parallel forward; reference: AG at megatron/core/tensor_parallel/
//                         layers.py:399-413 followed by torch.matmul :417): the A operand's row blocks are TMA-loaded
//                         (no multicast) straight from the peer that owns them, own block first, each peer's block
//                         only after that peer has announced it.
//   GEMM -> reduce-scatter (row-parallel forward and column-parallel input gradient; reference layers.py:1092-1109,
//                         :462-494): the epilogue stores every output tile into the workspace of the rank that owns
//                         those rows, into the slot of the producing rank; gv_reduce_slots on the owner finishes.
//   Ulysses: projection -> sequence/head exchange (epilogue stores each 32-column chunk to the rank that owns that
//                         head group; reference transformer.py:731-866,1928-1987) and head/sequence exchange ->
//                         output projection (A operand K-slices TMA-loaded from the peers that computed those heads;
//                         reference transformer.py:2163-2173,898).
// The transfers ride inside the GEMM's own load / store pipeline, tile by tile, so they overlap the tensor-core
// work. Same kernel skeleton as csrc/gemm_sm100.cu: 6 warps, 128x256x64 tiles, 4-stage TMA ring, tcgen05.mma into
// double-buffered TMEM accumulators.
#include "include/gv_kernels.h"
#include "include/gv_comm.cuh"

namespace gv {

int num_sms();
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                      uint32_t box_rows);

constexpr int FBM = 128, FBN = 256, FBK = 64, FSTAGES = 4, FTHREADS = 192, FGROUP_M = 8;
constexpr int FA_BYTES = FBM * FBK * 2, FB_BYTES = FBN * FBK * 2, FSTAGE_BYTES = FA_BYTES + FB_BYTES;
constexpr int FBAR_OFFSET = FSTAGES * FSTAGE_BYTES;
constexpr int FSMEM_TOTAL = FBAR_OFFSET + 256 + 1024;

struct TmapArray {
  CUtensorMap m[GV_MAX_RANKS];
};

struct FusedDev {
  PeerTable pt;
  void* C;
  const __nv_bfloat16* bias;
  const int* col_map;        // c_mode 2: per 32-column chunk, (dest_rank << 24) | dest_col
  int M, N, K, ldc;
  int a_mode, c_mode;
  long long c_off;
  int dest_cols;             // c_mode 2: row length of the destination buffer
  int slot_in;
  uint32_t epoch;
};

__device__ __forceinline__ void ftile_coords(int tile, int num_m, int num_n, int& tm, int& tn) {
  const int span = FGROUP_M * num_n;
  const int group = tile / span;
  const int first = group * FGROUP_M;
  const int gsize = min(num_m - first, FGROUP_M);
  const int in_group = tile - group * span;
  tm = first + in_group % gsize;
  tn = in_group / gsize;
}

template <bool B_MN>
__global__ void __launch_bounds__(FTHREADS, 1)
fused_gemm_kernel(const __grid_constant__ TmapArray tmA, const __grid_constant__ CUtensorMap tmB, FusedDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + FBAR_OFFSET);
  uint64_t* empty_bar = full_bar + FSTAGES;
  uint64_t* acc_full = empty_bar + FSTAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + FBM - 1) / FBM, num_n = (p.N + FBN - 1) / FBN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + FBK - 1) / FBK;
  const int world = p.pt.world, rank = p.pt.rank;
  // a_mode 1: M row tiles per source rank; a_mode 2: K blocks per source rank
  const int m_tiles_per_src = p.a_mode == 1 ? num_m / world : num_m;
  const int kb_per_src = p.a_mode == 2 ? num_kb / world : num_kb;
  constexpr uint32_t TMEM_COLS = 2 * FBN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < FSTAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
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

  // Row-tile rotation: every rank starts with the tiles whose A rows it owns (a_mode 1).
  // With a scattered output (c_mode 1) every rank starts on a different owner so no owner's ingress is a hot spot.
  const int rot = p.a_mode == 1 ? rank * m_tiles_per_src
                  : (p.c_mode == 1 && num_m % world == 0) ? ((rank + 1) % world) * (num_m / world) : 0;
  auto rotate_m = [&](int tm) { return rot ? (tm + rot) % num_m : tm; };

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t ready_mask = (p.a_mode == 0) ? 0xffu : (1u << rank);   // own data needs no flag
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        ftile_coords(tile, num_m, num_n, tm, tn);
        tm = rotate_m(tm);
        const int m0 = tm * FBM, n0 = tn * FBN;
        for (int kbi = 0; kbi < num_kb && ok; ++kbi) {
          const int kb = p.a_mode == 2 ? (kbi + rank * kb_per_src) % num_kb : kbi;
          int src = rank;
          if (p.a_mode == 1) src = tm / m_tiles_per_src;
          if (p.a_mode == 2) src = kb / kb_per_src;
          if (!((ready_mask >> src) & 1u)) {
            if (!wait_flag(p.pt, p.slot_in, src, p.epoch, 0x41)) { *abort_flag = 1; ok = false; break; }
            ready_mask |= 1u << src;
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, 0x42)) { ok = false; break; }
          uint8_t* sA = smem + stage * FSTAGE_BYTES;
          uint8_t* sB = sA + FA_BYTES;
          mbar_expect_tx(&full_bar[stage], FSTAGE_BYTES);
          if (p.a_mode == 0) {
            tma_load_2d(sA, &tmA.m[0], &full_bar[stage], kb * FBK, m0);
          } else if (p.a_mode == 1) {
            tma_load_2d(sA, &tmA.m[src], &full_bar[stage], kb * FBK, m0 - src * m_tiles_per_src * FBM);
          } else {
            tma_load_2d(sA, &tmA.m[src], &full_bar[stage], (kb - src * kb_per_src) * FBK, rank * p.M + m0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sB, &tmB, &full_bar[stage], kb * FBK, n0);
          } else {
#pragma unroll
            for (int q = 0; q < FBN / 64; ++q) tma_load_2d(sB + q * (FBK * 128), &tmB, &full_bar[stage], n0 + q * 64, kb * FBK);
          }
          if (++stage == FSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(FBM, FBN, 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, 0x43)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * FBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, 0x44)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * FSTAGE_BYTES);
          const uint32_t b_addr = a_addr + FA_BYTES;
#pragma unroll
          for (int k = 0; k < FBK / 16; ++k) {
            const uint64_t da = make_smem_desc_sw128(a_addr + k * 32, 0, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_addr + k * 2048, FBK * 128, 1024)
                                     : make_smem_desc_sw128(b_addr + k * 32, 0, 1024);
            umma_f16_ss<1>(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit<1>(&empty_bar[stage]);
          if (++stage == FSTAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit<1>(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const int rows_per = p.c_mode == 1 ? p.M / world : p.M;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      ftile_coords(tile, num_m, num_n, tm, tn);
      tm = rotate_m(tm);
      const int row = tm * FBM + quarter * 32 + lane;
      const int n0 = tn * FBN;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, 0x45)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * FBN + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool row_ok = row < p.M;
      // destination row base for this thread's row
      __nv_bfloat16* row_base = nullptr;
      if (row_ok) {
        if (p.c_mode == 0) {
          row_base = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc;
        } else if (p.c_mode == 1) {
          const int owner = row / rows_per;
          char* ws = reinterpret_cast<char*>(p.pt.base[owner]) + p.c_off;
          row_base = reinterpret_cast<__nv_bfloat16*>(ws) +
                     (static_cast<size_t>(rank) * rows_per + (row - owner * rows_per)) * p.N;
        }
      }
#pragma unroll 1
      for (int c = 0; c < FBN / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row_ok && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          const bool full = col0 + 32 <= p.N;
          if (p.bias != nullptr && full) {
            const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 b = __ldg(bp + j);
              float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
              v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
              v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
            }
          }
          __nv_bfloat16* dst;
          if (p.c_mode == 2) {
            const int e = p.col_map[col0 >> 5];
            char* ws = reinterpret_cast<char*>(p.pt.base[e >> 24]) + p.c_off;
            dst = reinterpret_cast<__nv_bfloat16*>(ws) + (static_cast<size_t>(rank) * p.M + row) * p.dest_cols + (e & 0xffffff);
          } else {
            dst = row_base + col0;
          }
          if (full) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
              o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
              o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
              o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
              d4[j] = o;
            }
          } else {
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) dst[i] = __float2bfloat16(v[i] + (p.bias ? __bfloat162float(p.bias[col0 + i]) : 0.f));
          }
        }
      }
      __syncwarp();
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    __threadfence_system();   // peer stores of this thread are performed before the kernel ends
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

__global__ void fused_signal_kernel(PeerTable pt, int slot, uint32_t epoch) {
  if (threadIdx.x == 0) signal_all(pt, slot, epoch);
}

template <bool B_MN>
static int launch_fused(const gv_peers* peers, const gv_fused_gemm_args* a, const int* col_map, int dest_cols, cudaStream_t stream) {
  const int world = peers->world, rank = peers->rank;
  TmapArray tmA;
  CUtensorMap tmB;
  int rc = 0;
  if (a->a_mode == 0) {
    rc = make_tmap_bf16_2d(&tmA.m[0], a->A, a->M, a->K, a->lda, 64, FBM);
    for (int r = 1; r < GV_MAX_RANKS; ++r) tmA.m[r] = tmA.m[0];
  } else if (a->a_mode == 1) {
    const int rows_per = a->M / world;
    for (int r = 0; r < GV_MAX_RANKS && !rc; ++r) {
      const int rr = r < world ? r : 0;
      rc = make_tmap_bf16_2d(&tmA.m[r], reinterpret_cast<const char*>(peers->bases[rr]) + a->a_off, rows_per, a->K, a->K, 64, FBM);
    }
  } else {
    const int k_per = a->K / world;
    for (int r = 0; r < GV_MAX_RANKS && !rc; ++r) {
      const int rr = r < world ? r : 0;
      rc = make_tmap_bf16_2d(&tmA.m[r], reinterpret_cast<const char*>(peers->bases[rr]) + a->a_off,
                             static_cast<uint64_t>(a->M) * world, k_per, k_per, 64, FBM);
    }
  }
  if (rc) return rc;
  if (!B_MN)
    rc = make_tmap_bf16_2d(&tmB, a->B, a->N, a->K, a->ldb, 64, FBN);
  else
    rc = make_tmap_bf16_2d(&tmB, a->B, a->K, a->N, a->ldb, 64, FBK);
  if (rc) return rc;
  FusedDev p;
  for (int i = 0; i < GV_MAX_RANKS; ++i) p.pt.base[i] = i < world ? peers->bases[i] : nullptr;
  p.pt.world = world;
  p.pt.rank = rank;
  p.C = a->C;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  p.col_map = col_map;
  p.M = a->M; p.N = a->N; p.K = a->K; p.ldc = a->ldc;
  p.a_mode = a->a_mode; p.c_mode = a->c_mode;
  p.c_off = a->c_off;
  p.dest_cols = dest_cols;
  p.slot_in = a->slot_in;
  p.epoch = a->epoch;
  auto kern = fused_gemm_kernel<B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FSMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
  }
  const int tiles = ((a->M + FBM - 1) / FBM) * ((a->N + FBN - 1) / FBN);
  const int grid = tiles < num_sms() ? tiles : num_sms();
  kern<<<grid, FTHREADS, FSMEM_TOTAL, stream>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (a->c_mode != 0 && a->slot_out >= 0) {
    fused_signal_kernel<<<1, 32, 0, stream>>>(p.pt, a->slot_out, a->epoch);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

}  // namespace gv

GV_DEFINE_ERROR_READER(gv_read_error_fgemm)

// b_mn_major != 0: B stored [K, N] (the weight of a linear layer used for its input gradient).
// col_map / dest_cols are only read for c_mode 2.
extern "C" int gv_fused_gemm_ex(const gv_peers* peers, const gv_fused_gemm_args* a, int b_mn_major, const int* col_map,
                                int dest_cols, gv_stream_t s) {
  using namespace gv;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
  const int world = peers->world;
  if (world < 1 || world > GV_MAX_RANKS) return 2601;
  if ((a->K % 8) || (a->ldb % 8) || (a->c_mode == 0 && (a->ldc % 8))) return 2602;
  if (a->a_mode == 1 && ((a->M % world) || ((a->M / world) % FBM))) return 2603;
  if (a->a_mode == 2 && ((a->K % world) || ((a->K / world) % FBK))) return 2604;
  if (a->c_mode == 1 && ((a->M % world) || (a->N % 8))) return 2605;
  if (a->c_mode == 2 && (col_map == nullptr || (a->N % 32) || (dest_cols % 8))) return 2606;
  if ((a->a_off % 16) || (a->c_off % 16)) return 2607;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(s);
  return b_mn_major ? launch_fused<true>(peers, a, col_map, dest_cols, stream)
                    : launch_fused<false>(peers, a, col_map, dest_cols, stream);
}

extern "C" int gv_fused_gemm(const gv_peers* peers, const gv_fused_gemm_args* a, gv_stream_t s) {
  return gv_fused_gemm_ex(peers, a, 0, nullptr, 0, s);
}
