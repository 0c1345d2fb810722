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
// work. Kernel skeleton of csrc/gemm_sm100.cu (128x256x64 tiles, 4-stage TMA ring, tcgen05.mma into double-buffered
// TMEM accumulators) with two additions:
//   * warps 6-9 are copy warps: for all-gather -> GEMM they pull every remote row block over NVLink exactly once
//     into a local [M, K] buffer, 16 KB units in the order the tiles are consumed, and count finished units per
//     128-row tile; the TMA producer waits for a tile's count, then loads it from local memory (L2 resident), so a
//     remote row never crosses the link once per N tile;
//   * the epilogue stages 128x64 bf16 chunks in swizzled shared memory and writes them with TMA stores, which
//     reach a peer's slot as full 128-byte lines instead of 16-byte scattered stores.
#include "include/gv_kernels.h"
#include "include/gv_host.h"
#include "include/gv_comm.cuh"

namespace gv {

int num_sms();
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                      uint32_t box_rows);

constexpr int FBM = 128, FBN = 256, FBK = 64, FSTAGES = 4, FTHREADS = 320, FGROUP_M = 8;
constexpr int FA_BYTES = FBM * FBK * 2, FB_BYTES = FBN * FBK * 2, FSTAGE_BYTES = FA_BYTES + FB_BYTES;
constexpr int FOUT_CHUNK = 64;                          // columns per TMA-store chunk (128 bytes of bf16)
constexpr int FOUT_BYTES = FBM * FOUT_CHUNK * 2;        // one staged chunk
constexpr int FOUT_OFFSET = FSTAGES * FSTAGE_BYTES;     // two staged chunks follow the operand ring
constexpr int FBAR_OFFSET = FOUT_OFFSET + 2 * FOUT_BYTES;
constexpr int FSMEM_TOTAL = FBAR_OFFSET + 256 + 1024;
constexpr int FCOPY_WARPS = 4, FCOPY_UNIT = 16384;      // copy warps per CTA, bytes per copy unit
static_assert(FSMEM_TOTAL <= 232448, "shared memory budget");

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
  long long a_off;
  int dest_cols;             // c_mode 2: row length of the destination buffer
  int slot_in;
  uint32_t epoch;
  int tma_store;             // epilogue through shared memory + TMA store (c_mode 0 / 1)
  char* gather_buf;          // a_mode 1: local [M, K]
  uint32_t* gather_ctr;      // a_mode 1: finished copy units per 128-row tile
  int units_per_tile;
};

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier over the 128 epilogue threads that also ANDs a predicate: a wait that gave up in one thread makes every
// thread leave the loop together, so nobody is left alone at a later epilogue_bar().
__device__ __forceinline__ bool epilogue_all(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return out != 0;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait until a tile's copy-unit counter reaches `target`.
__device__ __forceinline__ bool wait_counter(const uint32_t* ctr, uint32_t target, unsigned site) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (ld_acquire_gpu(ctr) >= target) return true;
    if ((spin & 0x3f) == 0x3f) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > GV_WAIT_NS) {
        record_error((site << 16) | 3u, target, ld_acquire_gpu(ctr));
        return false;
      }
      __nanosleep(32);
    }
  }
}

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
fused_gemm_kernel(const __grid_constant__ TmapArray tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ TmapArray tmC, FusedDev p) {
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
      uint32_t ready_mask = (p.a_mode == 2) ? (1u << rank) : 0xffu;   // own data needs no flag
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        ftile_coords(tile, num_m, num_n, tm, tn);
        tm = rotate_m(tm);
        const int m0 = tm * FBM, n0 = tn * FBN;
        const int row_src = p.a_mode == 1 ? tm / m_tiles_per_src : rank;
        if (p.a_mode == 1 && row_src != rank) {
          // rows of a peer: wait until the copy warps have landed this 128-row tile in the local gather buffer
          if (!wait_counter(p.gather_ctr + tm, static_cast<uint32_t>(p.units_per_tile), 0x47)) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          fence_proxy_async_all();
        }
        for (int kbi = 0; kbi < num_kb && ok; ++kbi) {
          const int kb = p.a_mode == 2 ? (kbi + rank * kb_per_src) % num_kb : kbi;
          int src = rank;
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
            if (row_src == rank)
              tma_load_2d(sA, &tmA.m[0], &full_bar[stage], kb * FBK, m0 - rank * m_tiles_per_src * FBM);   // own payload
            else
              tma_load_2d(sA, &tmA.m[1], &full_bar[stage], kb * FBK, m0);                                // gather buffer
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
  } else if (warp < 6) {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const int rows_per = p.c_mode == 1 ? p.M / world : p.M;
    if (p.tma_store) {
      // ---- staged epilogue: TMEM -> registers -> swizzled shared memory -> TMA store (local C or a peer's slot)
      uint8_t* stage_buf = smem + FOUT_OFFSET;
      const bool issuer = threadIdx.x == 64;          // first epilogue thread issues and tracks the bulk stores
      const int r_in_tile = quarter * 32 + lane;
      uint32_t chunk_no = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        ftile_coords(tile, num_m, num_n, tm, tn);
        tm = rotate_m(tm);
        const int m0 = tm * FBM, n0 = tn * FBN;
        if (!epilogue_all(mbar_wait(&acc_full[acc], acc_phase, abort_flag, 0x45))) { ok = false; break; }
        tc_fence_after();
        const uint32_t t_addr = tmem_base + acc * FBN + (static_cast<uint32_t>(quarter * 32) << 16);
        const int owner = p.c_mode == 1 ? m0 / rows_per : 0;
        const int row_in_dest = p.c_mode == 1 ? m0 - owner * rows_per : m0;
#pragma unroll 1
        for (int c = 0; c < FBN / FOUT_CHUNK; ++c) {
          const int col0 = n0 + c * FOUT_CHUNK;
          if (col0 >= p.N) break;                      // uniform over the epilogue warps
          uint8_t* buf = stage_buf + (chunk_no & 1) * FOUT_BYTES;
          if (issuer) tma_store_wait_read<1>();        // the store that last read this buffer has drained it
          epilogue_bar();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_addr + c * FOUT_CHUNK + half * 32, r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            const int colh = col0 + half * 32;
            if (p.bias != nullptr) {
              if (colh + 32 <= p.N) {
                const uint4* bp = reinterpret_cast<const uint4*>(p.bias + colh);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 bq = __ldg(bp + j);
                  float2 f0 = unpack_bf16x2(bq.x), f1 = unpack_bf16x2(bq.y), f2 = unpack_bf16x2(bq.z), f3 = unpack_bf16x2(bq.w);
                  v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
                  v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
                }
              } else {
                for (int i = 0; i < 32; ++i)
                  if (colh + i < p.N) v[i] += __bfloat162float(p.bias[colh + i]);
              }
            }
            // row r of the chunk is 128 bytes; its 16-byte pieces are XOR-swizzled with (r & 7) (SWIZZLE_128B)
            uint8_t* row_ptr = buf + r_in_tile * 128;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
              o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
              o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
              o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
              const int piece = (half * 4 + j) ^ (r_in_tile & 7);
              *reinterpret_cast<uint4*>(row_ptr + piece * 16) = o;
            }
          }
          fence_async_smem();
          epilogue_bar();
          if (issuer) {
            tma_store_2d(&tmC.m[owner], buf, col0, row_in_dest);
            tma_store_commit();
          }
          ++chunk_no;
        }
        __syncwarp();
        tc_fence_before();
        mbar_arrive(&acc_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (issuer) tma_store_wait<0>();                // every bulk store of this CTA has completed its writes
    } else {
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
    }
    __threadfence_system();   // peer stores of this thread are performed before the kernel ends
  } else {
    // ---- copy warps (all-gather -> GEMM): land the peers' row blocks in the local gather buffer, tile by tile
    if (p.a_mode == 1 && world > 1) {
      const int cw = blockIdx.x * FCOPY_WARPS + (warp - 6), n_cw = gridDim.x * FCOPY_WARPS;
      const long long tile_bytes = static_cast<long long>(FBM) * p.K * 2;
      const int upt = p.units_per_tile;
      const long long units_per_src = static_cast<long long>(m_tiles_per_src) * upt;
      const long long total_units = static_cast<long long>(world - 1) * units_per_src;
      uint32_t ready = 0;
      for (long long u = cw; u < total_units; u += n_cw) {
        const int k = static_cast<int>(u / units_per_src);
        const long long rem = u - k * units_per_src;
        const int t = static_cast<int>(rem / upt), sub = static_cast<int>(rem % upt);
        const int src = (rank + 1 + k) % world;
        if (!((ready >> src) & 1u)) {
          int okw = 1;
          if (lane == 0) okw = wait_flag(p.pt, p.slot_in, src, p.epoch, 0x46) ? 1 : 0;
          okw = __shfl_sync(0xffffffffu, okw, 0);
          if (!okw) {
            if (lane == 0) *abort_flag = 1;
            break;
          }
          ready |= 1u << src;
        }
        const long long off = static_cast<long long>(t) * tile_bytes + static_cast<long long>(sub) * FCOPY_UNIT;
        long long nbytes = tile_bytes - static_cast<long long>(sub) * FCOPY_UNIT;
        if (nbytes > FCOPY_UNIT) nbytes = FCOPY_UNIT;
        const uint4* in = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.pt.base[src]) + p.a_off + off);
        uint4* out = reinterpret_cast<uint4*>(p.gather_buf + static_cast<long long>(src) * m_tiles_per_src * tile_bytes + off);
        const int nvec = static_cast<int>(nbytes >> 4);
        for (int i0 = 0; i0 < nvec; i0 += 32 * 8) {
          uint4 tmp[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int i = i0 + q * 32 + lane;
            if (i < nvec) tmp[q] = in[i];
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int i = i0 + q * 32 + lane;
            if (i < nvec) out[i] = tmp[q];
          }
        }
        __threadfence();
        fence_proxy_async_all();
        __syncwarp();
        if (lane == 0) red_release_gpu_add(p.gather_ctr + src * m_tiles_per_src + t, 1u);
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
    rc = make_tmap_bf16_2d(&tmA.m[0], reinterpret_cast<const char*>(peers->bases[rank]) + a->a_off, rows_per, a->K, a->K, 64, FBM);
    if (!rc) rc = make_tmap_bf16_2d(&tmA.m[1], a->gather_buf, a->M, a->K, a->K, 64, FBM);
    for (int r = 2; r < GV_MAX_RANKS; ++r) tmA.m[r] = tmA.m[0];
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
  // destination maps of the staged epilogue
  TmapArray tmC;
  int tma_store = 0;
  if (a->c_mode == 0 && (reinterpret_cast<uintptr_t>(a->C) & 15) == 0) {
    rc = make_tmap_bf16_2d(&tmC.m[0], a->C, a->M, a->N, a->ldc, FOUT_CHUNK, FBM);
    for (int r = 1; r < GV_MAX_RANKS; ++r) tmC.m[r] = tmC.m[0];
    tma_store = 1;
  } else if (a->c_mode == 1 && (a->M / world) % FBM == 0) {
    const long long rows_per = a->M / world;
    for (int r = 0; r < GV_MAX_RANKS && !rc; ++r) {
      const int rr = r < world ? r : 0;
      char* base = reinterpret_cast<char*>(peers->bases[rr]) + a->c_off + static_cast<long long>(rank) * rows_per * a->N * 2;
      rc = make_tmap_bf16_2d(&tmC.m[r], base, rows_per, a->N, a->N, FOUT_CHUNK, FBM);
    }
    tma_store = 1;
  } else {
    rc = make_tmap_bf16_2d(&tmC.m[0], a->B, a->N, a->K, a->ldb, 64, 64);   // unused placeholder with valid contents
    for (int r = 1; r < GV_MAX_RANKS; ++r) tmC.m[r] = tmC.m[0];
  }
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
  p.a_off = a->a_off;
  p.dest_cols = dest_cols;
  p.slot_in = a->slot_in;
  p.epoch = a->epoch;
  p.tma_store = tma_store;
  p.gather_buf = reinterpret_cast<char*>(a->gather_buf);
  p.gather_ctr = a->gather_ctr;
  p.units_per_tile = static_cast<int>((static_cast<long long>(FBM) * a->K * 2 + FCOPY_UNIT - 1) / FCOPY_UNIT);
  auto kern = fused_gemm_kernel<B_MN>;
  static PerDeviceOnce smem_once;
  {
    cudaError_t e = ensure_max_dynamic_smem(smem_once, kern, FSMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int tiles = ((a->M + FBM - 1) / FBM) * ((a->N + FBN - 1) / FBN);
  int grid = tiles < num_sms() ? tiles : num_sms();
  cudaError_t e;
  if (a->a_mode == 1) {
    // The producers of this mode wait on tile counters that copy warps of OTHER CTAs fill, so every CTA of the grid
    // has to be resident at the same time. A cooperative launch guarantees exactly that (it is gang-scheduled once
    // the whole grid fits, whatever other streams of the job hold SMs at the moment); the grid is capped at what the
    // device can hold at once.
    static int max_resident = 0;
    if (max_resident == 0) {
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, FTHREADS, FSMEM_TOTAL) != cudaSuccess || per_sm <= 0) {
        cudaGetLastError();
        per_sm = 1;
      }
      max_resident = per_sm * num_sms();
    }
    if (grid > max_resident) grid = max_resident;
    void* args[] = {&tmA, &tmB, &tmC, &p};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), dim3(grid), dim3(FTHREADS), args, FSMEM_TOTAL, stream);
  } else {
    kern<<<grid, FTHREADS, FSMEM_TOTAL, stream>>>(tmA, tmB, tmC, p);
    e = cudaGetLastError();
  }
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
  if (a->a_mode == 1 && ((a->M % world) || ((a->M / world) % FBM) || a->gather_buf == nullptr || a->gather_ctr == nullptr ||
                         (reinterpret_cast<uintptr_t>(a->gather_buf) & 15)))
    return 2603;
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
