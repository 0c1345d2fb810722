// C launch API of the sm_100a kernel library. Every launcher takes raw device
// pointers and a stream, allocates nothing, and returns a cudaError_t-compatible int
// (0 = launched). Shapes are in elements; bf16 buffers are `void*` to keep this
// header free of CUDA types for the binding layer.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* gv_stream_t;

// ---- error reporting (bounded waits record here instead of hanging) ----------
// Reads and clears the device-side error record. Returns 0 when no kernel reported an error.
int gv_read_error(unsigned int out[4]);

// ---- GEMM (tcgen05 + TMEM + TMA) ---------------------------------------------
// C[M,N] = alpha * A[M,K] * B[N,K]^T  (+ bias[N]) (+ residual[M,N]) (+ beta * C)
//   a_mn_major = 0: A stored row-major [M, lda>=K] (K contiguous)
//   a_mn_major = 1: A stored row-major [K, lda>=M] (M contiguous; e.g. dY for a weight gradient)
//   b_mn_major = 0: B stored row-major [N, ldb>=K]
//   b_mn_major = 1: B stored row-major [K, ldb>=N]
//   c_f32 = 0: C is bf16 [M, ldc]; c_f32 = 1: C is fp32 [M, ldc]
//   accumulate != 0: C += result (used to accumulate weight gradients over micro-batches)
//   act: 0 none, 1 GELU(tanh) applied after bias
// Requirements: K, lda, ldb, ldc multiples of 8; all base pointers 16-byte aligned.
typedef struct {
  const void* A;
  const void* B;
  void* C;
  const void* bias;      // bf16 [N] or NULL
  const void* residual;  // bf16 [M, ldr] or NULL
  int M, N, K;
  int lda, ldb, ldc, ldr;
  int a_mn_major, b_mn_major;
  int c_f32;
  int accumulate;
  int act;
  float alpha;
  // Rotary embedding in the epilogue (0 = off): the leading rope_cols columns of C are heads of rope_dh (64 or 128)
  // columns whose halves are rotated by the row's position (rope_pos[row], or (row / rope_pos_div) % rope_pos_mod +
  // rope_pos_offset when rope_pos is NULL; div / mod <= 0 mean 1 / none) with frequencies rope_inv_freq[rope_dh / 2].
  // Needs alpha == 1 and no bias / residual / activation / accumulate.
  int rope_cols, rope_dh;
  const float* rope_inv_freq;
  const int* rope_pos;
  int rope_pos_div, rope_pos_mod, rope_pos_offset;
  // Gated activation in the epilogue (NULL = off): B = [gate rows (f) | up rows (f)] with N = 2 f, f a multiple of 128.
  // C receives [gate | up] as usual (the backward pass needs it) and swiglu_out [M, swiglu_ld >= f] (bf16) receives
  // silu(gate) * up. Needs K-major A and B, bf16 C, no bias / residual / activation / accumulate.
  void* swiglu_out;
  int swiglu_ld;
} gv_gemm_args;
int gv_gemm_bf16(const gv_gemm_args* args, gv_stream_t stream);

// Language-model head GEMM (logits = A * B^T, both K-major) with the cross entropy in its epilogue; the logits
// themselves are never stored.
//   mode 1: per row and per 256-column tile t of this vocabulary shard, stats[row, t, 0] = max and
//           stats[row, t, 1] = sum exp(logit - max) (the caller merges tiles and ranks); target[row] = logit of the
//           label when its column lies in this shard (written by exactly one tile; the caller zero-fills target).
//   mode 2: C[row, col] (bf16) = (exp(logit - lse[row]) - [col == label]) * gscale[row]: the gradient w.r.t. the
//           logits from recomputed logits (lse = log-sum-exp over the whole vocabulary, gscale = upstream gradient).
// labels are global ids; column c of this shard is id vocab_start + c; rows with label == ignore_index match nothing.
typedef struct {
  int mode;
  const long long* labels;
  long long vocab_start;
  long long ignore_index;
  float* stats;
  float* target;
  const float* lse;
  const float* gscale;
} gv_xent_args;
int gv_gemm_xent(const gv_gemm_args* args, const gv_xent_args* xent, gv_stream_t stream);

// ---- normalisation -------------------------------------------------------------
// y = x * rsqrt(mean(x^2)+eps) * w ; optional residual: h = x + res (written to h_out), y = norm(h)
int gv_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd, int rows,
                   int cols, float eps, gv_stream_t stream);
// dx = grad wrt normalised input (+ dres_in if given); dw_accum[cols] (fp32) += weight gradient, summed in a fixed
// order (two stages through `scratch`, no atomics: bitwise repeatable). `scratch` is caller-provided fp32 memory of
// at least gv_norm_bwd_scratch_elems(rows, cols, layer) elements; its contents need not be initialised.
long long gv_norm_bwd_scratch_elems(int rows, int cols, int layer);
int gv_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in, void* dx,
                   float* dw_accum, float* scratch, long long scratch_elems, int rows, int cols, gv_stream_t stream);
int gv_layernorm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* h_out, float* mean,
                     float* rstd, int rows, int cols, float eps, gv_stream_t stream);
int gv_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                     const void* dres_in, void* dx, float* dw_accum, float* db_accum, float* scratch,
                     long long scratch_elems, int rows, int cols, gv_stream_t stream);

// ---- rotary embedding (non-interleaved halves), in place on q and k -----------------
// x: [tokens, heads, dh] with token stride `ld` elements; pos[tokens] int32 absolute positions.
// inv_freq[dh/2] fp32 are the per-pair angular frequencies; pos == NULL means
// position = (token / pos_div) % pos_mod + pos_offset (batch-major tokens: div 1, mod seq; sequence-major
// tokens: div batch, mod 0 = none). inverse != 0 applies the transpose rotation (backward).
int gv_rope(void* x, const int* pos, const float* inv_freq, long long tokens, int heads, int dh, long long ld,
            int pos_div, int pos_mod, int pos_offset, int inverse, gv_stream_t stream);

// ---- gated / plain activations ---------------------------------------------------
// gate_up: [rows, 2*f] (gate | up halves) -> out [rows, f] = silu(gate) * up
int gv_swiglu_fwd(const void* gate_up, void* out, long long rows, int f, gv_stream_t stream);
int gv_swiglu_bwd(const void* dout, const void* gate_up, void* dgate_up, long long rows, int f, gv_stream_t stream);
int gv_gelu_fwd(const void* x, void* y, long long n, gv_stream_t stream);
int gv_gelu_bwd(const void* dy, const void* x, void* dx, long long n, gv_stream_t stream);
// bias gradient: db_accum[cols] += sum over rows of dy[rows, cols]
int gv_colsum_accum(const void* dy, float* db_accum, long long rows, int cols, gv_stream_t stream);

// ---- embedding -----------------------------------------------------------------------
// out[t, :] = table[ids[t] - vocab_start, :] (zero if outside [vocab_start, vocab_start+vocab_rows))
//             (+ pos_table[pos_ids[t], :] if pos_table)
int gv_embedding_fwd(const long long* ids, const void* table, const int* pos_ids, const void* pos_table, void* out,
                     long long tokens, int hidden, long long vocab_start, long long vocab_rows, gv_stream_t stream);
// dtable_accum[ids[t]-vocab_start, :] += dout[t, :]  (fp32 accumulate, atomic)
int gv_embedding_bwd(const long long* ids, const void* dout, float* dtable_accum, long long tokens, int hidden,
                     long long vocab_start, long long vocab_rows, gv_stream_t stream);

// ---- cross entropy over (a vocab shard of) logits -------------------------------------
// Pass 1: per-row partial statistics over the local vocab shard: row_max, row_sumexp (relative to row_max),
//         target_logit (0 if the label is not in this shard).
int gv_xent_stats(const void* logits, const long long* labels, float* row_max, float* row_sumexp, float* tgt_logit,
                  long long rows, int vocab_local, long long ld, long long vocab_start, gv_stream_t stream);
// Pass 2 (after the cross-shard reduction of the statistics): loss[row] = log(sumexp) + max - tgt and, in place,
//         logits <- (softmax - onehot) * grad_scale * (grad_scale_ptr[row] if given); rows with
//         label == ignore_index give 0. loss may be NULL.
int gv_xent_loss_grad(void* logits, const long long* labels, const float* row_max, const float* row_sumexp,
                      const float* tgt_logit, float* loss, float grad_scale, const float* grad_scale_ptr,
                      long long rows, int vocab_local, long long ld, long long vocab_start, long long ignore_index,
                      gv_stream_t stream);

// ---- optimizer ----------------------------------------------------------------------
// Fused AdamW on a flat shard: fp32 master/m/v, fp32 or bf16 grads, bf16 parameter write-back.
// grad_scale multiplies the gradient first (1/world, loss scale, clip coefficient pointer optional).
int gv_adamw(float* master, float* m, float* v, const void* grad, int grad_is_bf16, void* param_bf16, long long n,
             float lr, float beta1, float beta2, float eps, float weight_decay, float bias_corr1, float bias_corr2,
             float grad_scale, const float* clip_coef, gv_stream_t stream);
// sum of squares of a flat buffer accumulated into out[0] (fp32, atomic)
int gv_sumsq_accum(const void* x, int is_bf16, long long n, float* out, gv_stream_t stream);
// casts / scaling
int gv_cast_f32_to_bf16(const float* in, void* out, long long n, float scale, gv_stream_t stream);
int gv_cast_bf16_to_f32(const void* in, float* out, long long n, float scale, int accumulate, gv_stream_t stream);

// ---- flash attention (tcgen05) ----------------------------------------------------------
// q: [b, sq, hq, dh], k/v: [b, sk, hk, dh] (strides in elements given), o: [b, sq, hq, dh], lse: [b, hq, sq] fp32.
// causal aligns the last query with the last key (sq <= sk). dh must be 64 or 128.
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;
  // backward only
  const void* dout;
  void* dq;       // bf16 output
  void* dk;       // bf16 output
  void* dv;       // bf16 output
  float* dq_accum;  // fp32 scratch [b, sq, hq, dh], zeroed by the launcher
  float* delta;     // fp32 scratch [b, hq, sq]
  int b, sq, sk, hq, hk, dh;
  long long q_stride_b, q_stride_s, q_stride_h;
  long long k_stride_b, k_stride_s, k_stride_h;
  long long v_stride_b, v_stride_s, v_stride_h;
  long long o_stride_b, o_stride_s, o_stride_h;
  long long do_stride_b, do_stride_s, do_stride_h;
  long long dq_stride_b, dq_stride_s, dq_stride_h;
  long long dk_stride_b, dk_stride_s, dk_stride_h;
  long long dv_stride_b, dv_stride_s, dv_stride_h;
  int causal;
  float scale;
  // optional int32 [b] (device): per batch element, the number of leading keys that are real; keys at or beyond it
  // are padding and take no part in the softmax (padding masks of BERT / T5 batches). NULL = every key is real.
  const int* kv_lens;
  // backward only, optional: fold the inverse rotary rotation of the query gradient into the final fp32 -> bf16
  // conversion of dq. dq_rope_inv_freq fp32 [dh / 2] (NULL = off); position of query s of batch element b is
  // dq_rope_pos[s * batch + b] (int32) or s + dq_rope_pos_offset when dq_rope_pos is NULL.
  const float* dq_rope_inv_freq;
  const int* dq_rope_pos;
  int dq_rope_pos_offset;
  // dropout of the attention probabilities (0 = off): entry (q, k) of head (h + dropout_head_offset) of batch element
  // b is dropped with probability dropout_p as a pure function of (dropout_seed, b, head, q, k); the same mask is
  // re-drawn by the backward kernel (and by a recomputed forward), nothing is stored.
  float dropout_p;
  unsigned long long dropout_seed;
  int dropout_head_offset;
  // optional terms on the scaled scores before the softmax (windowed attention: relative-position bias and
  // shifted-window mask); batch elements are windows, image-major. All row strides below are `bias_ld`, a multiple of
  // 64 that covers max(sq, sk): padding columns are read (keep them finite / -1) but never used. NULL = absent.
  //   bias    bf16 [hq, sq, bias_ld]   additive, shared by all batch elements (the forward pass reads rows of it)
  //   bias_t  bf16 [hq, sk, bias_ld]   the same values transposed (the backward pass reads rows of it; required there
  //                                    whenever bias is given)
  //   mask    fp32 [mask_n, sq, bias_ld]   additive, batch element i uses mask[i % mask_n] (general, slower path)
  //   ids     int32 [mask_n, bias_ld]  group ids (sq == sk): key j is visible to query i iff ids[i] == ids[j], batch
  //                                    element i uses ids[i % mask_n]; padding entries -1
  //   dbias   fp32 [hq, sq, bias_ld]   backward, optional: gradient of `bias` summed over the batch (accumulated with
  //                                    atomic adds: zero it first)
  const void* bias;
  const void* bias_t;
  const float* mask;
  const int* ids;
  int mask_n;
  int bias_ld;
  float* dbias;
} gv_attn_args;
int gv_attn_fwd(const gv_attn_args* args, gv_stream_t stream);
int gv_attn_bwd(const gv_attn_args* args, gv_stream_t stream);

// Log-sum-exp merge of a partial attention result into fp32 accumulators (ring / context-parallel attention):
// acc fp32 [b, s, h, dh] contiguous, lse_acc fp32 [b, h, s]; partial o_blk bf16 [b, sb, h, dh] (element strides
// o_s*), lse_blk fp32 [b, h, sb], covering rows [s_off, s_off + sb) of the accumulators.
int gv_lse_merge(float* acc, float* lse_acc, const void* o_blk, const float* lse_blk, int b, int s, int sb, int s_off,
                 int h, int dh, long long o_sb, long long o_ss, long long o_sh, gv_stream_t stream);

// ---- peer-memory collectives and fused compute + collective kernels -----------------------------
// A symmetric workspace is the same-sized buffer on every rank of a group, mapped into every peer. `bases[r]`
// is rank r's workspace as addressed from THIS process; the first 512 bytes of each workspace are the flag area
// (see include/gv_comm.cuh), payload offsets below are in bytes from the workspace base and must be 16-aligned.
typedef struct {
  void* bases[8];
  int world;
  int rank;
} gv_peers;

// All ranks announce `epoch` on flag `slot` and wait for everyone (bounded; timeout_ms <= 0 uses the default).
int gv_comm_barrier(const gv_peers* peers, int slot, unsigned int epoch, int timeout_ms, gv_stream_t stream);
// Wait (bounded by timeout_ms) until rank `src` announced `epoch` on `slot`; used by the failure-detection tests.
int gv_comm_wait(const gv_peers* peers, int slot, int src, unsigned int epoch, int timeout_ms, gv_stream_t stream);
// Announce only.
int gv_comm_signal(const gv_peers* peers, int slot, unsigned int epoch, gv_stream_t stream);

// All-gather by pulling: out[r * n .. (r+1) * n) = peer r's n elements (2-byte) at byte offset `src_off`.
// Waits for flag (slot, epoch) of each source before reading it; local shard first.
int gv_allgather_pull(const gv_peers* peers, long long src_off, void* out, long long n_elems, int slot,
                      unsigned int epoch, gv_stream_t stream);

// out[rows, cols] (bf16) = sum_{r < world} slots[r][rows, cols] (+ residual) (+ bias[cols]), where slot r sits at
// byte offset slots_off + r * rows * cols * 2 of the LOCAL workspace (filled by peers). Waits for flag
// (slot, epoch) of every rank first.
int gv_reduce_slots(const gv_peers* peers, long long slots_off, void* out, const void* residual, const void* bias,
                    long long rows, int cols, int slot, unsigned int epoch, gv_stream_t stream);

// ZeRO gradient reduce-scatter fused with the AdamW update of this rank's shard (and, optionally, the all-gather
// of the updated bf16 parameters): for i in [0, n): g = sum_r peer_r.grad[lo + i]; AdamW on (master, m, v)[i];
// param shard written locally and, when push_params != 0, into every peer's parameter buffer at param_off.
// grads are bf16 (grad_is_bf16) or fp32 at byte offset grad_off of every workspace.
int gv_rs_adamw(const gv_peers* peers, long long grad_off, int grad_is_bf16, long long lo, long long n, float* master,
                float* m, float* v, long long param_off, int push_params, float lr, float beta1, float beta2, float eps,
                float weight_decay, float bias_corr1, float bias_corr2, float grad_scale, const float* clip_coef,
                float* sumsq_out, int slot, unsigned int epoch, gv_stream_t stream);

// ---- ZeRO gradient path as two peer-memory kernels (csrc/comm_kernels.cu) -----------------------------------
// Phase A. Every rank's gradient bucket sits at byte offset grad_off of its workspace. The kernel announces
// (slot_ready, epoch) = "my bucket is final", waits for the peers, sums elements [lo, lo + n) over all ranks in
// fp32 into `out` (out += sum when accumulate; out may be NULL), adds the sum of squares of the reduced slice
// into sumsq_out (may be NULL), and with write_back != 0 stores the sum into every rank's bucket (all-reduce).
// When all of that is complete it announces (slot_done, epoch): the owner of a bucket may clear or overwrite it
// once every peer has announced DONE. ctr_off: byte offset of a zero-initialised 4-byte counter in the workspace.
// max_blocks <= 0 picks a small grid (the kernel is meant to run next to the backward pass).
int gv_grad_reduce(const gv_peers* peers, long long grad_off, int grad_is_bf16, long long lo, long long n, float* out,
                   int accumulate, int write_back, float* sumsq_out, long long ctr_off, int slot_ready, int slot_done,
                   unsigned int epoch, int timeout_ms, int max_blocks, gv_stream_t stream);
// Phase B. AdamW on this rank's fp32 shard (master, m, v, grad: n elements each); the new bf16 values are stored
// at element lo of the parameter buffer at byte offset param_off of EVERY rank's workspace (push_all != 0) or of
// this rank's only. Announces (slot_param, epoch) when done. The caller orders it after phase A of the same
// bucket: a peer announces READY only after its last use of the old parameters in the step.
int gv_adamw_push(const gv_peers* peers, long long param_off, long long lo, long long n, float* master, float* m, float* v,
                  const float* grad, int push_all, float lr, float beta1, float beta2, float eps, float weight_decay,
                  float bias_corr1, float bias_corr2, float grad_scale, const float* clip_coef, long long ctr_off,
                  int slot_param, unsigned int epoch, gv_stream_t stream);
// Wait until every PEER (this rank excluded) announced `epoch` on `slot`.
int gv_comm_wait_peers(const gv_peers* peers, int slot, unsigned int epoch, int timeout_ms, gv_stream_t stream);
// Clear nbytes at ptr (16-byte aligned, multiple of 16) once every peer announced `epoch` on `slot`.
int gv_wait_zero(const gv_peers* peers, int slot, unsigned int epoch, void* ptr, long long nbytes, int timeout_ms,
                 gv_stream_t stream);
// gv_allgather_pull with a caller-chosen wait budget.
int gv_allgather_pull_ex(const gv_peers* peers, long long src_off, void* out, long long n_elems, int slot,
                         unsigned int epoch, int timeout_ms, gv_stream_t stream);

// Inter-layer reshard: out[(s, b), :] = peer[src_rank[s * bn + b]] payload row (src_row[s] * b_old + src_col[b]).
// Index arrays are device int32; `hidden` elements (2-byte) per row; payload at byte offset src_off.
int gv_reshard_gather(const gv_peers* peers, long long src_off, void* out, const int* src_rank, const int* src_row,
                      const int* src_col, int s_new, int b_new, int b_old, int hidden, int slot, unsigned int epoch,
                      gv_stream_t stream);

// NVLink collectives as plain kernels (csrc/nvlink_bench.cu); same flag protocol as above.
// Pull `nbytes` from peer `src`'s payload at src_off into local `out` after src announced (slot, epoch).
int gv_p2p_pull(const gv_peers* peers, int src, long long src_off, void* out, long long nbytes, int slot,
                unsigned int epoch, gv_stream_t stream);
// The same with at most max_blocks CTAs (<= 0: as many as gv_p2p_pull), for transfers that run beside a compute kernel.
int gv_p2p_pull_ex(const gv_peers* peers, int src, long long src_off, void* out, long long nbytes, int slot,
                   unsigned int epoch, int max_blocks, gv_stream_t stream);
// out[s * bytes_per_rank ...] = peer s's payload block [rank * bytes_per_rank, ...) at src_off, for every s.
int gv_alltoall_pull(const gv_peers* peers, long long src_off, void* out, long long bytes_per_rank, int slot,
                     unsigned int epoch, gv_stream_t stream);
// First shot of an in-place two-shot all-reduce of the bf16 buffer at `off`: this rank sums its shard over all
// peers and writes it back to all of them (mc_base != NULL: multimem.ld_reduce / multimem.st through NVSwitch on
// the multicast mapping). Follow with gv_comm_barrier on another slot.
int gv_allreduce_shard(const gv_peers* peers, void* mc_base, long long off, long long n_elems, int slot,
                       unsigned int epoch, gv_stream_t stream);

// Fused GEMM + collective (tcgen05). C = A * B^T with
//   a_mode 0: A local [M, K];  a_mode 1: A rows gathered from peers (all-gather -> GEMM): rows [r*M/world, ...) come
//             from peer r's payload at a_off (waits flag (slot_in, epoch) of r). Copy warps of the same kernel pull
//             every remote row block ONCE into the local buffer `gather_buf` [M, K] (each 128-row tile counted in
//             `gather_ctr`, which the caller zeroes per call) and the tensor-core pipeline reads the tile from there
//             as soon as it is complete; own rows are read from the own payload;  a_mode 2: A K-slices gathered from
//             peers (Ulysses head -> sequence): columns [r*K/world, ...) of my M rows come from peer r's payload rows
//             [rank*M, (rank+1)*M) at a_off.
//   c_mode 0: C local [M, N];  c_mode 1: row block o of C is stored into peer o's workspace at
//             c_off + rank * (M/world) * N * 2 (GEMM -> reduce-scatter; finish with gv_reduce_slots);
//             c_mode 2: column block o of C is stored into peer o's workspace at c_off, rows [rank*M, (rank+1)*M)
//             (projection -> Ulysses sequence -> head exchange).
// After the last tile every rank announces (slot_out, epoch).
typedef struct {
  const void* A;      // local A (a_mode 0) -- ignored otherwise
  const void* B;      // [N, K] row-major
  void* C;            // local C (c_mode 0)
  const void* bias;   // bf16 [N] or NULL
  int M, N, K;
  int lda, ldb, ldc;
  int a_mode, c_mode;
  long long a_off, c_off;
  int slot_in, slot_out;
  unsigned int epoch;
  void* gather_buf;            // a_mode 1: local [M, K] bf16 (rows of peers land here; own rows are not copied)
  unsigned int* gather_ctr;    // a_mode 1: one counter per 128-row tile of A, zero on entry
} gv_fused_gemm_args;
int gv_fused_gemm(const gv_peers* peers, const gv_fused_gemm_args* args, gv_stream_t stream);
// Extended form: b_mn_major != 0 reads B stored [K, N] (a layer's weight used for its input gradient);
// col_map (device int32, one entry per 32-column chunk: (dest_rank << 24) | dest_col) and dest_cols (row length of
// the destination buffer) drive c_mode 2.
int gv_fused_gemm_ex(const gv_peers* peers, const gv_fused_gemm_args* args, int b_mn_major, const int* col_map,
                     int dest_cols, gv_stream_t stream);

#ifdef __cplusplus
}
#endif
