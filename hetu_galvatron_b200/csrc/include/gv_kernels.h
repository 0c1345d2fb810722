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
} gv_gemm_args;
int gv_gemm_bf16(const gv_gemm_args* args, gv_stream_t stream);

// ---- normalisation -------------------------------------------------------------
// y = x * rsqrt(mean(x^2)+eps) * w ; optional residual: h = x + res (written to h_out), y = norm(h)
int gv_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd, int rows,
                   int cols, float eps, gv_stream_t stream);
// dx = grad wrt normalised input (+ dres_in if given); dw accumulated into fp32 dw_accum[cols] (atomic)
int gv_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in, void* dx,
                   float* dw_accum, int rows, int cols, gv_stream_t stream);
int gv_layernorm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* h_out, float* mean,
                     float* rstd, int rows, int cols, float eps, gv_stream_t stream);
int gv_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                     const void* dres_in, void* dx, float* dw_accum, float* db_accum, int rows, int cols,
                     gv_stream_t stream);

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
} gv_attn_args;
int gv_attn_fwd(const gv_attn_args* args, gv_stream_t stream);
int gv_attn_bwd(const gv_attn_args* args, gv_stream_t stream);

#ifdef __cplusplus
}
#endif
