/*
 * rte_b200.h -- C ABI of the B200 (sm_100a) kernels behind the Recursive
 * Training Engine's `recursive_macro` / `dense_exact` training step.
 *
 * The reference project has no FFI: its seam is a Python operator table
 * (src/recursive_training_engine/kernels/optimized.py:58-154, definitions in
 * kernels/reference.py:9-157) plus inline `nn.Linear`/`@`/`bmm` calls in
 * layers.py / macro.py / models.py and `torch.optim.AdamW`
 * (training.py:341-354).  Each entry point below names the reference
 * function(s) whose arithmetic it replaces.
 *
 * Conventions
 *  - plain device pointers, sizes and strides; no framework types.
 *  - every call is asynchronous on `stream` (a cudaStream_t passed as void*),
 *    never synchronises, never allocates; scratch memory is passed in.
 *  - return value: 0 = launched; <0 = argument error (see rte_status_string).
 *  - `status` arguments point to one device int32 that a kernel sets non-zero
 *    when a bounded wait ran out or an index was out of range; the host reads
 *    it when it next synchronises.  May be NULL.
 *  - bf16 = 16-bit brain float, row-major unless stated; "ld" = row stride in
 *    elements.  TMA operands need 16-byte aligned bases and ld % 8 == 0.
 */
#ifndef RTE_B200_H_
#define RTE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* rte_stream_t;

enum {
  RTE_OK = 0,
  RTE_ERR_BAD_ARG = -1,
  RTE_ERR_ALIGNMENT = -2,
  RTE_ERR_TENSOR_MAP = -3,
  RTE_ERR_LAUNCH = -4,
  RTE_ERR_UNSUPPORTED = -5,
  RTE_ERR_NO_DEVICE = -6,
  RTE_ERR_SCRATCH_CAPACITY = -7
};

/* Name of the backend ("cuda_sm100a_ext") for the reference's
 * backend_status() manifest block (kernels/optimized.py:27-43). */
const char* rte_backend_name(void);
const char* rte_status_string(int code);
/* Number of SMs of the current device (grid sizing); <0 on error. */
int rte_device_sm_count(void);

/* ---------------------------------------------------------------- GEMM ---
 * C[M,N] (+)= A[M,K] * B[N,K]^T on the tcgen05 tensor cores, bf16 inputs,
 * fp32 accumulation in tensor memory, operands fetched by TMA.
 * Replaces: nn.Linear of the fused QKV / wo / W_ug / W_d / tied logits
 * (layers.py:66,75,86-87; models.py:185) and their autograd backward GEMMs.
 *
 * a_mn_major = 0: A is stored [M,K] (K contiguous);  1: stored [K,M] (M contiguous).
 * b_mn_major = 0: B is stored [N,K] (K contiguous);  1: stored [K,N] (N contiguous).
 * lda / ldb are the row strides of the STORED matrices.
 */
enum {
  RTE_EPI_BF16 = 0,        /* C bf16 = acc                                                   */
  RTE_EPI_F32 = 1,         /* C f32 = acc (+ R f32 when R != NULL; R may alias C).            */
                           /* With splits > 1 partial s goes to C + s*split_stride (no R).    */
  RTE_EPI_SWIGLU_FWD = 2,  /* B rows [0,F) = up, [F,2F) = gate, F = b_pair_offset (N = 2F): */
                           /* C2 bf16 [M,2F] = (up | gate), C bf16 [M,F] = up * silu(gate)    */
  RTE_EPI_SWIGLU_BWD = 3   /* acc = dz [M,F]; R bf16 [M,2F] = saved (up | gate):              */
                           /* C bf16 [M,2F] = (dz*silu(g) | dz*up*sig(g)*(1+g*(1-sig(g))))    */
};

typedef struct rte_gemm_args {
  int32_t M, N, K;
  const void* A; int32_t lda; int32_t a_mn_major;
  const void* B; int32_t ldb; int32_t b_mn_major;
  int32_t epilogue;
  void* C; int32_t ldc;
  const void* R; int32_t ldr;
  void* C2; int32_t ldc2;
  int32_t b_pair_offset;    /* F for the SwiGLU epilogues, else 0 */
  int32_t splits;           /* >= 1; > 1 only with RTE_EPI_F32 (split along K) */
  int64_t split_stride;     /* elements between partial results */
  int32_t max_ctas;         /* 0 = one CTA per SM */
  int32_t* status;
  /* Grouped mode (cluster-pool FFN, cluster_pool_ffn.py:206-241): the rows of A/C are packed by group in blocks of
   * 128 rows; tile_group int32 [M/128] (device) names each block's group (< 0: unused block, skipped).  B is the
   * stack of all groups' matrices; group g's matrix starts b_group_stride rows further (rows of the stored B: its
   * N rows when K-major, its K rows when MN-major).  M must be a multiple of 128.  NULL = ordinary GEMM.        */
  const int32_t* tile_group;
  int32_t n_groups;
  int32_t b_group_stride;
  /* Ragged split-K (per-group weight gradients over packed rows): split s reduces the 64-wide k-blocks
   * [split_kblocks[s], split_kblocks[s+1]) (device int32 [splits+1]) into C + s*split_stride; an empty range gives
   * zeros.  RTE_EPI_F32 only.  NULL = equal splits.                                                             */
  const int32_t* split_kblocks;
  /* Tile shape (0 = chosen by the library).  tile_n: 128 or 256 columns per tile.  cta_pair: 1 = every tile is
   * 128 rows on one CTA; otherwise a product with more than 128 rows (and neither grouping nor ragged splits) runs
   * 256-row tiles on pairs of CTAs (tcgen05 cta_group::2), each CTA loading half of the tile's B operand.       */
  int32_t tile_n;
  int32_t cta_pair;
  /* rte_gemm_bf16_small with splits > 1 only: reduce the partial results inside the launch.  The CTA that finishes
   * last for an output tile (a counter per tile in split_counters: device int32, at least 1024, zero before the first
   * use; the kernel leaves them zero) sums the tile's `splits` partials from C in split order and writes
   * split_out[M,N] (row stride N; += when split_accumulate != 0).  NULL = the caller reduces (rte_reduce_splits).   */
  int32_t* split_counters;
  float* split_out;
  int32_t split_accumulate;
} rte_gemm_args;

int rte_gemm_bf16(const rte_gemm_args* args, rte_stream_t stream);
/* The tile shape rte_gemm_bf16 would use for `args` (M, N, epilogue, grouping, tile hints and max_ctas are read) and
 * how many tiles run at the same time: what a caller needs to choose a split count.  Any output may be NULL.  */
int rte_gemm_tile_plan(const rte_gemm_args* args, int32_t* tile_m, int32_t* tile_n, int32_t* concurrent_tiles);
/* The same product for FEW ROWS (the audited samples' replay, models.py:605-679: M = one or two samples): one
 * 128-thread CTA per 64x64 output tile, cp.async + mma.sync, no tensor maps or TMEM set-up, so a dependent chain of
 * such launches is not dominated by set-up time.  Subset of rte_gemm_args: A K-major, B either major, RTE_EPI_BF16
 * or RTE_EPI_F32 (+R), equal split-K (fp32, no R), no grouping; K % 8 == 0 (and N % 8 == 0 when B is MN-major).   */
int rte_gemm_bf16_small(const rte_gemm_args* args, rte_stream_t stream);

/* out[i] = (accumulate ? out[i] : 0) + sum_s ws[s*split_stride + i], i < n (deterministic order). */
int rte_reduce_splits(const float* ws, int32_t splits, int64_t split_stride, int64_t n, float* out,
                      int32_t accumulate, rte_stream_t stream);

/* ---------------------------------------------------- embedding (models.py:136,693) */
int rte_embed_fwd(const int64_t* tokens, const float* table, float* out, int32_t n_tokens, int32_t d,
                  int32_t vocab, int32_t* status, rte_stream_t stream);
/* dtable[tokens[i], :] += dx[i, :].  Reproducible bit for bit: the addends meet in `accum` (scratch, vocab*d int64,
 * any contents) as 64-bit fixed point (2^-40 resolution, order-free integer atomics) and are added to dtable once. */
int rte_embed_bwd(const int64_t* tokens, const float* dx, float* dtable, int64_t* accum, int32_t n_tokens, int32_t d,
                  int32_t vocab, int32_t* status, rte_stream_t stream);

/* ------------------------------------------------- RMSNorm (kernels/reference.py:9-17)
 * y = x * rsqrt(mean(x^2) + eps) * w [* (1 + film_gamma) + film_beta]  (FiLM: layers.py:841-847)
 * x f32 [rows,d]; y bf16 and/or f32 (either may be NULL); rstd f32 [rows] saved for backward.
 * w may be NULL (macro.py:16-18).                                                       */
int rte_rmsnorm_fwd(const float* x, const float* w, const float* film_gamma, const float* film_beta,
                    void* y_bf16, float* y_f32, float* rstd, int32_t rows, int32_t d, float eps,
                    rte_stream_t stream);
/* dx = rmsnorm_backward(dy) + dres;  dy is bf16 (dy_bf16) or f32 (dy_f32), dres f32 or NULL.
 * dx written as f32 (dx_f32) and/or bf16 (dx_bf16).  dw_partial f32 [grid_rows, d] receives
 * per-CTA partial sums of dy * xhat (and dfilm_* likewise) -- reduce with rte_colsum_partials.
 * Returns the number of partial rows written through *n_partials (host value).          */
/* Residual update(s) of the banked recurrent core fused in front of the norm (layers.py:831-870: "h + alpha*h0",
 * "h + s*branch", frozen samples passed through), one launch instead of two or three:
 *   x1 = (active == NULL || active[row / S]) ? base + *scale * branch : passthrough      -> x1_out (optional)
 *   x  = add2 ? x1 + *scale2 * add2 : x1                                                  -> x_out
 *   y  = rmsnorm(x) * w [* (1 + film_gamma) + film_beta]                                  -> y_bf16, rstd
 * scale / scale2 are device scalars; active is per sample (S rows each).                                        */
int rte_residual_rmsnorm_fwd(const float* base, const float* branch, const float* scale, const int32_t* active,
                             const float* passthrough, int32_t S, const float* add2, const float* scale2,
                             float* x1_out, float* x_out, const float* w, const float* film_gamma,
                             const float* film_beta, void* y_bf16, float* rstd, int32_t rows, int32_t d, float eps,
                             rte_stream_t stream);
int rte_rmsnorm_bwd(const float* x, const float* w, const float* film_gamma, const float* rstd,
                    const void* dy_bf16, const float* dy_f32, const float* dres,
                    float* dx_f32, void* dx_bf16, float* dw_partial, float* dgamma_partial,
                    float* dbeta_partial, int32_t rows, int32_t d, int32_t max_partials,
                    int32_t* n_partials, rte_stream_t stream);
/* The two launches above fed with the split-K partials of a few-row product instead of its reduced result (the audit
 * replay's chain: one dependent launch less per product).  `branch` / `dy_f32` then point at `*_splits` partials of
 * rows*d floats each, `*_split_stride` floats apart (a multiple of 4), which the kernel sums in split order -- the
 * bits rte_reduce_splits would have produced.  branch_out (optional) receives the summed branch.  With one split
 * they are the launches above.                                                                                     */
int rte_residual_rmsnorm_fwd_splits(const float* base, const float* branch, int32_t branch_splits,
                                    int64_t branch_split_stride, float* branch_out, const float* scale,
                                    const int32_t* active, const float* passthrough, int32_t S, const float* add2,
                                    const float* scale2, float* x1_out, float* x_out, const float* w,
                                    const float* film_gamma, const float* film_beta, void* y_bf16, float* rstd,
                                    int32_t rows, int32_t d, float eps, rte_stream_t stream);
int rte_rmsnorm_bwd_splits(const float* x, const float* w, const float* film_gamma, const float* rstd,
                           const void* dy_bf16, const float* dy_f32, int32_t dy_splits, int64_t dy_split_stride,
                           const float* dres, float* dx_f32, void* dx_bf16, float* dw_partial, float* dgamma_partial,
                           float* dbeta_partial, int32_t rows, int32_t d, int32_t max_partials, int32_t* n_partials,
                           rte_stream_t stream);
/* out[c] = (accumulate ? out[c] : 0) + sum_r partial[r, c] */
int rte_colsum_partials(const float* partial, int32_t n_rows, int32_t d, float* out, int32_t accumulate,
                        rte_stream_t stream);
/* The same for up to three equally shaped partial buffers in ONE launch (norm weight + the two FiLM vectors):
 * host arrays of `count` device pointers / flags.                                                                */
int rte_colsum_partials3(const float* const* partials, float* const* outs, const int32_t* accumulate, int32_t count,
                         int32_t n_rows, int32_t d, rte_stream_t stream);

/* --------------------- causal attention with RoPE (layers.py:36-50,64-75; reference.py:20-28,40-41)
 * qkv bf16 [B*S, 3*d] with columns (q | k | v), head-major inside each; adjacent-pair rotary
 * embedding (base 10000, positions 0..S-1) applied to q and k inside the kernel; softmax scale
 * 1/sqrt(head_dim).  y bf16 [B*S, d]; lse f32 [B, H, S] saved for backward.
 * n_heads may be fewer than d/head_dim when only the first `n_heads` heads of a packed buffer
 * exist (banked attention, layers.py:702-728): row stride stays `ld_qkv`, section stride `sec`.
 * rope_table (optional, may be NULL): f32 [S, head_dim/2, 2] = (cos, sin) of pos * 10000^(-2i/head_dim) as
 * written by rte_rope_table (the reference's cached buffers, layers.py:37-44); without it the kernels compute
 * the angles themselves.                                                                                       */
int rte_rope_table(float* out, int32_t S, int32_t head_dim, rte_stream_t stream);
/* k_rope_apply (kernels/reference.py:20-28) as an operator of its own: out = x*cos + rotate_half(x)*sin over
 * x [rows, S, head_dim] (rows = B*H), cos/sin f32 [S, head_dim]; f32 or bf16 data; adjoint != 0 applies the
 * transposed rotation (the operator's backward).  out may alias x.                                              */
int rte_rope_apply(const void* x, const float* cos_tab, const float* sin_tab, void* out, int64_t rows, int32_t S,
                   int32_t head_dim, int32_t is_bf16, int32_t adjoint, rte_stream_t stream);
int rte_attn_fwd(const void* qkv, int32_t ld_qkv, int32_t sec, void* y, int32_t ld_y, float* lse,
                 const float* rope_table, int32_t B, int32_t S, int32_t n_heads, int32_t head_dim,
                 rte_stream_t stream);
/* Forward with a second, column-masked copy of the output: y_masked[row, c] = y[row, c] * mask_table[mask_row[row / S]][c]
 * (the banked core's recipe mask, layers.py:702-728; mask_table f32 [n_rows_of_table, n_heads*head_dim]).  One launch
 * on the tensor-core path, otherwise rte_attn_fwd + rte_colmask_mul_bf16.  ld_y must equal n_heads*head_dim.     */
int rte_attn_fwd_masked(const void* qkv, int32_t ld_qkv, int32_t sec, void* y, void* y_masked, int32_t ld_y, float* lse,
                        const float* rope_table, const int32_t* mask_row, const float* mask_table, int32_t B, int32_t S,
                        int32_t n_heads, int32_t head_dim, rte_stream_t stream);
int rte_attn_bwd(const void* qkv, int32_t ld_qkv, int32_t sec, const void* y, const void* dy, int32_t ld_y,
                 const float* lse, void* dqkv, const float* rope_table, int32_t B, int32_t S, int32_t n_heads,
                 int32_t head_dim, rte_stream_t stream);
/* The same backward for an upstream gradient dy * mask_table[mask_row[sample]] (the mask of rte_attn_fwd_masked on the
 * way back, layers.py:702-728).  One launch on the tensor-core path, dy untouched; otherwise dy is masked in place
 * (rte_colmask_mul_bf16) and rte_attn_bwd follows.  ld_y must equal n_heads*head_dim.                              */
int rte_attn_bwd_masked(const void* qkv, int32_t ld_qkv, int32_t sec, const void* y, void* dy, int32_t ld_y,
                        const float* lse, void* dqkv, const float* rope_table, const int32_t* mask_row,
                        const float* mask_table, int32_t B, int32_t S, int32_t n_heads, int32_t head_dim,
                        rte_stream_t stream);

/* ------------- per-token cross entropy + its gradient (models.py:73-75; training.py:1381-1385)
 * logits bf16 [rows, V] (ld = ldl).  loss_tok f32 [rows] = logsumexp - logit[target].
 * If dlogits != NULL: dlogits bf16 [rows, V] = row_weight[row / S] * (softmax - onehot); may
 * alias logits.                                                                          */
int rte_ce_fwd_bwd(const void* logits, int32_t ldl, const int64_t* targets, const float* row_weight,
                   int32_t S, float* loss_tok, void* dlogits, int32_t rows, int32_t V, int32_t* status,
                   rte_stream_t stream);
/* out[b] = sum_s in[b*S + s]  (per-sample loss sums, models.py:75) */
int rte_segment_sum(const float* in, float* out, int32_t n_seg, int32_t seg_len, rte_stream_t stream);

/* ---------------------------------------------- router (routing.py:88-188; metrics.py:97-112)
 * One decision per sample from pooled = mean_S(h0).  Weights f32 in nn.Linear layout.
 * out_f f32 [B, RTE_ROUTER_F_STRIDE] and out_i int32 [B, RTE_ROUTER_I_STRIDE] are laid out as the
 * offsets below say.  argmax ties go to the LOWEST index.  fixed_recipe / fixed_depth_id < 0 = unset. */
enum { RTE_ROUTER_MAX_R = 32, RTE_ROUTER_MAX_K = 8, RTE_ROUTER_MAX_T = 128, RTE_ROUTER_DPOOLED_PARTS = 4 };
typedef struct rte_router_weights {
  const float *r_w0, *r_b0, *r_w2, *r_b2;   /* recipe_mlp */
  const float *d_w0, *d_b0, *d_w2, *d_b2;   /* depth_mlp  */
  const float* pass_recipe_bias;            /* [T, R] */
} rte_router_weights;
typedef struct rte_router_out {
  float* pooled;         /* [B, d]   */
  float* r_hidden_pre;   /* [B, hid] pre-activation of recipe_mlp.0 (saved for backward) */
  float* d_hidden_pre;   /* [B, hid] */
  float* recipe_logits;  /* [B, R]   */
  float* recipe_probs;   /* [B, R]   */
  float* depth_probs;    /* [B, K]   */
  float* expected_depth; /* [B]      */
  float* router_entropy; /* [B]      */
  int32_t* recipe_id;         /* [B]    */
  int32_t* recipe_id_by_pass; /* [B, T] */
  int32_t* depth_id;          /* [B]    */
  int32_t* depth;             /* [B]    */
} rte_router_out;
int rte_router_fwd(const float* h0, const rte_router_weights* w, const int32_t* depth_values,
                   const rte_router_out* out, int32_t B, int32_t S, int32_t d, int32_t hid, int32_t R,
                   int32_t K, int32_t T, int32_t fixed_recipe, int32_t fixed_depth_id, rte_stream_t stream);
/* aux[0] = lambda_load * (R * sum_r mean_B(p_r)^2 - 1), aux[1] = lambda_depth * mean_B E[depth]
 * (metrics.py:103-111).  Backward of both through the two MLPs: weight/bias grads (f32, overwritten)
 * and dh0[b,s,:] += dpooled[b,:] / S.  scratch f32 (16-byte aligned) >= RTE_ROUTER_MAX_R + B*(2*hid + R + K + RTE_ROUTER_DPOOLED_PARTS*d) + 4.      */
typedef struct rte_router_grads {
  float *r_w0, *r_b0, *r_w2, *r_b2, *d_w0, *d_b0, *d_w2, *d_b2;
} rte_router_grads;
int rte_router_aux_bwd(const rte_router_weights* w, const rte_router_out* fwd, const int32_t* depth_values,
                       float lambda_load, float lambda_depth, float* aux, const rte_router_grads* grads,
                       float* dh0, float* scratch, int32_t B, int32_t S, int32_t d, int32_t hid, int32_t R,
                       int32_t K, rte_stream_t stream);
/* The same backward in two halves (parameter gradients on another stream, ordered after _data, same `scratch`).
 * mean_prob_in (device f32 [R], may be NULL): the batch mean of the recipe probabilities to use instead of this
 * call's own.  The load-balance loss squares a BATCH mean (metrics.py:103-105), so under data parallelism the
 * global-batch step needs the mean over all shards: every rank writes scale * sum_b p with rte_router_mean_prob
 * (scale = 1 / (B * world)), the ranks sum those R floats, and each passes the result here.                       */
int rte_router_mean_prob(const float* recipe_probs, float* out, float scale, int32_t B, int32_t R, rte_stream_t stream);
int rte_router_aux_bwd_data(const rte_router_weights* w, const rte_router_out* fwd, const int32_t* depth_values,
                            float lambda_load, float lambda_depth, float* aux, float* dh0, float* scratch,
                            const float* mean_prob_in, int32_t B, int32_t S, int32_t d, int32_t hid, int32_t R,
                            int32_t K, rte_stream_t stream);
/* With dh0 == NULL the call above leaves out its last step; this performs it later (the rest needs no upstream
 * gradient and can run right after the router's forward): dh0[b,s,:] += dpooled[b,:] / S, read from `scratch`.  */
int rte_router_aux_add_dh0(float* dh0, const float* scratch, int32_t B, int32_t S, int32_t d, int32_t hid, int32_t R,
                           int32_t K, rte_stream_t stream);
int rte_router_aux_bwd_params(const rte_router_out* fwd, const rte_router_grads* grads, float* scratch, int32_t B,
                              int32_t d, int32_t hid, int32_t R, int32_t K, rte_stream_t stream);

/* ---------------------------------- top-k with ties to the lowest index (output.py:78; layers.py:602-627)
 * scores f32 [rows, n]; idx int32 [rows, k] and vals f32 [rows, k] (either may be NULL), descending. */
int rte_topk_lowest_index(const float* scores, int32_t ld, int32_t rows, int32_t n, int32_t k,
                          int32_t* idx, float* vals, rte_stream_t stream);

/* ------------------------------------------ macro operator Phi (macro.py:201-236, legacy shape)
 * out = h + s_cfg * scale[r,k] * tanh(gain[r,k]*h + silu([rmsnorm(h), mean_S rmsnorm(h), h0] @ v[r,k]) @ u[r,k] + bias[r,k])
 * with h == h0 (models.py:695).  Per-sample (recipe, stride) ids int32.  m = rank <= 64.
 * Saved for backward: rstd [B*S], pooled [B*d + B*m] (mean_S rmsnorm(h), then its product with
 * v[d:2d]), act [B*S, m] (pre-activation z @ v).                                             */
typedef struct rte_phi_params {
  const float *gain, *v, *u, *bias, *scale;   /* [R,K,d], [R,K,3d,m], [R,K,m,d], [R,K,d], [R,K,d] */
  const float* wt;                            /* optional: transposed v and u from rte_macro_phi_prepare (NULL: scalar kernels) */
  int32_t n_keys;                             /* R*K, the row count behind wt's leading dimensions */
} rte_phi_params;
/* wt f32 [n_keys*(3d*m + m*d)] = v^T as [m][n_keys*3d] followed by u^T as [d][n_keys*m]; call once per optimiser
 * step (after the parameters changed).  With it, d % 32 == 0 and rank % 4 == 0 the forward products and the
 * first backward product run on tensor cores (TF32 with hi/lo split: fp32 accuracy).                            */
int rte_macro_phi_prepare(const float* v, const float* u, float* wt, int32_t n_keys, int32_t d, int32_t m,
                          rte_stream_t stream);
int rte_macro_phi_fwd(const float* h0, const rte_phi_params* p, const int32_t* recipe_id,
                      const int32_t* stride_id, float s_cfg, float* out, float* rstd, float* pooled,
                      float* act, int32_t B, int32_t S, int32_t d, int32_t m, int32_t K_strides,
                      float eps, rte_stream_t stream);
/* dh0 f32 [B*S,d] (overwritten), parameter grads f32 (zeroed then accumulated, full [R,K,...] tensors).
 * scratch f32 >= B*S*d + B*S*m + 3*B*d + B*m*d + B*3*d*m.                                           */
typedef struct rte_phi_grads { float *gain, *v, *u, *bias; } rte_phi_grads;
int rte_macro_phi_bwd(const float* h0, const float* dout, const rte_phi_params* p, const int32_t* recipe_id,
                      const int32_t* stride_id, float s_cfg, const float* rstd, const float* pooled,
                      const float* act, float* dh0, const rte_phi_grads* g, float* scratch, int32_t B,
                      int32_t S, int32_t d, int32_t m, int32_t R, int32_t K_strides, float eps,
                      rte_stream_t stream);
/* Phi applied to a state h that is NOT the injected h0 (macro.py:201-236 with h != h0; the second application inside
 * MacroOperators.consistency_loss, macro.py:342-359): same buffers as above, `h` drives the norm, the pooled mean, the
 * gain and the residual term, `h0` only the third slice of z.  Backward: dh is overwritten, dh0 is ACCUMULATED into
 * (dh != dh0), parameter gradients as in rte_macro_phi_bwd (full tensors, overwritten).                            */
int rte_macro_phi_fwd_hx(const float* h, const float* h0, const rte_phi_params* p, const int32_t* recipe_id,
                         const int32_t* stride_id, float s_cfg, float* out, float* rstd, float* pooled,
                         float* act, int32_t B, int32_t S, int32_t d, int32_t m, int32_t K_strides,
                         float eps, rte_stream_t stream);
int rte_macro_phi_bwd_hx(const float* h, const float* h0, const float* dout, const rte_phi_params* p,
                         const int32_t* recipe_id, const int32_t* stride_id, float s_cfg, const float* rstd,
                         const float* pooled, const float* act, float* dh, float* dh0, const rte_phi_grads* g,
                         float* scratch, int32_t B, int32_t S, int32_t d, int32_t m, int32_t R, int32_t K_strides,
                         rte_stream_t stream);
/* Mean-squared-error pieces of the consistency term (F.mse_loss, macro.py:359): g = coef * (a - b) and
 * sum_out (+)= sum (a - b)^2, summed in a fixed order.  `partial`: scratch of >= 1024 floats.                       */
int rte_sqdiff_grad(const float* a, const float* b, int64_t n, float coef, float* g, float* partial, float* sum_out,
                    int32_t accumulate, rte_stream_t stream);
/* The same backward in two halves, so that a caller can put the parameter gradients on another stream: _data
 * computes dh0 (what the rest of backward waits for) and leaves its intermediates in `scratch`; _params (ordered
 * after _data, same `scratch`) reduces the per-sample parameter gradients per (recipe, stride) key.             */
int rte_macro_phi_bwd_data(const float* h0, const float* dout, const rte_phi_params* p, const int32_t* recipe_id,
                           const int32_t* stride_id, float s_cfg, const float* rstd, const float* act, float* dh0,
                           float* scratch, int32_t B, int32_t S, int32_t d, int32_t m, int32_t K_strides,
                           rte_stream_t stream);
int rte_macro_phi_bwd_params(const float* h0, const int32_t* recipe_id, const int32_t* stride_id, const float* rstd,
                             const float* pooled, const float* act, const rte_phi_grads* g, float* scratch,
                             int32_t B, int32_t S, int32_t d, int32_t m, int32_t R, int32_t K_strides,
                             rte_stream_t stream);

/* -------------------------------------------------- SwiGLU as its own pass (layers.py:78-87), for callers that
 * keep the W_ug GEMM's plain bf16 output: ug bf16 [rows, 2F] = (up | gate); z bf16 [rows, F] = up * silu(gate);
 * backward: dug = (dz * gate*sigmoid(gate) | dz * up * d silu(gate)).  The same arithmetic exists as GEMM
 * epilogues (RTE_EPI_SWIGLU_FWD/BWD); the step picks whichever is faster at its size.                         */
int rte_swiglu_fwd(const void* ug, void* z, int64_t rows, int32_t F, rte_stream_t stream);
int rte_swiglu_bwd(const void* ug, const void* dz, void* dug, int64_t rows, int32_t F, rte_stream_t stream);

/* -------------------------------------------------- fp32 -> bf16 shadow copies of weights */
int rte_cast_f32_bf16(const float* src, void* dst, int64_t n, rte_stream_t stream);
int rte_add_f32(float* dst, const float* src, int64_t n, rte_stream_t stream);   /* dst += src */
int rte_fill_f32(float* dst, float value, int64_t n, rte_stream_t stream);        /* dst[:] = value */
int rte_axpy_rows_f32(float* dst, const float* vec, float alpha, int32_t rows, int32_t seg, int32_t d,
                      rte_stream_t stream);  /* dst[r,:] += alpha * vec[r / seg, :] */

/* ------------------------------- fused multi-tensor AdamW (training.py:341-354,445-468)
 * torch.optim.AdamW semantics per tensor: p *= 1 - lr*wd; m,v EMA; bias correction with the
 * tensor's own step count; p -= lr/bc1 * m / (sqrt(v)/sqrt(bc2) + eps).  Tensors absent from the
 * table are untouched (the reference skips grad-less parameters).  One launch for all tensors.
 * table: device array of rte_adamw_tensor; lr_table f32 [n_groups] on device (LR schedule is written
 * there by the host); step_count int32 [n_tensors] on device, incremented by the kernel.
 * grad_scale: device f32 scalar multiplied into every gradient (clip coefficient / 1/world), or NULL.
 * bf16_shadow (per tensor, may be NULL) receives the updated weights as bf16 for the next forward.   */
typedef struct rte_adamw_tensor {
  float* p; const float* g; float* m; float* v; void* bf16_shadow;
  int64_t n; int32_t lr_group; int32_t step_slot;
} rte_adamw_tensor;
int rte_adamw_multi_tensor(const rte_adamw_tensor* table, int32_t n_tensors, int64_t total_chunks,
                           const int32_t* chunk_tensor, const int32_t* chunk_index, const float* lr_table,
                           int32_t* step_count, float beta1, float beta2, float eps, float weight_decay,
                           const float* grad_scale, rte_stream_t stream);
enum { RTE_ADAMW_CHUNK = 4096 };
/* The same update with the optional parts of the reference's `_finish_step` (training.py:445-468, 386-443):
 *  skip: device int32; non-zero makes the launch a no-op (no parameter, moment, shadow or step-count change): the
 *        step whose loss was not finite is dropped.  Written by rte_nonfinite_guard.
 *  metric_out f32 [n_metric_groups][2]: sum of (grad_scale*g)^2 and of p^2 (before the update) per metric group,
 *        metric_group int32 [n_tensors] (device) naming each table tensor's group; metric_partial f32
 *        [total_chunks][2] is scratch.  All three NULL = no metrics.  Deterministic two-stage sums.          */
typedef struct rte_adamw_extras {
  const int32_t* skip;
  float* metric_partial;
  const int32_t* metric_group;
  float* metric_out;
  int32_t n_metric_groups;
  /* tensors that may receive NO gradient in a step (the recurrent core when the Bernoulli sampler audited nobody):
   * while *absent_flag != 0 the tensors with absent_mask[i] != 0 are left untouched -- no decay, no moment update, no
   * step count -- as torch.optim.AdamW skips `grad is None`.  Both NULL = every tensor has a gradient.           */
  const int32_t* absent_flag;
  const uint8_t* absent_mask;   /* [n_tensors], device */
} rte_adamw_extras;
int rte_adamw_multi_tensor_ex(const rte_adamw_tensor* table, int32_t n_tensors, int64_t total_chunks,
                              const int32_t* chunk_tensor, const int32_t* chunk_index, const float* lr_table,
                              int32_t* step_count, float beta1, float beta2, float eps, float weight_decay,
                              const float* grad_scale, const rte_adamw_extras* extras, rte_stream_t stream);
/* *skip = 1 if any of a[0..na), b[0..nb) or c[0..nc) is NaN or infinite, else 0 (`torch.isfinite(loss)`,
 * training.py:448, applied to the pieces the loss is assembled from); *flag_out (optional f32) receives the same as
 * 1.0 / 0.0.  Ranges with a zero count may be NULL.                                                          */
int rte_nonfinite_guard(const float* a, int32_t na, const float* b, int32_t nb, const float* c, int32_t nc,
                        int32_t* skip, float* flag_out, rte_stream_t stream);
/* dst += src unless *skip != 0 (gradient accumulation over micro-batches, training.py:445-455: a micro-batch whose loss
 * is not finite contributes nothing).                                                                         */
int rte_add_f32_guarded(float* dst, const float* src, int64_t n, const int32_t* skip, rte_stream_t stream);
/* sumsq[0] = sum over all table tensors of g^2 (deterministic two-stage); clip_coef[0] =
 * min(1, max_norm / (sqrt(sumsq) + 1e-6)) (torch.nn.utils.clip_grad_norm_, training.py:456-462).
 * partial f32 >= total_chunks.                                                                       */
int rte_grad_norm_multi_tensor(const rte_adamw_tensor* table, int64_t total_chunks, const int32_t* chunk_tensor,
                               const int32_t* chunk_index, float* partial, float* sumsq, float max_norm,
                               float* clip_coef, rte_stream_t stream);

/* ------------------------------------------------ vocabulary shortlist (output.py:46-136, `recursive_macro_shortlist`)
 * rte_shortlist_build: shortlist int32 [rows, K] = the first K distinct ids, in order of first appearance, of
 *   [target | members of the TC top clusters (cluster c = ids c, c+C, ...; ceil(V/C) slots each, padded with id 0) |
 *    hard negatives 0..HN-1 (mod V) | random_negs[row, 0..RN) | filler 0..K-1 (mod V) | (target + 0..2K-1) mod V]
 *   (= ShortlistHead.build_shortlist + _dedupe_preserve_first; the target is always slot 0).
 *   top_clusters int32 [rows, TC] (e.g. from rte_topk_lowest_index over the cluster-router logits);
 *   dup_count int32 [rows] (optional) = candidates minus distinct candidates.  Indices are bit-exact.
 * rte_shortlist_ce: logits[k] = hidden . W[shortlist[k]] (k_logits_shortlist, reference.py:141-143), cross entropy
 *   against slot 0 -> loss_tok; logits_out bf16 [rows, K] optional; dlogits_dense bf16 [rows, V] (optional) receives
 *   row_weight[row/S] * (softmax - onehot(0)) at the shortlisted ids and zero elsewhere.
 * rte_random_tokens: counter-based pseudo-random ids in [0, vocab) from a device-resident seed.                 */
int rte_shortlist_build(const int64_t* targets, const int32_t* top_clusters, const int32_t* random_negs,
                        int32_t* shortlist, int32_t* dup_count, int32_t rows, int32_t V, int32_t C, int32_t TC,
                        int32_t HN, int32_t RN, int32_t K, int32_t* status, rte_stream_t stream);
int rte_shortlist_ce(const void* hidden, const void* W, const int32_t* shortlist, const float* row_weight, int32_t S,
                     float* loss_tok, void* logits_out, void* dlogits_dense, int32_t rows, int32_t d, int32_t V,
                     int32_t K, rte_stream_t stream);
/* rte_shortlist_ce with the dot products taken from FULL logits (bf16 [rows, V], e.g. hidden . W^T from rte_gemm_bf16):
 * the same loss and the same dense gradient, written in place over the logits row.  While the vocabulary is small
 * one GEMM over all V columns is cheaper than gathering K weight rows per token (2*d*V FLOP against K*d*2 bytes).  */
int rte_shortlist_ce_from_logits(void* logits_inout, const int32_t* shortlist, const float* row_weight, int32_t S,
                                 float* loss_tok, int32_t rows, int32_t V, int32_t K, rte_stream_t stream);
int rte_random_tokens(int32_t* out, int64_t n, int32_t vocab, const int64_t* seed, rte_stream_t stream);
/* dense bf16 [rows, V] = 0 except dense[r, ids[r, k]] = vals[r, k] (ids distinct per row): turns a gradient over
 * shortlist slots (backward of k_logits_shortlist, reference.py:141-143) into rows the dense GEMMs can consume. */
int rte_scatter_cols_bf16(const void* vals, const int32_t* ids, void* dense, int32_t rows, int32_t V, int32_t K,
                          rte_stream_t stream);

/* ------------------------------------------------ static cluster-pool sparse FFN (layers.py:188-220;
 * kernels/cluster_pool_ffn.py:90-241).  The pooled SwiGLU itself runs as rte_gemm_bf16 in grouped mode.
 * rte_cluster_route: assignments[t] = argmax_c q[t,:] . centers[c,:] with the lowest index on ties
 *   (route_to_static_centers; q = x @ [up_a | gate_a] from a GEMM; the reference's L2 normalisation of q is a
 *   positive per-token scale and cannot change the arg-max).  scores_out f32 [n, C] optional.
 * rte_cluster_pack: stable counting sort of tokens by cluster (build_static_pack_gather_indices) into one packed
 *   row order where cluster c owns rows [offsets[c], offsets[c] + counts[c]) and offsets are multiples of 128:
 *   perm int32 [capacity] (packed row -> token, -1 = padding), pos int32 [n] (token -> packed row),
 *   tile_group int32 [capacity/128] and kblocks int32 [C+1] for rte_gemm_bf16's grouped / ragged-split modes.
 *   capacity_rows >= n rounded up to 128, plus 128 per cluster, always suffices; overflow sets *status (202).
 * rte_gather_rows_convert: dst[i,:] = src[idx[i],:] converted f32<->bf16, zeros where idx[i] < 0.
 * rte_csr_row_reduce_f32: dense[f,:] (+)= sum_k src[rows[k],:], k in [row_ptr[f], row_ptr[f+1]) in that order
 *   (scatter_cluster_pool_grads as a gather: no atomics, reproducible).
 * rte_transpose_f32: dst [cols, rows] (bf16 or f32, optionally +=) = src f32 [rows, cols]^T.                  */
int rte_cluster_route(const float* q, int32_t ldq, const float* centers, int32_t* assignments, float* scores_out,
                      int32_t n_tokens, int32_t width, int32_t n_clusters, rte_stream_t stream);
int rte_cluster_pack(const int32_t* assignments, int32_t n_tokens, int32_t n_clusters, int32_t capacity_rows,
                     int32_t* perm, int32_t* pos, int32_t* counts, int32_t* offsets, int32_t* tile_group,
                     int32_t* kblocks, int32_t* status, rte_stream_t stream);
int rte_gather_rows_convert(const void* src, int32_t src_bf16, const int32_t* idx, void* dst, int32_t dst_bf16,
                            int64_t n_out, int32_t d, rte_stream_t stream);
int rte_csr_row_reduce_f32(const float* src, const int32_t* row_ptr, const int32_t* rows, float* dense,
                           int64_t n_dense_rows, int32_t d, int32_t accumulate, rte_stream_t stream);
int rte_transpose_f32(const float* src, void* dst, int32_t rows, int32_t cols, int32_t dst_bf16, int32_t accumulate,
                      rte_stream_t stream);

/* ------------------------------------------------ SVD-factor sparse FFN, mask mode (layers.py:342-643;
 * kernels/svd_sparse_ffn_triton.py:480-714).  The selector factors, the exact up/gate pre-activations of all F
 * neurons and the down projection are rte_gemm_bf16 launches; this is the per-token selection between them.
 * hats f32 [rows, 2F] = (x@up_a@up_b | x@gate_a@gate_b); ug bf16 [rows, 2F] = exact (up | gate); wd_norm f32 [F] =
 * row norms of w_down.  Candidates = union of the top up_m / gate_m / product_m neurons under |up_hat|*wn,
 * |silu(gate_hat)|*wn, |up_hat*silu(gate_hat)|*wn; selected = top top_k candidates under |up*silu(gate)|*wn
 * (ties: lowest index).  z_masked bf16 [rows, F] = selected ? up*silu(gate) : 0; selected uint8 [rows, F] and
 * cand_count int32 [rows] optional.  max(up_m, gate_m, product_m) >= top_k is required.
 * rte_svd_ffn_swiglu_bwd: dug bf16 [rows, 2F] = SwiGLU backward of dz bf16 [rows, F] on selected neurons, else 0.
 * rte_row_norm_f32: out[r] = ||w[r, :]||_2.                                                                    */
int rte_svd_ffn_select(const float* hats, const void* ug, const float* wd_norm, void* z_masked, uint8_t* selected,
                       int32_t* cand_count, int32_t rows, int32_t F, int32_t up_m, int32_t gate_m, int32_t product_m,
                       int32_t top_k, rte_stream_t stream);
int rte_svd_ffn_swiglu_bwd(const void* ug, const void* dz, const uint8_t* selected, void* dug, int64_t rows, int32_t F,
                           rte_stream_t stream);
int rte_row_norm_f32(const float* w, float* out, int32_t rows, int32_t d, rte_stream_t stream);

/* ------------------------------------------------ offline cluster-pool codebook build (cli.py:3297-3389, 4703-4782)
 * The step before the static cluster-pool FFN: cosine k-means over the selector features of a calibration window,
 * per-cluster aggregation of the per-neuron pool scores, candidate lists by rte_topk_lowest_index.  All reductions
 * run in a fixed order (reproducible).
 * rte_normalize_rows_f32: out[r,:] = x[r,:] / max(||x[r,:]||, 1e-12)                      (F.normalize, cli.py:3308)
 * rte_kmeans_update: centers_new[c,:] = normalise(mean of x_normed[t,:] over assignments[t] == c); a cluster without
 *   members keeps centers_old[c,:] (normalised) (cli.py:3315-3322); counts int32 [C] optional; W <= 256.
 *   One k-means round = rte_cluster_route (assignment, ties to the lowest centre) + this.
 * rte_cluster_aggregate: out[c,:] = mean (use_max = 0) or max (1) of scores[t,:] over the members of c, zeros for an
 *   empty cluster (cli.py:3326-3351).
 * rte_cluster_pool_scores: out[t,j] = wd_norm[j] * (|up| + |silu(gate)| + |up*silu(gate)|) (mode 0 "sum"),
 *   (|up| + |silu(gate)|) (1 "upgate") or |up*silu(gate)| (2 "product") of the low-rank estimates up_hat / gate_hat
 *   f32 [n, F] (cli.py:3369-3385).                                                                               */
int rte_normalize_rows_f32(const float* x, float* out, int32_t n, int32_t W, rte_stream_t stream);
int rte_kmeans_update(const float* x_normed, const int32_t* assignments, const float* centers_old, float* centers_new,
                      int32_t* counts, int32_t n, int32_t W, int32_t C, rte_stream_t stream);
int rte_cluster_aggregate(const float* scores, const int32_t* assignments, float* out, int32_t n, int32_t F, int32_t C,
                          int32_t use_max, rte_stream_t stream);
int rte_cluster_pool_scores(const float* up_hat, const float* gate_hat, const float* wd_norm, float* out, int64_t n,
                            int32_t F, int32_t mode, rte_stream_t stream);

/* ------------------------------------------------ exact-audit replay helpers (audit.py:245-387; models.py:605-679;
 * layers.py:831-870).  The audited subset has a fixed size n (fixed-count sampler), chosen on the host.
 * Per-sample recipe choices stay on the device: every kernel below looks the recipe of (pass, sample) up in
 * `rid` and applies the recipe's column mask (already multiplied by 1/len(banks) when the bank takes part, 0 when
 * not) from a table [R, cols], so tensor shapes never depend on the routing decision.                           */
/* dst[i, :] = src[idx[i], :], rows of row_bytes bytes (multiple of 16, 16-byte aligned). */
int rte_gather_rows(const void* src, const int32_t* idx, void* dst, int32_t n, int64_t row_bytes, rte_stream_t stream);
/* dst[idx[i], :] += src[i, :] (f32; idx entries distinct). */
int rte_scatter_add_rows_f32(float* dst, const int32_t* idx, const float* src, int32_t n, int64_t row_elems,
                             rte_stream_t stream);
/* rid_out[t, i] = recipe_id_by_pass[idx[i], t];  active_out[t, i] = depth[idx[i]] > t. */
int rte_audit_route(const int32_t* recipe_id_by_pass, const int32_t* depth, const int32_t* idx, int32_t* rid_out,
                    int32_t* active_out, int32_t n, int32_t T, rte_stream_t stream);
/* out[r, c] = x[r, c] * table[rid[r / S], c]   (bf16 in/out; used for y and, in backward, for dy) */
int rte_colmask_mul_bf16(const void* x, const int32_t* rid, const float* table, int32_t S, void* out, int32_t rows,
                         int32_t cols, rte_stream_t stream);
/* z[r, j] = up*silu(gate)*table[rid[r/S], j] from ug = (up | gate) [rows, 2F];  backward writes dug [rows, 2F]. */
int rte_swiglu_masked_fwd(const void* ug, const int32_t* rid, const float* table, int32_t S, void* z, int32_t rows,
                          int32_t F, rte_stream_t stream);
int rte_swiglu_masked_bwd(const void* ug, const void* dz, const int32_t* rid, const float* table, int32_t S, void* dug,
                          int32_t rows, int32_t F, rte_stream_t stream);
/* out = base + (*scale) * branch  where `active` (per sample, may be NULL) holds, else out = passthrough.
 * base/branch/passthrough/out f32 [n*S*d] (out may alias base).  layers.py:831-852,862-870.                      */
int rte_scaled_residual_fwd(const float* base, const float* branch, const float* scale, const int32_t* active,
                            const float* passthrough, float* out, int32_t n, int64_t sample_elems, rte_stream_t stream);
/* Backward of the above for gradient dout: dbase (=) dout where active else 0 (may alias dout);
 * dbranch_bf16 = scale*dout where active else 0 (NULL to skip); dbranch_f32_accum += scale*dout (NULL to skip);
 * dpassthrough += dout where inactive (NULL if no mask); dscale_partial[blockIdx] = sum dout*branch over active
 * samples (one f32 per CTA; *n_partials CTAs, host value).  frozen_active / frozen_src (both or neither): dbase
 * additionally receives frozen_src where frozen_active[sample] == 0 -- the hand-through of samples that were
 * frozen in the pass, folded into the pass's last launch.                                                      */
int rte_scaled_residual_bwd(const float* dout, const float* branch, const float* scale, const int32_t* active,
                            float* dbase, void* dbranch_bf16, float* dbranch_f32_accum, float* dpassthrough,
                            float* dscale_partial, int32_t max_partials, int32_t* n_partials,
                            const int32_t* frozen_active, const float* frozen_src, int32_t n,
                            int64_t sample_elems, rte_stream_t stream);
/* Distillation terms of the audited samples (macro.py:394-469, delta objective) and their gradient wrt the hot
 * endpoint.  hot/exact/h0 f32 [n, S, d].  terms f32 [n, 4] = per-sample (1 - cos, log-rms diff^2, sum smooth_l1 of
 * normed rows, sum smooth_l1 raw); dhot f32 [n,S,d] = gradient of
 *   l_dir*mean(1-cos) + l_rms*mean(diff^2) + l_normed*mean_elem(sl1 normed) + l_raw*mean_elem(sl1 raw).          */
int rte_macro_distill(const float* hot, const float* exact, const float* h0, float l_dir, float l_rms, float l_normed,
                      float l_raw, float* terms, float* dhot, int32_t n, int32_t S, int32_t d, rte_stream_t stream);
/* KL(exact || hot) at temperature temp per token row; adds coef*(p_hot - p_exact) into the rows
 * idx[i]*S + s of dlogits_hot (bf16).  hot/exact logits bf16 [n*S, V]; kl_rows f32 [n*S].                        */
int rte_kl_distill(const void* hot_logits, const void* exact_logits, float temp, float coef, const int32_t* idx,
                   int32_t S, void* dlogits_hot, int32_t ld_dlogits, float* kl_rows, int32_t rows, int32_t V,
                   rte_stream_t stream);
/* The same term with the gradient kept apart: dgrad f32 [rows, V] = coef*(p_hot - p_exact), to be added to the hot
 * dlogits by rte_add_rows_f32_to_bf16 once the hot pass's cross-entropy kernel has written them (the two then run
 * on different streams; the sum and its single bf16 rounding are those of rte_kl_distill).  dgrad may be NULL: only
 * the rows' KL is written.  kl1_rows (optional, f32 [rows]): the same divergence at temperature 1, the quantity
 * macro_alignment_metrics reports (macro.py:538-543), computed in the same pass over the rows.                      */
int rte_kl_distill_grad(const void* hot_logits, const void* exact_logits, float temp, float coef, float* dgrad,
                        float* kl_rows, float* kl1_rows, int32_t rows, int32_t V, rte_stream_t stream);
/* Residual clip of the control variate (audit.py:306-321): corrected = hot + clamp(exact - hot, -clip, clip) / p.
 * For each audited sample j (hot row idx[j]) with |exact - hot| <= clip: f_hot = 1 - inv_p, f_exact = 1; otherwise
 * f_hot = 1, f_exact = 0 -- the factors to apply (rte_scale_rows_bf16) to cross-entropy gradients that were written
 * with the weights 1 (hot) and 1/p (exact).                                                                        */
int rte_audit_clip(const float* hot_loss, const float* exact_loss, const int32_t* idx, int32_t n, float inv_p,
                   const float* inv_p_slot /* per-sample 1/p, or NULL: inv_p for all */, float clip, float* f_hot,
                   float* f_exact, rte_stream_t stream);
/* Bernoulli audit sampler with adaptive probability and cap (AuditEngine.compute_audit_prob / sample_mask_with_prob /
 * _update_audit_coverage, audit.py:62-132), on the device so that the audited subset can depend on this step's routing:
 *   p_b = clamp(p_min + alpha * entropy_b * inv_r_plus_k + beta * recent[0] + gamma * deficit(recipe_b), p_min, p_max),
 *   audited_b = u_b < p_b (u: the uniforms of torch.bernoulli, drawn by the host from the step's seed); with cap >= 0 and
 *   more candidates than cap, the candidates at positions perm_table[candidates - cap - 1][0..cap) of the ascending
 *   candidate list, inclusion probability p_b * cap / candidates.
 * The replay has n_cap slots: idx[j] = idx_scatter[j] = j-th audited sample (ascending), valid[j] = 1, inv_p[j] = 1 / p_inc,
 * dist_scale[j] = n_cap / audited, row_weight_a[j] = w0 / p_inc; unused slots: idx 0 (gathers stay in range),
 * idx_scatter -1 (rte_scatter_add_rows_f32, rte_add_rows_f32_to_bf16 and rte_scale_rows_bf16 skip negative
 * indices), weights 0.  row_weight[b] =
 * w0 * (1 - 1/p_inc) on audited rows when weight_mode = 1, else w0.  ema[R] (audit-coverage average) is read, then
 * updated.  stats = (candidates, audited, mean requested p, mean inclusion p).  More audited samples than n_cap set
 * *status to 202.  B <= 1024, R <= 64.                                                                              */
typedef struct rte_audit_sample_params {
  float p_min, p_max, alpha, beta, gamma, coverage_min, coverage_beta, inv_r_plus_k, w0;
  int32_t B, R, cap, n_cap, weight_mode;
} rte_audit_sample_params;
int rte_audit_sample_bernoulli(const float* entropy, const int32_t* recipe_id, const float* u, const int32_t* perm_table,
                               float* ema, const float* recent, const rte_audit_sample_params* prm, int32_t* idx,
                               int32_t* idx_scatter, float* valid, float* inv_p, float* dist_scale, float* row_weight,
                               float* row_weight_a, float* stats,
                               int32_t* none_audited /* optional: 1 when nobody was audited, else 0 */, int32_t* status,
                               rte_stream_t stream);
/* Per audited sample j the sums behind macro_alignment_metrics (macro.py:499-546): with a = macro endpoint, b = exact
 * endpoint, z = h0 (rows of row_len floats): out[j][0..7) = (a.b, a.a, b.b, |a-b|^2, |a-z|^2, |b-z|^2, (a-z).(b-z));
 * out[j][7] is left as it is (the caller's: the engine keeps the summed temperature-1 logit KL in out[0][7]).       */
int rte_audit_alignment_sums(const float* hot_end, const float* exact_end, const float* h0, int32_t n, int64_t row_len,
                             float* out, rte_stream_t stream);
/* x[j, 0..row_len) *= factor[j], j < n (fp32).                                                                      */
int rte_scale_rows_f32(float* x, const float* factor, int32_t n, int64_t row_len, rte_stream_t stream);
/* recent[0] = max(1 - mean over valid slots of cosine(hot_end_j, exact_end_j), 0) (audit.py:213-218; rows of row_len
 * floats, F.cosine_similarity with eps 1e-8); unchanged when no slot is valid.  cos_scratch: n floats.              */
int rte_audit_recent_residual(const float* hot_end, const float* exact_end, const float* valid, int32_t n, int64_t row_len,
                              float* cos_scratch, float* recent, rte_stream_t stream);
/* x[row_of(r) * ld + c] = bf16(x[...] * scale[r / S]),  r < rows, c < V;  row_of(r) = idx ? idx[r / S] * S + r % S : r */
int rte_scale_rows_bf16(void* x_bf16, int32_t ld, const int32_t* idx, int32_t S, const float* scale, int32_t rows, int32_t V,
                        rte_stream_t stream);
/* dst[(idx[r / S] * S + r % S) * ld + c] = bf16(dst[...] + src[r * V + c]),  r < rows, c < V                      */
int rte_add_rows_f32_to_bf16(void* dst_bf16, int32_t ld, const int32_t* idx, int32_t S, const float* src, int32_t rows,
                             int32_t V, rte_stream_t stream);

/* ------------------------------------------------ gradient exchange over NVLink peer memory (data parallelism)
 * Replaces the NCCL all-reduce a DistributedDataParallel wrapper of the reference would issue per gradient bucket
 * (the reference has no multi-GPU path of its own; its gradient-accumulation parity, tests/test_training_fixes.py:53-75,
 * is the arithmetic this reproduces across ranks).
 * rte_peer_allreduce_sum_f32: in place, buf[q][offset .. offset+n) <- sum over ranks, on every rank, by ONE kernel per
 * rank; everything that crosses the link is a plain peer store (each rank pushes its values of the other ranks' parts
 * into their staging buffers, sums its own part locally in rank order, and stores the result into every buffer).  All
 * ranks must launch it with the same (offset, n, slot).  `buf[q]` / `stage[q]` / `flags[q]` are THIS process's mappings
 * (rte_peer_open) of rank q's gradient buffer, staging buffer (as large as the gradient buffer plus
 * 4 * RTE_COMM_MAX_RANKS floats) and flag array (uint32 [RTE_COMM_MAX_SLOTS][2][RTE_COMM_MAX_RANKS], zero-initialised
 * once); `epoch` (uint32 [RTE_COMM_MAX_SLOTS]) and `done_count` (uint32 [RTE_COMM_MAX_SLOTS][2]) are this rank's own,
 * zero-initialised.  `slot` separates exchanges that may be in flight at the same time; such exchanges must also be
 * at least 4 * RTE_COMM_MAX_RANKS floats apart in the buffer (a part's row in the staging buffer may overhang the range
 * by that much).  Sums run in rank order, so every rank ends with bit-identical values.  Waits on peers are bounded; on
 * expiry *status becomes 104 and the range is left unreduced.  n and offset are multiples of 4; max_ctas (0 = 64)
 * bounds the grid. */
enum { RTE_COMM_MAX_RANKS = 8, RTE_COMM_MAX_SLOTS = 64 };
typedef struct rte_peer_comm {
  float* buf[RTE_COMM_MAX_RANKS];
  float* stage[RTE_COMM_MAX_RANKS];
  uint32_t* flags[RTE_COMM_MAX_RANKS];
  uint32_t* epoch;
  uint32_t* done_count;
  int32_t world, rank;
} rte_peer_comm;
int rte_peer_allreduce_sum_f32(const rte_peer_comm* comm, int64_t offset, int64_t n, int32_t slot, int32_t max_ctas,
                               int32_t* status, rte_stream_t stream);

/* Device memory the other ranks of the node can map (what rte_peer_comm's pointers point into).
 * rte_peer_alloc: zero-filled allocation on the current device plus its 64-byte inter-process handle (send the
 *   handle to the peers by any host channel).  rte_peer_free releases it, after every peer has closed its mapping.
 * rte_peer_open: maps a peer's allocation for kernels of the CURRENT device (`owner_device` = the owner's device
 *   ordinal, or -1 to skip the can-access check; RTE_ERR_UNSUPPORTED when the two devices have no peer path).
 *   rte_peer_close unmaps it. */
enum { RTE_IPC_HANDLE_BYTES = 64 };
int rte_peer_alloc(int64_t bytes, void** ptr, uint8_t* handle);
int rte_peer_open(const uint8_t* handle, int32_t owner_device, void** ptr);
int rte_peer_close(void* ptr);
int rte_peer_free(void* ptr);

/* Global gradient norm and clip coefficient WITHOUT any caller-provided or allocated scratch.
 * (No counterpart in the reference: it exists for embedders of this library, see below.)
 * Same outputs as rte_grad_norm_multi_tensor.  The per-chunk partial sums live in a 256 KB array built into
 * the library, so this is the variant for callers that own no spare device memory and must not create any:
 * a clipping hook bound from another language into the reference's `_finish_step`, say, holds only the
 * parameter and gradient pointers the framework gave it, while the framework's caching allocator owns the
 * rest of the device -- a raw cudaMalloc there can fail outright, and it stalls the whole device.
 * Limits and rules:
 *  - total_chunks <= 65536 (268M gradient elements); larger tables return RTE_ERR_SCRATCH_CAPACITY.
 *  - the first call on each device resolves the array's device address on the host; make that first call
 *    with the right device current and outside any stream capture.
 *  - every GPU that loads the library holds the array until the process exits.
 *  - calls on the same device share the array: do not let two of them overlap on the GPU (issue them on
 *    one stream, or order the streams), otherwise they race.  Nothing needs clearing between calls.       */
int rte_grad_norm_multi_tensor_static(const rte_adamw_tensor* table, int64_t total_chunks,
                                      const int32_t* chunk_tensor, const int32_t* chunk_index, float* sumsq,
                                      float max_norm, float* clip_coef, rte_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* RTE_B200_H_ */
