/*
 * lewi_moe.h -- C ABI of liblewi_moe.so: the MoE-layer hot path of Lewi Surge as sm_100a CUDA kernels.
 *
 * Conventions (all entry points):
 *   - every pointer is a DEVICE pointer unless the parameter name ends in `_host`;
 *   - `stream` is a cudaStream_t passed as void*; calls only enqueue work, never synchronise,
 *     never allocate: the caller owns inputs, outputs and workspaces;
 *   - return value: 0 = enqueued; negative = rejected argument (nothing was launched);
 *     device-side problems (a bounded wait that ran out, an index out of range) are recorded in a
 *     per-device status word read with lewi_last_status();
 *   - row-major tensors; `bf16` = __nv_bfloat16 bits; dtype codes LEWI_BF16 / LEWI_F32.
 *
 * Slot numbering: routed slot i = t*k + j (token t, j-th choice), as in the reference's
 * `selected_experts.reshape(-1)` (modal/moe_permute.py:401).
 *
 * Padded-block layout: the rows of expert e occupy padded rows [pad_offsets[e], pad_offsets[e+1]),
 * every group start is a multiple of `block` (128); unused rows of the last block of a group are
 * zero rows.  Static bound on padded rows: lewi_padded_rows_bound().
 */
#ifndef LEWI_MOE_H_
#define LEWI_MOE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LEWI_BF16 0
#define LEWI_F32 1

/* error codes (negative return values) */
#define LEWI_OK 0
#define LEWI_ERR_ARG (-1)       /* null pointer / non-positive size / unsupported dtype          */
#define LEWI_ERR_SHAPE (-2)     /* shape not supported by the kernels (alignment, limits)        */
#define LEWI_ERR_WORKSPACE (-3) /* workspace too small                                           */
#define LEWI_ERR_CUDA (-4)      /* a CUDA runtime / driver call failed at launch                 */
#define LEWI_ERR_LIMIT (-5)     /* size beyond a compiled-in maximum                             */
#define LEWI_ERR_STATIC_SCRATCH (-6) /* problem does not fit the built-in scratch (static variant) */

/* device status bits (lewi_last_status) */
#define LEWI_STATUS_WAIT_TIMEOUT 1 /* a bounded device-side wait ran out */
#define LEWI_STATUS_BAD_INDEX 2    /* an index read from a table was out of range and skipped */
#define LEWI_STATUS_EP_OVERFLOW 4  /* expert-parallel receive buffer too small for the routed rows (rows dropped) */
#define LEWI_STATUS_SMEM_LAYOUT 8  /* a GEMM kernel found its shared memory not 1024-byte aligned and did nothing */

int lewi_version(void);
const char* lewi_error_string(int code);

/* Number of kernels this library has launched in this process (host-side counter; not thread-safe). */
int64_t lewi_launch_count(void);

/* Reads (and clears) the status word of the current device.  Synchronises `stream`. */
int lewi_last_status(void* stream);

/* Static bound on padded rows: floor((m + num_experts*(block-1)) / block) * block. */
int64_t lewi_padded_rows_bound(int64_t m, int num_experts, int block);

/* Bytes of scratch that lewi_router_topk / lewi_sort_indices need for M = T*k slots.  The bound is deliberately
 * conservative (it assumes the smallest chunk the kernels ever use, 128 slots); lewi_router_topk actually works in
 * chunks of 128*k slots and touches about 1/k of it. */
int64_t lewi_route_workspace_bytes(int64_t num_slots, int num_experts);

/* ------------------------------------------------------------------------------------------------
 * Router.  Replaces the router of maxtext.layers.moe.RoutedMoE as configured by
 * configs/stage1.yml:33-41 (softmax -> top-k -> renormalise), plus the slot sort of
 * modal/moe_permute.py:240-264 and the padded-block table, in one call.
 * ---------------------------------------------------------------------------------------------- */

/* logits[T,E] (f32) = x[T,d] (bf16) . w_router[d,E] (f32) (+ bias[E] if not null), f32 accumulate.
 * With a workspace of lewi_router_logits_workspace_bytes(d,E) bytes (and d, E multiples of 64) the
 * product runs on the tensor cores without losing float32 precision: the weight is split into
 * three bf16 pieces whose sum is the f32 value, and every bf16 x bf16 product is exact in f32.
 * Without a workspace a CUDA-core float32 kernel is used. */
int64_t lewi_router_logits_workspace_bytes(int d, int E);
int lewi_router_logits(void* stream, const void* x, const float* w_router, const float* bias,
                       float* logits, int64_t T, int d, int E, void* workspace,
                       int64_t workspace_bytes);

/* Fused softmax + top-k + renormalise + stable counting sort + block table.
 *   logits   f32 [T,E]
 *   topk_idx i32 [T,k]  experts by probability descending, lower index first on ties
 *   topk_w   f32 [T,k]  renormalised probabilities
 *   counts i32 [E], offsets i32 [E+1], pad_offsets i32 [E+1]
 *   block_expert i32 [Mpad/block] (-1 past n_blocks), n_blocks i32 [1]
 *   order i32 [M], pos i32 [M]      exactly sort_indices() of the reference (pos = inverse of order)
 *   pad_pos i32 [M]                 padded row of slot i
 *   row_slot i32 [Mpad]             slot held by padded row r, -1 for a padding row
 *   probs_sum f32 [E] or null       column sums of the soft-max probabilities (for the load-balance loss)
 *   aux_loss f32 [1] or null        load-balance loss E * sum_e (counts[e] / (T*k)) * (probs_sum[e] / T), unweighted
 *                                   (configs/stage1.yml:41 weights it by load_balance_loss_weight; needs probs_sum)
 */
int lewi_router_topk(void* stream, const float* logits, int64_t T, int E, int k, int block,
                     int32_t* topk_idx, float* topk_w, int32_t* counts, int32_t* offsets,
                     int32_t* pad_offsets, int32_t* block_expert, int32_t* n_blocks, int32_t* order,
                     int32_t* pos, int32_t* pad_pos, int32_t* row_slot, float* probs_sum, float* aux_loss,
                     void* workspace, int64_t workspace_bytes);

/* lewi_router_topk without a workspace argument.  It has no counterpart in the reference: it exists
 * for callers that are not allowed to allocate device memory and have no scratch buffer to hand in --
 * for example a custom-call handler running under a compiled XLA program, where every buffer was
 * planned when the program was compiled, or a host runtime with a fixed memory budget that forbids
 * cudaMalloc on its serving path.  The scratch is a fixed array inside the library image
 * (lewi_router_topk_static_max_bytes() bytes, currently 4 MiB, resident on every GPU that loads the
 * library until the process exits).  Inputs, outputs and semantics are exactly those of
 * lewi_router_topk.
 *   - The problem must satisfy lewi_route_workspace_bytes(T*k, E) <= lewi_router_topk_static_max_bytes();
 *     otherwise LEWI_ERR_STATIC_SCRATCH is returned and nothing is launched.
 *   - The first call on each device looks up the array's device address (a host-side CUDA runtime
 *     query, made with that device current).  Make that first call outside any stream capture.
 *   - The call itself allocates nothing: no cudaMalloc/cudaFree, no allocating library routine.
 *   - All calls on one device share the one array and it keeps the previous call's contents; every
 *     word that is read is written first within the same call, so nothing needs clearing.  Two calls
 *     whose kernels overlap on the GPU (different streams, or different host threads) race on it:
 *     issue them on one stream or serialise them yourself. */
int64_t lewi_router_topk_static_max_bytes(void);
int lewi_router_topk_static(void* stream, const float* logits, int64_t T, int E, int k, int block,
                            int32_t* topk_idx, float* topk_w, int32_t* counts, int32_t* offsets,
                            int32_t* pad_offsets, int32_t* block_expert, int32_t* n_blocks,
                            int32_t* order, int32_t* pos, int32_t* pad_pos, int32_t* row_slot,
                            float* probs_sum);

/* sort_indices(flat_experts, num_experts, method) of modal/moe_permute.py:240-264 (both methods give
 * the same result; this is the counting sort).  Padded-layout outputs may be null (block <= 0 too). */
int lewi_sort_indices(void* stream, const int32_t* flat_experts, int64_t M, int E, int block,
                      int32_t* order, int32_t* pos, int32_t* counts, int32_t* offsets,
                      int32_t* pad_offsets, int32_t* block_expert, int32_t* n_blocks,
                      int32_t* pad_pos, int32_t* row_slot, void* workspace, int64_t workspace_bytes);

/* Gradient of the renormalised top-k weights with respect to the logits: dlogits f32 [T,E] and/or
 * a bf16 copy dlogits_bf16 [T,E] (either may be null) that feeds the tensor-core GEMMs for the
 * router-weight and input gradients. */
int lewi_router_topk_bwd(void* stream, const float* logits, const int32_t* topk_idx, const float* dw,
                         float* dlogits, void* dlogits_bf16, int64_t T, int E, int k);

/* Same, with the routing-weight gradient given as pieces: dw[t,j] = sum_p dw_partial[pad_pos[t*k+j], p]
 * (the pieces are written by lewi_grouped_gemm_dh_dswiglu_scaled).  dw may then be null; dw_out [T,k]
 * (optional) receives the summed gradient. */
int lewi_router_topk_bwd_partial(void* stream, const float* logits, const int32_t* topk_idx, const float* dw,
                                 const float* dw_partial, int dw_parts, const int32_t* pad_pos, float* dw_out,
                                 float* dlogits, void* dlogits_bf16, int64_t T, int E, int k);

/* The complete router backward.  On top of lewi_router_topk_bwd_partial:
 *   counts i32 [E] + aux_grad    adds the gradient of aux_grad * (the load-balance loss lewi_router_topk reports) to
 *                                dlogits; the token fractions counts/(T*k) are constants of that loss (counts null or
 *                                aux_grad 0: no such term);
 *   d_bias f32 [E] (optional)    column sums of dlogits = gradient of a router logit bias; needs a workspace of
 *                                lewi_router_bias_grad_workspace_bytes(T, E) bytes; summed in a fixed order. */
int64_t lewi_router_bias_grad_workspace_bytes(int64_t T, int E);
int lewi_router_topk_bwd_full(void* stream, const float* logits, const int32_t* topk_idx, const float* dw,
                              const float* dw_partial, int dw_parts, const int32_t* pad_pos, float* dw_out,
                              float* dlogits, void* dlogits_bf16, int64_t T, int E, int k,
                              const int32_t* counts, float aux_grad, float* d_bias, void* workspace,
                              int64_t workspace_bytes);

/* dst (bf16) = round-to-nearest-even(src (f32)), n elements.  Used for the bf16 copy of the f32 router
 * weight (the reference casts rhs to the lhs dtype before its GEMMs: modal/padded_gmm.py:67). */
int lewi_cast_f32_to_bf16(void* stream, const float* src, void* dst, int64_t n);

/* Row/group tables for a drop-in ragged_dot: from group_sizes[E] (rows already sorted by expert)
 * builds pad_offsets, block_expert, n_blocks, row_of_padded[Mpad] (-1 = padding) and
 * padded_of_row[M] (-1 for rows past sum(group_sizes)).  Replaces the index arithmetic of
 * modal/padded_gmm.py:51-64 with a dropless layout. */
int lewi_group_tables(void* stream, const int32_t* group_sizes, int64_t M, int E, int block,
                      int32_t* pad_offsets, int32_t* block_expert, int32_t* n_blocks,
                      int32_t* row_of_padded, int32_t* padded_of_row);

/* ------------------------------------------------------------------------------------------------
 * Gather kernels.  Replace gather_rows / gather_reduce / gather_dot of
 * modal/moe_permute.py:116-158, 214-225, 228-234.
 * ---------------------------------------------------------------------------------------------- */

/* out[i] = x[idx[i]] * scale[i] (scale may be null; multiply in f32, cast back).
 * idx[i] < 0 writes a zero row.  If idx_div > 1 the source row is idx[i] / idx_div (dispatch uses
 * order // k).  If scale_by_idx != 0, scale is indexed by idx[i] instead of i.
 * If n_rows_dev is not null only the first (*n_rows_dev * rows_per_unit) rows are produced. */
int lewi_gather_rows(void* stream, const void* x, const int32_t* idx, const float* scale, void* out,
                     int64_t n_src, int64_t m, int d, int dtype, int idx_div, int scale_by_idx,
                     const int32_t* n_rows_dev, int rows_per_unit);

/* The dispatch of `_route_activations` (modal/moe_permute.py:399-404) in token order: out[pos[t,j]] = x[t] for the k
 * slots of token t (pos i32 [T,k] = padded row of every slot), and padded rows without a slot (row_slot[r] < 0,
 * row_slot i32 [out_rows]) become zero rows.  Every output row has exactly one writer (pos is a bijection onto the
 * occupied rows), so the result is reproducible and equals lewi_gather_rows(x, row_slot, idx_div = k); each source
 * row is read once instead of k times.  bf16 rows; n_rows_dev / rows_per_unit as in lewi_gather_rows. */
int lewi_dispatch_rows(void* stream, const void* x, const int32_t* pos, const int32_t* row_slot, void* out,
                       int64_t T, int k, int d, int64_t out_rows, const int32_t* n_rows_dev, int rows_per_unit);

/* out[t] = sum_j w[t,j] * y[pos[t,j]] (+ add0[t] + add1[t]) accumulated in f32.
 * w, add0, add1 may be null.  in_dtype: dtype of y/add0/add1; out_dtype: dtype of out.
 * y has n_y_rows rows; a negative pos contributes nothing, a pos >= n_y_rows is skipped and
 * raises LEWI_STATUS_BAD_INDEX. */
int lewi_gather_reduce(void* stream, const void* y, const int32_t* pos, const float* w,
                       const void* add0, const void* add1, void* out, int64_t n, int k, int d,
                       int in_dtype, int out_dtype, int64_t n_y_rows);

/* out[t,j] = <g[t], y[pos[t,j]]> in f32. */
int lewi_gather_dot(void* stream, const void* y, const int32_t* pos, const void* g, float* out,
                    int64_t n, int k, int d, int dtype, int64_t n_y_rows);

/* ------------------------------------------------------------------------------------------------
 * Grouped GEMMs on the padded-block layout (tcgen05 tensor cores, TMEM accumulators, TMA loads).
 * Replace jax.lax.ragged_dot as patched by modal/padded_gmm.py:45-69 and modal/te_gmm.py:12-19 and
 * the expert SwiGLU of maxtext.layers.moe.RoutedMoE (weights wi_0/wi_1 [E,d,f], wo [E,f,d],
 * modal/stage2.py:338-341).  `a` has `rows` rows; row block b (128 rows) belongs to expert
 * block_expert[b]; only the first *n_blocks blocks are processed.  block_expert == null means a
 * single group (expert 0) of `rows` rows (the shared expert); then n_blocks may be null too.
 * pad_offsets i32 [E+1] (the padded row range of every expert, as the router call produces it) lets
 * the library run CTA pairs (tcgen05 cta_group::2: two SMs share one 256-row tile and each loads half
 * of the weight tile); when it is null but block_expert is given, single-CTA kernels are used.
 * K and N extents must be multiples of 8; all operands bf16.  With several groups (E > 1) a call needs
 * block_expert, or pad_offsets with CTA pairs enabled; otherwise it is rejected with LEWI_ERR_SHAPE.
 * E <= 512 when pad_offsets is given (LEWI_ERR_LIMIT beyond).
 * ---------------------------------------------------------------------------------------------- */

/* out[r, :] = a[r, :] . b[e]      a [rows,K], b [E,K,N], out [rows,N] (out_dtype), optional f32 row_scale[rows]. */
int lewi_grouped_gemm_nn(void* stream, const void* a, const void* b, void* out, const float* row_scale,
                         const int32_t* block_expert, const int32_t* n_blocks,
                         const int32_t* pad_offsets, int64_t rows, int K, int N, int E, int out_dtype);

/* out[r, :] = a[r, :] . b[e]^T    a [rows,K], b [E,N,K], out [rows,N]. */
int lewi_grouped_gemm_nt(void* stream, const void* a, const void* b, void* out, const float* row_scale,
                         const int32_t* block_expert, const int32_t* n_blocks,
                         const int32_t* pad_offsets, int64_t rows, int K, int N, int E, int out_dtype);

/* out[e] = a[rows of e]^T . b[rows of e]   a [rows,Ma], b [rows,Nb], out [E,Ma,Nb] (out_dtype).
 * pad_offsets i32 [E+1] gives each expert's padded row range (null: one group of all rows).
 * Experts without rows get zeros.  If out2 is not null, columns >= Nb/2 of the product go to
 * out2 [E,Ma,Nb/2] and out is [E,Ma,Nb/2] (used for dW_gate | dW_up from one pass).
 * workspace: optional scratch, see lewi_grouped_gemm_tn_workspace_bytes(). */
int lewi_grouped_gemm_tn(void* stream, const void* a, const void* b, void* out, void* out2,
                         const int32_t* pad_offsets, int64_t rows, int Ma, int Nb, int E,
                         int out_dtype, void* workspace, int64_t workspace_bytes);

/* Scratch that lets lewi_grouped_gemm_tn cut the contraction into parts when there are too few
 * output tiles to fill the GPU (one group, long contraction: the shared expert's and the router's
 * weight gradients).  Partial products are summed in a fixed order, so results are reproducible.
 * 0 means no split is wanted; the workspace argument may always be null. */
int64_t lewi_grouped_gemm_tn_workspace_bytes(int64_t rows, int Ma, int Nb, int E, int split_out);

/* Fused gate/up projection + SwiGLU:  g = xs.Wg[e], u = xs.Wu[e], h = silu(g)*u.
 * xs [rows,d], w_gate/w_up [E,d,f], gu [rows,2f] (g | u, bf16, may be null), h [rows,f] bf16. */
int lewi_grouped_gemm_gateup_swiglu(void* stream, const void* xs, const void* w_gate,
                                    const void* w_up, void* gu, void* h,
                                    const int32_t* block_expert, const int32_t* n_blocks,
                                    const int32_t* pad_offsets, int64_t rows, int d, int f, int E);

/* lewi_grouped_gemm_gateup_swiglu whose epilogue also multiplies h by a per-row factor:
 * h[r] *= h_scale_src[scale_idx[r]] (scale_idx[r] < 0: factor 0; scale_idx null: h_scale_src[r]).
 * With the router weights there (scale_idx = row_slot, h_scale_src = topk_w flattened) the down projection yields
 * already-weighted expert outputs and the combine (`unpermute`, modal/moe_permute.py:417-433) needs no weights.
 * gu keeps the unscaled pre-activations. */
int lewi_grouped_gemm_gateup_swiglu_scaled(void* stream, const void* xs, const int32_t* scale_idx,
                                           const float* h_scale_src, const void* w_gate, const void* w_up,
                                           void* gu, void* h, const int32_t* block_expert,
                                           const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows,
                                           int d, int f, int E);

/* Backward of the down projection fused with the SwiGLU derivative:
 * dh = dys.Wd[e]^T; dg = dh*u*silu'(g); du = dh*silu(g).  dys [rows,d], w_down [E,f,d],
 * gu [rows,2f], dgu [rows,2f] (dg | du). */
int lewi_grouped_gemm_dh_dswiglu(void* stream, const void* dys, const void* w_down, const void* gu,
                                 void* dgu, const int32_t* block_expert, const int32_t* n_blocks,
                                 const int32_t* pad_offsets, int64_t rows, int d, int f, int E);

/* Same with dh multiplied by scale_src[scale_idx[r]] (the router weight of the row's slot; indexing as in
 * lewi_grouped_gemm_gateup_swiglu_scaled) and, if dw_partial is not null,
 * dw_partial[r, p] = sum over a column range of dh_unscaled * silu(g) * u: the pieces of the routing-weight
 * gradient <dout[t], y[row]> (reference: gather_dot in `_combine_bwd`, modal/moe_permute.py:303-309).
 * dw_partial is [rows, lewi_dw_partial_parts(f)] f32. */
int lewi_dw_partial_parts(int f);
int lewi_grouped_gemm_dh_dswiglu_scaled(void* stream, const void* dys, const int32_t* scale_idx,
                                        const float* scale_src, float* dw_partial, const void* w_down,
                                        const void* gu, void* dgu, const int32_t* block_expert,
                                        const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows,
                                        int d, int f, int E);

/* dxs = dg.Wg[e]^T + du.Wu[e]^T.  dgu [rows,2f], w_gate/w_up [E,d,f], dxs [rows,d] bf16. */
int lewi_grouped_gemm_dx(void* stream, const void* dgu, const void* w_gate, const void* w_up,
                         void* dxs, const int32_t* block_expert, const int32_t* n_blocks,
                         const int32_t* pad_offsets, int64_t rows, int d, int f, int E);

/* ------------------------------------------------------------------------------------------------
 * Sequence mixing beside the MoE layer: the causal depthwise 1-D convolution of the Gated-DeltaNet block.
 * Replaces the reference's shift-add rewrite of flax `nnx.Conv(padding="CAUSAL", feature_group_count=C)`
 * (modal/fast_conv.py:14-31):  y[b,t,c] = sum_{j<K} w[j,c] * x[b, t-(K-1)+j, c], inputs before t = 0 are zero.
 * x, y, g, dx bf16 [B,T,C]; w bf16 [K,1,C] (flax kernel layout, read as [K,C]); K <= 8; C a multiple of 8.
 * Products and sums in f32, one rounding at the end.  The backward call gives dx (the same convolution run
 * backwards in time over g) and/or dw [K,C] (dw_dtype; needs lewi_causal_conv1d_workspace_bytes of scratch;
 * partial sums are added in a fixed order).
 * ---------------------------------------------------------------------------------------------- */
int64_t lewi_causal_conv1d_workspace_bytes(int B, int T, int C, int K);
int lewi_causal_conv1d_fwd(void* stream, const void* x, const void* w, void* y, int B, int T, int C, int K);
int lewi_causal_conv1d_bwd(void* stream, const void* x, const void* w, const void* g, void* dx, void* dw,
                           int dw_dtype, void* workspace, int64_t workspace_bytes, int B, int T, int C, int K);

/* Chunked gated delta rule, forward: replaces the reference's `fast_chunk_gated_delta_rule`
 * (modal/gdn_fast.py:37-113) for compute_dtype = bfloat16, chunk size 64, no context parallelism.
 *   per (batch, head):  h <- h*exp(g_t) + k_t (x) beta_t*(v_t - k_t^T h),   o_t = (q_t / sqrt(K))^T h
 * q, k bf16 [B,S,H,K]; v, o bf16 [B,S,H,V]; g f32 [B,S,H] (log decay, <= 0); beta bf16 [B,S,H];
 * h0 f32 [B,H,K,V] or null (zero state); h_final f32 [B,H,K,V] or null.  K <= 128 and a multiple of 8, V a
 * multiple of 8.  S need not be a multiple of 64 (the tail is padded with empty tokens, as the reference pads).
 * workspace: lewi_gdn_chunk_workspace_bytes(...) bytes (per-chunk u, w, in-chunk attention and cumulative decay).
 * The reference differentiates this function through JAX autodiff; lewi_gdn_chunk_bwd below is its gradient here. */
int64_t lewi_gdn_chunk_workspace_bytes(int B, int S, int H, int K, int V);
int lewi_gdn_chunk_fwd(void* stream, const void* q, const void* k, const void* v, const float* g, const void* beta,
                       const float* h0, void* o, float* h_final, void* workspace, int64_t workspace_bytes, int B,
                       int S, int H, int K, int V);

/* Backward of lewi_gdn_chunk_fwd: gradients of q, k, v, beta (bf16, shapes of the inputs), g (f32 [B,S,H]) and,
 * optionally, of the initial state (dh0 f32 [B,H,K,V], may be null) from d_o (bf16 [B,S,H,V]) and, optionally, the
 * gradient of the final state (dh_final f32 [B,H,K,V], may be null).  fwd_workspace is the workspace lewi_gdn_chunk_fwd
 * filled for the same inputs (it holds u, w, the in-chunk attention and the cumulative decay of every chunk); workspace
 * is scratch of lewi_gdn_chunk_bwd_workspace_bytes (the state at the start of every chunk, which the first kernel
 * recomputes, and per-column-block partial sums that are added in a fixed order: no atomics, reproducible).  The
 * forward pass's roundings to bf16 are kept in the values and differentiated as the identity, which is what automatic
 * differentiation of the reference's forward (modal/gdn_fast.py:37-113) does with its casts; the reference has no
 * backward of its own to compare with.  K, V <= 128, multiples of 8. */
int64_t lewi_gdn_chunk_bwd_workspace_bytes(int B, int S, int H, int K, int V);
int lewi_gdn_chunk_bwd(void* stream, const void* q, const void* k, const void* v, const float* g, const void* beta,
                       const float* h0, const void* d_o, const float* dh_final, const void* fwd_workspace,
                       int64_t fwd_workspace_bytes, void* workspace, int64_t workspace_bytes, void* dq, void* dk, void* dv,
                       float* dg, void* dbeta, float* dh0, int B, int S, int H, int K, int V);

/* ------------------------------------------------------------------------------------------------
 * The whole layer in two calls.  lewi_moe_fwd / lewi_moe_bwd queue the complete launch sequence of the MoE layer of
 * the MaxText `qwen3_5` block as the reference patches it: router (softmax -> top-k -> renormalise,
 * configs/stage1.yml:33-41) -> `_route_activations` (modal/moe_permute.py:399-404) -> the three `ragged_dot`s of the
 * SwiGLU experts (modal/padded_gmm.py:45-69) -> `unpermute` (modal/moe_permute.py:417-433), plus the always-on shared
 * expert (configs/stage1.yml:32,35), and the gradient of all of it with the gather-only structure of
 * `_combine_bwd` / `_dispatch_bwd` (modal/moe_permute.py:282-309).
 *
 * Shapes: x, out, dout, dx bf16 [T,d]; w_router f32 [d,E], router_bias f32 [E] or null; w_gate, w_up bf16 [E,d,f],
 * w_down bf16 [E,f,d] (wi_0, wi_1, wo: modal/stage2.py:338-341); shared expert ws_gate, ws_up bf16 [d,fs],
 * ws_down bf16 [fs,d] (fs = 0: no shared expert, pointers null); w_sg f32 [d] or null: optional gate of the shared
 * expert, out = routed + sigmoid(x . w_sg) * shared (the Hugging Face twin has it, tools/grow_7b.py:85; null = gate 1).
 *
 * Buffers the caller owns:
 *   residual   lewi_moe_residual_layout(...) bytes; written by fwd, read by bwd (logits, routing tables, the permuted
 *              rows xs, pre-activations g|u, h, the shared expert's g|u and h, the gate).  Item i of the
 *              LEWI_MOE_RES_* list starts at byte offsets_host[i]; offsets_host has LEWI_MOE_RES_COUNT + 1 entries,
 *              the last is the total.  The routing tables are those of lewi_router_topk.
 *   workspace  lewi_moe_workspace_bytes(...) bytes of scratch; contents are undefined after a call, and one
 *              workspace can serve fwd and bwd of any number of layers on the same stream.
 * Both buffers must be 16-byte aligned.  `has_gate` (layout functions) = whether w_sg will be passed.
 *
 * side_stream (may be null or equal to stream): the shared expert, which needs only x / dout, is queued there
 * between two events so that it overlaps the memory-bound routing, dispatch and gather kernels; the call
 * returns with `stream` waiting for it.  The four events per device are created on first use and kept.
 *
 * router_prepared (may be null): the bf16 pieces of w_router that the router GEMMs read, as written by
 * lewi_moe_prepare_router (lewi_moe_router_prepared_bytes(d,E) bytes); pass it to skip that conversion in
 * every call while the router weight is unchanged.
 *
 * aux_loss f32 [1] (may be null) receives the load-balance loss of lewi_router_topk; bwd adds aux_grad times its
 * gradient to the router gradient (aux_grad = load_balance_loss_weight x the upstream gradient of the loss; 0: none).
 * dw_topk f32 [T,k] (may be null) receives the gradient of the routing weights; d_router_bias f32 [E] (may be null);
 * dw_sg f32 [d] (given exactly when w_sg is); weight gradients of the experts and the shared expert have
 * wgrad_dtype (LEWI_BF16 or LEWI_F32), dw_router is f32 [d,E].  Experts without rows get exactly-zero gradients.
 * ---------------------------------------------------------------------------------------------- */
#define LEWI_MOE_RES_LOGITS 0       /* f32 [T,E]        */
#define LEWI_MOE_RES_TOPK_IDX 1     /* i32 [T,k]        */
#define LEWI_MOE_RES_TOPK_W 2       /* f32 [T,k]        */
#define LEWI_MOE_RES_COUNTS 3       /* i32 [E]          */
#define LEWI_MOE_RES_OFFSETS 4      /* i32 [E+1]        */
#define LEWI_MOE_RES_PAD_OFFSETS 5  /* i32 [E+1]        */
#define LEWI_MOE_RES_N_BLOCKS 6     /* i32 [1]          */
#define LEWI_MOE_RES_PROBS_SUM 7    /* f32 [E]          */
#define LEWI_MOE_RES_BLOCK_EXPERT 8 /* i32 [Mpad/128]   */
#define LEWI_MOE_RES_ORDER 9        /* i32 [T*k]        */
#define LEWI_MOE_RES_POS 10         /* i32 [T*k]        */
#define LEWI_MOE_RES_PAD_POS 11     /* i32 [T*k]        */
#define LEWI_MOE_RES_ROW_SLOT 12    /* i32 [Mpad]       */
#define LEWI_MOE_RES_XS 13          /* bf16 [Mpad,d]    */
#define LEWI_MOE_RES_GU 14          /* bf16 [Mpad,2f]   */
#define LEWI_MOE_RES_H 15           /* bf16 [Mpad,f] (times the router weight of the row) */
#define LEWI_MOE_RES_GUS 16         /* bf16 [T,2fs]     */
#define LEWI_MOE_RES_HS 17          /* bf16 [T,fs] (times the gate, if any) */
#define LEWI_MOE_RES_GATE 18        /* f32 [T] (only with w_sg) */
#define LEWI_MOE_RES_COUNT 19

int64_t lewi_moe_residual_layout(int64_t T, int d, int E, int f, int k, int fs, int has_gate,
                                 int64_t* offsets_host);
int64_t lewi_moe_workspace_bytes(int64_t T, int d, int E, int f, int k, int fs, int has_gate);
int64_t lewi_moe_router_prepared_bytes(int d, int E);
int lewi_moe_prepare_router(void* stream, const float* w_router, void* prepared, int d, int E);

int lewi_moe_fwd(void* stream, void* side_stream, const void* x, const float* w_router,
                 const float* router_bias, const void* router_prepared, const void* w_gate, const void* w_up,
                 const void* w_down, const void* ws_gate, const void* ws_up, const void* ws_down,
                 const float* w_sg, void* out, float* aux_loss, void* residual, int64_t residual_bytes,
                 void* workspace, int64_t workspace_bytes, int64_t T, int d, int E, int f, int k, int fs);

int lewi_moe_bwd(void* stream, void* side_stream, const void* dout, const void* x, const float* w_router,
                 const void* router_prepared, const void* w_gate, const void* w_up, const void* w_down,
                 const void* ws_gate, const void* ws_up, const void* ws_down, const float* w_sg,
                 const void* residual, int64_t residual_bytes, void* workspace, int64_t workspace_bytes,
                 void* dx, float* dw_router, float* d_router_bias, void* dw_gate, void* dw_up, void* dw_down,
                 void* dws_gate, void* dws_up, void* dws_down, float* dw_sg, float* dw_topk, float aux_grad,
                 int wgrad_dtype, int64_t T, int d, int E, int f, int k, int fs);

/* Profiling hook: fn(name, stream) is called on the host after each kernel (or kernel group) that lewi_moe_fwd /
 * lewi_moe_bwd queue, with the stream it went to; a timing harness records events there.  null disables (default). */
int lewi_moe_set_mark_callback(void (*fn)(const char*, void*));

/* ------------------------------------------------------------------------------------------------
 * Expert parallelism over peer memory (one process per GPU on an NVSwitch node).  The reference never ran
 * expert parallelism (configs/stage1.yml:102 keeps ici_expert_parallelism at 1), so these entry points
 * have no counterpart there; they implement the sharded form of `_route_activations` / `unpermute`.
 * Buffers that peers write or read are allocated with lewi_ep_alloc (cudaMalloc) and shared through
 * CUDA IPC handles (64 bytes each, exchanged by the host code).  `peers` arguments are HOST arrays of G
 * device pointers (index = rank; the rank's own buffer at its own index).  G <= 8.
 * ---------------------------------------------------------------------------------------------- */
int lewi_ep_alloc(int64_t bytes, void** out_host);
int lewi_ep_free(void* ptr);
int lewi_ep_ipc_export(void* ptr, void* handle64_host);
int lewi_ep_ipc_import(const void* handle64_host, void** out_host);
int lewi_ep_ipc_release(void* ptr);

/* From all ranks' expert histograms counts_all i32 [G,E] (device) computes, for rank `me`:
 *   dst_base i32 [E]            first row, in the owner's padded buffer, of this rank's rows of expert e
 *   pad_offsets i32 [E/G + 1]   this rank's own padded layout as an owner (rows source-major inside an expert)
 *   valid_end i32 [E/G]         end of the real rows of each local expert (the rest of its last block is padding)
 *   n_blocks i32 [1], block_expert i32 [rmax_pad/block] (may be null), recv_rows i32 [1]
 * Raises LEWI_STATUS_EP_OVERFLOW if the padded rows exceed rmax_pad. */
int lewi_ep_plan(void* stream, const int32_t* counts_all, int G, int E, int me, int block, int64_t rmax_pad,
                 int32_t* dst_base, int32_t* pad_offsets, int32_t* valid_end, int32_t* n_blocks,
                 int32_t* block_expert, int32_t* recv_rows);

/* Dispatch fused with the exchange: sorted position p (slot order[p], token order[p]/k, expert
 * flat_expert[slot]) is stored to row dst_base[e] + (p - offsets[e]) of peers_rows[owner]; offsets i32 [E+1].
 * With the row go slot_w[slot] (optional, f32) to peers_w[owner][row] and the row's return address
 * (me << 28 | slot, i32) to peers_ret[owner][row] (optional).  Only the rows of local experts (e mod E/G) in
 * [el_lo, el_hi) are moved: launching once per range of local experts lets the owners start on the first
 * range while the next one is still in flight.  M = T*k < 2^28.  The kernel is one small CTA per SM that
 * fits beside a resident grouped-GEMM CTA, so it overlaps GEMMs running on another stream.  threads = CTA size
 * (a multiple of 32 up to 256; 0 = 256): fewer warps keep fewer remote stores in flight per SM, which slows the
 * transfer and disturbs a GEMM on the same SM less. */
int lewi_ep_push_rows(void* stream, const void* x, const int32_t* order, const int32_t* flat_expert,
                      const int32_t* offsets, const int32_t* dst_base, const float* slot_w,
                      void* const* peers_rows_host, void* const* peers_w_host, void* const* peers_ret_host, int me,
                      int64_t M, int k, int d, int E, int G, int64_t rmax_pad, int64_t T, int el_lo, int el_hi,
                      int threads);

/* Owner side of the way back: rows [pad_offsets[el_lo], pad_offsets[el_hi]) of `rows` [rmax_pad,d] bf16 are
 * stored to row `slot` of peers_slot_rows[source] ([M,d] bf16 on every rank), slot and source taken from the
 * return addresses ret i32 [rmax_pad] (-1 = padding row, skipped).  `pieces` f32 [rmax_pad,parts] (optional)
 * go to peers_slot_pieces[source][slot, :parts].  Either of rows / pieces may be null.  On the source rank
 * the combine is then a sum over k consecutive rows (lewi_gather_reduce with the identity index).  threads as in
 * lewi_ep_push_rows. */
int lewi_ep_return_rows(void* stream, const void* rows, const float* pieces, const int32_t* ret,
                        const int32_t* pad_offsets, int el_lo, int el_hi, void* const* peers_slot_rows_host,
                        void* const* peers_slot_pieces_host, int d, int parts, int G, int64_t M, int64_t rmax_pad,
                        int threads);

/* The same way back fused into the GEMM that makes the rows: lewi_grouped_gemm_nn (down projection) and
 * lewi_grouped_gemm_dx with an epilogue that stores row r of the bf16 product to row `slot` of out_ptrs[source]
 * ([out_rows, N] bf16 each: this GPU's buffer or a peer's) for ret[r] = source << 28 | slot, and nowhere for
 * ret[r] < 0; ret is indexed like the GEMM's rows.  A tile's rows leave while the tensor cores work on the next
 * tile, the product is never written to local memory, and no separate transfer kernel runs.  out_ptrs_host: host
 * array of `ranks` (<= 8) device pointers.  Other arguments as in the GEMM they extend.  There is no reference
 * counterpart (the reference never ran expert-parallel). */
int lewi_grouped_gemm_nn_return(void* stream, const void* a, const void* b, const int32_t* ret,
                                void* const* out_ptrs_host, int ranks, int64_t out_rows, const int32_t* block_expert,
                                const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows, int K, int N, int E);
int lewi_grouped_gemm_dx_return(void* stream, const void* dgu, const void* w_gate, const void* w_up, const int32_t* ret,
                                void* const* out_ptrs_host, int ranks, int64_t out_rows, const int32_t* block_expert,
                                const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows, int d, int f, int E);

/* ---- A token travels once per destination rank instead of once per (token, expert) slot.
 * top-6 over 2 / 4 / 8 ranks: 0.99 / 2.5 / 3.9 rows per token cross NVLink instead of 3 / 4.5 / 5.25.  The owner copies
 * a received ("unique") row to the padded rows of its local experts, runs the grouped GEMMs, adds up the token's local
 * expert outputs and returns ONE partial row; the source adds the partial rows of the ranks it sent the token to
 * (lewi_gather_reduce over comb).  The exchange stays pipelined over ranges of local experts (bounds_host
 * [n_ranges+1], 0 = first, E/G = last, n_ranges <= 8): a row is pushed with the first range it is needed for and its
 * partial row returns after the last.  No reference counterpart.
 *
 * lewi_ep_unique_tables: from topk_idx [T,k] (global expert ids): info [T,G] (-1 = token not sent to that rank, else
 * first range | last range << 8), uidx [T,G] (rank of the token among those sent to the rank, token order; -1),
 * comb [T,G] (r*T + uidx: row of this rank's [G*T,d] return buffer; -1), ucount [G] (tokens sent to each rank).
 * workspace: lewi_ep_unique_workspace_bytes(T, G). */
int64_t lewi_ep_unique_workspace_bytes(int64_t T, int G);
int lewi_ep_unique_tables(void* stream, const int32_t* topk_idx, int64_t T, int k, int E, int G,
                          const int32_t* bounds_host, int n_ranges, int32_t* info, int32_t* uidx, int32_t* comb,
                          int32_t* ucount, void* workspace, int64_t workspace_bytes);
/* ucount_all [G,G] (row = source rank, gathered with lewi_ep_put_i32) -> usrc_base [G]: first row of THIS rank's unique
 * rows in every owner's buffer; utotal [1]: unique rows this rank receives (more than umax: LEWI_STATUS_EP_OVERFLOW). */
int lewi_ep_unique_plan(void* stream, const int32_t* ucount_all, int G, int me, int64_t umax, int32_t* usrc_base,
                        int32_t* utotal);
/* Stores into the owners' tables what they need besides the rows: per padded row the routing weight (w f32
 * [rmax_pad]), the slot's return address (ret, as lewi_ep_push_rows) and its unique row (rowu i32 [rmax_pad]); per
 * unique row its padded rows (urows i32 [umax,k], -1 padded), last range (umeta i32 [umax]) and return address
 * (uret i32 [umax] = source << 28 | row of the source's return buffer).  pos / offsets / dst_base as in
 * lewi_ep_push_rows (pos = sorted position of a slot). */
int lewi_ep_unique_meta(void* stream, const int32_t* topk_idx, const float* topk_w, const int32_t* pos,
                        const int32_t* offsets, const int32_t* dst_base, const int32_t* info, const int32_t* uidx,
                        const int32_t* usrc_base, void* const* peers_w_host, void* const* peers_ret_host,
                        void* const* peers_rowu_host, void* const* peers_urows_host, void* const* peers_umeta_host,
                        void* const* peers_uret_host, int me, int64_t T, int k, int E, int G, int64_t rmax_pad,
                        int64_t umax);
/* Rows x[t] of the tokens whose first range on the destination is `group` (negative: every token) go to row
 * usrc_base[r] + uidx[t,r] of peers_ux[r] ([umax,d] bf16).  Thin kernel, threads as in lewi_ep_push_rows. */
int lewi_ep_push_unique(void* stream, const void* x, const int32_t* info, const int32_t* uidx, const int32_t* usrc_base,
                        void* const* peers_ux_host, int me, int64_t T, int d, int G, int group, int64_t umax,
                        int threads);
/* Owner, local memory: out[row] = ux[rowu[row]] (zero row where rowu[row] < 0) for the padded rows of local experts
 * [el_lo, el_hi). */
int lewi_ep_local_rows(void* stream, const void* ux, const int32_t* rowu, const int32_t* pad_offsets, int el_lo, int el_hi,
                       void* out, int d, int64_t rmax_pad, int64_t umax);
/* Owner: for every unique row u < utotal[0] whose last range is `group` (negative: all), the f32 sum of rows[urows[u,:]]
 * goes as bf16 to row (uret[u] & slot mask) of peers_out[uret[u] >> 28] ([out_rows,d] bf16).  Thin kernel. */
int lewi_ep_combine_return(void* stream, const void* rows, const int32_t* urows, const int32_t* umeta,
                           const int32_t* uret, const int32_t* utotal, int group, void* const* peers_out_host, int k,
                           int d, int G, int64_t rmax_pad, int64_t out_rows, int threads);

/* Zero rows [valid_end[el], pad_offsets[el+1]) of buf [rmax_pad,d] bf16 for every local expert and, with
 * ret (i32 [rmax_pad], optional), mark them as having no return address. */
int lewi_ep_zero_pad(void* stream, void* buf, int32_t* ret, const int32_t* valid_end, const int32_t* pad_offsets,
                     int E_local, int d, int64_t rmax_pad);

/* 1: the grouped-GEMM CTAs launched from now on leave room on their SM (1 KB of shared memory, 2 warps of 40
 * registers per scheduler) for one CTA of an exchange kernel running on another stream, so that transfers overlap
 * the GEMMs; 0 (default): a GEMM CTA has its SM to itself, which measured faster when nothing needs to overlap.
 * Host-side switch read at launch time; not thread-safe against concurrent launches. */
int lewi_set_sm_sharing(int on);

/* n >= 2: the grouped-GEMM launches that follow use at most n CTAs (an odd n counts as n-1 for the CTA-pair kernels);
 * 0 (default): one CTA per SM.  With limits that add up to the SM count, two GEMMs launched on different streams run
 * side by side, each on its share of the GPU: the expert-parallel layer gives the GEMM whose epilogue sends rows to
 * peers (and therefore runs at the speed of the links) a part of the SMs and the next range's first GEMM the rest.
 * Host-side switch read at launch time; not thread-safe against concurrent launches. */
int lewi_set_gemm_cta_limit(int n);

/* All-gather of a small table by peer stores: src i32 [n] goes to elements [dst_offset, dst_offset+n) of every
 * peer's buffer (used for the expert histograms: dst_offset = me*E).  Follow it with lewi_ep_barrier. */
int lewi_ep_put_i32(void* stream, const int32_t* src, void* const* peers_dst_host, int64_t dst_offset, int n, int G);

/* Barrier between the G ranks in stream order: adds one to *epoch_counter (i32 on this device, zero-initialised;
 * it counts this rank's barriers), stores the new epoch into slot `me` of every peer's flag array (peers_flags[g],
 * i32 [G], zero-initialised, lewi_ep_alloc'ed) and waits until my_flags[g] >= epoch for every g.  Every rank must
 * run the same sequence of barriers.  Nothing is passed from the host per call, so a captured launch can be
 * replayed.  The wait gives up after timeout_ms (<= 10000) with LEWI_STATUS_WAIT_TIMEOUT in lewi_last_status();
 * the kernel then returns normally. */
int lewi_ep_barrier(void* stream, void* const* peers_flags_host, int32_t* my_flags, int32_t* epoch_counter, int me,
                    int G, int64_t timeout_ms);

/* A/B switch: 0 forces the single-CTA (cta_group::1) GEMM kernels everywhere, 1 (default) allows CTA pairs
 * (cta_group::2) where pad_offsets is given.  Host-side, read at launch time. */
int lewi_set_cta_pair(int on);

#ifdef __cplusplus
}
#endif
#endif /* LEWI_MOE_H_ */
