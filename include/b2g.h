/* C ABI of libb2g: hand-written sm_100a kernels for the GGUF-quantized LoRA path.
 *
 * Conventions
 *   - every function returns 0 on success or a negative B2G_E_* code; the message is available
 *     from b2g_last_error() on the calling thread.  Nothing throws, aborts or synchronises the
 *     device.
 *   - all tensor pointers are borrowed DEVICE pointers on the current device, row-major and
 *     contiguous; `stream` is a cudaStream_t passed as void*.  Unless a function says otherwise it
 *     allocates nothing: outputs and workspaces come from the caller.
 *   - bf16 activations / outputs, uint8 GGUF payloads in their on-disk block layout
 *     ([rows, K / block * block_bytes]); quant types use the GGML ids (8 = Q8_0, 10 = Q2_K,
 *     11 = Q3_K, 12 = Q4_K, 13 = Q5_K, 14 = Q6_K, 16 = IQ2_XXS, 22 = IQ2_S).
 *   - `status` (nullable) is a device int32 the kernels write a non-zero code into when a bounded
 *     device-side wait runs out (1xx-4xx) or an input is out of range (901 receive buffer too small, 902 label
 *     outside the vocabulary, 903 expert id outside [0, E), 904 expert offsets beyond the row count); it is
 *     never written on a healthy run and only the first code is kept.
 *
 * Each entry names the reference interface it stands in for (file:line in
 * woct0rdho/transformers5-qwen3.5-recipe).  The reference reaches these through the third-party
 * torch_ggml_ops / AITER ops, named at each entry below.
 */
#ifndef B2G_H_
#define B2G_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B2G_API __attribute__((visibility("default")))
#else
#define B2G_API
#endif

#define B2G_E_ARG (-1)     /* bad argument: shape, alignment, unsupported type */
#define B2G_E_CUDA (-2)    /* a CUDA runtime / driver call failed */
#define B2G_E_STATE (-3)   /* library state missing (e.g. IQ2_XXS grid not uploaded) */

#define B2G_Q8_0 8
#define B2G_Q4_K 12
#define B2G_IQ2_XXS 16
#define B2G_Q6_K 14
#define B2G_Q5_K 13
#define B2G_Q2_K 10
#define B2G_Q3_K 11
#define B2G_IQ2_S 22
/* OR-ed into the `qtype` argument of the matrix products: every payload row is padded to the next multiple of 16 bytes
 * (TMA needs 16-byte row pitches; 66-, 82-, 84-, 110- and 210-byte blocks give them only for some K).  b2g_dequant takes
 * plain type ids and unpadded rows only. */
#define B2G_PADDED_ROWS 0x100

#define B2G_LORA_PAD 16    /* LoRA rank operands are zero-padded to 16 columns / rows */

B2G_API const char* b2g_last_error(void);
B2G_API int b2g_abi_version(void);

/* Upload the IQ2_XXS magnitude table (256 rows x 8 bytes, HOST pointer) to the current device.
 * The table is third-party data owned by the gguf package; the caller reads it from there
 * (gguf.quants.IQ2_XXS.grid) and hands it in once per device before any IQ2_XXS call. */
B2G_API int b2g_set_iq2xxs_grid(const uint8_t* host_grid_256x8);

/* The same for IQ2_S (type 22 of the reference's allow-list, fast_lora.py:24-27): its 1024 rows x 8 bytes table
 * (gguf.quants.IQ2_S.grid), once per device before any IQ2_S call. */
B2G_API int b2g_set_iq2s_grid(const uint8_t* host_grid_1024x8);

/* Logical bf16 weight from a packed payload, bit-exact with float32 decode + round-to-nearest-even.
 * Replaces transformers.integrations.gguf_dequant.dequantize_gguf_tensor as used at
 * fast_moe_lora.py:163,235,264 and as the oracle of test_fast_lora.py:110-115. */
B2G_API int b2g_dequant(int qtype, const void* payload, int64_t rows, int64_t cols, void* out_bf16, void* stream);

/* ---- dense path ------------------------------------------------------------------------------ */

/* Y[M,N] = X[M,K] . deq(W[N,K])^T (+ bias[N]) (+ XAs[M,16] . Bp[N,16]^T).
 * Replaces torch_ggml_ops.mmq (fast_lora.py:155-160) and, with the two LoRA operands, the addmm of
 * _fused_lora_add (fast_lora.py:55-61): XAs is the already scaled s*(X.A^T) from b2g_lora_down and
 * Bp is lora_B zero-padded to 16 columns.  bias, xas/lora_b16 are nullable (xas and lora_b16 together). */
B2G_API int b2g_qlinear_fwd(int qtype, const void* x, const void* payload, const void* bias, const void* xas,
                    const void* lora_b16, void* y, int64_t M, int64_t N, int64_t K, int* status, void* stream);

/* dX[M,K] = dY[M,N] . deq(W[N,K]) (+ dYBs[M,16] . Ap[16,K]).
 * Replaces torch_ggml_ops.mmq_grad_input (registered autograd of mmq, test_fast_lora.py:104-105;
 * direct call at gguf_liger_loss.py:172) plus the LoRA input-gradient term of fast_lora.py:50-61's
 * autograd: dYBs = s*(dY.B) from b2g_lora_down, Ap = lora_A zero-padded to 16 rows. */
B2G_API int b2g_qlinear_dgrad(int qtype, const void* dy, const void* payload, const void* dybs, const void* lora_a16,
                      void* dx, int64_t M, int64_t N, int64_t K, int* status, void* stream);

/* TEST HOOK (no counterpart in the reference): b2g_qlinear_fwd without LoRA whose packed-weight producer is held back and whose
 * bounded waits give up after spin_limit polls (16..65536) instead of the library's 2^22.  The wait for packed bytes runs out,
 * every role of the kernel drains, TMEM is released, the kernel returns and *status holds 401; Y is unspecified.  It exists so
 * that the give-up path of the bounded waits can be exercised without a faulting, trapping or hanging GPU. */
B2G_API int b2g_debug_stalled_qlinear_fwd(int qtype, const void* x, const void* payload, void* y, int64_t M, int64_t N, int64_t K,
                                  int spin_limit, int* status, void* stream);

/* Fixed groups: Y[M,g,:] = X[M,g,:] . deq(W_g[N,K])^T for g < groups, with X [M, groups, K], the payload
 * [groups, N, row bytes] and Y [M, groups, N] all contiguous: `groups` independent dense products that read and write
 * column blocks of the shared tensors in place (no per-group copies), each the same kernel and the same arithmetic as
 * b2g_qlinear_fwd on a contiguous slice.  Replaces torch_ggml_ops.fixed_grouped_mmq(input[...,8,4096],
 * payload[8,1024,.]) of DeepSeek's frozen eight-group Q8_0 o_a_proj (deepseek_v4_lora.py:123); the group count, widths
 * and quant type are not fixed here (any type of this library, widths multiples of 16). */
B2G_API int b2g_fixed_grouped_fwd(int qtype, const void* x, const void* payload, void* y, int64_t M, int groups, int64_t N,
                          int64_t K, int* status, void* stream);

/* dX[M,g,:] = dY[M,g,:] . deq(W_g[N,K]): the registered autograd of fixed_grouped_mmq (the reference checks it
 * against per-group mmq_grad_input, test_deepseek_v4_lora.py:101-152). */
B2G_API int b2g_fixed_grouped_dgrad(int qtype, const void* dy, const void* payload, void* dx, int64_t M, int groups, int64_t N,
                            int64_t K, int* status, void* stream);

/* Cross-entropy of a chunk of bf16 logits [rows, V] (row pitch ld elements), IN PLACE: loss[row] = (logsumexp - logit
 * of the target) * scale and the logits are overwritten by (softmax - onehot) * scale in bf16, scale = 1 / *count for
 * mean (count: device scalar, the number of non-ignored targets of the WHOLE batch) or 1 for sum.  Rows whose target
 * is ignore_index give zero loss and zero gradient; predicted[row] (argmax, -1 when ignored) and correct[row] (0/1) are
 * optional.  Replaces the Liger Triton cross-entropy kernel that the packed LM-head loss runs between mmq and
 * mmq_grad_input (gguf_liger_loss.py:138-170, deepseek_v4_liger_loss.py:129-158).  A target outside [0, V) sets status
 * 902 and is treated as ignored. */
B2G_API int b2g_cross_entropy_inplace(void* logits, int64_t ld, const int64_t* target, float* loss, int64_t* predicted, float* correct,
                              int64_t rows, int64_t V, int64_t ignore_index, const int64_t* count, int mean, int* status,
                              void* stream);

/* Skinny projection onto the LoRA rank: P[M,r] = X[M,C] . W^T with W given as [r,C] (w_is_cr = 0,
 * lora_A for X.A^T) or as [C,r] (w_is_cr = 1, lora_B for dY.B); r <= 16.
 * Writes out_plain[M,16] = bf16(P) and out_scaled[M,16] = bf16(scale*P), zero in columns >= r
 * (either may be null).  Replaces the torch.matmul of fast_lora.py:50-53 and its autograd twin. */
B2G_API int b2g_lora_down(const void* x, const void* w, int w_is_cr, float scale, void* out_plain, void* out_scaled,
                  int64_t M, int64_t C, int r, void* stream);

/* LoRA factor gradient, a contraction over the M rows:
 *   G[r,C] = scale * S[M,16]^T . T[M,C]   (only the first r rows of S^T are used)
 * stored as [r,C] (transpose_out = 0: dA = s*(dY.B)^T.X) or as [C,r] (transpose_out = 1:
 * dB = s*dY^T.(X.A^T)).  Replaces the addmm/matmul autograd of fast_lora.py:50-61.
 * `workspace` is fp32 scratch of at least b2g_lora_wgrad_workspace_bytes(M, C) bytes. */
B2G_API int64_t b2g_lora_wgrad_workspace_bytes(int64_t M, int64_t C);
B2G_API int b2g_lora_wgrad(const void* s, const void* t, float scale, void* out, int transpose_out, void* workspace,
                   int64_t workspace_bytes, int64_t M, int64_t C, int r, void* stream);

/* The same factor gradient for callers that cannot allocate device memory (a plug-in inside another
 * framework's memory plan, a host that was handed only input and output buffers, a process whose pool is
 * fully committed): the split partials live in a fixed 8 MiB array inside the library image, which every
 * GPU that loads the library holds until exit.  This entry has no counterpart in the reference.
 *   - allocates nothing on the device: no cudaMalloc / cudaFree, no allocating library routine (the two tensor maps of its
 *     kernel are 128-byte host structures filled by cuTensorMapEncodeTiled, kept in a host-side table and passed as kernel
 *     parameters);
 *   - shapes whose scratch need (b2g_lora_wgrad_workspace_bytes) exceeds b2g_lora_wgrad_static_max_bytes()
 *     are rejected with B2G_E_ARG; use b2g_lora_wgrad with your own workspace for those;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current) and caches it: make that first call before any stream capture begins;
 *   - all calls share the one array.  It keeps the previous call's partials; each call overwrites every
 *     entry it later reads, so nothing needs clearing, but two calls that overlap on the GPU (different
 *     streams, or threads without ordering) race on it: order them. */
B2G_API int64_t b2g_lora_wgrad_static_max_bytes(void);
B2G_API int b2g_lora_wgrad_static(const void* s, const void* t, float scale, void* out, int transpose_out, int64_t M,
                          int64_t C, int r, void* stream);

/* ---- router / routing ------------------------------------------------------------------------ */

/* Top-k expert ids per token, best first, ties to the smaller id.  logits_dtype: 0 = bf16, 1 = fp32;
 * score_fn: 0 = identity, 1 = sqrt(softplus(x)) (+ bias[E], nullable, fp32).  E must be 256.
 * Replaces router_topk_indices / _router_topk_kernel (fast_moe_ranking.py:166-270). */
B2G_API int b2g_router_topk(const void* logits, int logits_dtype, const float* bias, int score_fn, int64_t* indices,
                    int64_t T, int E, int top_k, void* stream);

/* Stable counting sort of the flat [T*top_k] expert ids.  idx_dtype: 0 = int32, 1 = int64.
 * Outputs: sorted_expert[R], perm[R], inv_perm[R] (int64), group_sizes[E], offsets[E] (int32,
 * cumulative ends).  `workspace` is int32 scratch of b2g_route_plan_workspace_bytes(T*top_k, E).
 * An id outside [0, E) is neither counted nor placed and sets status 903: its inv_perm entry and the last
 * positions of sorted_expert / perm keep what the caller put there (pass zero-filled arrays to keep them in range).
 * Replaces torch.sort + _inverse_permutation_kernel (fast_moe_routing.py:400-410) and the expert
 * histogram of GGUFExperts._prepare_expert_execution (called at fast_moe_lora.py:709). */
B2G_API int64_t b2g_route_plan_workspace_bytes(int64_t R, int E);
B2G_API int b2g_route_plan(const void* topk_idx, int idx_dtype, int64_t T, int top_k, int E, int64_t* sorted_expert,
                   int64_t* perm, int64_t* inv_perm, int32_t* group_sizes, int32_t* offsets, void* workspace,
                   int64_t workspace_bytes, int* status, void* stream);

/* sel[s,:] = hidden[perm[s] / top_k, :]            (_route_gather_forward_kernel, fast_moe_routing.py:101-123) */
B2G_API int b2g_route_gather(const void* hidden, const int64_t* perm, void* selected, int64_t T, int top_k, int H, void* stream);
/* dHidden[t,:] = sum over the token's k routes in ascending sorted position, bf16 rounding after
 * every add                                        (_route_gather_backward_kernel, :126-159) */
B2G_API int b2g_route_gather_bwd(const void* grad_selected, const int64_t* inv_perm, void* grad_hidden, int64_t T,
                         int top_k, int H, void* stream);
/* out[t,:] = sum_j expert_out[inv[t*k+j],:] * bf16(w[t,j]); w_dtype 0 = bf16, 1 = fp32
 *                                                  (_route_combine_forward_kernel, :162-194) */
B2G_API int b2g_route_combine(const void* expert_out, const void* weights, int w_dtype, const int64_t* inv_perm, void* out,
                      int64_t T, int top_k, int H, void* stream);
/* dExpertOut[s,:] = bf16(dFinal[t,:]*bf16(w)); dW[route] = sum_h dFinal*expert_out (in w's dtype)
 *                                                  (_route_combine_backward_kernel, :197-226) */
B2G_API int b2g_route_combine_bwd(const void* expert_out, const void* weights, int w_dtype, const int64_t* perm,
                          const void* grad_final, void* grad_expert_out, void* grad_weights, int64_t T, int top_k,
                          int H, void* stream);

/* ---- grouped (MoE) path ---------------------------------------------------------------------- */

/* Tile table for the persistent grouped kernels: one entry per (active expert, block of rows).
 * expert_indices[G] int64, offsets[G] int32 cumulative ends (the pair produced by
 * GGUFExperts._prepare_expert_execution, fast_moe_lora.py:709-719).  `tiles` is int32 scratch of
 * b2g_grouped_tiles_bytes(R, G) bytes that the grouped calls below consume.  Offsets beyond R are clamped to R (no
 * tile ever reaches past the R activation rows, nor past the table) and set status 904.  first_row (device int32, nullable):
 * where the first listed expert's rows begin (0 when null), for a table over a sub-range of a larger sorted buffer. */
B2G_API int64_t b2g_grouped_tiles_bytes(int64_t R, int G);
B2G_API int b2g_grouped_schedule(const int64_t* expert_indices, const int32_t* offsets, const int32_t* first_row, int G, int64_t R,
                         int32_t* tiles, int* status, void* stream);

/* One persistent launch over the ragged expert segments:
 *   Y0[rows_g, N] = X[rows_g, K] . deq(W0[e_g])^T   and, when payload1 != NULL, Y1 likewise from W1.
 * Optional fused LoRA: + XAs[R,16] . Bp[e_g][n,16]^T where lora_b16 is [E, lora_rows, 16] and the
 * rows used for output j are lora_rows_offset_j + n (Y0: 0, Y1: N).
 * Replaces torch_ggml_ops.grouped_mmq (fast_moe_lora.py:221-228) and grouped_mmq_pair (:339-347),
 * and with the LoRA operands the second AITER gmm + torch.add of :737-745 / :756-763. */
B2G_API int b2g_grouped_fwd(int qtype, const void* x, const void* payload0, const void* payload1, const int32_t* tiles,
                    const void* xas, const void* lora_b16, int64_t lora_rows, void* y0, void* y1, int64_t R,
                    int64_t N, int64_t K, int num_experts, int* status, void* stream);

/* dX[rows_g, K] = dY0[rows_g, N] . deq(W0[e_g]) (+ dY1 . deq(W1[e_g]) in the same fp32 accumulator)
 * (+ dYBs[R,16] . Ap[e_g][16,K]).  Replaces grouped_mmq_grad_input (fast_moe_lora.py:255-262) and
 * grouped_mmq_pair_grad_input (:364-375) plus the gmm input-gradient of :126-131. */
B2G_API int b2g_grouped_dgrad(int qtype, const void* dy0, const void* dy1, const void* payload0, const void* payload1,
                      const int32_t* tiles, const void* dybs, const void* lora_a16, void* dx, int64_t R, int64_t N,
                      int64_t K, int num_experts, int* status, void* stream);

/* Per-expert skinny projection P[rows_g, r] = X[rows_g, C] . W[e_g]^T, W given per expert as [r,C]
 * (w_is_cr = 0) or [C,r] (w_is_cr = 1); with x1 != NULL the reduction runs over [x | x1] (two
 * [R,C] halves against a [r,2C] or [2C,r] factor: dGate|dUp against gate_up_b).  Outputs as b2g_lora_down.
 * Replaces the first AITER gmm of _lora_grouped_linear (fast_moe_lora.py:675-682) and gmm's use in
 * _AiterGroupedMM.backward (:126-131). */
B2G_API int b2g_grouped_lora_down(const void* x, const void* x1, const void* w, int w_is_cr, float scale, const int32_t* tiles,
                          void* out_plain, void* out_scaled, int64_t R, int64_t C, int r, int num_experts,
                          void* stream);

/* Per-expert LoRA factor gradients over all E experts (zero rows -> exactly zero output):
 *   G[e][r,C] = scale * S[rows_e,16]^T . T[rows_e, C], stored [E,r,C] or (transpose_out) [E,C,r].
 * `offsets_full` is the cumulative-end array over ALL E experts (fast_moe_lora.py:663-672); first_row (device int32,
 * nullable) is where the first expert's rows begin (0 when null).
 * Replaces AITER ptgmm via _aiter_weight_grad (fast_moe_lora.py:76-87,132-139). */
B2G_API int b2g_grouped_lora_wgrad(const void* s, const void* t, float scale, const int32_t* offsets_full, const int32_t* first_row,
                           void* out, int transpose_out, int64_t R, int64_t C, int r, int num_experts, int64_t out_col_offset,
                           int64_t out_cols_total, void* stream);

/* Per-expert up-projection from the rank: Y[rows_e, N] = P[rows_e, :r] . W[e]^T with P of row stride
 * `ldp` and W per expert as [N,r] (w_is_nr = 1) or [r,N] (w_is_nr = 0).  Replaces the second AITER gmm
 * of _lora_grouped_linear (fast_moe_lora.py:675-682) where a caller wants it as a separate operator;
 * the fused expert path folds this product into b2g_grouped_fwd instead. */
B2G_API int b2g_grouped_lora_up(const void* p, int64_t ldp, const void* w, int w_is_nr, const int32_t* offsets_full, void* y,
                        int64_t R, int64_t N, int r, int num_experts, void* stream);

/* ---- expert-parallel row exchange over peer memory (new design: the reference is single-GPU,
 *      docs/plan_qwen3.5.md:23) -------------------------------------------------------------------------- */

/* Source side.  For every routed row s (rows sorted by global expert id, sorted_expert[R]) whose local expert index
 * (id modulo experts_per_rank) lies in [group_lo, group_hi), copy the row into the receive buffer of the expert's owner rank:
 * peer_ptrs[owner] (device array of one base address per rank, NVLink peer pointers of a symmetric allocation) at row
 * dest_base[e] + (s - my_start[e]).  With perm != NULL the row is gathered from the token matrix (row perm[s] / top_k of
 * src): the token permute of _route_gather_forward_kernel (fast_moe_routing.py:101-123) and the inter-GPU dispatch in one
 * pass; with perm == NULL row s of src is sent.  A slot at or beyond capacity_rows is never written; the status word is set to
 * 901 instead (b2g_ep_peer_plan clamps the owner's segments to the same capacity, so the rows that were dropped are not read
 * either).  The owners are visited in the order rank+1, rank+2, ..., so that the ranks do not all store to the same owner at
 * once.  One launch per expert group lets the caller overlap a group's transfer with another group's expert products.
 * spread > 0: a small kernel (128 threads of 32 registers, no shared memory) with that many CTAs per SM: 1 shares every SM
 * with the quantized GEMM, 8 is for an exchange that runs alone.  spread < 0: a wide kernel (1024 threads) as -spread clusters
 * of two CTAs, which occupy the two SMs of -spread TPCs entirely: for an exchange that runs beside a GEMM told to leave those
 * SMs free (b2g_set_gemm_sm_margin), so that the two share no SM. */
B2G_API int b2g_ep_scatter_rows(const void* src, const int64_t* perm, int top_k, const int64_t* sorted_expert,
                        const int32_t* my_start, const int32_t* dest_base, const uint64_t* peer_ptrs, int experts_per_rank,
                        int world, int rank, int group_lo, int group_hi, int64_t R, int H, int64_t capacity_rows, int spread,
                        int* status, void* stream);

/* Owner side, the inverse: rows of the grouped buffer (blocks ordered by (local expert, source rank), block b
 * spanning rows [blk_start[b], blk_start[b+1]), source rank b % world) go back to their source rank at row
 * src_pos[b] + offset inside the block; the call moves the blocks [block_lo, block_hi) (whole experts: multiples of world).
 * Pairs with the weighted un-permute of fast_moe_routing.py:162-194 on the source rank. */
B2G_API int b2g_ep_return_rows(const void* rows, const int32_t* blk_start, const int32_t* src_pos, const uint64_t* peer_ptrs,
                       int world, int block_lo, int block_hi, int H, int64_t capacity_rows, int spread, void* stream);

/* SMs that every later launch of the persistent quantized GEMM (dense and grouped) leaves free: an even number, 0 by default.
 * The expert-parallel layer sets it while its exchange kernels run beside the expert products on SMs of their own, and clears
 * it afterwards.  Process-wide.  This entry has no counterpart in the reference (which is single-GPU, docs/plan_qwen3.5.md:23). */
B2G_API int b2g_set_gemm_sm_margin(int sms);

/* Slots of the two exchange kernels for rank `rank`, from the all-gathered histograms counts[world][num_experts]
 * (int32, row g = rows of rank g per global expert, rows count_stride elements apart; rank g owns experts
 * [g*E/world, (g+1)*E/world)).  One launch;
 * no value visits the host.  Outputs (int32, device): my_start[E], dest_base[E] as b2g_ep_scatter_rows reads them;
 * blk_start[E/world*world + 1], src_pos[E/world*world] as b2g_ep_return_rows reads them; local_sizes[E/world] and
 * local_offsets[E/world] (cumulative ends) = the expert segments of the rows this rank receives, in the form the
 * grouped products take (the role that the expert histogram of GGUFExperts._prepare_expert_execution, called at
 * fast_moe_lora.py:709, plays on a single GPU).  blk_start, local_sizes and local_offsets are clamped to capacity_rows, the
 * row count of this rank's receive buffer; when the rows sent to this rank exceed it, status 901 is set and the rows past
 * the capacity are neither stored (b2g_ep_scatter_rows) nor read by anything that follows this plan. */
B2G_API int b2g_ep_peer_plan(const int32_t* counts, int64_t count_stride, int world, int num_experts, int rank, int32_t* my_start,
                     int32_t* dest_base, int32_t* blk_start, int32_t* src_pos, int32_t* local_sizes, int32_t* local_offsets,
                     int64_t capacity_rows, int* status, void* stream);

/* SwiGLU between the two grouped products: z = silu(g) * u (optionally clamped as the DeepSeek
 * experts do: g <= limit, |u| <= limit; limit <= 0 disables).  Replaces GGUFExperts._apply_split_gate
 * (called at fast_moe_lora.py:747; clamp semantics at test_deepseek_v4_moe_lora.py:194-196).  n = elements of each tensor.
 * row_begin / row_end (nullable, device int32): only the rows [*row_begin, *row_end) of `cols` elements are processed (0 and
 * all rows when null), for tensors that are the partly filled receive buffer of an expert-parallel exchange, whose fill
 * counts never visit the host. */
B2G_API int b2g_swiglu_fwd(const void* gate, const void* up, void* z, int64_t n, float limit, const int32_t* row_begin,
                   const int32_t* row_end, int64_t cols, void* stream);
B2G_API int b2g_swiglu_bwd(const void* gate, const void* up, const void* dz, void* dgate, void* dup, int64_t n, float limit,
                   const int32_t* row_begin, const int32_t* row_end, int64_t cols, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B2G_H_ */
