/*
 * fmoe_b200 -- C ABI of the sm_100a implementation of the FastMoE forward hot path.
 *
 * The reference (meta-recsys/fast_moe) is a pure-Python operator library; its "FFI" for this path
 * is the set of Python callables in kernels/moe.py, kernels/moe_fp8.py and the routing code of
 * modules/fast_moe_module.py. Each entry point below is what a binding of one of those callables
 * needs from native code; the comment above it cites the reference interface it stands in for
 * (paths are relative to the reference repository).
 *
 * Conventions
 *  - All pointers are DEVICE pointers unless a comment says "host". The library never allocates,
 *    frees or copies on the caller's behalf: outputs and scratch buffers are passed in.
 *  - Every function enqueues work on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 *    default stream) and returns without synchronising. Return value: FMOE_OK or a negative
 *    fmoe_status; fmoe_last_error() gives the message of the calling thread's last failure.
 *  - Index tensors are int64 ("long"), as in the reference. Row strides (ld*) are in elements.
 *  - Weights are logical [E, K, N] tensors described by element strides (se, sk, sn). The tensor
 *    core path needs K contiguous (sk == 1), which is the layout FastMoELayer hands to the
 *    operators (a permuted view of [E, N, K] storage, modules/fast_moe_module.py:167,177).
 *  - Kernels never trap. A kernel that meets an out-of-range index or a wait that runs out
 *    records a code in a per-device status word and returns; fmoe_device_status() reads it.
 */
#ifndef FMOE_B200_H_
#define FMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  FMOE_OK = 0,
  FMOE_ERR_BAD_ARG = -1,     /* shape / pointer / dtype relation violated (the reference asserts) */
  FMOE_ERR_UNSUPPORTED = -2, /* valid for the reference, not for this kernel (e.g. stride not 16-byte aligned) */
  FMOE_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed */
  FMOE_ERR_DEVICE = -4       /* the device status word is non-zero (see fmoe_device_status) */
} fmoe_status;

/* element types */
enum { FMOE_F32 = 0, FMOE_BF16 = 1, FMOE_E4M3 = 3 };

/* GEMM epilogues */
enum { FMOE_EPI_NONE = 0, FMOE_EPI_SILU = 1, FMOE_EPI_SWIGLU = 2 };

/* codes a kernel may leave in the device status word */
enum {
  FMOE_DEV_OK = 0,
  FMOE_DEV_BAD_INDEX = 1,      /* an index / expert id outside its range was skipped */
  FMOE_DEV_WAIT_PRODUCER = 2,  /* bounded waits that gave up, by pipeline role */
  FMOE_DEV_WAIT_MMA = 3,
  FMOE_DEV_WAIT_EPILOGUE = 4
};

int fmoe_version(void);
/* Message of the last failure on the calling thread (host string, never NULL). */
const char* fmoe_last_error(void);
/* Copies the device status word of the current device to *status_out (host), after synchronising
 * `stream`; clears it when reset != 0. */
int fmoe_device_status(int* status_out, int reset, void* stream);
/* Failure-path self test: one CTA waits, with the bounded wait every pipeline role uses, on a
 * barrier that is never signalled; after limit_us it gives up, records FMOE_DEV_WAIT_PRODUCER in
 * the device status word and returns. Nothing traps, the context stays usable. */
int fmoe_selftest_bounded_wait(int64_t limit_us, void* stream);
/* Number of kernels this library has launched in this process (all entry points). */
long long fmoe_kernel_launch_count(void);

/* ---------------------------------------------------------------------------------------------
 * Routing.
 * Replaces GatingNetwork.forward + FastMoELayer._select_top_k_experts
 * (modules/fast_moe_module.py:21-27, :93-105): logits = x @ Wg^T + bg in fp32, softmax over the
 * E experts, top-k (slots in descending score order, ties to the lower expert id), scores of the
 * chosen experts renormalised to sum 1 (F.normalize p=1, eps 1e-12).
 *   x         [L, d] bf16 or f32 (x_dtype), row stride ldx; may be NULL when logits_in is given
 *   gate_w    [E, d] f32 row-major (nn.Linear weight), gate_b [E] f32 or NULL
 *   logits_in f32 or NULL: when non-NULL the matrix product is skipped and row t of the logits is
 *             read at logits_in + t * ld_logits (gate_b is still added). With logits_split != 0 the
 *             row holds two halves [E | E] that are summed: the product was computed with tensor
 *             cores on a two-term bf16 expansion (hi + lo) of the fp32 gate weights.
 *   logits_out[L, E] f32 or NULL
 *   topk_idx  [L, k] int64, topk_score [L, k] f32
 * 1 <= k <= E <= 256.
 * bf16 x with 16-byte-aligned rows, E <= 32 and gate weights that fit in shared memory run the
 * product on the warp-level tensor cores with the fp32 weights expanded on the fly into three
 * bf16 terms (exact products, fp32 accumulation); other cases use fp32 FMAs. Both give the same
 * scores for the same logits, bit for bit.
 */
int fmoe_gate_topk(const void* x, int x_dtype, int64_t ldx, const float* gate_w, const float* gate_b,
                   const float* logits_in, int64_t ld_logits, int logits_split, int64_t L, int d, int E, int k,
                   float* logits_out, int64_t* topk_idx, float* topk_score, void* stream);

/* The router of the sparsely-gated ("MRN" / SGMoE) layer, OrigSGMoEImpl._orig_noisy_gating without
 * noise (kernels/pytorch/mrn.py:236-252; the same steps as _compute_top_logits,
 * utils/utils.py:139-164): logits = x @ Wg^T (+ bias), divided by max(||logits||_2, 1e-12) per token
 * (F.normalize), softmax over ALL experts, the k largest probabilities taken in descending order
 * (ties to the lower expert id: a stable descending sort) and kept as they are - no
 * renormalisation. Arguments as fmoe_gate_topk; gate_w is [E, d] (the reference stores [d, E]:
 * pass its transpose); logits_in, when given, are the un-normalised logits. */
int fmoe_gate_topk_normalized(const void* x, int x_dtype, int64_t ldx, const float* gate_w, const float* gate_b,
                              const float* logits_in, int64_t ld_logits, int64_t L, int d, int E, int k,
                              float* logits_out, int64_t* topk_idx, float* topk_score, void* stream);

/* Token normalisation in front of that router and of the experts (kernels/pytorch/mrn.py:301-318):
 * layer norm over the d features (num_groups = 1, weight / bias [d], per_group_affine = 0), or
 * F.group_norm of x viewed as [L, num_groups, d / num_groups] with one weight / bias per group
 * (per_group_affine = 1). fp32 statistics (biased variance), result in the token dtype.
 * weight / bias are f32 and may be NULL. */
int fmoe_token_norm(const void* x, int dtype, int64_t L, int d, int64_t ldx, int num_groups, const float* weight,
                    const float* bias, int per_group_affine, float eps, void* out, int64_t ldo, void* stream);

/* Load fractions and training loss of the sparsely-gated layer (kernels/pytorch/mrn.py:186-189,
 * :253-287): importance[e] = sum of the gate values routed to expert e (in the order of the
 * expert-sorted rows; with round_bf16 the gates and the sum are rounded to bf16 as bf16 tokens make
 * the reference do), load[e] = rows of expert e; load_frac [E] = load / sum(load);
 * loss [1] = loss_coef * (cv2(importance) + cv2(load)), cv2 = unbiased variance / (mean^2 + 1e-6),
 * or 0 when want_loss == 0 (evaluation). offsets [E+1], gate_index [rows] as fmoe_route_metadata
 * produced them; topk_score [L, k] f32. With noisy gating the loss uses the smooth load instead of
 * the row counts: load_partials [n_partials, E] as fmoe_sg_noisy_load wrote them (NULL otherwise);
 * load_frac stays the row fractions, as in the reference. */
int fmoe_sg_load_loss(const int64_t* offsets, const int64_t* gate_index, const float* topk_score, int E,
                      int round_bf16, float loss_coef, int want_loss, const float* load_partials, int n_partials,
                      float* load_frac, float* loss, void* stream);

/* Training-time noise on the router logits of the sparsely-gated layer
 * (OrigSGMoEImpl._orig_noisy_gating, kernels/pytorch/mrn.py:229-237). logits2 [L, >= 2E] f32 holds
 * x @ w_gate in columns [0, E) and x @ w_noise in columns [E, 2E) (one gate product on the two
 * weights stacked); noise [L, E] f32 is the caller's standard-normal draw.
 *   stddev = softplus(x @ w_noise) + noise_eps,  noisy = clean + noise * stddev   (both [L, E] f32)
 * The noisy logits then go through fmoe_gate_topk_normalized (logits_in). */
int fmoe_sg_noisy_logits(const float* logits2, int64_t ld_logits, const float* noise, int64_t L, int E,
                         float noise_eps, float* noisy, float* stddev, void* stream);

/* Backward of the sparsely-gated layer's own pieces. The reference obtains them from torch autograd
 * through its eager code (kernels/pytorch/mrn.py:221-333) and its test compares the gradients of x,
 * every parameter and the norm's weight / bias (kernels/tests/mrn_test.py:816-860).
 *   fmoe_token_norm_backward: d_x of fmoe_token_norm and, when d_weight / d_bias are given, the
 *     gradients of its weight / bias ([d] per feature, or [num_groups] with per_group_affine) as
 *     fixed-order sums over the tokens. Scratch: stats [L * num_groups * 2] f32,
 *     partial [chunks * 2 * d] f32 (1 <= chunks <= 1024).
 *   fmoe_sg_router_backward: d_logits [L, E] of fmoe_gate_topk_normalized from the gradient of its
 *     k scores (softmax over all experts, then the L2 normalisation of the logits); logits are the
 *     un-normalised ones it returned.
 *   fmoe_sg_loss_backward: d_score [L, k] of fmoe_sg_load_loss's loss (through the importance only;
 *     the load is a count), scaled by *d_loss (1 when NULL). */
int fmoe_token_norm_backward(const void* x, const void* d_out, int dtype, int64_t L, int d, int64_t ldx, int64_t ld_dout,
                             int num_groups, const float* weight, int per_group_affine, float eps, void* d_x,
                             int64_t ld_dx, float* stats, float* partial, int chunks, float* d_weight, float* d_bias,
                             void* stream);
int fmoe_sg_router_backward(const float* logits, const int64_t* topk_idx, const float* d_score, int64_t L, int E, int k,
                            float* d_logits, void* stream);
int fmoe_sg_loss_backward(const int64_t* offsets, const int64_t* gate_index, const float* topk_score, int E,
                          int round_bf16, float loss_coef, const float* d_loss, float* d_score,
                          const float* load_partials, int n_partials, float* d_load, void* stream);
/* Noisy gating (training): fmoe_sg_loss_backward also returns d loss / d load [E] when the loss was
 * built on the smooth load (load_partials as fmoe_sg_noisy_load wrote them; NULL otherwise), and
 * fmoe_sg_noisy_router_backward turns the gradient of the k scores and that d_load into
 * d_logits2 [L, 2E] = (d clean | d raw) for the stacked gate product x @ [w_gate | w_noise]
 * (through the softmax, the L2 normalisation, the thresholds of the load estimate, noise * stddev
 * and softplus); fmoe_gate_linear_backward on the stacked weight finishes the job. d_load NULL:
 * the load takes no part (k == E). */
int fmoe_sg_noisy_router_backward(const float* logits2, int64_t ld_logits, const float* noise, const float* noisy,
                                  const float* stddev, const int64_t* topk_idx, const float* d_score,
                                  const float* d_load, int64_t L, int E, int k, float* d_logits2, int64_t ld_d,
                                  void* stream);

/* Smooth load of the noisy router (OrigSGMoEImpl._prob_in_top_k, kernels/pytorch/mrn.py:191-219):
 * per token and expert Phi((clean - threshold) / stddev), the threshold being the (k+1)-th largest
 * L2-normalised noisy logit where the expert's noisy logit exceeds it and the k-th largest elsewhere,
 * summed over the tokens. partials [n_partials, E] f32 receives one row of sums per block
 * (n_partials blocks, 1..1024; fmoe_sg_load_loss adds them up in order). 1 <= k < E <= 256. */
int fmoe_sg_noisy_load(const float* logits2, int64_t ld_logits, const float* noisy, const float* stddev, int64_t L,
                       int E, int k, float* partials, int n_partials, void* stream);

/* Replaces FastMoELayer._compute_routing_metadata (modules/fast_moe_module.py:107-144) and the
 * fbgemm op asynchronous_complete_cumsum it calls (:131): a stable counting sort of the L*k
 * (token, slot) pairs by expert id.
 *   topk_idx      [L, k] int64 in
 *   lengths       [E]    rows per expert
 *   offsets       [E+1]  exclusive prefix of lengths, offsets[E] = L*k
 *   gate_index    [L*k]  stable argsort of topk_idx.view(-1): value = token*k + slot
 *   token_index   [L*k]  gate_index / k
 *   reverse_index [L, k] stable argsort of token_index, i.e. for each token the sorted positions
 *                        of its k rows (ascending expert id)
 *   max_len       [1]    max(lengths) (stays on the device: no kernel here needs it on the host)
 *   workspace            fmoe_route_workspace_bytes(L, E, k) bytes of scratch
 * Any output pointer except offsets may be NULL.
 */
size_t fmoe_route_workspace_bytes(int64_t L, int E, int k);
int fmoe_route_metadata(const int64_t* topk_idx, int64_t L, int E, int k, int64_t* lengths, int64_t* offsets,
                        int64_t* gate_index, int64_t* token_index, int64_t* reverse_index, int64_t* max_len,
                        void* workspace, size_t workspace_bytes, void* stream);

/* Small batches: the two routing steps chained so that the indices are read once, plus the two
 * memory passes the layers run right after routing. No counterpart in the reference beyond the
 * functions fmoe_gate_topk and fmoe_route_metadata already stand in for
 * (modules/fast_moe_module.py:93-144) and the index_select of the up projection
 * (kernels/pytorch/moe.py:69-73); results are bit-identical to those entry points.
 *   fmoe_gate_topk_counts_supported: 1 when fmoe_gate_topk_counts can run on these arguments (bf16
 *     tokens with 16-byte aligned rows, E <= 32, d a multiple of 8, ceil(L/32) * 2 * E <= 16384).
 *   fmoe_gate_topk_counts: fmoe_gate_topk (x given, no precomputed logits) that also writes, for
 *     every group of 16 tokens, the rows per expert: group_counts, fmoe_route_group_counts_bytes(L, E)
 *     bytes. It optionally clears rows 0..L-1 of zero_rows ([L, zero_cols] bf16 / f32, 16-byte
 *     aligned rows): the buffer a fused combine accumulates into; the stores ride under the
 *     kernel's load latency. zero_rows may be NULL.
 *   fmoe_route_metadata_gather: fmoe_route_metadata from those counts (one launch, no workspace),
 *     which optionally also (a) writes x_sorted[p, :] = x[token_index[p], :] for every sorted row p
 *     - the row gather of the up projection, x read once - and (b) clears rows 0..L-1 of zero_rows
 *     ([L, zero_cols], the buffer a fused combine accumulates into). Either may be NULL. */
int fmoe_gate_topk_counts_supported(const void* x, int x_dtype, int64_t ldx, const float* gate_w, int64_t L, int d,
                                    int E);
size_t fmoe_route_group_counts_bytes(int64_t L, int E);
int fmoe_gate_topk_counts(const void* x, int x_dtype, int64_t ldx, const float* gate_w, const float* gate_b,
                          int64_t L, int d, int E, int k, float* logits_out, int64_t* topk_idx, float* topk_score,
                          int* group_counts, void* zero_rows, int zero_dtype, int64_t ld_zero, int zero_cols,
                          void* stream);
int fmoe_route_metadata_gather(const int64_t* topk_idx, int64_t L, int E, int k, const int* group_counts,
                               int64_t* lengths, int64_t* offsets, int64_t* gate_index, int64_t* token_index,
                               int64_t* reverse_index, int64_t* max_len, const void* x, int x_dtype, int64_t ldx,
                               int cols, void* x_sorted, int64_t ld_sorted, void* zero_rows, int zero_dtype,
                               int64_t ld_zero, int zero_cols, void* stream);

/* fmoe_route_metadata without a workspace argument, for callers that cannot allocate device
 * memory (code inside a pre-planned memory region, plugins that only receive their input and
 * output buffers, fixed-budget services). It has no counterpart in the reference. The scratch
 * table lives in a 256 KiB array inside the library image (held by every GPU that loads the
 * library, until exit), so sizes are limited to ceil(L/256) * E <= 65536; larger problems get
 * FMOE_ERR_UNSUPPORTED and should use fmoe_route_metadata. No cudaMalloc / cudaFree or other
 * allocating call is made. The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current): make that first call outside any stream
 * capture. All calls on a device share the one array, so two calls whose kernels can overlap on
 * the GPU (different streams) race; calls on one stream are ordered and need no clearing between
 * them. Results are identical to fmoe_route_metadata. */
int fmoe_route_metadata_static(const int64_t* topk_idx, int64_t L, int E, int k, int64_t* lengths,
                               int64_t* offsets, int64_t* gate_index, int64_t* token_index,
                               int64_t* reverse_index, int64_t* max_len, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Up projection.
 * index_select_jagged_bmm (kernels/moe.py:39-68 -> kernels/pytorch/moe.py:40-84):
 *   out[r, :] = jagged[index[r] / index_div, :] @ weight[e] + bias[e],  offsets[e] <= r < offsets[e+1]
 *   offsets [E+1] int64; index [rows] int64 (the flattened [L, A] tensor, index_div = A);
 *   index may be NULL when jagged already holds the rows in expert-sorted order (L = rows).
 *   With an index the kernel gathers the rows itself (16-byte cp.async, once per column block);
 *   from about 1024 rows and 1024 output columns on, fmoe_gather_rows into a scratch followed
 *   by this call with index = NULL is faster (contiguous TMA tiles, CTA pairs) - the Python
 *   mirror does that.
 *   jagged  [L, K] dtype (bf16, or f32 computed with tf32 tensor-core math), row stride ldj
 *   weight  logical [E, K, N], element strides (w_se, w_sk, w_sn), same dtype
 *   bias    [E, N] same dtype as out, expert stride bias_se, or NULL
 *   out     [rows, N] out_dtype (bf16 or f32), row stride ldo; rows = offsets[E] (<= total_rows)
 * `epilogue` = FMOE_EPI_NONE for the reference operator; FMOE_EPI_SILU additionally applies SiLU
 * (used by the layer to fold the activation that silu_jagged_bmm_combine would otherwise apply to
 * its input, kernels/pytorch/moe.py:262-263).
 */
int fmoe_index_select_jagged_bmm(const int64_t* offsets, const int64_t* index, int index_div, int64_t total_rows,
                                 const void* jagged, int dtype, int64_t L, int64_t ldj, const void* weight,
                                 int64_t w_se, int64_t w_sk, int64_t w_sn, const void* bias, int64_t bias_se,
                                 int E, int K, int N, int epilogue, void* out, int out_dtype, int64_t ldo,
                                 void* stream);

/* Second product of index_select_jagged_gating_bmm (kernels/moe.py:192-233 ->
 * kernels/pytorch/moe.py:149-221: silu(A_g Wa + ba) * (B_g Wb + bb) on two different inputs):
 * fmoe_index_select_jagged_bmm whose result is multiplied elementwise, in the epilogue, by
 * `multiplier` [total_rows, N] (out_dtype, row stride ld_mul) - the SiLU'd first product, computed
 * by fmoe_index_select_jagged_bmm with FMOE_EPI_SILU. No separate multiply pass. */
int fmoe_index_select_jagged_bmm_mul(const int64_t* offsets, const int64_t* index, int index_div, int64_t total_rows,
                                     const void* jagged, int dtype, int64_t L, int64_t ldj, const void* weight,
                                     int64_t w_se, int64_t w_sk, int64_t w_sn, const void* bias, int64_t bias_se, int E,
                                     int K, int N, const void* multiplier, int64_t ld_mul, void* out, int out_dtype,
                                     int64_t ldo, void* stream);

/* index_select_jagged_bmm_swiglu (kernels/moe.py:156-189 -> kernels/pytorch/moe.py:87-146):
 *   out[r, :] = silu(x_r @ weight[e] + bias[e]) * (x_r @ weight_p[e] + bias_p[e])
 * weight and weight_p share shape and strides. */
int fmoe_index_select_jagged_bmm_swiglu(const int64_t* offsets, const int64_t* index, int index_div,
                                        int64_t total_rows, const void* jagged, int dtype, int64_t L, int64_t ldj,
                                        const void* weight, const void* weight_p, int64_t w_se, int64_t w_sk,
                                        int64_t w_sn, const void* bias, const void* bias_p, int64_t bias_se, int E,
                                        int K, int N, void* out, int out_dtype, int64_t ldo, void* stream);

/* moe_fp8.index_select_jagged_bmm(fp8=True) (kernels/moe_fp8.py:185-248 ->
 * kernels/pytorch/moe_fp8.py:98-139) on operands that are already quantised with
 * fmoe_rowwise_quant_fp8: jagged_q [L, K] e4m3 with jagged_scale [L]; weight_q logical [E, K, N]
 * e4m3, K contiguous, with weight_scale [E, N] (expert stride ws_se). Scales are the multipliers
 * used at quantisation; the epilogue divides by their product, then adds bias.
 * weight_p_q / weight_p_scale non-NULL selects the SwiGLU form of the same product.
 * index may be NULL (rows and their scales already gathered, L = rows). */
int fmoe_index_select_jagged_bmm_fp8(const int64_t* offsets, const int64_t* index, int index_div,
                                     int64_t total_rows, const void* jagged_q, const float* jagged_scale, int64_t L,
                                     int64_t ldj, const void* weight_q, const float* weight_scale,
                                     const void* weight_p_q, const float* weight_p_scale, int64_t w_se, int64_t w_sk,
                                     int64_t w_sn, int64_t ws_se, const void* bias, const void* bias_p,
                                     int64_t bias_se, int E, int K, int N, int epilogue, void* out, int out_dtype,
                                     int64_t ldo, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Down projection.
 * pytorch_silu_jagged_bmm (kernels/pytorch/moe.py:255-275), the GEMM half of
 * silu_jagged_bmm_combine: out[r, :] = act(jagged[r, :]) @ weight[e] + bias[e] with act = SiLU
 * when has_silu != 0. The activation cannot be applied between shared memory and the tensor core,
 * so with has_silu the caller passes act_scratch ([rows, K], same dtype, row stride K) which
 * receives silu(jagged) first. jagged_scale / weight_scale non-NULL select the FP8 form (jagged
 * and weight are then e4m3 and has_silu must be 0).
 * jagged_index / out_row_index (both [total_rows] int64, nullable) are not part of the reference
 * operator: when given, row r reads jagged[jagged_index[r]] and is stored at out[out_row_index[r]].
 * The expert-parallel layer uses them to consume rows in the order the all-to-all delivered them
 * and to hand results back in that order, without a separate permutation pass.
 */
int fmoe_silu_jagged_bmm(const int64_t* offsets, int64_t total_rows, const void* jagged, int dtype, int64_t ldj,
                         const float* jagged_scale, const void* weight, const float* weight_scale, int64_t w_se,
                         int64_t w_sk, int64_t w_sn, int64_t ws_se, const void* bias, int64_t bias_se, int E, int K,
                         int N, int has_silu, void* act_scratch, const int64_t* jagged_index,
                         const int64_t* out_row_index, void* out, int out_dtype, int64_t ldo, void* stream);

/* mul_merge_k_add (kernels/moe.py:71-115 -> kernels/pytorch/moe.py:14-37):
 *   out[t, :] = sum_j value[p_j, :] * weight[weight_index[p_j]],  p_j = reverse_index[t, j], j = 0..k-1
 * accumulated in fp32 in that order (ascending row, the order index_add visits them), the product
 * rounded to the value type first when value and weight are both bf16 (what Tensor.mul does).
 *   value [L*k, D] v_dtype, row stride ldv; reverse_index [L, k] int64
 *   weight: flat array of w_dtype (bf16/f32) or NULL; weight_index [L*k] int64 or NULL (identity)
 *   out [L, D] out_dtype, row stride ldo
 */
int fmoe_mul_merge_k_add(const int64_t* reverse_index, const void* value, int v_dtype, int64_t ldv,
                         const void* weight, int w_dtype, const int64_t* weight_index, int64_t L, int k, int D,
                         void* out, int out_dtype, int64_t ldo, void* stream);

/* silu_jagged_bmm_combine (kernels/moe.py:236-292 -> kernels/pytorch/moe.py:278-303):
 * fmoe_silu_jagged_bmm into bmm_scratch ([rows, N], out_dtype, row stride N) followed by
 * fmoe_mul_merge_k_add with gating_scores / gates_index. */
int fmoe_silu_jagged_bmm_combine(const int64_t* offsets, int64_t total_rows, const void* jagged, int dtype,
                                 int64_t ldj, const void* weight, int64_t w_se, int64_t w_sk, int64_t w_sn,
                                 const void* bias, int64_t bias_se, const int64_t* reverse_index,
                                 const void* gating_scores, int g_dtype, const int64_t* gates_index, int64_t L, int k,
                                 int E, int K, int N, int has_silu, void* act_scratch, void* bmm_scratch, void* out,
                                 int out_dtype, int64_t ldo, void* stream);

/* silu_jagged_bmm_combine with the combine folded into the GEMM's epilogue: no [rows, N]
 * intermediate and no second kernel. `out` [L, N] is zeroed (memset on `stream`), then every
 * expert row r is rounded to the activation type, multiplied by
 * gating_scores.view(-1)[gates_index[r]], rounded again and ADDED (red.global.add) to
 * out[gates_index[r] / k]. For k <= 2 this equals fmoe_silu_jagged_bmm_combine bit for bit in
 * bf16 (two commutative additions); for k > 2 the order of the additions, hence the last bit, is
 * not fixed - use the two-kernel form when reproducibility matters. jagged_scale / weight_scale
 * select the FP8 form as in fmoe_silu_jagged_bmm.
 * flags: FMOE_COMBINE_ACCUMULATE - `out` is not cleared; the rows are added to what it holds (a
 *   buffer the caller zeroed earlier, off the critical path, or a residual to add the layer to);
 *   FMOE_COMBINE_ROUND_GATE - f32 gating_scores are rounded to the output type before use: the
 *   operand types the reference's own layer produces, whose gate runs in the dtype of the tokens
 *   (modules/fast_moe_module.py:21-27) so that bf16 tokens come with bf16 scores. The layers
 *   here route in fp32 and round in the epilogue instead of running a separate cast. */
#define FMOE_COMBINE_ACCUMULATE 1
#define FMOE_COMBINE_ROUND_GATE 2
int fmoe_silu_jagged_bmm_combine_fused(const int64_t* offsets, int64_t total_rows, const void* jagged, int dtype,
                                       int64_t ldj, const float* jagged_scale, const void* weight,
                                       const float* weight_scale, int64_t w_se, int64_t w_sk, int64_t w_sn,
                                       int64_t ws_se, const void* bias, int64_t bias_se, const void* gating_scores,
                                       int g_dtype, const int64_t* gates_index, int64_t L, int k, int E, int K, int N,
                                       int has_silu, void* act_scratch, void* out, int out_dtype, int64_t ldo,
                                       int flags, void* stream);

/* Row index of index_select_jagged_bmm_3D (kernels/moe.py:118-153 -> kernels/pytorch/moe.py:224-252):
 * the rows of expert e read slice e of their token in a [L, E, K] input. out[p] = (index[p] / A) * E
 * + e(p), e(p) the expert whose segment of `offsets` holds sorted row p; fmoe_index_select_jagged_bmm
 * on the [L * E, K] view with this index (index_div = 1) is the operator. */
int fmoe_expand_3d_index(const int64_t* offsets, const int64_t* index, int A, int E, int64_t rows, int64_t* out,
                         void* stream);

/* fp32 operands without TF32. The tensor-core path for FMOE_F32 operands rounds them to tf32
 * (10 mantissa bits); the reference's kernels do that only when
 * torch.backends.cuda.matmul.allow_tf32 is set (kernels/triton/triton_moe.py:592, default off) and
 * otherwise multiply in full fp32, which is also what its PYTORCH path does. For that case the
 * operands are expanded into three bf16 terms each (hi + mid + lo = x to about 2^-24) and laid out
 * so that ONE bf16 grouped GEMM over a reduction dimension of 6 * cols_padded reproduces the fp32
 * product: left operand rows [hi | hi | mid | hi | lo | mid] (pattern 0), right operand rows
 * [hi | mid | hi | lo | hi | mid] (pattern 1); every partial product is exact in the fp32
 * accumulator. in [rows, cols] f32 (row stride ldi); out [rows, 6 * cols_padded] bf16 (row stride
 * ldo), columns cols..cols_padded-1 of every term are zero. apply_silu != 0 expands silu(in). */
int fmoe_split_f32_bf16x3(const float* in, int64_t rows, int cols, int64_t ldi, int cols_padded, int pattern,
                          int apply_silu, void* out, int64_t ldo, void* stream);

/* Row gather: dst[r, :] = src[index[r] / index_div, :], r < rows. The index_select step of
 * pytorch_index_select_jagged_bmm (kernels/pytorch/moe.py:69-73: jagged[index]) as a standalone
 * kernel; the expert-parallel layer uses it to pack the rows it sends, already in
 * (destination rank, expert, token) order, which is the order of gate_index.
 *   src [src_rows, cols] dtype (element size 1, 2 or 4 bytes), row stride lds; dst row stride ldd. */
int fmoe_gather_rows(const void* src, int dtype, int64_t src_rows, int64_t lds, const int64_t* index,
                     int index_div, int64_t rows, int cols, void* dst, int64_t ldd, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Expert parallelism over peer memory (one process per GPU, experts split in contiguous blocks of
 * E / world over the ranks, tokens stay on their rank). The reference names an expert-parallel
 * layer in its README (README.md:100-113, :162) but ships no such file, so these four entry points
 * have no reference interface to cite; the contract is that the sharded layer equals the
 * single-GPU one. Peer buffers (receive rows, route table, return rows) are allocated and mapped
 * by the caller (e.g. torch symmetric memory); the library only needs their addresses, passed as
 * DEVICE arrays of `world` int64 pointers. Kernels touch peer memory with plain loads and stores
 * only. The caller orders the steps across ranks (a collective on the same stream after
 * fmoe_ep_dispatch and after fmoe_ep_down_projection).
 *
 * fmoe_ep_plan: counts [world, E] int64, counts[s, e] = rows rank s routes to global expert e
 *   (every rank's `lengths`, all-gathered). Outputs, for the calling rank:
 *   dst_base [E]: row of the owner's receive buffer where this rank's rows for expert e start.
 *   The receive buffer is expert-major: (local expert, source rank, source's row order).
 *   offsets_local [E/world + 1]: jagged offsets of the local experts over the rows received.
 *   A total beyond `capacity` rows sets FMOE_DEV_BAD_INDEX in the device status word.
 * fmoe_ep_dispatch: one row per entry of this rank's expert-sorted order (offsets [E+1],
 *   token_index [rows], as fmoe_route_metadata produced them): row p of expert e is copied from
 *   x[token_index[p]] to recv_ptrs[e / (E/world)] + (dst_base[e] + p - offsets[e]) * ld_recv, and
 *   route_ptrs[owner][that row] = (rank << 40) | p, the row's return address.
 * fmoe_ep_up_projection: the SwiGLU up projection (fmoe_index_select_jagged_bmm_swiglu without an
 *   index) on the receive buffer; `capacity` bounds the rows, offsets_local[E_local] is their
 *   number, rows_hint (> 0) the expected number (chooses the tile shape).
 *   weight / weight_p: [E_local, N, K] storage, K contiguous, strides (w_se, w_sn) in elements.
 * fmoe_ep_down_projection: the down projection whose epilogue stores result row r at its return
 *   address: back_ptrs[route[r] >> 40] + (route[r] & (2^40 - 1)) * ld_back. back_rows = rows of
 *   each return buffer (addresses beyond it are recorded in the status word and skipped). */
int fmoe_ep_plan(const int64_t* counts, int world, int E, int rank, int64_t capacity, int64_t* dst_base,
                 int64_t* offsets_local, void* stream);
int fmoe_ep_dispatch(const void* x, int dtype, int64_t x_rows, int64_t ldx, int cols, const int64_t* offsets,
                     const int64_t* token_index, int64_t rows, int E, int world, int rank, const int64_t* dst_base,
                     const int64_t* recv_ptrs, const int64_t* route_ptrs, int64_t ld_recv, int64_t capacity,
                     void* stream);
int fmoe_ep_up_projection(const int64_t* offsets_local, int64_t capacity, int64_t rows_hint, const void* recv,
                          int dtype, int64_t ld_recv, const void* weight, const void* weight_p, int64_t w_se,
                          int64_t w_sn, int E_local, int K, int N, void* out, int64_t ldo, void* stream);
int fmoe_ep_down_projection(const int64_t* offsets_local, int64_t capacity, int64_t rows_hint, const void* hidden,
                            int dtype, int64_t ldh, const void* weight, int64_t w_se, int64_t w_sn, int E_local,
                            int K, int N, const int64_t* route, const int64_t* back_ptrs, int world,
                            int64_t back_rows, int64_t ld_back, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Backward pass of the expert products. The reference implements each operator's backward as
 * Triton kernels of its own; here every matrix product of the backward pass is the grouped GEMM
 * above on differently laid out operands, and these entry points provide the layouts and the
 * elementwise derivatives. The Python mirror (fast_moe_b200/kernels/autograd.py) assembles them
 * into torch.autograd.Functions with the reference operators' signatures.
 *
 * d_jagged (kernels/triton/triton_moe.py:290-381 _jagged_bmm_index_add, :3474-3559): rows of d_out
 *   times weight[e]^T is fmoe_silu_jagged_bmm / fmoe_index_select_jagged_bmm on the transposed
 *   weight; fmoe_batched_transpose produces it (out[b, c, r] = in[b, r, c]; strides in elements),
 *   and fmoe_mul_merge_k_add sums the k rows of every token.
 * d_weight (:389-516, :1576-1976 _jagged_jagged_bmm*): dW[e] = A_e^T B_e, a product whose reduction
 *   runs over the rows of expert e. fmoe_jagged_pad_offsets turns offsets [E+1] into kseg [E+1], each
 *   expert's row count rounded up to whole K steps of 128 bytes (at least one);
 *   fmoe_jagged_transpose_pad writes out[c, kseg[e] + j] = in[src(offsets[e] + j), c] (zeros in
 *   the padding; src(r) = index[r] / index_div when index is given, else r; ld_out >= rows + E * 128 /
 *   element size); fmoe_jagged_jagged_bmm multiplies the two transposed operands a_t [M, padded],
 *   b_t [N, padded] in the grouped GEMM's reduction-over-rows mode: out[e * M + m, n] = sum over
 *   expert e's padded range of a_t[m, r] * b_t[n, r]. group_offsets is the uniform [0, M, 2M, ...].
 * d_bias (:1997-2140 _jagged_reduce_sum): fmoe_jagged_colsum, out[e, n] = sum of x[r, n] over the
 *   rows of expert e (fp32 accumulation).
 * combine backward (:922-983 _mul_merge_k_add_bwd): fmoe_gather_scale_rows,
 *   out[p, :] = src[index[p] / index_div, :] * weight[weight_index[p]] (weight NULL: plain gather),
 *   and fmoe_row_dot, out[p] = <a[p, :], b[index[p] / index_div, :]> in fp32 (index NULL: b[p]).
 * activations (:62-106 _fused_swiglu_backward_kernel; triton_general_ops.py:325-344 SiLU backward):
 *   fmoe_activation_backward mode 0: d_alpha = d_out * silu'(alpha); mode 1 (out = silu(alpha) *
 *   beta): d_alpha = d_out * beta * silu'(alpha), d_beta = d_out * silu(alpha). */
/* Router backward (the reference differentiates its eager routing code with autograd,
 * modules/fast_moe_module.py:93-135). The renormalised top-k scores are the softmax over the k
 * selected logits, so d_logits[t, e_j] = y_j (dy_j - sum_i y_i dy_i) and 0 for unselected experts:
 * fmoe_router_backward (topk_idx [L, k], topk_score = y, d_score = dy, all as fmoe_gate_topk wrote
 * them; d_logits [L, E] f32). fmoe_gate_linear_backward then gives the gradients of the gate's
 * Linear: d_x [L, d] (dtype of x, may be NULL) = d_logits @ gate_w, d_gate_w [E, d] f32 = d_logits^T @ x,
 * d_gate_b [E] f32 = column sums (both cleared first; either may be NULL). The two parameter
 * gradients are accumulated with fp32 atomics over chunks of 256 tokens: their last bits can
 * differ from run to run. */
int fmoe_router_backward(const int64_t* topk_idx, const float* topk_score, const float* d_score, int64_t L, int E, int k,
                         float* d_logits, void* stream);
int fmoe_gate_linear_backward(const float* d_logits, const void* x, int x_dtype, int64_t ldx, const float* gate_w,
                              int64_t L, int d, int E, void* d_x, int64_t lddx, float* d_gate_w, float* d_gate_b,
                              void* stream);
/* out[r, :] = jagged[r, :k_split] @ weight0[e] + jagged[r, k_split:] @ weight1[e] for the rows r of expert
 * e: one grouped product whose reduction walks two weights (logical [E, k_split, N] and
 * [E, K - k_split, N], same strides). The backward of the gated up projection uses it for
 * d_x = d_alpha @ W^T + d_beta @ Wp^T (kernels/triton/triton_moe.py:2378-2511) without building the
 * concatenated weight; k_split a multiple of 128 bytes of K. */
int fmoe_jagged_bmm_two_weights(const int64_t* offsets, int64_t total_rows, const void* jagged, int dtype, int64_t ldj,
                                const void* weight0, const void* weight1, int k_split, int64_t w_se, int64_t w_sk,
                                int64_t w_sn, int E, int K, int N, void* out, int out_dtype, int64_t ldo, void* stream);
int fmoe_batched_transpose(const void* in, int dtype, int batch, int64_t in_sb, int64_t ld_in, int rows, int cols,
                           void* out, int64_t out_sb, int64_t ld_out, void* stream);
int fmoe_jagged_pad_offsets(const int64_t* offsets, int E, int dtype, int64_t* kseg, void* stream);
int fmoe_jagged_transpose_pad(const void* in, int dtype, int64_t in_rows, int64_t ld_in, const int64_t* index,
                              int index_div, const int64_t* offsets, const int64_t* kseg, int E, int64_t rows, int cols,
                              void* out, int64_t ld_out, void* stream);
int fmoe_jagged_jagged_bmm(const int64_t* group_offsets, const int64_t* kseg, int64_t padded_rows, const void* a_t,
                           int64_t lda, const void* b_t, int64_t ldb, int dtype, int E, int M, int N, void* out,
                           int out_dtype, int64_t ldo, void* stream);
int fmoe_jagged_colsum(const void* x, int dtype, int64_t ldx, const int64_t* offsets, int E, int N, void* out,
                       int out_dtype, void* stream);
int fmoe_gather_scale_rows(const void* src, int dtype, int64_t src_rows, int64_t lds, const int64_t* index,
                           int index_div, const void* weight, int w_dtype, const int64_t* weight_index,
                           int64_t weight_count, int64_t rows, int cols, void* out, int64_t ldo, void* stream);
int fmoe_row_dot(const void* a, int64_t lda, const void* b, int64_t b_rows, int64_t ldb, int dtype,
                 const int64_t* index, int index_div, int64_t rows, int cols, float* out, void* stream);
int fmoe_activation_backward(int mode, const void* d_out, int64_t ldd, const void* alpha, int64_t lda, const void* beta,
                             int64_t ldb, int dtype, int64_t rows, int cols, void* d_alpha, int64_t ldda, void* d_beta,
                             int64_t lddb, void* stream);

/* ---------------------------------------------------------------------------------------------
 * FP8 rowwise quantisation.
 * pytorch_rowwise_quant_fp8 + calculate_scale (kernels/pytorch/quant_fp8.py:13-34), and with
 * apply_silu != 0 pytorch_silu_jagged_fp8 (kernels/pytorch/moe_fp8.py:17-33):
 *   amax = max|row|; scale = 2^floor(log2(448/amax)), 2^127 when that is not finite;
 *   q = e4m3fn(row * scale) (round to nearest even, no saturation: |v| > 464 gives NaN as
 *   Tensor.to(float8_e4m3fn) does)
 *   in [rows, cols] in_dtype (bf16/f32) row stride ldi; q [rows, cols] bytes, row stride ldq;
 *   scale_out [rows] f32 receives scale, or 1/scale when store_reciprocal != 0; may be NULL.
 */
int fmoe_rowwise_quant_fp8(const void* in, int in_dtype, int64_t rows, int cols, int64_t ldi, int apply_silu,
                           int store_reciprocal, void* q, int64_t ldq, float* scale_out, void* stream);

/* pytorch_bmm_weight_rowwise_quant_fp8 (kernels/pytorch/moe_fp8.py:36-43): weight [E, K, D]
 * contiguous, absmax over K for every (e, d), q = e4m3fn(weight * scale[e, d]).
 * scale_out [E, D] may be NULL (the reference returns only the quantised tensor). */
int fmoe_bmm_weight_quant_fp8(const void* weight, int dtype, int E, int K, int D, void* q, float* scale_out,
                              void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FMOE_B200_H_ */
