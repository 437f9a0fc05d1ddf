/*
 * C ABI of librbf_b200.so: fused RBF attention forward / backward on NVIDIA B200 (sm_100a).
 *
 * These entry points are what a foreign-function binding of the reference project's operator
 * boundary would call in place of its Triton launchers. The reference registers four operators
 * (file paths are inside the reference project):
 *
 *   rbf_attn_v5::scaled_fwd       rbf_attention.py:651-690    -> rbf_b200_fwd(softmax = 1)
 *   rbf_attn_v5::scaled_bwd       rbf_attention.py:702-810    -> rbf_b200_bwd(softmax = 1)
 *   rbf_attn_v5::non_softmax_fwd  rbf_attention.py:1355-1391  -> rbf_b200_fwd(softmax = 0)
 *   rbf_attn_v5::non_softmax_bwd  rbf_attention.py:1399-1480  -> rbf_b200_bwd(softmax = 0)
 *
 * Conventions
 *   - All tensors are (B, H, N, D) with unit stride on D; `*_strides` point at three element strides
 *     for the dims (b, h, n), exactly what the reference passes to its kernels
 *     (rbf_attention.py:671-682). D must be 64 or 128. Base addresses must be 16-byte aligned and the
 *     strides multiples of 8 elements (TMA addressing).
 *   - dtype: 0 = bfloat16, 1 = float16. Accumulation is fp32. `lse` and the workspace are fp32. The forward
 *     also takes dtype 2 = float32 tensors at D = 64: TF32 tensor-core operands like the reference's Triton path for
 *     fp32 inputs (rbf_attention.py:183), strides counted in fp32 elements (multiples of 4), fp32 output.
 *   - The library never allocates device memory: the caller passes a workspace of at least
 *     rbf_b200_workspace_bytes() bytes, 256-byte aligned, which the call may overwrite entirely.
 *   - Launches go to `stream` (a cudaStream_t passed as void*; NULL = legacy default stream) on the
 *     current device. No call synchronises except rbf_b200_read_device_status().
 *   - Every function returns 0 on success or a positive rbf_b200 status code; nothing throws or aborts.
 *     rbf_b200_last_error() returns a thread-local message for the last failing call.
 */
#ifndef RBF_B200_H_
#define RBF_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RBF_B200_ABI_VERSION 3

enum {
  RBF_B200_OK = 0,
  RBF_B200_ERR_BAD_ARGUMENT = 1,
  RBF_B200_ERR_BAD_LAYOUT = 2,
  RBF_B200_ERR_WORKSPACE = 3,
  RBF_B200_ERR_TENSOR_MAP = 4,
  RBF_B200_ERR_LAUNCH = 5,
  RBF_B200_ERR_DEVICE = 6
};

/* ABI version of the loaded library (RBF_B200_ABI_VERSION at build time). */
int rbf_b200_abi_version(void);

/* Message describing the last error raised on the calling thread ("" if none). */
const char* rbf_b200_last_error(void);

/* Bytes of scratch the forward (backward = 0) or backward (backward = 1) call needs.
 * Replaces the reference launchers' internal torch.empty calls for L-adjacent scratch
 * (rbf_attention.py:716 `Delta`) and holds the pre-computed key / query norm bias. */
size_t rbf_b200_workspace_bytes(int B, int H, int N, int D, int softmax, int backward);

/* Forward. Replaces rbf_scaled_fwd (rbf_attention.py:651-690) when softmax = 1 and
 * rbf_non_softmax_fwd (rbf_attention.py:1355-1391) when softmax = 0.
 *   out : (B, H, N, D) in `dtype`, strides o_strides.
 *   lse : (B, H, N) contiguous fp32, base-2 log-sum-exp of the base-2-scaled logits
 *         (rbf_attention.py:217-219); ignored (may be NULL) when softmax = 0.
 *   sm_scale : gamma; the reference always uses 1/sqrt(D) (rbf_attention.py:660). */
int rbf_b200_fwd(const void* q, const void* k, const void* v, void* out, float* lse, void* workspace,
                 size_t workspace_bytes, int B, int H, int N, int D, const int64_t* q_strides,
                 const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides, int dtype,
                 int causal, int softmax, float sm_scale, void* stream);

/* Backward. Replaces rbf_scaled_bwd (rbf_attention.py:702-810: _bwd_preprocess, dK/dV kernel, dQ kernel)
 * when softmax = 1 and rbf_non_softmax_bwd (rbf_attention.py:1399-1480) when softmax = 0.
 *   out, lse : the forward's results. lse is ignored (may be NULL) when softmax = 0. out is optional when
 *              softmax = 0 (the reference's operator does not have it): with it the backward runs as one kernel
 *              (rowsum_j dS_ij = dO_i . O_i feeds the query-norm term), without it as the reference's two.
 *   dq, dk, dv : (B, H, N, D) in `dtype`. dk includes the gradient through the key-norm term
 *                (rbf_attention.py:447); for softmax = 0, dq includes the query-norm term (:1336). */
int rbf_b200_bwd(const void* q, const void* k, const void* v, const void* out, const float* lse, const void* dout,
                 void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes, int B, int H, int N, int D,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const int64_t* o_strides, const int64_t* do_strides, const int64_t* dq_strides,
                 const int64_t* dk_strides, const int64_t* dv_strides, int dtype, int causal, int softmax,
                 float sm_scale, void* stream);

/* The same calls restricted to some of their kernels, for per-kernel timing and profiling. `phases` is a
 * mask of RBF_B200_PHASE_*: the pre-pass (key / query norms, delta, bias slabs; in the backward it also clears
 * the fp32 dQ accumulator), the main kernel (forward; the single-kernel backward with its dQ conversion, or dK/dV
 * of the two-kernel backward) and the two-kernel backward's second kernel (dQ). Skipped phases leave the workspace
 * contents of an earlier call in place: a backward MAIN without its PREPASS adds to the accumulator of the
 * previous call, which is fine for timing and wrong for results. No counterpart in the reference, whose launchers
 * always run every kernel. */
#define RBF_B200_PHASE_PREPASS 1
#define RBF_B200_PHASE_MAIN 2
#define RBF_B200_PHASE_MAIN2 4
#define RBF_B200_PHASE_ALL 7
int rbf_b200_fwd_phases(const void* q, const void* k, const void* v, void* out, float* lse, void* workspace,
                        size_t workspace_bytes, int B, int H, int N, int D, const int64_t* q_strides,
                        const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides, int dtype,
                        int causal, int softmax, float sm_scale, void* stream, int phases);
int rbf_b200_bwd_phases(const void* q, const void* k, const void* v, const void* out, const float* lse,
                        const void* dout, void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes, int B,
                        int H, int N, int D, const int64_t* q_strides, const int64_t* k_strides,
                        const int64_t* v_strides, const int64_t* o_strides, const int64_t* do_strides,
                        const int64_t* dq_strides, const int64_t* dk_strides, const int64_t* dv_strides, int dtype,
                        int causal, int softmax, float sm_scale, void* stream, int phases);

/* Forward for callers that cannot hand over device memory of their own. It has no counterpart in the reference,
 * whose launchers allocate freely through torch. Some hosts of this library cannot do that: a plug-in running
 * inside an engine that owns all device memory and forbids allocation after start-up, a real-time or serving loop
 * where cudaMalloc's implicit device synchronisation is not acceptable, or a thin foreign-function caller that has
 * no allocator at hand for the few megabytes of scratch. For them the scratch of the forward (status word, key-norm
 * bias slabs, and the query norms of the non-softmax variant) lives in a fixed array of
 * RBF_B200_STATIC_SCRATCH_BYTES inside the library's device image; every GPU that loads the library keeps it
 * reserved until the process exits. The call makes no cudaMalloc / cudaFree and calls nothing that allocates.
 *   - Problems whose scratch (rbf_b200_workspace_bytes(..., backward = 0)) exceeds the array are refused with
 *     RBF_B200_ERR_WORKSPACE; configuration 2 of the benchmark (B8 H16 N4096) just fits.
 *   - The first call on each device looks up the array's device address (with that device current); make that
 *     first call outside any stream capture.
 *   - All calls share the one array, and it keeps what the last call left. Each call rewrites everything it
 *     later reads, so consecutive calls on one stream are independent; two calls that may run on the GPU at the
 *     same time (different streams, different host threads) race on it and must not be made.
 * Inputs, outputs and all other arguments are those of rbf_b200_fwd. */
#define RBF_B200_STATIC_SCRATCH_BYTES (20u * 1024u * 1024u)
size_t rbf_b200_static_scratch_bytes(void);
int rbf_b200_fwd_static(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int N, int D,
                        const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                        const int64_t* o_strides, int dtype, int causal, int softmax, float sm_scale, void* stream);

/* Fused preparation of the attention block's operands. Replaces the torch ops between the fused projection and the
 * attention call in CustomCausalAttention.forward (rbf_attention.py:1659-1688; parameters :1642-1654): it reads the
 * projection output `qkv` (B, S, 3, H, D contiguous: the reference's "b s (qkv h n)" layout), adds to q and k the
 * SuSiE position term `susie_table[t, :] * [w_h | w_h]` on the text rows (w_h = row h of `pos_weight`, (H, D/2); t
 * counts text rows, which follow the R register rows) and row (h, r) of `reg_pos_emb` (H, R, D) on the register rows,
 * and writes q', k' as (B, H, S, D) tensors through `q_strides`, `k_strides` (v needs nothing: pass the v part of
 * `qkv` to the forward as a strided view). In the same pass it fills `fwd_workspace` (rbf_b200_workspace_bytes(...,
 * backward = 0) bytes) with what the forward's pre-pass would compute from k' (and q' when softmax = 0) and clears its
 * status word, so that the forward that follows runs as rbf_b200_fwd_phases(..., RBF_B200_PHASE_MAIN) alone.
 * `params_fp32` != 0: the two parameter arrays are fp32 (autocast training); otherwise they have type `dtype`.
 * `susie_table` is fp32, (at least S - R, D), [sin | cos] as rbf_attention.py:1539-1544 builds it. */
int rbf_b200_qkv_prep(const void* qkv, const void* pos_weight, const void* reg_pos_emb, int params_fp32,
                      const float* susie_table, void* q_out, void* k_out, const int64_t* q_strides,
                      const int64_t* k_strides, void* fwd_workspace, size_t fwd_workspace_bytes, int B, int S, int H,
                      int D, int R, int dtype, int softmax, float sm_scale, void* stream);

/* Gradients of the block's position parameters from dq', dk' (the attention backward's dq, dk; (B, H, S, D) through
 * strides): d_pos_weight (H, D/2) and d_reg_pos_emb (H, R, D), both fp32, summed in a fixed order (bitwise
 * reproducible). Replaces what autograd derives from rbf_attention.py:1667-1688 (broadcast sums over batch and
 * sequence). The gradient of the fused projection output is dq', dk', dv themselves: let the attention backward
 * write them into one (B, S, 3, H, D) buffer through its output strides. `workspace`: at least
 * rbf_b200_qkv_prep_bwd_workspace_bytes() bytes, 256-byte aligned. */
size_t rbf_b200_qkv_prep_bwd_workspace_bytes(int B, int S, int H, int D, int R);
int rbf_b200_qkv_prep_bwd(const void* dq, const void* dk, const int64_t* dq_strides, const int64_t* dk_strides,
                          const float* susie_table, float* d_pos_weight, float* d_reg_pos_emb, void* workspace,
                          size_t workspace_bytes, int B, int S, int H, int D, int R, int dtype, void* stream);

/* Exclusive self attention, the attention block's apply_xsa option (rbf_attention.py:1757-1759):
 * out = o - (o . vh) vh per row, with vh = v / max(|v|, 1e-12) the normalised value row of the same position; all
 * tensors (B, H, N, D) through strides, arithmetic in fp32, one pass over the rows. The backward call returns, from
 * the gradient g of `out`, d_o = g - (g . vh) vh and the contribution to d_v of this step (the attention backward's
 * own d_v is added by the caller); it needs o as the attention produced it, which is why this is a separate pass and
 * not part of the attention kernel's output stage: the attention backward needs that same unprojected o. */
int rbf_b200_xsa_fwd(const void* o, const void* v, void* out, const int64_t* o_strides, const int64_t* v_strides,
                     const int64_t* out_strides, int B, int H, int N, int D, int dtype, void* stream);
int rbf_b200_xsa_bwd(const void* g, const void* o, const void* v, void* d_o, void* d_v, const int64_t* g_strides,
                     const int64_t* o_strides, const int64_t* v_strides, const int64_t* do_strides,
                     const int64_t* dv_strides, int B, int H, int N, int D, int dtype, void* stream);

/* LayerNorm of the language model's blocks (nn.LayerNorm(emb_dim), train_rbf_transformer.py:139-150, 215, 241) for 16-bit
 * activations: x, y (rows, cols) contiguous, gamma and beta (cols) in the dtype of x (0 = bfloat16, 1 = float16), cols
 * 256, 512, 768 or 1024, all 16-byte aligned. Statistics in fp32; `mean` and `rstd` (rows, fp32) are saved for the
 * backward, which returns dx in the dtype of x and dgamma, dbeta in fp32, summed in a fixed order (bitwise
 * reproducible). The backward's workspace holds one fp32 partial row per thread block. */
int rbf_b200_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                            int64_t rows, int cols, float eps, int dtype, void* stream);
size_t rbf_b200_layer_norm_bwd_workspace_bytes(int64_t rows, int cols);
int rbf_b200_layer_norm_bwd(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                            void* dx, float* dgamma, float* dbeta, void* workspace, size_t workspace_bytes,
                            int64_t rows, int cols, int dtype, void* stream);

/* The same two passes with the block's residual connection folded in (x = x + f(x) followed by the next LayerNorm,
 * train_rbf_transformer.py:147-151). Forward: sum_out = x + residual rounded to the dtype (exactly what the separate
 * addition leaves; sum_out may be x or residual itself, not y) and y = LayerNorm(sum_out); residual and sum_out are
 * both NULL (then this is rbf_b200_layer_norm_fwd) or both set. Backward: x is the forward's sum_out, and `dres`
 * (NULL, or the gradient that reaches sum_out from its other consumers; may be dx itself) is added to dx in fp32
 * before dx is rounded - dx is then the gradient of both x and residual. */
int rbf_b200_add_layer_norm_fwd(const void* x, const void* residual, void* sum_out, const void* gamma, const void* beta,
                                void* y, float* mean, float* rstd, int64_t rows, int cols, float eps, int dtype,
                                void* stream);
int rbf_b200_layer_norm_bwd_add(const void* x, const void* dy, const void* dres, const void* gamma, const float* mean,
                                const float* rstd, void* dx, float* dgamma, float* dbeta, void* workspace,
                                size_t workspace_bytes, int64_t rows, int cols, int dtype, void* stream);

/* out[c] = sum over r of x[r, c] in fp32 for a 16-bit matrix (rows x cols, row pitch `ld` elements, cols and ld
 * multiples of 8, 16-byte aligned base; dtype 0 = bfloat16, 1 = float16): the bias gradient of a linear layer
 * (`nn.Linear` in train_rbf_transformer.py:143, 216 and rbf_attention.py:1625-1626), which PyTorch computes with a
 * generic reduction. Summed in a fixed order. The workspace holds one fp32 partial row per band of rows. */
size_t rbf_b200_column_sums_workspace_bytes(int64_t rows, int cols);
int rbf_b200_column_sums(const void* x, float* out, void* workspace, size_t workspace_bytes, int64_t rows, int cols,
                         int64_t ld, int dtype, void* stream);

/* GELU in its exact (erf) form, nn.GELU() of the model's MLP (train_rbf_transformer.py:143), for 16-bit activations
 * (dtype 0 = bfloat16, 1 = float16; 16-byte aligned, contiguous). Forward: out[i] = h[i] Phi(h[i]) for n elements, n a
 * multiple of 8. Backward: dh = dy * (Phi(h) + h phi(h)) for a (rows x cols) matrix, cols a multiple of 8; with
 * dbias != NULL the same pass also gives dbias[c] = sum over rows of dh[r, c] in fp32 (the bias gradient of the
 * projection that produced h), through a workspace of rbf_b200_column_sums_workspace_bytes(rows, cols) bytes. Phi comes
 * from a rational approximation with an absolute error below 1.5e-7. */
int rbf_b200_gelu_fwd(const void* h, void* out, int64_t n, int dtype, void* stream);
int rbf_b200_gelu_bwd(const void* h, const void* dy, void* dh, float* dbias, void* workspace, size_t workspace_bytes,
                      int64_t rows, int cols, int dtype, void* stream);

/* Cross entropy of the language-model training step: replaces torch.nn.CrossEntropyLoss(ignore_index=-100) and its
 * backward (train_rbf_transformer.py:282, 335-345). One kernel reads the logits (rows x cols, row pitch `ld` elements,
 * dtype 0 = bfloat16, 1 = float16, 2 = float32), writes loss_rows[r] = logsumexp(logits[r]) - logits[r, targets[r]] and
 * dlogits[r, :] = (softmax(logits[r]) - onehot(targets[r])) * (*grad_scale), in the dtype of the logits with row pitch
 * `ld_out`. `grad_scale` is a device scalar (the caller's 1 / number of counted rows), so that the mean loss's
 * gradient needs no second pass. A row whose target equals `ignore_index` or lies outside [0, cols) gets loss 0 and a
 * zero gradient. Columns holding -inf have probability and gradient zero. 16-byte aligned bases and pitches that are
 * multiples of 16 bytes take the vector path; anything else runs element by element. */
int rbf_b200_cross_entropy(const void* logits, const int64_t* targets, const float* grad_scale, float* loss_rows,
                           void* dlogits, int rows, int cols, int64_t ld, int64_t ld_out, int64_t ignore_index,
                           int dtype, void* stream);

/* x[0..n) *= *factor, decided on the device: when *factor == 1 (the gradient of a loss that is the graph's output)
 * the kernel returns without touching x. Used by the backward of the cross entropy above. */
int rbf_b200_scale_unless_one(void* x, const float* factor, int64_t n, int dtype, void* stream);

/* Synchronises `stream` and reads the device status word that the last call using `workspace` left:
 * 0 = ok, otherwise (site << 24 | work unit) of the bounded wait that ran out; the work unit is the linear block
 * index of the launch or, for the persistent kernels (head dim 64), the work item the block was on. Returns
 * RBF_B200_ERR_DEVICE when the word is non-zero. `workspace` = NULL reads the built-in scratch of the current
 * device, i.e. the status the last rbf_b200_fwd_static call left. No counterpart in the reference (its kernels have
 * no device-side waits). */
int rbf_b200_read_device_status(const void* workspace, void* stream, unsigned int* code);

/* Asynchronous form of the status read: enqueues on `stream` a one-thread kernel that stores the status word at the
 * start of `workspace` into `*host_slot`, a 4-byte slot in page-locked host memory that is mapped into the device's
 * address space (cudaHostAlloc / cudaHostRegister; the function resolves the device-side address itself). Nothing
 * synchronises and no copy engine is used, so the word is not queued behind the caller's own bulk transfers; the host
 * reads the slot once an event recorded after this call has completed. No counterpart in the reference. */
int rbf_b200_post_device_status(const void* workspace, unsigned int* host_slot, void* stream);

/* Process-wide switch for run-to-run bitwise reproducible gradients. Off (default): the backward runs as one kernel
 * per call whose dQ partials are added in fp32 in arrival order (dQ then differs by rounding between runs; O, L, dK,
 * dV never do). On: the backward runs as the reference's two kernels (key-stationary dK/dV, rbf_attention.py:279-477,
 * and query-stationary dQ, :480-642), which sum in a fixed order like the reference's, at about 7/5 of the tensor
 * work. Returns the previous setting. */
int rbf_b200_set_deterministic(int on);
int rbf_b200_get_deterministic(void);

/* Self-test of the bounded device waits every kernel of the library relies on: launches one block that waits, with
 * the kernels' own wait routine, on a barrier that nothing arms. After `limit_cycles` SM clocks (at most 2e9) the
 * wait gives up, records site 250 in the status word at the start of `workspace` (at least 256 bytes, 256-byte
 * aligned) and the kernel returns by itself; rbf_b200_read_device_status then reports RBF_B200_ERR_DEVICE. A later
 * forward or backward call on the same workspace clears the word. Nothing traps, faults or spins without bound.
 * No counterpart in the reference. */
int rbf_b200_selftest_wait_timeout(void* workspace, size_t workspace_bytes, long long limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* RBF_B200_H_ */
