// Host-side launch interfaces between the C ABI (capi.cu) and the kernel translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "common.cuh"

namespace rbf {

// One pre-pass launch: any subset of the four row statistics (null input pointer = skip).
struct RowStatsArgs {
  const void* k;          // -> ksq_out = scale * |k|^2, +inf on padding rows
  const void* q;          // -> qsq_out = scale * |q|^2, qsq_pad on padding rows
  const void* o;          // with dout -> delta_out = rowsum(o * dout), 0 on padding rows
  const void* dout;
  const float* lse;       // (B, H, N) -> lse_pad_out re-pitched to n_pad, +inf on padding rows
  float* ksq_out;
  float* qsq_out;
  float* delta_out;
  float* lse_pad_out;
  // "bias slabs": 16 x 16-bit per row (hi, mid, lo parts of an fp32 value, then zeros), consumed as one extra
  // K = 16 step of an MMA against a slab of constants `slab_w`, so that the product adds the fp32 value back.
  void* kslab_out;        // -ksq / (scale2 * slab_w); -slab_big on padding rows
  void* lslab_out;        // -lse / (scale2 * slab_w); -slab_big on padding rows
  void* dslab_out;        // -delta / slab_w; 0 on padding rows
  float* zero_rows;       // optional (B, H, N, D) fp32 array to clear (the backward's dQ accumulator)
  int lslab_from_qsq;     // non-softmax variant: the L slab carries -qsq / (scale2 * slab_w) instead
  int dslab_zero;         // non-softmax variant: dS = P * dP, nothing is subtracted
  float scale2, slab_w, slab_big;
  int64_t ks[3], qs[3], os[3], dos[3];   // element strides of dims b, h, n
  int B, H, N, n_pad;
  float scale;
  float qsq_pad;
  int iters;              // set by the launcher
  DeviceStatus* status_to_clear;  // optional: the 256-byte status block (status word, work counters) is zeroed
};
cudaError_t launch_row_stats(const RowStatsArgs& a, bool bf16, int D, cudaStream_t stream);

// Fused preparation of the attention block's operands (the reference does this with torch ops, rbf_attention.py:
// 1659-1688): splits the fused projection output qkv (B, S, 3, H, D), adds the SuSiE position term to the text rows
// of q and k (table[t, :] * [w | w] with one learnable weight row w per head) and the learned register-position
// rows to the first R rows, writes q' and k' through strides, and in the same pass emits what the forward's pre-pass
// would compute from k' (and q'): the key-norm bias slabs and, for the non-softmax variant, the query norms.
struct QkvPrepArgs {
  const void* qkv;          // (B, S, 3, H, D) contiguous, 16-bit
  const void* pos_weight;   // (H, D/2)
  const void* reg_pos;      // (H, R, D); unused when R == 0
  int params_fp32;          // the two parameter arrays are fp32 (otherwise the 16-bit type of qkv)
  const float* table;       // (>= S - R, D) fp32 SuSiE table [sin | cos], row t for text position t
  void* q_out;              // (B, H, S, D) through strides qo (elements, dims b, h, n)
  void* k_out;
  int64_t qo[3], ko[3];
  void* kslab_out;          // (B*H, n_pad, 16) bias slabs of -c|k'|^2 / (scale2 * slab_w); -slab_big on padding rows
  float* qsq_out;           // optional (B*H, n_pad): c|q'|^2, 0 on padding rows
  DeviceStatus* status_to_clear;
  int B, S, H, D, R, n_pad;
  float scale, scale2, slab_w, slab_big;
};
cudaError_t launch_qkv_prep(const QkvPrepArgs& a, bool bf16, cudaStream_t stream);

// Gradients of the SuSiE parameters from the gradients of q' and k' (both (B, H, S, D) through strides):
//   d_pos_weight[h, i] = sum_{b, t} (dq' + dk')[b, h, R + t, i] * sin-part[t, i] + (dq' + dk')[b, h, R + t, i + D/2] * cos-part[t, i]
//   d_reg_pos[h, r, :] = sum_b (dq' + dk')[b, h, r, :]
// in two launches with a fixed summation order (block partials in `partials`, then one sum per output element).
struct QkvPrepBwdArgs {
  const void* dq;
  const void* dk;
  int64_t dqs[3], dks[3];
  const float* table;
  float* partials;          // (B * chunks, H * D/2) fp32 scratch
  float* d_pos_weight;      // (H, D/2) fp32
  float* d_reg_pos;         // (H, R, D) fp32; unused when R == 0
  int B, S, H, D, R;
  int chunks;               // set by the launcher
};
int qkv_prep_bwd_chunks(int S, int R);
cudaError_t launch_qkv_prep_bwd(QkvPrepBwdArgs a, bool bf16, cudaStream_t stream);

// Exclusive self attention (the attention block's `apply_xsa` option, rbf_attention.py:1757-1759): every output row
// loses its component along the value row of the same position, out = o - (o . vh) vh with vh = v / max(|v|, 1e-12).
// One pass forward; one pass backward giving d_o = g - (g . vh) vh and d_v = (-(o . vh) g - (g . vh) o +
// 2 (o . vh)(g . vh) vh) / |v|. All tensors (B, H, N, D) through strides (elements, dims b, h, n).
struct XsaArgs {
  const void* o;
  const void* v;
  const void* g;           // backward only: gradient of the projected output
  void* out;               // forward: projected output; backward: d_o
  void* dv;                // backward only
  int64_t os[3], vs[3], gs[3], outs[3], dvs[3];
  int B, H, N;
};
cudaError_t launch_xsa(const XsaArgs& a, bool backward, bool bf16, int D, cudaStream_t stream);

// Self-test of the bounded waits: one block waits on a barrier that nothing arms; when the wait runs out after `limit`
// SM clocks it records site kSiteSelfTest in `status` exactly as the attention kernels do, and the kernel returns.
static constexpr uint32_t kSiteSelfTest = 250;
// LayerNorm of the language model's blocks (layer_norm.cu): 16-bit rows of 256, 512, 768 or 1024 columns.
struct LayerNormArgs {
  const void* x;             // (rows, cols) contiguous
  const void* gamma;         // (cols), dtype of x
  const void* beta;          // (cols)
  void* y;                   // (rows, cols)
  float* mean;               // (rows) saved for the backward
  float* rstd;               // (rows)
  int64_t rows;
  float eps;
  const void* residual;      // optional (rows, cols): y = LayerNorm(round(x + residual)) and
  void* sum_out;             // the rounded sum goes here (may be x or residual itself); both NULL or both set
};
struct LayerNormBwdArgs {
  const void* x;
  const void* dy;
  const void* gamma;
  const float* mean;
  const float* rstd;
  void* dx;                  // (rows, cols), dtype of x
  float* dgamma;             // (cols) fp32
  float* dbeta;              // (cols) fp32
  float* partials;           // layer_norm_bwd_blocks() x 2 x cols floats
  int64_t rows;
  const void* dres;          // optional (rows, cols): added to dx before it is rounded (may be dx itself)
};
bool layer_norm_supported(int cols);
int layer_norm_bwd_blocks(int64_t rows, int sms);
cudaError_t launch_layer_norm_fwd(const LayerNormArgs& a, int cols, bool bf16, int sms, cudaStream_t stream);
cudaError_t launch_layer_norm_bwd(const LayerNormBwdArgs& a, int cols, bool bf16, int sms, cudaStream_t stream);

// Column sums of a 16-bit (rows x cols) matrix, row pitch ld elements, into out (cols, fp32): col_sums.cu.
// `partials` holds col_sums_bands() x cols floats.
int col_sums_bands(int64_t rows, int cols, int sms);
cudaError_t launch_col_sums(const void* x, int64_t ld, int64_t rows, int cols, bool bf16, float* partials, float* out,
                            int sms, cudaStream_t stream);

cudaError_t launch_col_sums_final(const float* partials, int bands, int cols, float* out, cudaStream_t stream);

// GELU (erf form) of 16-bit activations, gelu.cu. Forward: n elements, n a multiple of 8. Backward: dh = dy * gelu'(h)
// for a contiguous (rows x cols) matrix, cols a multiple of 8; with dbias != nullptr also dbias[c] = sum_r dh[r, c]
// (fp32), through `partials` (col_sums_bands() x cols floats).
cudaError_t launch_gelu_fwd(const void* h, void* out, int64_t n, bool bf16, int sms, cudaStream_t stream);
cudaError_t launch_gelu_bwd(const void* h, const void* dy, void* dh, int64_t rows, int cols, bool bf16, float* partials,
                            float* dbias, int sms, cudaStream_t stream);

// Cross entropy of the language-model step (ce_loss.cu): per-row losses and d(mean loss)/d(logits) in one kernel.
struct CrossEntropyArgs {
  const void* logits;        // (rows, cols), row pitch ld elements
  int64_t ld;
  const int64_t* targets;    // (rows); ignore_index or out-of-range: the row has no loss and a zero gradient
  void* dlogits;             // (rows, cols), row pitch ld_out elements, dtype of the logits
  int64_t ld_out;
  float* loss_rows;          // (rows)
  const float* grad_scale;   // device scalar multiplied into every gradient (1 / number of rows that count)
  int rows, cols;
  int64_t ignore_index;
};
cudaError_t launch_cross_entropy(const CrossEntropyArgs& a, int dtype, int sms, cudaStream_t stream);
// x *= *factor unless *factor == 1 (decided on the device: nothing synchronises).
cudaError_t launch_scale_unless_one(void* x, const float* factor, int64_t n, int dtype, int sms, cudaStream_t stream);

cudaError_t launch_wait_selftest(DeviceStatus* status, long long limit, cudaStream_t stream);
// One thread stores the status word into mapped page-locked host memory (device-side address of the slot).
cudaError_t launch_post_status(const DeviceStatus* status, unsigned int* host_slot_device_ptr, cudaStream_t stream);

// Forward pass. Tensor maps use a 64-element x 128-row box with the 128-byte swizzle.
struct FwdArgs {
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  CUtensorMap tm_kslab;   // (B*H, n_pad, 16) key-norm bias slabs, box 16 x 128, 32-byte swizzle
  float slab_w;           // constant the other operand's slab holds
  const float* qsq;       // (B*H, n_pad): gamma*log2(e)*|q|^2; non-softmax variant only
  float* lse;             // (B, H, N) base-2 log-sum-exp; softmax variant only
  DeviceStatus* status;
  int B, H, N, n_pad;
  int causal;
  float scale2;           // 2 * gamma * log2(e)
};
cudaError_t launch_fwd(const FwdArgs& a, bool bf16, int D, bool softmax, cudaStream_t stream);
// fp32 tensors on TF32 operands, head dim 64 (tensor maps of fp32 tiles, slabs of 8 floats per row; slab_w unused)
cudaError_t launch_fwd_tf32(const FwdArgs& a, bool softmax, cudaStream_t stream);

// Pre-pass of the TF32 forward over fp32 K (and Q): key-norm bias slabs of 8 floats per row (three TF32 parts of
// -c|k|^2 / scale2, -1e30 on padding rows) and, for the non-softmax variant, c|q|^2 per row (0 on padding rows).
struct RowStatsF32Args {
  const float* k;
  const float* q;           // optional
  int64_t ks[3], qs[3];
  float* kslab_out;
  float* qsq_out;           // optional
  DeviceStatus* status_to_clear;
  int B, H, N, n_pad;
  float scale, scale2;
};
cudaError_t launch_row_stats_f32(const RowStatsF32Args& a, cudaStream_t stream);

// Backward pass (two kernels: key-stationary dK/dV, query-stationary dQ).
struct BwdArgs {
  CUtensorMap tm_q, tm_k, tm_v, tm_do, tm_dq, tm_dk, tm_dv;
  const float* ksq;       // (B*H, n_pad)
  const float* row_bias;  // (B*H, n_pad): softmax: L (base-2 LSE); non-softmax: c*|q|^2; +inf on padding rows
  int row_bias_pitch;     // row pitch of row_bias (n_pad)
  const float* delta;     // (B*H, n_pad): rowsum(O*dO); all zero for the non-softmax variant
  DeviceStatus* status;
  int B, H, N, n_pad;
  int causal;
  float scale2;           // 2 * gamma * log2(e)
  float grad_scale;       // 2 * gamma
};
cudaError_t launch_bwd_dkdv(const BwdArgs& a, bool bf16, int D, bool softmax, cudaStream_t stream);
cudaError_t launch_bwd_dq(const BwdArgs& a, bool bf16, int D, bool softmax, cudaStream_t stream);

// Single-kernel softmax backward (five MMAs per tile pair, dQ through an fp32 accumulator). The head-dim-64 kernel
// streams 128 query rows per step (Q, dO, slab and accumulator maps with 128-row boxes); the head-dim-128 kernel
// streams 64 (those four maps with 64-row boxes).
struct BwdFusedArgs {
  CUtensorMap tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv;
  CUtensorMap tm_lslab, tm_dslab;  // (B*H, n_pad, 16) bias slabs of -L / scale2 and -delta, box 16 x 128
  CUtensorMap tm_dq_acc;  // head dim 64: the accumulator as 32-float x 32-row boxes, 128-byte swizzle
  float* dq_acc;          // fp32 (B, H, N, D) contiguous accumulator
  void* dq;               // final dQ in the operand type
  int64_t dq_strides[3];
  const float* ksq;       // (B*H, n_pad); head dim 64 only (the head-dim-128 kernel takes the norms from its K tile)
  // non-softmax variant: dQ = 2 gamma (acc - delta * q) with delta = rowsum(O * dO) = rowsum_j dS_ij; null otherwise
  const void* q_rows;
  int64_t q_strides[3];
  const float* delta;     // (B*H, n_pad)
  DeviceStatus* status;
  unsigned int* work;     // two work counters of the persistent launch (zero at launch; D = 64 kernel)
  int sm_count;
  int B, H, N, n_pad;
  int causal;
  float scale2, grad_scale, slab_w;
};
cudaError_t launch_bwd_fused(const BwdFusedArgs& a, bool bf16, cudaStream_t stream);      // D = 64
cudaError_t launch_bwd_fused128(const BwdFusedArgs& a, bool bf16, cudaStream_t stream);   // D = 128

// cudaFuncSetAttribute applies to the current device only, so a kernel's dynamic shared-memory limit has to be raised
// once on every device the process launches it on. One flag per device and kernel instantiation; devices beyond the
// table are configured on every launch.
struct PerDeviceFlags {
  static constexpr int kMaxDevices = 64;
  std::atomic<int> done[kMaxDevices];
};
template <class Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kernel, int bytes, PerDeviceFlags& flags) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool cached = dev >= 0 && dev < PerDeviceFlags::kMaxDevices;
  if (cached && flags.done[dev].load(std::memory_order_acquire)) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && cached) flags.done[dev].store(1, std::memory_order_release);
  return e;
}

// SM count of the current device (-1 on error), cached per device.
inline int device_sm_count() {
  static std::atomic<int> cached[PerDeviceFlags::kMaxDevices];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return -1;
  const bool slot = dev < PerDeviceFlags::kMaxDevices;
  if (slot) {
    const int c = cached[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return -1;
  if (slot) cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

}  // namespace rbf
