// C ABI of the library (see include/rbf_b200.h): argument validation, workspace carving, TMA tensor
// maps, and the launch sequence of each call. No device memory is allocated here.
#include <math.h>
#include <stdarg.h>

#include <atomic>

#include <stdio.h>
#include <string.h>

#include "../../include/rbf_b200.h"
#include "common.cuh"
#include "launch.h"
#include "tmap.h"

namespace {

thread_local char g_last_error[512] = "";

int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

constexpr size_t kStatusBytes = 256;
size_t align256(size_t x) { return (x + 255) / 256 * 256; }

struct Workspace {
  rbf::DeviceStatus* status;
  void* kslab;       // forward: key-norm bias slabs, 32 bytes per row
  float* ksq;        // backward: c|k|^2 per row
  float* row_bias;   // query norms (non-softmax) or the forward's L re-pitched to n_pad (softmax backward)
  float* delta;      // backward only
  void* lslab;       // single-kernel backward only: L and delta bias slabs, fp32 (B, H, N, D) dQ accumulator
  void* dslab;
  float* dq_acc;
  size_t bytes;
};

// The backward runs as one kernel that accumulates dQ in fp32 global memory (a kernel per head dim). The non-softmax
// variant needs the forward output for it (rowsum_j dS_ij = dO_i . O_i); without `out` it takes the two-kernel path.
// The workspace is sized for the single kernel in every case.
// With the deterministic flag set (rbf_b200_set_deterministic) every backward takes the two-kernel path, whose
// summation order is fixed: the single kernel adds its dQ partials in arrival order.
std::atomic<int> g_deterministic{0};
bool use_fused_backward(int D, int softmax, bool have_out) {
  if (g_deterministic.load(std::memory_order_relaxed)) return false;
  return (softmax || have_out) && (D == 64 || D == 128);
}

// Constant held by the operand-side slab of a bias-slab MMA step, and the "minus infinity" the slabs use on padding
// rows. fp16 needs the range extension: a bias up to 65504 * 256 stays representable.
float slab_w(bool bf16) { return bf16 ? 1.0f : 256.0f; }
float slab_big(bool bf16) { return bf16 ? 1e30f : 60000.0f; }

Workspace carve(void* base, int B, int H, int N, int D, int softmax, int backward) {
  const size_t rows = static_cast<size_t>(B) * H * rbf::padded_rows(N);
  const size_t vec = align256(rows * sizeof(float));
  const size_t slab = align256(rows * 32);
  char* p = static_cast<char*>(base);
  Workspace w{};
  size_t off = 0;
  w.status = reinterpret_cast<rbf::DeviceStatus*>(p + off);
  off += kStatusBytes;
  if (!backward) {
    w.kslab = p + off;
    off += slab;
    if (!softmax) {
      w.row_bias = reinterpret_cast<float*>(p + off);
      off += vec;
    }
  } else {
    w.ksq = reinterpret_cast<float*>(p + off);
    off += vec;
    w.row_bias = reinterpret_cast<float*>(p + off);
    off += vec;
    w.delta = reinterpret_cast<float*>(p + off);
    off += vec;
    if (D == 64 || D == 128) {
      w.lslab = p + off;
      off += slab;
      w.dslab = p + off;
      off += slab;
      w.dq_acc = reinterpret_cast<float*>(p + off);
      off += align256(static_cast<size_t>(B) * H * N * D * sizeof(float));
    }
  }
  w.bytes = off;
  return w;
}

int check_common(int B, int H, int N, int D, int dtype, float sm_scale) {
  if (B <= 0 || H <= 0 || N <= 0) return fail(RBF_B200_ERR_BAD_ARGUMENT, "B, H, N must be positive (got %d, %d, %d)", B, H, N);
  if (static_cast<long long>(B) * H > 65535) return fail(RBF_B200_ERR_BAD_ARGUMENT, "B*H = %lld exceeds 65535", static_cast<long long>(B) * H);
  if (D != 64 && D != 128) return fail(RBF_B200_ERR_BAD_ARGUMENT, "head dim D = %d is not supported (64 or 128)", D);
  if (dtype != 0 && dtype != 1) return fail(RBF_B200_ERR_BAD_ARGUMENT, "dtype %d is not supported (0 = bf16, 1 = fp16)", dtype);
  if (!(sm_scale > 0.f) || !isfinite(sm_scale)) return fail(RBF_B200_ERR_BAD_ARGUMENT, "sm_scale must be positive and finite");
  return 0;
}

int check_tensor(const char* name, const void* p, const int64_t* s, int B, int H, int N, int D) {
  if (p == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "%s is NULL", name);
  if (s == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "%s strides are NULL", name);
  if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return fail(RBF_B200_ERR_BAD_LAYOUT, "%s base address is not 16-byte aligned", name);
  const int ext[3] = {B, H, N};
  for (int i = 0; i < 3; ++i) {
    if (ext[i] == 1) continue;  // stride of an extent-1 dim is never used
    if (s[i] <= 0 || s[i] % 8 != 0)
      return fail(RBF_B200_ERR_BAD_LAYOUT, "%s stride[%d] = %lld must be a positive multiple of 8 elements", name, i,
                  static_cast<long long>(s[i]));
    if (s[i] >= (1ll << 38)) return fail(RBF_B200_ERR_BAD_LAYOUT, "%s stride[%d] is too large for TMA", name, i);
  }
  if (N > 1 && s[2] < D) return fail(RBF_B200_ERR_BAD_LAYOUT, "%s row stride %lld is smaller than D", name, static_cast<long long>(s[2]));
  return 0;
}

int make_map(CUtensorMap* m, const char* name, const void* p, const int64_t* s, bool bf16, int B, int H, int N, int D,
             int box_rows = rbf::kTile) {
  const int r = rbf::make_tmap_bhnd(m, p, bf16, B, H, N, D, s[0], s[1], s[2], box_rows);
  if (r != 0) return fail(RBF_B200_ERR_TENSOR_MAP, "cuTensorMapEncodeTiled failed for %s (code %d)", name, r);
  return 0;
}

// SM count of the current device (cached per device)
int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    cached[dev] = n;
  }
  return cached[dev];
}

void set_strides(int64_t (&dst)[3], const int64_t* src) {
  dst[0] = src[0]; dst[1] = src[1]; dst[2] = src[2];
}

}  // namespace

extern "C" {

int rbf_b200_abi_version(void) { return RBF_B200_ABI_VERSION; }

const char* rbf_b200_last_error(void) { return g_last_error; }

size_t rbf_b200_workspace_bytes(int B, int H, int N, int D, int softmax, int backward) {
  if (B <= 0 || H <= 0 || N <= 0) return 0;
  return carve(nullptr, B, H, N, D, softmax, backward).bytes;
}

// Forward for fp32 tensors on TF32 operands (dtype 2, head dim 64): the tensors' strides count fp32 elements.
static int fwd_tf32(const void* q, const void* k, const void* v, void* out, float* lse, void* workspace,
                    size_t workspace_bytes, int B, int H, int N, int D, const int64_t* q_strides,
                    const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides, int causal,
                    int softmax, float sm_scale, void* stream_v, int phases) {
  int rc;
  if ((rc = check_common(B, H, N, 64, 0, sm_scale))) return rc;
  if (D != 64) return fail(RBF_B200_ERR_BAD_ARGUMENT, "fp32 tensors (TF32 operands) are supported at head dim 64, got %d", D);
  const void* ptrs[4] = {q, k, v, out};
  const int64_t* strs[4] = {q_strides, k_strides, v_strides, o_strides};
  const char* names[4] = {"q", "k", "v", "out"};
  for (int t = 0; t < 4; ++t) {
    if (ptrs[t] == nullptr || strs[t] == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "%s or its strides are NULL", names[t]);
    if (reinterpret_cast<uintptr_t>(ptrs[t]) % 16 != 0) return fail(RBF_B200_ERR_BAD_LAYOUT, "%s base address is not 16-byte aligned", names[t]);
    const int ext[3] = {B, H, N};
    for (int i = 0; i < 3; ++i)
      if (ext[i] > 1 && (strs[t][i] <= 0 || strs[t][i] % 4 != 0))
        return fail(RBF_B200_ERR_BAD_LAYOUT, "%s stride[%d] = %lld must be a positive multiple of 4 fp32 elements", names[t], i,
                    static_cast<long long>(strs[t][i]));
    if (N > 1 && strs[t][2] < D) return fail(RBF_B200_ERR_BAD_LAYOUT, "%s row stride is smaller than D", names[t]);
  }
  if (softmax && lse == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "lse is NULL");
  if (workspace == nullptr || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace is NULL or not 256-byte aligned");
  const Workspace ws = carve(workspace, B, H, N, D, softmax, 0);       // same sizes: 32 bytes of slab per padded row
  if (workspace_bytes < ws.bytes)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, ws.bytes);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int n_pad = rbf::padded_rows(N);
  const float c = sm_scale * rbf::kLog2e;
  cudaError_t e = cudaSuccess;
  if (phases & RBF_B200_PHASE_PREPASS) {
    rbf::RowStatsF32Args r{};
    r.k = static_cast<const float*>(k); set_strides(r.ks, k_strides);
    if (!softmax) { r.q = static_cast<const float*>(q); set_strides(r.qs, q_strides); r.qsq_out = ws.row_bias; }
    r.kslab_out = static_cast<float*>(ws.kslab); r.status_to_clear = ws.status;
    r.B = B; r.H = H; r.N = N; r.n_pad = n_pad; r.scale = c; r.scale2 = 2.f * c;
    e = rbf::launch_row_stats_f32(r, stream);
    if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "pre-pass launch failed: %s", cudaGetErrorString(e));
  }
  if (!(phases & RBF_B200_PHASE_MAIN)) return RBF_B200_OK;
  rbf::FwdArgs a{};
  const void* bases[4] = {q, k, v, out};
  CUtensorMap* maps[4] = {&a.tm_q, &a.tm_k, &a.tm_v, &a.tm_o};
  const int rows[4] = {rbf::kTile, 64, 64, rbf::kTile};
  for (int t = 0; t < 4; ++t) {
    const int r = rbf::make_tmap_bhnd_f32(maps[t], bases[t], B, H, N, D, strs[t][0], strs[t][1], strs[t][2], rows[t]);
    if (r != 0) return fail(RBF_B200_ERR_TENSOR_MAP, "cuTensorMapEncodeTiled failed for %s (code %d)", names[t], r);
  }
  const int sr = rbf::make_tmap_slab8_f32(&a.tm_kslab, ws.kslab, B * H, n_pad, 64);
  if (sr != 0) return fail(RBF_B200_ERR_TENSOR_MAP, "cuTensorMapEncodeTiled failed for the key-norm slabs (code %d)", sr);
  a.qsq = ws.row_bias; a.lse = lse; a.status = ws.status;
  a.B = B; a.H = H; a.N = N; a.n_pad = n_pad; a.causal = causal ? 1 : 0; a.scale2 = 2.f * c; a.slab_w = 1.0f;
  e = rbf::launch_fwd_tf32(a, softmax != 0, stream);
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "forward launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_fwd_phases(const void* q, const void* k, const void* v, void* out, float* lse, void* workspace,
                        size_t workspace_bytes, int B, int H, int N, int D, const int64_t* q_strides,
                        const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides, int dtype,
                        int causal, int softmax, float sm_scale, void* stream_v, int phases) {
  g_last_error[0] = 0;
  int rc;
  if (dtype == 2)
    return fwd_tf32(q, k, v, out, lse, workspace, workspace_bytes, B, H, N, D, q_strides, k_strides, v_strides,
                    o_strides, causal, softmax, sm_scale, stream_v, phases);
  if ((rc = check_common(B, H, N, D, dtype, sm_scale))) return rc;
  if ((rc = check_tensor("q", q, q_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("k", k, k_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("v", v, v_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("out", out, o_strides, B, H, N, D))) return rc;
  if (softmax && lse == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "lse is NULL");
  if (workspace == nullptr || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace is NULL or not 256-byte aligned");
  const Workspace ws = carve(workspace, B, H, N, D, softmax, 0);
  if (workspace_bytes < ws.bytes)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, ws.bytes);

  const bool bf16 = dtype == 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  rbf::FwdArgs a{};
  // the forward streams keys in tiles of 128 at D = 64 and of 64 at D = 128
  const int key_rows = D == 128 ? 64 : rbf::kTile;
  if ((rc = make_map(&a.tm_q, "q", q, q_strides, bf16, B, H, N, D))) return rc;
  if ((rc = make_map(&a.tm_k, "k", k, k_strides, bf16, B, H, N, D, key_rows))) return rc;
  if ((rc = make_map(&a.tm_v, "v", v, v_strides, bf16, B, H, N, D, key_rows))) return rc;
  if ((rc = make_map(&a.tm_o, "out", out, o_strides, bf16, B, H, N, D))) return rc;

  const int n_pad = rbf::padded_rows(N);
  const float c = sm_scale * rbf::kLog2e;
  cudaError_t e = cudaSuccess;
  if (phases & RBF_B200_PHASE_PREPASS) {
    rbf::RowStatsArgs r{};
    r.B = B; r.H = H; r.N = N; r.n_pad = n_pad; r.scale = c; r.status_to_clear = ws.status;
    r.scale2 = 2.f * c; r.slab_w = slab_w(bf16); r.slab_big = slab_big(bf16);
    r.k = k; r.kslab_out = ws.kslab; set_strides(r.ks, k_strides);
    if (!softmax) {
      r.q = q; r.qsq_out = ws.row_bias; r.qsq_pad = 0.f; set_strides(r.qs, q_strides);
    }
    e = rbf::launch_row_stats(r, bf16, D, stream);
    if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "pre-pass launch failed: %s", cudaGetErrorString(e));
  }
  if (!(phases & RBF_B200_PHASE_MAIN)) return RBF_B200_OK;

  const int sr = rbf::make_tmap_slab16(&a.tm_kslab, ws.kslab, bf16, B * H, n_pad, key_rows);
  if (sr != 0) return fail(RBF_B200_ERR_TENSOR_MAP, "cuTensorMapEncodeTiled failed for the key-norm slabs (code %d)", sr);
  a.slab_w = slab_w(bf16);
  a.qsq = ws.row_bias; a.lse = lse; a.status = ws.status;
  a.B = B; a.H = H; a.N = N; a.n_pad = n_pad; a.causal = causal ? 1 : 0; a.scale2 = 2.f * c;
  e = rbf::launch_fwd(a, bf16, D, softmax != 0, stream);
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "forward launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_fwd(const void* q, const void* k, const void* v, void* out, float* lse, void* workspace,
                 size_t workspace_bytes, int B, int H, int N, int D, const int64_t* q_strides,
                 const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides, int dtype,
                 int causal, int softmax, float sm_scale, void* stream_v) {
  return rbf_b200_fwd_phases(q, k, v, out, lse, workspace, workspace_bytes, B, H, N, D, q_strides, k_strides,
                             v_strides, o_strides, dtype, causal, softmax, sm_scale, stream_v, RBF_B200_PHASE_ALL);
}

int rbf_b200_bwd_phases(const void* q, const void* k, const void* v, const void* out, const float* lse,
                        const void* dout, void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes, int B,
                        int H, int N, int D, const int64_t* q_strides, const int64_t* k_strides,
                        const int64_t* v_strides, const int64_t* o_strides, const int64_t* do_strides,
                        const int64_t* dq_strides, const int64_t* dk_strides, const int64_t* dv_strides, int dtype,
                        int causal, int softmax, float sm_scale, void* stream_v, int phases) {
  g_last_error[0] = 0;
  int rc;
  if ((rc = check_common(B, H, N, D, dtype, sm_scale))) return rc;
  if ((rc = check_tensor("q", q, q_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("k", k, k_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("v", v, v_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("dout", dout, do_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("dq", dq, dq_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("dk", dk, dk_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("dv", dv, dv_strides, B, H, N, D))) return rc;
  if (softmax || out != nullptr) {
    if ((rc = check_tensor("out", out, o_strides, B, H, N, D))) return rc;
  }
  if (softmax && lse == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "lse is NULL");
  const bool fused = use_fused_backward(D, softmax, out != nullptr);
  if (workspace == nullptr || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace is NULL or not 256-byte aligned");
  const Workspace ws = carve(workspace, B, H, N, D, softmax, 1);
  if (workspace_bytes < ws.bytes)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, ws.bytes);

  const bool bf16 = dtype == 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  rbf::BwdArgs a{};
  if ((rc = make_map(&a.tm_q, "q", q, q_strides, bf16, B, H, N, D))) return rc;
  if ((rc = make_map(&a.tm_k, "k", k, k_strides, bf16, B, H, N, D))) return rc;
  if ((rc = make_map(&a.tm_v, "v", v, v_strides, bf16, B, H, N, D))) return rc;
  if ((rc = make_map(&a.tm_do, "dout", dout, do_strides, bf16, B, H, N, D))) return rc;
  if ((rc = make_map(&a.tm_dq, "dq", dq, dq_strides, bf16, B, H, N, D))) return rc;
  if ((rc = make_map(&a.tm_dk, "dk", dk, dk_strides, bf16, B, H, N, D))) return rc;
  if ((rc = make_map(&a.tm_dv, "dv", dv, dv_strides, bf16, B, H, N, D))) return rc;

  const int n_pad = rbf::padded_rows(N);
  const float c = sm_scale * rbf::kLog2e;
  cudaError_t e = cudaSuccess;
  if (phases & RBF_B200_PHASE_PREPASS) {
    rbf::RowStatsArgs r{};
    r.B = B; r.H = H; r.N = N; r.n_pad = n_pad; r.scale = c; r.status_to_clear = ws.status;
    r.scale2 = 2.f * c; r.slab_w = slab_w(bf16); r.slab_big = slab_big(bf16);
    if (fused) { r.lslab_out = ws.lslab; r.dslab_out = ws.dslab; r.zero_rows = ws.dq_acc; }
    // The head-dim-128 single kernel takes the key norms from its resident K tile, so K is not read here. (At head
    // dim 64 the same change slowed the main kernel by as much as the pre-pass gained: its compute warps have no
    // registers to spare and its other warps are on the critical path of the dQ hand-over.)
    if (!(fused && D == 128)) { r.k = k; r.ksq_out = ws.ksq; set_strides(r.ks, k_strides); }
    r.delta_out = ws.delta;                     // written as zeros when there is no O (non-softmax variant)
    if (softmax) {
      r.o = out; r.dout = dout; set_strides(r.os, o_strides); set_strides(r.dos, do_strides);
      r.lse = lse; r.lse_pad_out = ws.row_bias;
    } else {
      r.q = q; r.qsq_out = ws.row_bias; r.qsq_pad = INFINITY; set_strides(r.qs, q_strides);
      if (fused) {
        // single kernel: the L slab carries -qsq, nothing is subtracted from dP, delta feeds the dQ correction
        r.o = out; r.dout = dout; set_strides(r.os, o_strides); set_strides(r.dos, do_strides);
        r.lslab_from_qsq = 1; r.dslab_zero = 1;
      }
    }
    e = rbf::launch_row_stats(r, bf16, D, stream);
    if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "pre-pass launch failed: %s", cudaGetErrorString(e));
  }

  if (fused) {
    if (!(phases & (RBF_B200_PHASE_MAIN | RBF_B200_PHASE_MAIN2))) return RBF_B200_OK;
    rbf::BwdFusedArgs f{};
    f.tm_q = a.tm_q; f.tm_k = a.tm_k; f.tm_v = a.tm_v; f.tm_do = a.tm_do; f.tm_dk = a.tm_dk; f.tm_dv = a.tm_dv;
    // the head-dim-128 kernel streams the queries in steps of 64 rows
    const int q_rows = D == 128 ? 64 : rbf::kTile;
    if (q_rows != rbf::kTile) {
      if ((rc = make_map(&f.tm_q, "q", q, q_strides, bf16, B, H, N, D, q_rows))) return rc;
      if ((rc = make_map(&f.tm_do, "dout", dout, do_strides, bf16, B, H, N, D, q_rows))) return rc;
    }
    const int t1 = rbf::make_tmap_slab16(&f.tm_lslab, ws.lslab, bf16, B * H, n_pad, q_rows);
    const int t2 = rbf::make_tmap_slab16(&f.tm_dslab, ws.dslab, bf16, B * H, n_pad, q_rows);
    if (t1 != 0 || t2 != 0)
      return fail(RBF_B200_ERR_TENSOR_MAP, "cuTensorMapEncodeTiled failed for the bias slabs (codes %d, %d)", t1, t2);
    if (D == 64) {
      const int t3 = rbf::make_tmap_f32_bhnd(&f.tm_dq_acc, ws.dq_acc, B, H, N, D, 32);
      if (t3 != 0)
        return fail(RBF_B200_ERR_TENSOR_MAP, "cuTensorMapEncodeTiled failed for the dQ accumulator (code %d)", t3);
    }
    f.dq_acc = ws.dq_acc; f.dq = dq; set_strides(f.dq_strides, dq_strides);
    f.ksq = ws.ksq; f.status = ws.status;
    // work counters of the persistent launch live in the status block (words 16, 17), zeroed by the pre-pass
    f.work = reinterpret_cast<unsigned int*>(ws.status) + 16;
    f.sm_count = sm_count();
    if (f.sm_count <= 0) return fail(RBF_B200_ERR_LAUNCH, "cannot read the SM count of the current device");
    if (!softmax) { f.q_rows = q; set_strides(f.q_strides, q_strides); f.delta = ws.delta; }
    f.B = B; f.H = H; f.N = N; f.n_pad = n_pad; f.causal = causal ? 1 : 0;
    f.scale2 = 2.f * c; f.grad_scale = 2.f * sm_scale; f.slab_w = slab_w(bf16);
    e = D == 128 ? rbf::launch_bwd_fused128(f, bf16, stream) : rbf::launch_bwd_fused(f, bf16, stream);
    if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "backward launch failed: %s", cudaGetErrorString(e));
    return RBF_B200_OK;
  }

  a.ksq = ws.ksq;
  a.row_bias = ws.row_bias;
  a.row_bias_pitch = n_pad;
  a.delta = ws.delta;
  a.status = ws.status;
  a.B = B; a.H = H; a.N = N; a.n_pad = n_pad; a.causal = causal ? 1 : 0;
  a.scale2 = 2.f * c; a.grad_scale = 2.f * sm_scale;
  if (phases & RBF_B200_PHASE_MAIN) {
    e = rbf::launch_bwd_dkdv(a, bf16, D, softmax != 0, stream);
    if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "dK/dV launch failed: %s", cudaGetErrorString(e));
  }
  if (phases & RBF_B200_PHASE_MAIN2) {
    e = rbf::launch_bwd_dq(a, bf16, D, softmax != 0, stream);
    if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "dQ launch failed: %s", cudaGetErrorString(e));
  }
  return RBF_B200_OK;
}

int rbf_b200_bwd(const void* q, const void* k, const void* v, const void* out, const float* lse, const void* dout,
                 void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes, int B, int H, int N, int D,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const int64_t* o_strides, const int64_t* do_strides, const int64_t* dq_strides,
                 const int64_t* dk_strides, const int64_t* dv_strides, int dtype, int causal, int softmax,
                 float sm_scale, void* stream_v) {
  return rbf_b200_bwd_phases(q, k, v, out, lse, dout, dq, dk, dv, workspace, workspace_bytes, B, H, N, D, q_strides,
                             k_strides, v_strides, o_strides, do_strides, dq_strides, dk_strides, dv_strides, dtype,
                             causal, softmax, sm_scale, stream_v, RBF_B200_PHASE_ALL);
}

// ---------------------------------------------------------------------------------------------
// Forward without a caller-provided workspace: the scratch lives in a fixed device array of this library.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = RBF_B200_STATIC_SCRATCH_BYTES;
// Reserved on every GPU that loads the library, until the process exits. In host code this name is only a
// handle: the device address has to be asked for with cudaGetSymbolAddress (below), never taken with '&'.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_static_scratch_addr[kMaxDevices];

// Device address of the scratch array on the current device; looked up once per device.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(RBF_B200_ERR_BAD_ARGUMENT, "device index %d is out of range", dev);
  void* ptr = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    // the first call on a device: this may load the library's device image there
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(RBF_B200_ERR_LAUNCH, "cudaGetSymbolAddress failed for the static scratch: %s", cudaGetErrorString(e));
    g_static_scratch_addr[dev].store(ptr, std::memory_order_release);   // every thread would store the same address
  }
  *out = ptr;
  return 0;
}

}  // namespace

size_t rbf_b200_static_scratch_bytes(void) { return kStaticScratchBytes; }

int rbf_b200_fwd_static(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int N, int D,
                        const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                        const int64_t* o_strides, int dtype, int causal, int softmax, float sm_scale, void* stream_v) {
  g_last_error[0] = 0;
  int rc;
  if ((rc = check_common(B, H, N, D, dtype, sm_scale))) return rc;
  const size_t need = carve(nullptr, B, H, N, D, softmax, 0).bytes;
  if (need > kStaticScratchBytes)
    return fail(RBF_B200_ERR_WORKSPACE,
                "problem needs %zu bytes of scratch but the built-in scratch holds %zu: use rbf_b200_fwd with a "
                "caller-provided workspace", need, kStaticScratchBytes);
  void* scratch = nullptr;
  if ((rc = static_scratch_for_current_device(&scratch))) return rc;
  // The pre-pass rewrites every scratch word the main kernel reads and clears the status word, so nothing of an
  // earlier call leaks into this one.
  return rbf_b200_fwd_phases(q, k, v, out, lse, scratch, kStaticScratchBytes, B, H, N, D, q_strides, k_strides,
                             v_strides, o_strides, dtype, causal, softmax, sm_scale, stream_v, RBF_B200_PHASE_ALL);
}

// ---------------------------------------------------------------------------------------------
// Fused q/k preparation of the attention block and the gradients of its position parameters
// ---------------------------------------------------------------------------------------------
int rbf_b200_qkv_prep(const void* qkv, const void* pos_weight, const void* reg_pos_emb, int params_fp32,
                      const float* susie_table, void* q_out, void* k_out, const int64_t* q_strides,
                      const int64_t* k_strides, void* fwd_workspace, size_t fwd_workspace_bytes, int B, int S, int H,
                      int D, int R, int dtype, int softmax, float sm_scale, void* stream_v) {
  g_last_error[0] = 0;
  int rc;
  if ((rc = check_common(B, H, S, D, dtype, sm_scale))) return rc;
  if (R < 0 || R > S) return fail(RBF_B200_ERR_BAD_ARGUMENT, "register rows R = %d must be in [0, S = %d]", R, S);
  if (qkv == nullptr || pos_weight == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "qkv or pos_weight is NULL");
  if (R > 0 && reg_pos_emb == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "reg_pos_emb is NULL with R = %d", R);
  if (S > R && susie_table == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "susie_table is NULL");
  if (reinterpret_cast<uintptr_t>(qkv) % 16 != 0 || reinterpret_cast<uintptr_t>(susie_table) % 16 != 0)
    return fail(RBF_B200_ERR_BAD_LAYOUT, "qkv and susie_table must be 16-byte aligned");
  if ((rc = check_tensor("q_out", q_out, q_strides, B, H, S, D))) return rc;
  if ((rc = check_tensor("k_out", k_out, k_strides, B, H, S, D))) return rc;
  if (fwd_workspace == nullptr || reinterpret_cast<uintptr_t>(fwd_workspace) % 256 != 0)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace is NULL or not 256-byte aligned");
  const Workspace ws = carve(fwd_workspace, B, H, S, D, softmax, 0);
  if (fwd_workspace_bytes < ws.bytes)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", fwd_workspace_bytes, ws.bytes);
  const bool bf16 = dtype == 0;
  const float c = sm_scale * rbf::kLog2e;
  rbf::QkvPrepArgs a{};
  a.qkv = qkv; a.pos_weight = pos_weight; a.reg_pos = reg_pos_emb; a.params_fp32 = params_fp32 ? 1 : 0;
  a.table = susie_table; a.q_out = q_out; a.k_out = k_out;
  set_strides(a.qo, q_strides); set_strides(a.ko, k_strides);
  a.kslab_out = ws.kslab; a.qsq_out = softmax ? nullptr : ws.row_bias; a.status_to_clear = ws.status;
  a.B = B; a.S = S; a.H = H; a.D = D; a.R = R; a.n_pad = rbf::padded_rows(S);
  a.scale = c; a.scale2 = 2.f * c; a.slab_w = slab_w(bf16); a.slab_big = slab_big(bf16);
  const cudaError_t e = rbf::launch_qkv_prep(a, bf16, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "q/k preparation launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

size_t rbf_b200_qkv_prep_bwd_workspace_bytes(int B, int S, int H, int D, int R) {
  if (B <= 0 || S <= 0 || H <= 0 || D <= 0 || R < 0 || R > S) return 0;
  const size_t chunks = static_cast<size_t>(rbf::qkv_prep_bwd_chunks(S, R));
  return align256((chunks > 0 ? chunks : 1) * B * H * (D / 2) * sizeof(float));
}

int rbf_b200_qkv_prep_bwd(const void* dq, const void* dk, const int64_t* dq_strides, const int64_t* dk_strides,
                          const float* susie_table, float* d_pos_weight, float* d_reg_pos_emb, void* workspace,
                          size_t workspace_bytes, int B, int S, int H, int D, int R, int dtype, void* stream_v) {
  g_last_error[0] = 0;
  int rc;
  if ((rc = check_common(B, H, S, D, dtype, 1.0f))) return rc;
  if (R < 0 || R > S) return fail(RBF_B200_ERR_BAD_ARGUMENT, "register rows R = %d must be in [0, S = %d]", R, S);
  if ((rc = check_tensor("dq", dq, dq_strides, B, H, S, D))) return rc;
  if ((rc = check_tensor("dk", dk, dk_strides, B, H, S, D))) return rc;
  if (d_pos_weight == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "d_pos_weight is NULL");
  if (R > 0 && d_reg_pos_emb == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "d_reg_pos_emb is NULL with R = %d", R);
  if (S > R && (susie_table == nullptr || reinterpret_cast<uintptr_t>(susie_table) % 16 != 0))
    return fail(RBF_B200_ERR_BAD_ARGUMENT, "susie_table is NULL or not 16-byte aligned");
  if (H * (D / 8) > 1024) return fail(RBF_B200_ERR_BAD_ARGUMENT, "H * D = %d exceeds 8192", H * D);
  const size_t need = rbf_b200_qkv_prep_bwd_workspace_bytes(B, S, H, D, R);
  if (workspace == nullptr || reinterpret_cast<uintptr_t>(workspace) % 256 != 0 || workspace_bytes < need)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace is NULL, not 256-byte aligned or smaller than %zu bytes", need);
  rbf::QkvPrepBwdArgs a{};
  a.dq = dq; a.dk = dk; set_strides(a.dqs, dq_strides); set_strides(a.dks, dk_strides);
  a.table = susie_table; a.partials = static_cast<float*>(workspace);
  a.d_pos_weight = d_pos_weight; a.d_reg_pos = d_reg_pos_emb;
  a.B = B; a.S = S; a.H = H; a.D = D; a.R = R;
  const cudaError_t e = rbf::launch_qkv_prep_bwd(a, dtype == 0, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "position-gradient launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// Exclusive self attention (projection away from the position's own value row)
// ---------------------------------------------------------------------------------------------
int rbf_b200_xsa_fwd(const void* o, const void* v, void* out, const int64_t* o_strides, const int64_t* v_strides,
                     const int64_t* out_strides, int B, int H, int N, int D, int dtype, void* stream_v) {
  g_last_error[0] = 0;
  int rc;
  if ((rc = check_common(B, H, N, D, dtype, 1.0f))) return rc;
  if ((rc = check_tensor("o", o, o_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("v", v, v_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("out", out, out_strides, B, H, N, D))) return rc;
  rbf::XsaArgs a{};
  a.o = o; a.v = v; a.out = out; a.B = B; a.H = H; a.N = N;
  set_strides(a.os, o_strides); set_strides(a.vs, v_strides); set_strides(a.outs, out_strides);
  const cudaError_t e = rbf::launch_xsa(a, false, dtype == 0, D, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "xsa forward launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_xsa_bwd(const void* g, const void* o, const void* v, void* d_o, void* d_v, const int64_t* g_strides,
                     const int64_t* o_strides, const int64_t* v_strides, const int64_t* do_strides,
                     const int64_t* dv_strides, int B, int H, int N, int D, int dtype, void* stream_v) {
  g_last_error[0] = 0;
  int rc;
  if ((rc = check_common(B, H, N, D, dtype, 1.0f))) return rc;
  if ((rc = check_tensor("g", g, g_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("o", o, o_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("v", v, v_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("d_o", d_o, do_strides, B, H, N, D))) return rc;
  if ((rc = check_tensor("d_v", d_v, dv_strides, B, H, N, D))) return rc;
  rbf::XsaArgs a{};
  a.g = g; a.o = o; a.v = v; a.out = d_o; a.dv = d_v; a.B = B; a.H = H; a.N = N;
  set_strides(a.gs, g_strides); set_strides(a.os, o_strides); set_strides(a.vs, v_strides);
  set_strides(a.outs, do_strides); set_strides(a.dvs, dv_strides);
  const cudaError_t e = rbf::launch_xsa(a, true, dtype == 0, D, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "xsa backward launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_read_device_status(const void* workspace, void* stream_v, unsigned int* code) {
  g_last_error[0] = 0;
  if (code == nullptr) return fail(RBF_B200_ERR_BAD_ARGUMENT, "code is NULL");
  if (workspace == nullptr) {
    // the built-in scratch of the current device (what rbf_b200_fwd_static used)
    void* scratch = nullptr;
    int rc;
    if ((rc = static_scratch_for_current_device(&scratch))) return rc;
    workspace = scratch;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  rbf::DeviceStatus st{};
  cudaError_t e = cudaMemcpyAsync(&st, workspace, sizeof(st), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "status read failed: %s", cudaGetErrorString(e));
  *code = st.code;
  if (st.code != 0)
    return fail(RBF_B200_ERR_DEVICE, "device-side wait ran out: site %u, work unit %u", st.code >> 24,
                st.code & 0xffffffu);
  return RBF_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// LayerNorm of the language model's blocks
// ---------------------------------------------------------------------------------------------
static int check_layer_norm(int64_t rows, int cols, int dtype) {
  if (rows < 0) return fail(RBF_B200_ERR_BAD_ARGUMENT, "rows must be >= 0");
  if (!rbf::layer_norm_supported(cols))
    return fail(RBF_B200_ERR_BAD_ARGUMENT, "cols must be 256, 512, 768 or 1024, got %d", cols);
  if (dtype != 0 && dtype != 1) return fail(RBF_B200_ERR_BAD_ARGUMENT, "dtype must be 0 (bf16) or 1 (fp16)");
  return RBF_B200_OK;
}

int rbf_b200_add_layer_norm_fwd(const void* x, const void* residual, void* sum_out, const void* gamma, const void* beta,
                                void* y, float* mean, float* rstd, int64_t rows, int cols, float eps, int dtype,
                                void* stream_v) {
  g_last_error[0] = 0;
  int rc;
  if ((rc = check_layer_norm(rows, cols, dtype))) return rc;
  if ((residual == nullptr) != (sum_out == nullptr))
    return fail(RBF_B200_ERR_BAD_ARGUMENT, "residual and sum_out go together: both NULL or both set");
  if (rows == 0) return RBF_B200_OK;
  if (!x || !gamma || !beta || !y || !mean || !rstd) return fail(RBF_B200_ERR_BAD_ARGUMENT, "NULL tensor pointer");
  for (const void* ptr : {x, residual, static_cast<const void*>(sum_out), gamma, beta, static_cast<const void*>(y)})
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return fail(RBF_B200_ERR_BAD_LAYOUT, "tensors must be 16-byte aligned");
  if (sum_out != nullptr && sum_out == y) return fail(RBF_B200_ERR_BAD_ARGUMENT, "sum_out and y must be different tensors");
  const int sms = sm_count();
  if (sms <= 0) return fail(RBF_B200_ERR_LAUNCH, "cannot read the SM count of the current device");
  rbf::LayerNormArgs a{};
  a.x = x; a.gamma = gamma; a.beta = beta; a.y = y; a.mean = mean; a.rstd = rstd; a.rows = rows; a.eps = eps;
  a.residual = residual; a.sum_out = sum_out;
  const cudaError_t e = rbf::launch_layer_norm_fwd(a, cols, dtype == 0, sms, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "layer norm launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                            int64_t rows, int cols, float eps, int dtype, void* stream_v) {
  return rbf_b200_add_layer_norm_fwd(x, nullptr, nullptr, gamma, beta, y, mean, rstd, rows, cols, eps, dtype, stream_v);
}

size_t rbf_b200_layer_norm_bwd_workspace_bytes(int64_t rows, int cols) {
  const int sms = sm_count();
  if (sms <= 0 || rows < 0 || !rbf::layer_norm_supported(cols)) return 0;
  return static_cast<size_t>(rbf::layer_norm_bwd_blocks(rows, sms)) * 2 * cols * sizeof(float);
}

int rbf_b200_layer_norm_bwd_add(const void* x, const void* dy, const void* dres, const void* gamma, const float* mean,
                                const float* rstd, void* dx, float* dgamma, float* dbeta, void* workspace,
                                size_t workspace_bytes, int64_t rows, int cols, int dtype, void* stream_v) {
  g_last_error[0] = 0;
  int rc;
  if ((rc = check_layer_norm(rows, cols, dtype))) return rc;
  if (!dgamma || !dbeta || !workspace) return fail(RBF_B200_ERR_BAD_ARGUMENT, "NULL output pointer");
  if (rows > 0 && (!x || !dy || !gamma || !mean || !rstd || !dx))
    return fail(RBF_B200_ERR_BAD_ARGUMENT, "NULL tensor pointer");
  for (const void* ptr : {x, dy, dres, gamma, static_cast<const void*>(dx)})
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return fail(RBF_B200_ERR_BAD_LAYOUT, "tensors must be 16-byte aligned");
  if (workspace_bytes < rbf_b200_layer_norm_bwd_workspace_bytes(rows, cols))
    return fail(RBF_B200_ERR_WORKSPACE, "workspace too small: %zu bytes", workspace_bytes);
  const int sms = sm_count();
  if (sms <= 0) return fail(RBF_B200_ERR_LAUNCH, "cannot read the SM count of the current device");
  rbf::LayerNormBwdArgs a{};
  a.x = x; a.dy = dy; a.gamma = gamma; a.mean = mean; a.rstd = rstd; a.dx = dx; a.dgamma = dgamma; a.dbeta = dbeta;
  a.partials = static_cast<float*>(workspace); a.rows = rows; a.dres = dres;
  const cudaError_t e = rbf::launch_layer_norm_bwd(a, cols, dtype == 0, sms, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "layer norm backward launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_layer_norm_bwd(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                            void* dx, float* dgamma, float* dbeta, void* workspace, size_t workspace_bytes,
                            int64_t rows, int cols, int dtype, void* stream_v) {
  return rbf_b200_layer_norm_bwd_add(x, dy, nullptr, gamma, mean, rstd, dx, dgamma, dbeta, workspace, workspace_bytes, rows,
                                     cols, dtype, stream_v);
}

// ---------------------------------------------------------------------------------------------
// Column sums (bias gradients of the model's linear layers)
// ---------------------------------------------------------------------------------------------
size_t rbf_b200_column_sums_workspace_bytes(int64_t rows, int cols) {
  const int sms = sm_count();
  if (sms <= 0 || rows < 0 || cols <= 0) return 0;
  return static_cast<size_t>(rbf::col_sums_bands(rows, cols, sms)) * cols * sizeof(float);
}

int rbf_b200_column_sums(const void* x, float* out, void* workspace, size_t workspace_bytes, int64_t rows, int cols,
                         int64_t ld, int dtype, void* stream_v) {
  g_last_error[0] = 0;
  if (rows < 0 || cols <= 0 || cols % 8 != 0) return fail(RBF_B200_ERR_BAD_ARGUMENT, "cols must be a positive multiple of 8");
  if (dtype != 0 && dtype != 1) return fail(RBF_B200_ERR_BAD_ARGUMENT, "dtype must be 0 (bf16) or 1 (fp16)");
  if (ld < cols || ld % 8 != 0) return fail(RBF_B200_ERR_BAD_LAYOUT, "row pitch must be a multiple of 8 elements and >= cols");
  if (!out || !workspace || (rows > 0 && !x)) return fail(RBF_B200_ERR_BAD_ARGUMENT, "NULL pointer");
  if (reinterpret_cast<uintptr_t>(x) % 16 != 0) return fail(RBF_B200_ERR_BAD_LAYOUT, "x must be 16-byte aligned");
  if (workspace_bytes < rbf_b200_column_sums_workspace_bytes(rows, cols))
    return fail(RBF_B200_ERR_WORKSPACE, "workspace too small: %zu bytes", workspace_bytes);
  const int sms = sm_count();
  if (sms <= 0) return fail(RBF_B200_ERR_LAUNCH, "cannot read the SM count of the current device");
  const cudaError_t e = rbf::launch_col_sums(x, ld, rows, cols, dtype == 0, static_cast<float*>(workspace), out, sms,
                                             static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "column sums launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// GELU of the model's MLP
// ---------------------------------------------------------------------------------------------
int rbf_b200_gelu_fwd(const void* h, void* out, int64_t n, int dtype, void* stream_v) {
  g_last_error[0] = 0;
  if (n < 0 || n % 8 != 0) return fail(RBF_B200_ERR_BAD_ARGUMENT, "n must be a non-negative multiple of 8");
  if (dtype != 0 && dtype != 1) return fail(RBF_B200_ERR_BAD_ARGUMENT, "dtype must be 0 (bf16) or 1 (fp16)");
  if (n == 0) return RBF_B200_OK;
  if (!h || !out) return fail(RBF_B200_ERR_BAD_ARGUMENT, "NULL pointer");
  if (reinterpret_cast<uintptr_t>(h) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0)
    return fail(RBF_B200_ERR_BAD_LAYOUT, "tensors must be 16-byte aligned");
  const int sms = sm_count();
  if (sms <= 0) return fail(RBF_B200_ERR_LAUNCH, "cannot read the SM count of the current device");
  const cudaError_t e = rbf::launch_gelu_fwd(h, out, n, dtype == 0, sms, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "gelu launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_gelu_bwd(const void* h, const void* dy, void* dh, float* dbias, void* workspace, size_t workspace_bytes,
                      int64_t rows, int cols, int dtype, void* stream_v) {
  g_last_error[0] = 0;
  if (rows < 0 || cols <= 0 || cols % 8 != 0) return fail(RBF_B200_ERR_BAD_ARGUMENT, "cols must be a positive multiple of 8");
  if (dtype != 0 && dtype != 1) return fail(RBF_B200_ERR_BAD_ARGUMENT, "dtype must be 0 (bf16) or 1 (fp16)");
  if (rows > 0 && (!h || !dy || !dh)) return fail(RBF_B200_ERR_BAD_ARGUMENT, "NULL tensor pointer");
  for (const void* ptr : {h, dy, static_cast<const void*>(dh)})
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return fail(RBF_B200_ERR_BAD_LAYOUT, "tensors must be 16-byte aligned");
  if (dbias != nullptr && (!workspace || workspace_bytes < rbf_b200_column_sums_workspace_bytes(rows, cols)))
    return fail(RBF_B200_ERR_WORKSPACE, "workspace too small: %zu bytes", workspace_bytes);
  const int sms = sm_count();
  if (sms <= 0) return fail(RBF_B200_ERR_LAUNCH, "cannot read the SM count of the current device");
  const cudaError_t e = rbf::launch_gelu_bwd(h, dy, dh, rows, cols, dtype == 0, static_cast<float*>(workspace), dbias, sms,
                                             static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "gelu backward launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// Cross entropy of the language-model training step
// ---------------------------------------------------------------------------------------------
int rbf_b200_cross_entropy(const void* logits, const int64_t* targets, const float* grad_scale, float* loss_rows,
                           void* dlogits, int rows, int cols, int64_t ld, int64_t ld_out, int64_t ignore_index,
                           int dtype, void* stream_v) {
  g_last_error[0] = 0;
  if (rows < 0 || cols <= 0) return fail(RBF_B200_ERR_BAD_ARGUMENT, "rows must be >= 0 and cols > 0");
  if (dtype < 0 || dtype > 2) return fail(RBF_B200_ERR_BAD_ARGUMENT, "dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)");
  if (ld < cols || ld_out < cols) return fail(RBF_B200_ERR_BAD_ARGUMENT, "row pitches must be at least cols");
  if (rows == 0) return RBF_B200_OK;
  if (!logits || !targets || !grad_scale || !loss_rows || !dlogits)
    return fail(RBF_B200_ERR_BAD_ARGUMENT, "NULL tensor pointer");
  const int sms = sm_count();
  if (sms <= 0) return fail(RBF_B200_ERR_LAUNCH, "cannot read the SM count of the current device");
  rbf::CrossEntropyArgs a{};
  a.logits = logits; a.ld = ld; a.targets = targets; a.dlogits = dlogits; a.ld_out = ld_out;
  a.loss_rows = loss_rows; a.grad_scale = grad_scale; a.rows = rows; a.cols = cols; a.ignore_index = ignore_index;
  const cudaError_t e = rbf::launch_cross_entropy(a, dtype, sms, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "cross entropy launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_scale_unless_one(void* x, const float* factor, int64_t n, int dtype, void* stream_v) {
  g_last_error[0] = 0;
  if (n < 0) return fail(RBF_B200_ERR_BAD_ARGUMENT, "n must be >= 0");
  if (dtype < 0 || dtype > 2) return fail(RBF_B200_ERR_BAD_ARGUMENT, "dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)");
  if (n == 0) return RBF_B200_OK;
  if (!x || !factor) return fail(RBF_B200_ERR_BAD_ARGUMENT, "NULL pointer");
  const int sms = sm_count();
  if (sms <= 0) return fail(RBF_B200_ERR_LAUNCH, "cannot read the SM count of the current device");
  const cudaError_t e = rbf::launch_scale_unless_one(x, factor, n, dtype, sms, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "scale launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_post_device_status(const void* workspace, unsigned int* host_slot, void* stream_v) {
  g_last_error[0] = 0;
  if (workspace == nullptr || host_slot == nullptr)
    return fail(RBF_B200_ERR_BAD_ARGUMENT, "workspace and host_slot must not be NULL");
  // device-side address of the slot: resolved by the driver once per 256-byte block and thread (callers post into a
  // small ring of slots, and the driver call costs more than the launch)
  thread_local uintptr_t cached_page = 0;
  thread_local intptr_t cached_delta = 0;
  thread_local int cached_device = -1;
  const uintptr_t host_addr = reinterpret_cast<uintptr_t>(host_slot);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  void* dev_ptr = nullptr;
  if (cached_page != 0 && cached_page == (host_addr & ~uintptr_t(255)) && cached_device == device) {
    dev_ptr = reinterpret_cast<void*>(host_addr + cached_delta);
  } else {
    e = cudaHostGetDevicePointer(&dev_ptr, host_slot, 0);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(RBF_B200_ERR_BAD_ARGUMENT, "host_slot is not mapped page-locked host memory: %s",
                  cudaGetErrorString(e));
    }
    cached_page = host_addr & ~uintptr_t(255);
    cached_delta = static_cast<intptr_t>(reinterpret_cast<uintptr_t>(dev_ptr) - host_addr);
    cached_device = device;
  }
  e = rbf::launch_post_status(static_cast<const rbf::DeviceStatus*>(workspace), static_cast<unsigned int*>(dev_ptr),
                              static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "status post failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

int rbf_b200_set_deterministic(int on) { return g_deterministic.exchange(on ? 1 : 0); }

int rbf_b200_get_deterministic(void) { return g_deterministic.load(); }

int rbf_b200_selftest_wait_timeout(void* workspace, size_t workspace_bytes, long long limit_cycles, void* stream_v) {
  g_last_error[0] = 0;
  if (workspace == nullptr || reinterpret_cast<uintptr_t>(workspace) % 256 != 0 || workspace_bytes < kStatusBytes)
    return fail(RBF_B200_ERR_WORKSPACE, "workspace is NULL, not 256-byte aligned or smaller than %zu bytes", kStatusBytes);
  if (limit_cycles <= 0 || limit_cycles > 2000000000ll)
    return fail(RBF_B200_ERR_BAD_ARGUMENT, "limit_cycles must be in (0, 2e9]");
  const cudaError_t e = rbf::launch_wait_selftest(static_cast<rbf::DeviceStatus*>(workspace), limit_cycles,
                                                  static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(RBF_B200_ERR_LAUNCH, "self-test launch failed: %s", cudaGetErrorString(e));
  return RBF_B200_OK;
}

}  // extern "C"
