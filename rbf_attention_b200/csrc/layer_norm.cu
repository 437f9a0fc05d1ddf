// LayerNorm of the language model's blocks (nn.LayerNorm(emb_dim) before the attention and the MLP of every block and
// before the output projection, train_rbf_transformer.py:139-150, 215, 241) for 16-bit activations whose width is a multiple
// of 256: forward and backward as one streaming pass each. Roofline: HBM (forward: read x, write y; backward: read x
// and dy, write dx). A warp owns a row (8 elements per lane and 256 columns, 16-byte accesses), statistics in fp32 with
// the variance taken around the mean; the backward keeps the per-column sums for d(gamma), d(beta) in registers while a
// warp walks its rows, folds the eight warps of a block in shared memory and leaves one fp32 partial row per block
// for a second, small kernel (fixed order: bitwise reproducible).
// Both passes take the block's residual connection with them (x = x + f(x) followed by the next LayerNorm,
// train_rbf_transformer.py:147-151): the forward can add a second tensor to x first, writing the rounded sum (the new
// residual stream) beside the normalised rows, and the backward can add the gradient that reaches that sum along the
// skip path to dx before it rounds - one pass over the activations instead of two in either direction.
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "launch.h"

namespace rbf {
namespace {

constexpr int kLnThreads = 256;
constexpr int kLnWarps = kLnThreads / 32;

template <bool kBf16>
__device__ __forceinline__ float2 ln_unpack(uint32_t w) {
  if constexpr (kBf16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  const __half2 h = *reinterpret_cast<const __half2*>(&w);
  return __half22float2(h);
}
template <bool kBf16>
__device__ __forceinline__ uint32_t ln_pack(float a, float b) {
  if constexpr (kBf16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <bool kBf16>
__device__ __forceinline__ void ln_load8(const void* base, int64_t chunk, float (&out)[8]) {
  const uint4 raw = reinterpret_cast<const uint4*>(base)[chunk];
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = ln_unpack<kBf16>(w[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <bool kBf16, int kVecs>
__global__ void __launch_bounds__(kLnThreads) layer_norm_fwd_kernel(const LayerNormArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int kCols = kVecs * 256;
  float gamma[kVecs][8], beta[kVecs][8];
#pragma unroll
  for (int v = 0; v < kVecs; ++v) {
    ln_load8<kBf16>(a.gamma, v * 32 + lane, gamma[v]);
    ln_load8<kBf16>(a.beta, v * 32 + lane, beta[v]);
  }
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarps + warp; row < a.rows;
       row += static_cast<int64_t>(gridDim.x) * kLnWarps) {
    const uint16_t* x = static_cast<const uint16_t*>(a.x) + row * kCols;
    float xv[kVecs][8];
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      ln_load8<kBf16>(x, v * 32 + lane, xv[v]);
      if (a.residual != nullptr) {
        // the sum is rounded to the activations' type first, as the separate addition would have left it
        float rv[8];
        ln_load8<kBf16>(static_cast<const uint16_t*>(a.residual) + row * kCols, v * 32 + lane, rv);
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          w[i] = ln_pack<kBf16>(xv[v][2 * i] + rv[2 * i], xv[v][2 * i + 1] + rv[2 * i + 1]);
          const float2 f = ln_unpack<kBf16>(w[i]);
          xv[v][2 * i] = f.x;
          xv[v][2 * i + 1] = f.y;
        }
        reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.sum_out) + row * kCols)[v * 32 + lane] =
            make_uint4(w[0], w[1], w[2], w[3]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += xv[v][j];
    }
    const float mean = warp_sum(sum) * (1.f / kCols);
    float sq = 0.f;
#pragma unroll
    for (int v = 0; v < kVecs; ++v)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = xv[v][j] - mean;
        sq = fmaf(d, d, sq);
      }
    const float rstd = rsqrtf(warp_sum(sq) * (1.f / kCols) + a.eps);
    if (lane == 0) {
      a.mean[row] = mean;
      a.rstd[row] = rstd;
    }
    uint16_t* y = static_cast<uint16_t*>(a.y) + row * kCols;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[i] = ln_pack<kBf16>(fmaf((xv[v][2 * i] - mean) * rstd, gamma[v][2 * i], beta[v][2 * i]),
                              fmaf((xv[v][2 * i + 1] - mean) * rstd, gamma[v][2 * i + 1], beta[v][2 * i + 1]));
      reinterpret_cast<uint4*>(y)[v * 32 + lane] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

template <bool kBf16, int kVecs>
__global__ void __launch_bounds__(kLnThreads) layer_norm_bwd_kernel(const LayerNormBwdArgs a) {
  constexpr int kCols = kVecs * 256;
  extern __shared__ float s_part[];               // [kLnWarps][2][kCols]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float gamma[kVecs][8], dg[kVecs][8], db[kVecs][8];
#pragma unroll
  for (int v = 0; v < kVecs; ++v) {
    ln_load8<kBf16>(a.gamma, v * 32 + lane, gamma[v]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dg[v][j] = db[v][j] = 0.f;
  }
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarps + warp; row < a.rows;
       row += static_cast<int64_t>(gridDim.x) * kLnWarps) {
    const uint16_t* x = static_cast<const uint16_t*>(a.x) + row * kCols;
    const uint16_t* dy = static_cast<const uint16_t*>(a.dy) + row * kCols;
    const float mean = a.mean[row], rstd = a.rstd[row];
    float xh[kVecs][8], g[kVecs][8];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      float dyv[8];
      ln_load8<kBf16>(x, v * 32 + lane, xh[v]);
      ln_load8<kBf16>(dy, v * 32 + lane, dyv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[v][j] = (xh[v][j] - mean) * rstd;
        g[v][j] = dyv[j] * gamma[v][j];
        c1 += g[v][j];
        c2 = fmaf(g[v][j], xh[v][j], c2);
        dg[v][j] = fmaf(dyv[j], xh[v][j], dg[v][j]);
        db[v][j] += dyv[j];
      }
    }
    c1 = warp_sum(c1) * (1.f / kCols);
    c2 = warp_sum(c2) * (1.f / kCols);
    uint16_t* dx = static_cast<uint16_t*>(a.dx) + row * kCols;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      float skip[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (a.dres != nullptr) ln_load8<kBf16>(static_cast<const uint16_t*>(a.dres) + row * kCols, v * 32 + lane, skip);
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[i] = ln_pack<kBf16>(fmaf(rstd, g[v][2 * i] - c1 - xh[v][2 * i] * c2, skip[2 * i]),
                              fmaf(rstd, g[v][2 * i + 1] - c1 - xh[v][2 * i + 1] * c2, skip[2 * i + 1]));
      reinterpret_cast<uint4*>(dx)[v * 32 + lane] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  // fold the block's warps (fixed order), one fp32 partial row of d(gamma) and d(beta) per block
#pragma unroll
  for (int v = 0; v < kVecs; ++v)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = (v * 32 + lane) * 8 + j;
      s_part[(warp * 2 + 0) * kCols + col] = dg[v][j];
      s_part[(warp * 2 + 1) * kCols + col] = db[v][j];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * kCols; i += kLnThreads) {
    float sum = 0.f;
#pragma unroll
    for (int wv = 0; wv < kLnWarps; ++wv) sum += s_part[wv * 2 * kCols + i];
    a.partials[static_cast<int64_t>(blockIdx.x) * 2 * kCols + i] = sum;
  }
}

// out[i] = sum over blocks of partials[block][i], i in [0, 2 cols): 32 outputs x 8 partial-lanes per block of 256
__global__ void __launch_bounds__(256) layer_norm_bwd_final_kernel(const float* partials, int n_blocks, int n_out,
                                                                   float* dgamma, float* dbeta) {
  __shared__ float s[8][33];
  const int col = threadIdx.x & 31, lp = threadIdx.x >> 5;
  const int o = blockIdx.x * 32 + col;
  float sum = 0.f;
  if (o < n_out)
    for (int p = lp; p < n_blocks; p += 8) sum += partials[static_cast<int64_t>(p) * n_out + o];
  s[lp][col] = sum;
  __syncthreads();
  if (threadIdx.x < 32 && o < n_out) {
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += s[i][threadIdx.x];
    const int half = n_out / 2;
    if (o < half) dgamma[o] = total;
    else dbeta[o - half] = total;
  }
}

template <bool kBf16, int kVecs>
cudaError_t launch_fwd_t(const LayerNormArgs& a, int sms, cudaStream_t stream) {
  const int64_t want = (a.rows + kLnWarps - 1) / kLnWarps;
  const int grid = static_cast<int>(want < sms * 8ll ? want : sms * 8ll);
  layer_norm_fwd_kernel<kBf16, kVecs><<<grid, kLnThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

template <bool kBf16, int kVecs>
cudaError_t launch_bwd_t(const LayerNormBwdArgs& a, int grid, cudaStream_t stream) {
  constexpr int smem = kLnWarps * 2 * kVecs * 256 * sizeof(float);
  static PerDeviceFlags flags;
  cudaError_t e = ensure_dynamic_smem(layer_norm_bwd_kernel<kBf16, kVecs>, smem, flags);
  if (e != cudaSuccess) return e;
  layer_norm_bwd_kernel<kBf16, kVecs><<<grid, kLnThreads, smem, stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int n_out = 2 * kVecs * 256;
  layer_norm_bwd_final_kernel<<<(n_out + 31) / 32, 256, 0, stream>>>(a.partials, grid, n_out, a.dgamma, a.dbeta);
  return cudaGetLastError();
}

}  // namespace

bool layer_norm_supported(int cols) { return cols > 0 && cols % 256 == 0 && cols <= 1024; }

int layer_norm_bwd_blocks(int64_t rows, int sms) {
  const int64_t want = (rows + kLnWarps - 1) / kLnWarps;
  const int64_t cap = static_cast<int64_t>(sms) * 4;
  return static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
}

#define RBF_LN_DISPATCH(FN, ...)                                              \
  switch (cols / 256) {                                                       \
    case 1: return bf16 ? FN<true, 1>(__VA_ARGS__) : FN<false, 1>(__VA_ARGS__); \
    case 2: return bf16 ? FN<true, 2>(__VA_ARGS__) : FN<false, 2>(__VA_ARGS__); \
    case 3: return bf16 ? FN<true, 3>(__VA_ARGS__) : FN<false, 3>(__VA_ARGS__); \
    case 4: return bf16 ? FN<true, 4>(__VA_ARGS__) : FN<false, 4>(__VA_ARGS__); \
    default: return cudaErrorInvalidValue;                                    \
  }

cudaError_t launch_layer_norm_fwd(const LayerNormArgs& a, int cols, bool bf16, int sms, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  RBF_LN_DISPATCH(launch_fwd_t, a, sms, stream)
}

cudaError_t launch_layer_norm_bwd(const LayerNormBwdArgs& a, int cols, bool bf16, int sms, cudaStream_t stream) {
  const int grid = layer_norm_bwd_blocks(a.rows, sms);
  RBF_LN_DISPATCH(launch_bwd_t, a, grid, stream)
}

}  // namespace rbf
