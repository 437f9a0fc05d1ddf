// GELU of the model's MLP (nn.GELU() between the two projections of every block, train_rbf_transformer.py:143: the
// exact, erf-based form) for 16-bit activations, forward and backward as streaming kernels. Roofline: HBM (forward:
// read h, write a; backward: read h and dy, write dh). The normal distribution function comes from the rational
// approximation 7.1.26 of Abramowitz & Stegun, erfc(z) = t (a1 + t (a2 + t (a3 + t (a4 + t a5)))) exp(-z^2) with
// t = 1 / (1 + p z), absolute error below 1.5e-7 - a thousandth of a bf16 rounding step - at one reciprocal and one
// exponential on the special-function unit; erff() costs as many instructions as the rest of the element and makes
// the kernel issue-bound. The backward also sums its output over the rows (the bias gradient of the projection that
// feeds the GELU) in the same pass, with the column-sum kernel's layout: a block owns 256 columns and a band of rows.
#include <cstdint>
#include <cuda_runtime.h>

#include "launch.h"

namespace rbf {
namespace {

template <bool kBf16>
__device__ __forceinline__ float2 g_unpack(uint32_t w) {
  if constexpr (kBf16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  return make_float2(__half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu))),
                     __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16))));
}
template <bool kBf16>
__device__ __forceinline__ uint32_t g_pack(float a, float b) {
  if constexpr (kBf16) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
  }
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ float g_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float g_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Phi(x) = P(N(0,1) <= x) and e = exp(-x^2 / 2)
__device__ __forceinline__ float normal_cdf(float x, float& e) {
  const float ax = fabsf(x);
  const float t = g_rcp(fmaf(0.3275911f * 0.70710678f, ax, 1.0f));              // z = |x| / sqrt(2)
  e = g_ex2(x * x * (-0.5f * 1.4426950408889634f));
  float poly = fmaf(t, 1.061405429f, -1.453152027f);
  poly = fmaf(t, poly, 1.421413741f);
  poly = fmaf(t, poly, -0.284496736f);
  poly = fmaf(t, poly, 0.254829592f);
  const float q = 0.5f * t * poly * e;                                           // 0.5 erfc(z)
  return x >= 0.f ? 1.0f - q : q;
}

template <bool kBf16>
__global__ void __launch_bounds__(256) gelu_fwd_kernel(const uint4* __restrict__ h, uint4* __restrict__ out, int64_t n16) {
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n16; i += gridDim.x * 256ll) {
    const uint4 raw = h[i];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = g_unpack<kBf16>(w[j]);
      float e0, e1;
      o[j] = g_pack<kBf16>(x.x * normal_cdf(x.x, e0), x.y * normal_cdf(x.y, e1));
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// dh = dy * (Phi(h) + h phi(h)); partials[band][c] = sum over the band's rows of dh[:, c] (when partials != nullptr)
template <bool kBf16>
__global__ void __launch_bounds__(256) gelu_bwd_kernel(const uint16_t* __restrict__ h, const uint16_t* __restrict__ dy,
                                                       uint16_t* __restrict__ dh, int64_t rows, int cols, int64_t band,
                                                       float* __restrict__ partials) {
  __shared__ float s_acc[8][256 + 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + lane) * 8;
  const int64_t r0 = blockIdx.y * band, r1 = min(r0 + band, rows);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < cols) {
#pragma unroll 2
    for (int64_t r = r0 + warp; r < r1; r += 8) {
      const int64_t at = r * cols + col;
      const uint4 hr = *reinterpret_cast<const uint4*>(h + at);
      const uint4 gr = *reinterpret_cast<const uint4*>(dy + at);
      const uint32_t hw[4] = {hr.x, hr.y, hr.z, hr.w}, gw[4] = {gr.x, gr.y, gr.z, gr.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = g_unpack<kBf16>(hw[j]), g = g_unpack<kBf16>(gw[j]);
        float e0, e1;
        const float c0 = normal_cdf(x.x, e0), c1 = normal_cdf(x.y, e1);
        const float d0 = g.x * fmaf(x.x * 0.3989422804f, e0, c0), d1 = g.y * fmaf(x.y * 0.3989422804f, e1, c1);
        o[j] = g_pack<kBf16>(d0, d1);
        // the sums take the rounded values: what a reduction over the stored dh would see
        const float2 rd = g_unpack<kBf16>(o[j]);
        acc[2 * j] += rd.x;
        acc[2 * j + 1] += rd.y;
      }
      *reinterpret_cast<uint4*>(dh + at) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  if (partials == nullptr) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) s_acc[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < cols) {
    float sum = 0.f;
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) sum += s_acc[wv][threadIdx.x];
    partials[static_cast<int64_t>(blockIdx.y) * cols + c] = sum;
  }
}

}  // namespace

cudaError_t launch_gelu_fwd(const void* h, void* out, int64_t n, bool bf16, int sms, cudaStream_t stream) {
  const int64_t n16 = n / 8;
  if (n16 == 0) return cudaSuccess;
  const int64_t want = (n16 + 255) / 256;
  const int grid = static_cast<int>(want < sms * 16ll ? want : sms * 16ll);
  if (bf16) gelu_fwd_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(h), static_cast<uint4*>(out), n16);
  else gelu_fwd_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(h), static_cast<uint4*>(out), n16);
  return cudaGetLastError();
}

cudaError_t launch_gelu_bwd(const void* h, const void* dy, void* dh, int64_t rows, int cols, bool bf16, float* partials,
                            float* dbias, int sms, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  const int bands = col_sums_bands(rows, cols, sms);
  const int64_t band = (rows + bands - 1) / bands;
  const dim3 grid((cols + 255) / 256, bands);
  const uint16_t* hp = static_cast<const uint16_t*>(h);
  const uint16_t* gp = static_cast<const uint16_t*>(dy);
  uint16_t* op = static_cast<uint16_t*>(dh);
  float* part = dbias != nullptr ? partials : nullptr;
  if (bf16) gelu_bwd_kernel<true><<<grid, 256, 0, stream>>>(hp, gp, op, rows, cols, band, part);
  else gelu_bwd_kernel<false><<<grid, 256, 0, stream>>>(hp, gp, op, rows, cols, band, part);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || dbias == nullptr) return e;
  return launch_col_sums_final(partials, bands, cols, dbias, stream);
}

}  // namespace rbf
