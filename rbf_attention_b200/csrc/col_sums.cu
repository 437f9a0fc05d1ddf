// Column sums of a 16-bit (rows x cols) matrix in fp32: the bias gradient of a linear layer, sum over the rows of the
// layer's output gradient (the language model's projections, train_rbf_transformer.py:143, 216 and
// rbf_attention.py:1625-1626; PyTorch's generic reduction reaches 1 TB/s on 65792 x 512). Roofline: HBM, one read of
// the matrix. A block owns 256 columns and a band of rows: 32 lanes x 16 bytes along a row (512 contiguous bytes per
// warp), 8 warps on 8 consecutive rows, fp32 sums in registers, folded across the warps in shared memory; the bands'
// partial rows are summed by a second small kernel in a fixed order (bitwise reproducible).
#include <cstdint>
#include <cuda_runtime.h>

#include "launch.h"

namespace rbf {
namespace {

template <bool kBf16>
__device__ __forceinline__ float2 cs_unpack(uint32_t w) {
  if constexpr (kBf16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  return make_float2(__half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu))),
                     __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16))));
}

template <bool kBf16>
__global__ void __launch_bounds__(256) col_sums_partial_kernel(const uint16_t* __restrict__ x, int64_t ld, int64_t rows,
                                                               int cols, int64_t band, float* __restrict__ partials) {
  __shared__ float s_acc[8][256 + 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + lane) * 8;
  const int64_t r0 = blockIdx.y * band, r1 = min(r0 + band, rows);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < cols) {
    const uint16_t* p = x + col;
#pragma unroll 4                                    // independent rows: several 16-byte loads in flight per thread
    for (int64_t r = r0 + warp; r < r1; r += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p + r * ld);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = cs_unpack<kBf16>(w[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
  }
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

// out[c] = sum over bands of partials[band][c]: 32 columns x 8 band-lanes per block of 256
__global__ void __launch_bounds__(256) col_sums_final_kernel(const float* __restrict__ partials, int bands, int cols,
                                                             float* __restrict__ out) {
  __shared__ float s[8][33];
  const int col = threadIdx.x & 31, lp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + col;
  float sum = 0.f;
  if (c < cols)
    for (int b = lp; b < bands; b += 8) sum += partials[static_cast<int64_t>(b) * cols + c];
  s[lp][col] = sum;
  __syncthreads();
  if (threadIdx.x < 32 && c < cols) {
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += s[i][threadIdx.x];
    out[c] = total;
  }
}

}  // namespace

int col_sums_bands(int64_t rows, int cols, int sms) {
  const int col_blocks = (cols + 255) / 256;
  int64_t bands = (static_cast<int64_t>(sms) * 8 + col_blocks - 1) / col_blocks;   // about eight blocks per SM
  const int64_t most = (rows + 63) / 64;                                          // at least 64 rows per band
  if (bands > most) bands = most;
  if (bands > 65535) bands = 65535;
  return static_cast<int>(bands < 1 ? 1 : bands);
}

cudaError_t launch_col_sums_final(const float* partials, int bands, int cols, float* out, cudaStream_t stream) {
  col_sums_final_kernel<<<(cols + 31) / 32, 256, 0, stream>>>(partials, bands, cols, out);
  return cudaGetLastError();
}

cudaError_t launch_col_sums(const void* x, int64_t ld, int64_t rows, int cols, bool bf16, float* partials, float* out,
                            int sms, cudaStream_t stream) {
  const int bands = col_sums_bands(rows, cols, sms);
  const int64_t band = (rows + bands - 1) / bands;
  const dim3 grid((cols + 255) / 256, bands);
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  if (bf16) col_sums_partial_kernel<true><<<grid, 256, 0, stream>>>(xp, ld, rows, cols, band, partials);
  else col_sums_partial_kernel<false><<<grid, 256, 0, stream>>>(xp, ld, rows, cols, band, partials);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  col_sums_final_kernel<<<(cols + 31) / 32, 256, 0, stream>>>(partials, bands, cols, out);
  return cudaGetLastError();
}

}  // namespace rbf
