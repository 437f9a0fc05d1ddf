// Row-wise pre-passes over (B, H, N, D) tensors: scaled squared row norms (the RBF key / query bias)
// and the backward's delta = rowsum(O * dO). One warp per row; pure HBM streaming.
#include "common.cuh"
#include "launch.h"

namespace rbf {

template <bool kBf16, int D>
__device__ __forceinline__ void load_row_chunk(const void* base, int64_t row_off, int lane, float (&x)[D / 32]) {
  constexpr int kPer = D / 32;  // 2 (D=64) or 4 (D=128) consecutive elements per lane
  const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + row_off + lane * kPer;
  if constexpr (kPer == 2) {
    uint32_t w = *reinterpret_cast<const uint32_t*>(p);
    float2 f = unpack2<kBf16>(w);
    x[0] = f.x; x[1] = f.y;
  } else {
    uint2 w = *reinterpret_cast<const uint2*>(p);
    float2 f0 = unpack2<kBf16>(w.x), f1 = unpack2<kBf16>(w.y);
    x[0] = f0.x; x[1] = f0.y; x[2] = f1.x; x[3] = f1.y;
  }
}

// out[bh * n_pad + i] = scale * sum_d x[b,h,i,d]^2 for i < N, `pad_value` for N <= i < n_pad.
// With y != nullptr: out = sum_d x*y (scale ignored).
template <bool kBf16, int D>
__global__ void __launch_bounds__(256) row_reduce_kernel(const void* __restrict__ x, const void* __restrict__ y,
                                                         float* __restrict__ out, int H, int N, int n_pad,
                                                         int64_t xsb, int64_t xsh, int64_t xsn, int64_t ysb,
                                                         int64_t ysh, int64_t ysn, float scale, float pad_value,
                                                         DeviceStatus* status_to_clear) {
  if (status_to_clear != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) status_to_clear->code = 0;
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int bh = blockIdx.y;
  if (row >= n_pad) return;
  float acc;
  if (row < N) {
    const int b = bh / H, h = bh % H;
    float xv[D / 32];
    load_row_chunk<kBf16, D>(x, b * xsb + h * xsh + row * xsn, lane, xv);
    acc = 0.f;
    if (y != nullptr) {
      float yv[D / 32];
      load_row_chunk<kBf16, D>(y, b * ysb + h * ysh + row * ysn, lane, yv);
#pragma unroll
      for (int i = 0; i < D / 32; ++i) acc = fmaf(xv[i], yv[i], acc);
    } else {
#pragma unroll
      for (int i = 0; i < D / 32; ++i) acc = fmaf(xv[i], xv[i], acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (y == nullptr) acc *= scale;
  } else {
    acc = pad_value;
  }
  if (lane == 0) out[static_cast<int64_t>(bh) * n_pad + row] = acc;
}

template <bool kBf16, int D>
static cudaError_t launch_row_reduce_t(const RowReduceArgs& a, cudaStream_t stream) {
  dim3 grid((a.n_pad + 7) / 8, a.B * a.H);
  row_reduce_kernel<kBf16, D><<<grid, 256, 0, stream>>>(a.x, a.y, a.out, a.H, a.N, a.n_pad, a.xs[0], a.xs[1],
                                                         a.xs[2], a.ys[0], a.ys[1], a.ys[2], a.scale, a.pad_value,
                                                         a.status_to_clear);
  return cudaGetLastError();
}

cudaError_t launch_row_reduce(const RowReduceArgs& a, bool bf16, int D, cudaStream_t stream) {
  if (D == 64) return bf16 ? launch_row_reduce_t<true, 64>(a, stream) : launch_row_reduce_t<false, 64>(a, stream);
  return bf16 ? launch_row_reduce_t<true, 128>(a, stream) : launch_row_reduce_t<false, 128>(a, stream);
}

}  // namespace rbf
