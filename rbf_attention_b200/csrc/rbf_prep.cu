// Row-wise pre-pass over (B, H, N, D) tensors, one launch per forward / backward call:
//   ksq[row]     = c * |k_row|^2            (+inf on padding rows: a padded key then gets weight exp2(-inf) = 0)
//   qsq[row]     = c * |q_row|^2            (non-softmax variant)
//   delta[row]   = sum_d O[row,d] dO[row,d] (softmax backward; 0 on padding rows)
//   lse_pad[row] = lse[row]                 (softmax backward: the forward's L re-pitched to n_pad, +inf padding)
//   the backward's fp32 dQ accumulator is cleared on the way
//   bias slabs of -ksq, of -L (or -qsq, non-softmax variant) and of -delta (or zeros) for the MMA bias steps
// Pure HBM streaming: D/8 lanes per row with 16-byte loads, 32/(D/8) rows per warp per iteration.
#include "common.cuh"
#include "launch.h"

namespace rbf {

template <bool kBf16>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = unpack2<kBf16>(aw[i]), y = unpack2<kBf16>(bw[i]);
    acc = fmaf(x.x, y.x, acc);
    acc = fmaf(x.y, y.y, acc);
  }
  return acc;
}

// fp32 value -> three 16-bit floats whose sum reproduces it to ~24 bits, as one 32-byte slab row (13 zeros follow).
template <bool kBf16>
__device__ __forceinline__ void store_slab_row(void* slab, int64_t row, float x) {
  float hi, mid, lo;
  if constexpr (kBf16) {
    hi = __bfloat162float(__float2bfloat16_rn(x));
    mid = __bfloat162float(__float2bfloat16_rn(x - hi));
    lo = __bfloat162float(__float2bfloat16_rn(x - hi - mid));
  } else {
    hi = __half2float(__float2half_rn(x));
    mid = __half2float(__float2half_rn(x - hi));
    lo = __half2float(__float2half_rn(x - hi - mid));
  }
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(slab) + row * 32);
  dst[0] = make_uint4(pack2<kBf16>(hi, mid), pack2<kBf16>(lo, 0.f), 0u, 0u);
  dst[1] = make_uint4(0u, 0u, 0u, 0u);
}

__device__ __forceinline__ uint4 load_chunk(const void* base, const int64_t* s, int b, int h, int row, int part) {
  return *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + b * s[0] + h * s[1] +
                                         static_cast<int64_t>(row) * s[2] + part * 8);
}

template <bool kBf16, int D>
__global__ void __launch_bounds__(256) row_stats_kernel(const RowStatsArgs a) {
  constexpr int kLanesPerRow = D / 8;                 // 8 (D=64) or 16 (D=128)
  constexpr int kRowsPerWarp = 32 / kLanesPerRow;     // 4 or 2
  if (a.status_to_clear != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < 64)
    reinterpret_cast<unsigned int*>(a.status_to_clear)[threadIdx.x] = 0u;   // status word and work counters
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane / kLanesPerRow;                // row within the warp's group
  const int part = lane % kLanesPerRow;               // 16-byte chunk of the row
  const int bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int rows_per_block = 8 * kRowsPerWarp * a.iters;
  const int row_begin = blockIdx.x * rows_per_block;
  const int64_t out_base = static_cast<int64_t>(bh) * a.n_pad;

  if (a.zero_rows != nullptr) {
    // clear this block's rows of the fp32 accumulator: the writes ride along with a kernel that mostly reads
    const int rows_here = min(rows_per_block, a.N - row_begin);
    if (rows_here > 0) {
      float4* dst = reinterpret_cast<float4*>(a.zero_rows + (static_cast<int64_t>(bh) * a.N + row_begin) * D);
      const int n4 = rows_here * (D / 4);
      for (int i = threadIdx.x; i < n4; i += 256) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  for (int it = 0; it < a.iters; ++it) {
    const int row = row_begin + (it * 8 + warp) * kRowsPerWarp + sub;
    const bool valid = row < a.N;
    float ksq = 0.f, qsq = 0.f, delta = 0.f;
    if (valid) {
      if (a.k != nullptr) {
        const uint4 v = load_chunk(a.k, a.ks, b, h, row, part);
        ksq = dot8<kBf16>(v, v);
      }
      if (a.q != nullptr) {
        const uint4 v = load_chunk(a.q, a.qs, b, h, row, part);
        qsq = dot8<kBf16>(v, v);
      }
      if (a.o != nullptr) {
        const uint4 x = load_chunk(a.o, a.os, b, h, row, part);
        const uint4 y = load_chunk(a.dout, a.dos, b, h, row, part);
        delta = dot8<kBf16>(x, y);
      }
    }
#pragma unroll
    for (int o = kLanesPerRow / 2; o > 0; o >>= 1) {
      ksq += __shfl_xor_sync(0xffffffffu, ksq, o);
      qsq += __shfl_xor_sync(0xffffffffu, qsq, o);
      delta += __shfl_xor_sync(0xffffffffu, delta, o);
    }
    if (part == 0 && row < a.n_pad) {
      if (a.ksq_out != nullptr) a.ksq_out[out_base + row] = valid ? ksq * a.scale : INFINITY;
      if (a.qsq_out != nullptr) a.qsq_out[out_base + row] = valid ? qsq * a.scale : a.qsq_pad;
      if (a.delta_out != nullptr) a.delta_out[out_base + row] = delta;
      float lse = INFINITY;
      if (a.lse != nullptr && valid) lse = a.lse[static_cast<int64_t>(bh) * a.N + row];
      if (a.lse_pad_out != nullptr) a.lse_pad_out[out_base + row] = lse;
      const float inv = 1.0f / (a.scale2 * a.slab_w);
      if (a.kslab_out != nullptr) store_slab_row<kBf16>(a.kslab_out, out_base + row, valid ? -ksq * a.scale * inv : -a.slab_big);
      const float row_stat = a.lslab_from_qsq ? qsq * a.scale : lse;
      if (a.lslab_out != nullptr)
        store_slab_row<kBf16>(a.lslab_out, out_base + row, valid ? -row_stat * inv : -a.slab_big);
      if (a.dslab_out != nullptr)
        store_slab_row<kBf16>(a.dslab_out, out_base + row, a.dslab_zero ? 0.f : -delta / a.slab_w);
    }
  }
}

template <bool kBf16, int D>
static cudaError_t launch_row_stats_t(RowStatsArgs a, cudaStream_t stream) {
  constexpr int kRowsPerWarp = 32 / (D / 8);
  a.iters = 4;
  const int rows_per_block = 8 * kRowsPerWarp * a.iters;
  dim3 grid((a.n_pad + rows_per_block - 1) / rows_per_block, a.B * a.H);
  row_stats_kernel<kBf16, D><<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

__global__ void __launch_bounds__(32) wait_selftest_kernel(DeviceStatus* status, long long limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    abort_flag = 0;
  }
  __syncwarp();
  // nothing ever arrives on `bar`: the first lane whose limit runs out records the status and raises the flag, the
  // other lanes leave on the flag, and the block returns
  mbar_wait_limit(&bar, 0, &abort_flag, status, kSiteSelfTest, limit);
  __syncwarp();
  if (threadIdx.x == 0) mbar_inval(&bar);
}

cudaError_t launch_wait_selftest(DeviceStatus* status, long long limit, cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>(status, limit);
  return cudaGetLastError();
}

cudaError_t launch_row_stats(const RowStatsArgs& a, bool bf16, int D, cudaStream_t stream) {
  if (D == 64) return bf16 ? launch_row_stats_t<true, 64>(a, stream) : launch_row_stats_t<false, 64>(a, stream);
  return bf16 ? launch_row_stats_t<true, 128>(a, stream) : launch_row_stats_t<false, 128>(a, stream);
}

}  // namespace rbf
