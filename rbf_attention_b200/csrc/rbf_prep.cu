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

// ---------------------------------------------------------------------------------------------
// Pre-pass of the TF32 forward (fp32 tensors, head dim 64)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float tf32_part(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

__global__ void __launch_bounds__(256) row_stats_f32_kernel(const RowStatsF32Args a) {
  constexpr int D = 64;
  constexpr int kLanesPerRow = D / 4;                 // 16 lanes x 16 bytes
  constexpr int kRowsPerWarp = 32 / kLanesPerRow;     // 2
  if (a.status_to_clear != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < 64)
    reinterpret_cast<unsigned int*>(a.status_to_clear)[threadIdx.x] = 0u;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / kLanesPerRow, part = lane % kLanesPerRow;
  const int bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int row = (blockIdx.x * 8 + warp) * kRowsPerWarp + sub;
  const bool valid = row < a.N;
  float ksq = 0.f, qsq = 0.f;
  if (valid) {
    const float4 kv = *reinterpret_cast<const float4*>(a.k + b * a.ks[0] + h * a.ks[1] +
                                                       static_cast<int64_t>(row) * a.ks[2] + part * 4);
    ksq = kv.x * kv.x + kv.y * kv.y + kv.z * kv.z + kv.w * kv.w;
    if (a.q != nullptr) {
      const float4 qv = *reinterpret_cast<const float4*>(a.q + b * a.qs[0] + h * a.qs[1] +
                                                         static_cast<int64_t>(row) * a.qs[2] + part * 4);
      qsq = qv.x * qv.x + qv.y * qv.y + qv.z * qv.z + qv.w * qv.w;
    }
  }
#pragma unroll
  for (int o = kLanesPerRow / 2; o > 0; o >>= 1) {
    ksq += __shfl_xor_sync(0xffffffffu, ksq, o);
    qsq += __shfl_xor_sync(0xffffffffu, qsq, o);
  }
  if (part == 0 && row < a.n_pad) {
    const int64_t out_row = static_cast<int64_t>(bh) * a.n_pad + row;
    // three parts that the tensor core reads exactly (it keeps the upper 19 bits of an operand) and that add up to
    // the fp32 value
    const float x = valid ? -ksq * a.scale / a.scale2 : -1e30f;
    const float hi = tf32_part(x), mid = tf32_part(x - hi), lo = tf32_part(x - hi - mid);
    float4* dst = reinterpret_cast<float4*>(a.kslab_out + out_row * 8);
    dst[0] = make_float4(hi, mid, lo, 0.f);
    dst[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.qsq_out != nullptr) a.qsq_out[out_row] = valid ? qsq * a.scale : 0.f;
  }
}

cudaError_t launch_row_stats_f32(const RowStatsF32Args& a, cudaStream_t stream) {
  dim3 grid((a.n_pad + 15) / 16, a.B * a.H);
  row_stats_f32_kernel<<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Fused q/k preparation of the attention block (see QkvPrepArgs)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_param(const void* base, int64_t index, bool fp32, bool bf16) {
  if (fp32) return reinterpret_cast<const float*>(base)[index];
  const uint16_t raw = reinterpret_cast<const uint16_t*>(base)[index];
  if (bf16) return __uint_as_float(static_cast<uint32_t>(raw) << 16);
  return __half2float(__ushort_as_half(raw));
}

template <bool kBf16>
__device__ __forceinline__ uint4 add_round8(const uint4& x, const float (&e)[8], float& sumsq) {
  const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
  uint32_t ow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack2<kBf16>(xw[i]);
    ow[i] = pack2<kBf16>(f.x + e[2 * i], f.y + e[2 * i + 1]);
    const float2 r = unpack2<kBf16>(ow[i]);          // the norms are those of the rounded rows the kernels will read
    sumsq = fmaf(r.x, r.x, sumsq);
    sumsq = fmaf(r.y, r.y, sumsq);
  }
  return make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

static constexpr int kPrepRowsPerBlock = 8;      // sequence positions per block (all heads)

template <bool kBf16, int D>
__global__ void __launch_bounds__(256) qkv_prep_kernel(const QkvPrepArgs a) {
  constexpr int kLanesPerRow = D / 8;
  if (a.status_to_clear != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < 64)
    reinterpret_cast<unsigned int*>(a.status_to_clear)[threadIdx.x] = 0u;
  const int b = blockIdx.y;
  const int s0 = blockIdx.x * kPrepRowsPerBlock;
  const int per_pos = a.H * kLanesPerRow;                 // 16-byte chunks of q (or k) per sequence position
  const int items = kPrepRowsPerBlock * per_pos;
  const int64_t E = static_cast<int64_t>(a.H) * D;
  const float inv = 1.0f / (a.scale2 * a.slab_w);
  // whole warps stay in the loop: a row's lanes reduce with shuffles
  for (int base = 0; base < items; base += 256) {
    const int idx = base + threadIdx.x;
    const int s = s0 + idx / per_pos;
    const int rem = idx % per_pos;
    const int h = rem / kLanesPerRow, part = rem % kLanesPerRow;
    const bool in_range = idx < items && s < a.n_pad;
    const bool valid = in_range && s < a.S;
    float ksq = 0.f, qsq = 0.f;
    if (valid) {
      float e[8];
      if (s < a.R) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          e[j] = load_param(a.reg_pos, (static_cast<int64_t>(h) * a.R + s) * D + part * 8 + j, a.params_fp32, kBf16);
      } else {
        const float* trow = a.table + static_cast<int64_t>(s - a.R) * D + part * 8;
        const int i0 = (part * 8) % (D / 2);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          e[j] = trow[j] * load_param(a.pos_weight, static_cast<int64_t>(h) * (D / 2) + i0 + j, a.params_fp32, kBf16);
      }
      const uint16_t* src = reinterpret_cast<const uint16_t*>(a.qkv) + (static_cast<int64_t>(b) * a.S + s) * 3 * E +
                            static_cast<int64_t>(h) * D + part * 8;
      const uint4 qv = *reinterpret_cast<const uint4*>(src);
      const uint4 kv = *reinterpret_cast<const uint4*>(src + E);
      const uint4 qn = add_round8<kBf16>(qv, e, qsq);
      const uint4 kn = add_round8<kBf16>(kv, e, ksq);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.q_out) + b * a.qo[0] + h * a.qo[1] +
                                static_cast<int64_t>(s) * a.qo[2] + part * 8) = qn;
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.k_out) + b * a.ko[0] + h * a.ko[1] +
                                static_cast<int64_t>(s) * a.ko[2] + part * 8) = kn;
    }
#pragma unroll
    for (int o = kLanesPerRow / 2; o > 0; o >>= 1) {
      ksq += __shfl_xor_sync(0xffffffffu, ksq, o);
      qsq += __shfl_xor_sync(0xffffffffu, qsq, o);
    }
    if (in_range && part == 0) {
      const int64_t row = (static_cast<int64_t>(b) * a.H + h) * a.n_pad + s;
      if (a.kslab_out != nullptr) store_slab_row<kBf16>(a.kslab_out, row, valid ? -ksq * a.scale * inv : -a.slab_big);
      if (a.qsq_out != nullptr) a.qsq_out[row] = valid ? qsq * a.scale : 0.f;
    }
  }
}

cudaError_t launch_qkv_prep(const QkvPrepArgs& a, bool bf16, cudaStream_t stream) {
  dim3 grid((a.n_pad + kPrepRowsPerBlock - 1) / kPrepRowsPerBlock, a.B);
  if (a.D == 64) {
    if (bf16) qkv_prep_kernel<true, 64><<<grid, 256, 0, stream>>>(a);
    else qkv_prep_kernel<false, 64><<<grid, 256, 0, stream>>>(a);
  } else {
    if (bf16) qkv_prep_kernel<true, 128><<<grid, 256, 0, stream>>>(a);
    else qkv_prep_kernel<false, 128><<<grid, 256, 0, stream>>>(a);
  }
  return cudaGetLastError();
}

// ---- backward: gradients of pos_weight and of the register-position rows -----------------------------------------
static constexpr int kPrepBwdRows = 64;          // text rows per block of the first stage
static constexpr int kPrepBwdMaxSlots = 4;       // (head, chunk) columns per thread: H * D / 8 <= 1024

int qkv_prep_bwd_chunks(int S, int R) { return (S - R + kPrepBwdRows - 1) / kPrepBwdRows; }

template <bool kBf16>
__global__ void __launch_bounds__(256) qkv_prep_bwd_partial_kernel(const QkvPrepBwdArgs a) {
  extern __shared__ float s_cols[];              // groups x (H * D) column sums of this block
  const int D = a.D;
  const int lanes = D / 8;
  const int cols = a.H * lanes;                  // 16-byte columns of one text row over all heads
  const int groups = cols >= 256 ? 1 : 256 / cols;   // row groups: few columns leave threads for a split over the rows
  const int b = blockIdx.y;
  const int t0 = blockIdx.x * kPrepBwdRows;
  const int t1 = min(t0 + kPrepBwdRows, a.S - a.R);
#pragma unroll
  for (int u = 0; u < kPrepBwdMaxSlots; ++u) {
    const int idx = threadIdx.x + u * 256;
    if (idx >= cols * groups) break;
    const int c = idx % cols, rg = idx / cols;
    const int h = c / lanes, part = c % lanes;
    const uint16_t* pq = reinterpret_cast<const uint16_t*>(a.dq) + b * a.dqs[0] + h * a.dqs[1] + part * 8;
    const uint16_t* pk = reinterpret_cast<const uint16_t*>(a.dk) + b * a.dks[0] + h * a.dks[1] + part * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll 4                                   // independent rows: keep several 16-byte loads in flight
    for (int t = t0 + rg; t < t1; t += groups) {
      const uint4 x = *reinterpret_cast<const uint4*>(pq + static_cast<int64_t>(a.R + t) * a.dqs[2]);
      const uint4 y = *reinterpret_cast<const uint4*>(pk + static_cast<int64_t>(a.R + t) * a.dks[2]);
      const float4 w0 = *reinterpret_cast<const float4*>(a.table + static_cast<int64_t>(t) * D + part * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(a.table + static_cast<int64_t>(t) * D + part * 8 + 4);
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<kBf16>(xw[i]), g = unpack2<kBf16>(yw[i]);
        acc[2 * i] = fmaf(f.x + g.x, w[2 * i], acc[2 * i]);
        acc[2 * i + 1] = fmaf(f.y + g.y, w[2 * i + 1], acc[2 * i + 1]);
      }
    }
    float* mine = s_cols + (rg * cols + c) * 8;
    *reinterpret_cast<float4*>(mine) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(mine + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  __syncthreads();
  // fold the row groups (fixed order), then the sine half and the cosine half of every head onto its D/2 weights
  const int half = D / 2;
  float* dst = a.partials + (static_cast<int64_t>(b) * gridDim.x + blockIdx.x) * a.H * half;
  for (int o = threadIdx.x; o < a.H * half; o += 256) {
    const int h = o / half, i = o % half;
    float sum = 0.f;
    for (int g = 0; g < groups; ++g) {
      const float* src = s_cols + g * cols * 8;
      sum += src[h * D + i] + src[h * D + half + i];
    }
    dst[o] = sum;
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(1024) qkv_prep_bwd_final_kernel(const QkvPrepBwdArgs a) {
  // blocks [0, nw): 32 weight gradients each; 32 partial-lanes per output stride over the block partials with four
  // independent sums (the loads of a lane are independent: several stay in flight), then a fixed-order tree in shared
  // memory. The remaining blocks: register-position gradients, one thread per element, summed over the batch.
  const int half = a.D / 2;
  const int n_out = a.H * half;
  const int nw = (n_out + 31) / 32;
  if (static_cast<int>(blockIdx.x) < nw) {
    __shared__ float s_part[32][33];
    const int col = threadIdx.x & 31, lane_p = threadIdx.x >> 5;
    const int o = blockIdx.x * 32 + col;
    const int n_blocks = a.B * a.chunks;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (o < n_out) {
      const float* src = a.partials + o;
      int p = lane_p;
      for (; p + 96 < n_blocks; p += 128) {
        s0 += src[static_cast<int64_t>(p) * n_out];
        s1 += src[static_cast<int64_t>(p + 32) * n_out];
        s2 += src[static_cast<int64_t>(p + 64) * n_out];
        s3 += src[static_cast<int64_t>(p + 96) * n_out];
      }
      for (; p < n_blocks; p += 32) s0 += src[static_cast<int64_t>(p) * n_out];
    }
    s_part[lane_p][col] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (threadIdx.x < 32 && o < n_out) {
      float total = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) total += s_part[i][threadIdx.x];
      a.d_pos_weight[o] = total;
    }
  } else {
    const int e = (blockIdx.x - nw) * 1024 + threadIdx.x;
    if (e >= a.H * a.R * a.D) return;
    const int d = e % a.D, r = (e / a.D) % a.R, h = e / (a.D * a.R);
    const uint16_t* pq = reinterpret_cast<const uint16_t*>(a.dq) + h * a.dqs[1] + r * a.dqs[2] + d;
    const uint16_t* pk = reinterpret_cast<const uint16_t*>(a.dk) + h * a.dks[1] + r * a.dks[2] + d;
    float sum = 0.f;
    for (int b0 = 0; b0 < a.B; b0 += 8) {            // eight batches' loads in flight (each one a DRAM round trip)
      uint16_t x[8], y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool in = b0 + j < a.B;
        x[j] = in ? pq[(b0 + j) * a.dqs[0]] : uint16_t(0);
        y[j] = in ? pk[(b0 + j) * a.dks[0]] : uint16_t(0);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        sum += kBf16 ? __uint_as_float(static_cast<uint32_t>(x[j]) << 16) + __uint_as_float(static_cast<uint32_t>(y[j]) << 16)
                     : __half2float(__ushort_as_half(x[j])) + __half2float(__ushort_as_half(y[j]));
    }
    a.d_reg_pos[e] = sum;
  }
}

cudaError_t launch_qkv_prep_bwd(QkvPrepBwdArgs a, bool bf16, cudaStream_t stream) {
  if (a.H * (a.D / 8) > 256 * kPrepBwdMaxSlots) return cudaErrorInvalidValue;
  a.chunks = qkv_prep_bwd_chunks(a.S, a.R);
  const int cols = a.H * (a.D / 8);
  const int smem = (cols >= 256 ? 1 : 256 / cols) * a.H * a.D * sizeof(float);
  dim3 grid(a.chunks, a.B);
  if (bf16) qkv_prep_bwd_partial_kernel<true><<<grid, 256, smem, stream>>>(a);
  else qkv_prep_bwd_partial_kernel<false><<<grid, 256, smem, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int nw = (a.H * (a.D / 2) + 31) / 32;
  const int nr = (a.H * a.R * a.D + 1023) / 1024;
  if (bf16) qkv_prep_bwd_final_kernel<true><<<nw + nr, 1024, 0, stream>>>(a);
  else qkv_prep_bwd_final_kernel<false><<<nw + nr, 1024, 0, stream>>>(a);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Exclusive self attention: row-wise projection away from the position's own value row (see XsaArgs)
// ---------------------------------------------------------------------------------------------
template <bool kBf16>
__device__ __forceinline__ void unpack8(const uint4& x, float (&f)[8]) {
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack2<kBf16>(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <bool kBf16>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack2<kBf16>(f[0], f[1]), pack2<kBf16>(f[2], f[3]), pack2<kBf16>(f[4], f[5]),
                    pack2<kBf16>(f[6], f[7]));
}

template <bool kBf16, int D, bool kBackward>
__global__ void __launch_bounds__(256) xsa_kernel(const XsaArgs a) {
  constexpr int kLanesPerRow = D / 8;
  constexpr int kRowsPerBlock = 256 / kLanesPerRow;
  const int sub = threadIdx.x / kLanesPerRow, part = threadIdx.x % kLanesPerRow;
  const int bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int row = blockIdx.x * kRowsPerBlock + sub;
  const bool valid = row < a.N;
  float o[8] = {}, v[8] = {}, g[8] = {};
  if (valid) {
    unpack8<kBf16>(load_chunk(a.o, a.os, b, h, row, part), o);
    unpack8<kBf16>(load_chunk(a.v, a.vs, b, h, row, part), v);
    if (kBackward) unpack8<kBf16>(load_chunk(a.g, a.gs, b, h, row, part), g);
  }
  float vv = 0.f, ov = 0.f, gv = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    vv = fmaf(v[j], v[j], vv);
    ov = fmaf(o[j], v[j], ov);
    if (kBackward) gv = fmaf(g[j], v[j], gv);
  }
#pragma unroll
  for (int m = kLanesPerRow / 2; m > 0; m >>= 1) {
    vv += __shfl_xor_sync(0xffffffffu, vv, m);
    ov += __shfl_xor_sync(0xffffffffu, ov, m);
    if (kBackward) gv += __shfl_xor_sync(0xffffffffu, gv, m);
  }
  if (!valid) return;
  const float nrm = fmaxf(sqrtf(vv), 1e-12f);
  const float inv = 1.0f / nrm;
  const float alpha = ov * inv;                 // o . vh
  uint16_t* out = reinterpret_cast<uint16_t*>(a.out) + b * a.outs[0] + h * a.outs[1] +
                  static_cast<int64_t>(row) * a.outs[2] + part * 8;
  float r[8];
  if (!kBackward) {
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = fmaf(-alpha * inv, v[j], o[j]);
    *reinterpret_cast<uint4*>(out) = pack8<kBf16>(r);
  } else {
    const float beta = gv * inv;                // g . vh
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = fmaf(-beta * inv, v[j], g[j]);
    *reinterpret_cast<uint4*>(out) = pack8<kBf16>(r);
    // below the clamp vh = v / 1e-12 is linear in v: only the first two terms remain
    const float corr = sqrtf(vv) > 1e-12f ? 2.f * alpha * beta * inv : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = (fmaf(corr, v[j], -alpha * g[j]) - beta * o[j]) * inv;
    uint16_t* dv = reinterpret_cast<uint16_t*>(a.dv) + b * a.dvs[0] + h * a.dvs[1] +
                   static_cast<int64_t>(row) * a.dvs[2] + part * 8;
    *reinterpret_cast<uint4*>(dv) = pack8<kBf16>(r);
  }
}

template <bool kBf16, int D>
static cudaError_t launch_xsa_t(const XsaArgs& a, bool backward, cudaStream_t stream) {
  constexpr int kRowsPerBlock = 256 / (D / 8);
  dim3 grid((a.N + kRowsPerBlock - 1) / kRowsPerBlock, a.B * a.H);
  if (backward) xsa_kernel<kBf16, D, true><<<grid, 256, 0, stream>>>(a);
  else xsa_kernel<kBf16, D, false><<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_xsa(const XsaArgs& a, bool backward, bool bf16, int D, cudaStream_t stream) {
  if (D == 64) return bf16 ? launch_xsa_t<true, 64>(a, backward, stream) : launch_xsa_t<false, 64>(a, backward, stream);
  return bf16 ? launch_xsa_t<true, 128>(a, backward, stream) : launch_xsa_t<false, 128>(a, backward, stream);
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

__global__ void __launch_bounds__(32) post_status_kernel(const DeviceStatus* status, unsigned int* host_slot) {
  // a plain store into page-locked host memory mapped into the device's address space: no copy engine takes part,
  // so the word arrives even while the engines are busy with the caller's own bulk transfers
  if (threadIdx.x == 0) {
    *reinterpret_cast<volatile unsigned int*>(host_slot) = status->code;
    __threadfence_system();
  }
}

cudaError_t launch_post_status(const DeviceStatus* status, unsigned int* host_slot_device_ptr, cudaStream_t stream) {
  post_status_kernel<<<1, 32, 0, stream>>>(status, host_slot_device_ptr);
  return cudaGetLastError();
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
