// Cross entropy over the vocabulary for the language-model training step (the reference trains with
// torch.nn.CrossEntropyLoss(ignore_index=-100), train_rbf_transformer.py:282,335-345): one kernel produces the
// per-row losses AND the gradient of the mean loss with respect to the logits, so that log-softmax, the loss and their
// two backward kernels (four passes over 6.6 GB of logits at the benchmark's size, plus an fp32 copy of them) become
// one read and one write. Roofline: HBM. A block owns a row: pass 1 reads it from DRAM with an online maximum / sum
// and keeps it in shared memory (100 KB per row at the benchmark's vocabulary, two blocks per SM), pass 2 writes
// softmax - onehot, scaled by 1 / (rows that count), from there. Rows too long for that are read a second time
// (with two blocks per SM in flight they are L2 hits). Measured at 65536 x 50304 bf16: 2.84 ms, 4.65 TB/s = 71 % of the
// copy bandwidth (3.16 ms with exp2f() in place of the bare ex2.approx; block shapes of 256 to 512 threads, two to
// eight per SM, staged or re-read, all land within 10 % of each other); a variant with one block of 1024 threads per SM that streams the next row into a second buffer with
// cp.async while the current one is reduced was slower (3.82 ms) and is not kept.
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "launch.h"

namespace rbf {
namespace {

constexpr int kCeThreads = 512;
constexpr float kLog2e = 1.4426950408889634f;

// 2^x on the special-function unit (two ulp; ce_ex2() adds range fix-ups that cost as much as the rest of the element)
__device__ __forceinline__ float ce_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr float kLn2 = 0.6931471805599453f;

template <int kDtype> struct Elem;
template <> struct Elem<0> {                      // bfloat16
  using type = uint16_t;
  static constexpr int kPerVec = 8;
  static __device__ __forceinline__ float to_float(uint16_t x) { return __uint_as_float(static_cast<uint32_t>(x) << 16); }
  static __device__ __forceinline__ uint16_t from_float(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
};
template <> struct Elem<1> {                      // float16
  using type = uint16_t;
  static constexpr int kPerVec = 8;
  static __device__ __forceinline__ float to_float(uint16_t x) { return __half2float(__ushort_as_half(x)); }
  static __device__ __forceinline__ uint16_t from_float(float x) { return __half_as_ushort(__float2half_rn(x)); }
};
template <> struct Elem<2> {                      // float32
  using type = float;
  static constexpr int kPerVec = 4;
  static __device__ __forceinline__ float to_float(float x) { return x; }
  static __device__ __forceinline__ float from_float(float x) { return x; }
};

// (m, s): s = sum of 2^(y - m) over the values seen so far, y = x * log2(e); m = -inf and s = 0 before any finite value
__device__ __forceinline__ void merge(float& m, float& s, float m2, float s2) {
  const float M = fmaxf(m, m2);
  if (M == -INFINITY) return;                     // both empty
  s = s * ce_ex2(m - M) + s2 * ce_ex2(m2 - M);      // ce_ex2(-inf) = 0 for the empty side
  m = M;
}

constexpr int kCeStageBytes = 113 * 1024;          // a staged row leaves room for a second block on the SM

template <int kDtype, bool kVec, bool kStage>
__global__ void __launch_bounds__(kCeThreads, 2) cross_entropy_kernel(const CrossEntropyArgs a) {
  static_assert(kVec || !kStage, "staging uses the vector path");
  extern __shared__ uint4 s_row[];                // kStage: the row, every 16-byte chunk kept by the thread that read it
  using E = Elem<kDtype>;
  using T = typename E::type;
  constexpr int V = E::kPerVec;
  __shared__ float s_m[kCeThreads / 32], s_s[kCeThreads / 32];
  __shared__ float s_lse2;
  const float scale = *a.grad_scale;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const T* x = static_cast<const T*>(a.logits) + static_cast<int64_t>(row) * a.ld;
    T* dx = static_cast<T*>(a.dlogits) + static_cast<int64_t>(row) * a.ld_out;
    const int64_t t = a.targets[row];
    const bool counts = t != a.ignore_index && t >= 0 && t < a.cols;
    if (!counts) {                                // no loss, zero gradient: the row is not read
      if constexpr (kVec) {
        for (int c = threadIdx.x; c < a.cols / V; c += kCeThreads) reinterpret_cast<uint4*>(dx)[c] = make_uint4(0, 0, 0, 0);
      } else {
        for (int c = threadIdx.x; c < a.cols; c += kCeThreads) dx[c] = E::from_float(0.f);
      }
      if (threadIdx.x == 0) a.loss_rows[row] = 0.f;
      continue;
    }
    // ---- pass 1: online maximum and sum ------------------------------------------------------------------------
    float m = -INFINITY, s = 0.f;
    if constexpr (kVec) {
#pragma unroll 4                                    // two blocks per SM: 4 x 16 bytes per thread keep 64 KB in flight
      for (int c = threadIdx.x; c < a.cols / V; c += kCeThreads) {
        const uint4 raw = reinterpret_cast<const uint4*>(x)[c];
        if constexpr (kStage) s_row[c] = raw;
        const T* e = reinterpret_cast<const T*>(&raw);
        float xv[V];
        float cx = -INFINITY;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          xv[j] = E::to_float(e[j]);
          cx = fmaxf(cx, xv[j]);
        }
        const float cm = cx * kLog2e;               // the maximum in base-2 units (log2e > 0: same element)
        if (cm > m) {
          s *= ce_ex2(m - cm);
          m = cm;
        }
        if (m != -INFINITY) {
          const float neg_m = -m;
#pragma unroll
          for (int j = 0; j < V; ++j) s += ce_ex2(fmaf(xv[j], kLog2e, neg_m));
        }
      }
    } else {
      for (int c = threadIdx.x; c < a.cols; c += kCeThreads) {
        const float y = E::to_float(x[c]) * kLog2e;
        if (y > m) {
          s *= ce_ex2(m - y);
          m = y;
        }
        if (m != -INFINITY) s += ce_ex2(y - m);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      merge(m, s, m2, s2);
    }
    if (lane == 0) {
      s_m[warp] = m;
      s_s[warp] = s;
    }
    __syncthreads();
    if (warp == 0) {
      m = lane < kCeThreads / 32 ? s_m[lane] : -INFINITY;
      s = lane < kCeThreads / 32 ? s_s[lane] : 0.f;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        merge(m, s, m2, s2);
      }
      if (lane == 0) {
        const float lse2 = m + log2f(s);          // log2 of the sum of 2^y; +inf / nan rows propagate as they are
        s_lse2 = lse2;
        a.loss_rows[row] = (lse2 - E::to_float(x[t]) * kLog2e) * kLn2;
      }
    }
    __syncthreads();
    const float lse2 = s_lse2;
    const float shift = log2f(scale) - lse2;       // scale > 0 whenever a row counts
    // ---- pass 2: gradient of the mean loss ------------------------------------------------------------------------
    if constexpr (kVec) {
      const int tc = static_cast<int>(t) / V, tj = static_cast<int>(t) % V;
#pragma unroll 2
      for (int c = threadIdx.x; c < a.cols / V; c += kCeThreads) {
        uint4 raw;
        if constexpr (kStage) raw = s_row[c];
        else raw = reinterpret_cast<const uint4*>(x)[c];
        const T* e = reinterpret_cast<const T*>(&raw);
        float p[V];                                 // softmax * scale: the scale rides in the exponent
#pragma unroll
        for (int j = 0; j < V; ++j) p[j] = ce_ex2(fmaf(E::to_float(e[j]), kLog2e, shift));
        if (c == tc) {
#pragma unroll
          for (int j = 0; j < V; ++j)
            if (j == tj) p[j] -= scale;
        }
        uint4 out;
        T* o = reinterpret_cast<T*>(&out);
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = E::from_float(p[j]);
        reinterpret_cast<uint4*>(dx)[c] = out;
      }
    } else {
      for (int c = threadIdx.x; c < a.cols; c += kCeThreads) {
        float p = ce_ex2(fmaf(E::to_float(x[c]), kLog2e, -lse2));
        if (c == t) p -= 1.f;
        dx[c] = E::from_float(p * scale);
      }
    }
    __syncthreads();                              // s_lse2 and the per-warp slots are reused by the next row
  }
}

template <int kDtype>
__global__ void __launch_bounds__(256) scale_unless_one_kernel(void* x_v, const float* factor, int64_t n) {
  using E = Elem<kDtype>;
  using T = typename E::type;
  constexpr int V = E::kPerVec;
  const float f = *factor;
  if (f == 1.f) return;                           // the usual case (gradient of a loss that is the graph's output)
  T* x = static_cast<T*>(x_v);
  const int64_t stride = gridDim.x * 256ll, first = blockIdx.x * 256ll + threadIdx.x;
  int64_t head = 0;                               // elements before the first 16-byte boundary
  while ((reinterpret_cast<uintptr_t>(x + head) & 15) != 0 && head < n) ++head;
  const int64_t nvec = (n - head) / V;
  for (int64_t i = first; i < nvec; i += stride) {
    uint4 raw = reinterpret_cast<uint4*>(x + head)[i];
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int j = 0; j < V; ++j) e[j] = E::from_float(E::to_float(e[j]) * f);
    reinterpret_cast<uint4*>(x + head)[i] = raw;
  }
  const int64_t body_end = head + nvec * V;       // the few elements outside the vector body
  for (int64_t i = first; i < head + (n - body_end); i += stride) {
    const int64_t at = i < head ? i : body_end + (i - head);
    x[at] = E::from_float(E::to_float(x[at]) * f);
  }
}

template <int kDtype>
cudaError_t launch_ce_t(const CrossEntropyArgs& a, int sms, cudaStream_t stream) {
  using T = typename Elem<kDtype>::type;
  constexpr int V = Elem<kDtype>::kPerVec;
  const bool vec = a.cols % V == 0 && a.ld % V == 0 && a.ld_out % V == 0 &&
                   reinterpret_cast<uintptr_t>(a.logits) % 16 == 0 && reinterpret_cast<uintptr_t>(a.dlogits) % 16 == 0;
  const int64_t row_bytes = static_cast<int64_t>(a.cols) * sizeof(T);
  const int per_sm = 2;                                       // rows in flight per SM: staged, or re-read through L2
  const int grid = a.rows < sms * per_sm ? a.rows : sms * per_sm;
  if (vec && row_bytes <= kCeStageBytes) {
    static PerDeviceFlags flags;
    const cudaError_t e = ensure_dynamic_smem(cross_entropy_kernel<kDtype, true, true>, kCeStageBytes, flags);
    if (e != cudaSuccess) return e;
    cross_entropy_kernel<kDtype, true, true><<<grid, kCeThreads, row_bytes, stream>>>(a);
  } else if (vec) {
    cross_entropy_kernel<kDtype, true, false><<<grid, kCeThreads, 0, stream>>>(a);
  } else {
    cross_entropy_kernel<kDtype, false, false><<<grid, kCeThreads, 0, stream>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_cross_entropy(const CrossEntropyArgs& a, int dtype, int sms, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  switch (dtype) {
    case 0: return launch_ce_t<0>(a, sms, stream);
    case 1: return launch_ce_t<1>(a, sms, stream);
    case 2: return launch_ce_t<2>(a, sms, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_scale_unless_one(void* x, const float* factor, int64_t n, int dtype, int sms, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const int64_t want = (n + 255) / 256;
  const int grid = static_cast<int>(want < sms * 32ll ? want : sms * 32ll);
  switch (dtype) {
    case 0: scale_unless_one_kernel<0><<<grid, 256, 0, stream>>>(x, factor, n); break;
    case 1: scale_unless_one_kernel<1><<<grid, 256, 0, stream>>>(x, factor, n); break;
    case 2: scale_unless_one_kernel<2><<<grid, 256, 0, stream>>>(x, factor, n); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace rbf
