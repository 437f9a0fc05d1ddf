// Host-side construction of TMA tensor maps for (B, H, N, D) tensors with unit stride on D.
// The driver entry point is resolved through the CUDA runtime, so the library has no link-time
// dependency on libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rbf {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// Tensor map over a 16-bit (B, H, N, D) tensor; strides in elements for dims b, h, n. The box is
// 64 elements (128 bytes, the swizzle span) along D by `box_rows` along N.
// Returns 0 on success, otherwise a CUresult (or -1 when the entry point is missing).
inline int make_tmap_bhnd(CUtensorMap* out, const void* base, bool bf16, int B, int H, int N, int D,
                          int64_t sb, int64_t sh, int64_t sn, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  // A dimension of extent 1 can carry any stride in the caller's tensor; give it a harmless one.
  if (N == 1) sn = D;
  if (H == 1) sh = static_cast<int64_t>(N) * sn;
  if (B == 1) sb = static_cast<int64_t>(H) * sh;
  cuuint64_t gdim[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t gstr[3] = {static_cast<cuuint64_t>(sn) * 2, static_cast<cuuint64_t>(sh) * 2,
                        static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

// Tensor map over a contiguous 16-bit (rows_total / n_pad, n_pad, 16) array of "bias slabs": 16 elements (32 bytes)
// per row, loaded as a 16 x `box_rows` box with the 32-byte swizzle (an extra K = 16 step of an MMA).
inline int make_tmap_slab16(CUtensorMap* out, const void* base, bool bf16, int BH, int n_pad, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  cuuint64_t gdim[3] = {16, static_cast<cuuint64_t>(n_pad), static_cast<cuuint64_t>(BH)};
  cuuint64_t gstr[2] = {32, static_cast<cuuint64_t>(n_pad) * 32};
  cuuint32_t box[3] = {16, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                   const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

// Tensor map over an fp32 (B, H, N, D) tensor with unit stride on D; strides in elements for dims b, h, n. The box is
// 32 floats (128 bytes, the swizzle span) along D by `box_rows` along N.
inline int make_tmap_bhnd_f32(CUtensorMap* out, const void* base, int B, int H, int N, int D, int64_t sb, int64_t sh,
                              int64_t sn, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  if (N == 1) sn = D;
  if (H == 1) sh = static_cast<int64_t>(N) * sn;
  if (B == 1) sb = static_cast<int64_t>(H) * sh;
  cuuint64_t gdim[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t gstr[3] = {static_cast<cuuint64_t>(sn) * 4, static_cast<cuuint64_t>(sh) * 4,
                        static_cast<cuuint64_t>(sb) * 4};
  cuuint32_t box[4] = {32, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

// Bias slabs for the TF32 kernel: a contiguous fp32 (rows_total / n_pad, n_pad, 8) array, 8 floats (32 bytes) per row.
inline int make_tmap_slab8_f32(CUtensorMap* out, const void* base, int BH, int n_pad, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  cuuint64_t gdim[3] = {8, static_cast<cuuint64_t>(n_pad), static_cast<cuuint64_t>(BH)};
  cuuint64_t gstr[2] = {32, static_cast<cuuint64_t>(n_pad) * 32};
  cuuint32_t box[3] = {8, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

// Tensor map over a contiguous fp32 (B, H, N, D) accumulator; box = 32 floats (128 bytes) x `box_rows`.
inline int make_tmap_f32_bhnd(CUtensorMap* out, const void* base, int B, int H, int N, int D, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  cuuint64_t gdim[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t gstr[3] = {static_cast<cuuint64_t>(D) * 4, static_cast<cuuint64_t>(N) * D * 4,
                        static_cast<cuuint64_t>(H) * N * D * 4};
  cuuint32_t box[4] = {32, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

// Tensor map over a transposed contiguous fp32 accumulator (B, H, D, n_pad): queries innermost. The box is
// 32 queries (128 bytes, the swizzle span) by `box_rows` head-dim rows.
inline int make_tmap_f32_bhdn(CUtensorMap* out, const void* base, int B, int H, int n_pad, int D, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  cuuint64_t gdim[4] = {static_cast<cuuint64_t>(n_pad), static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t gstr[3] = {static_cast<cuuint64_t>(n_pad) * 4, static_cast<cuuint64_t>(n_pad) * D * 4,
                        static_cast<cuuint64_t>(H) * n_pad * D * 4};
  cuuint32_t box[4] = {32, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

}  // namespace rbf
