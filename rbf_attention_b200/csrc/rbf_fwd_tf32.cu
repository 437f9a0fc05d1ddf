// RBF attention forward for fp32 inputs on TF32 tensor-core operands (sm_100a, head dim 64).
//
// The reference runs fp32 tensors through its Triton kernels with TF32 dot products (rbf_attention.py:183, 201; its
// parity script does so for its second dtype, test_equivalence.py:124-125). This kernel is that path: operands keep
// fp32's exponent range (the 16-bit kernels do not: fp16 overflows at 65504), the tensor core reads the upper 19 bits
// of every operand (10-bit significand, like fp16; Q and K are truncated to it, P and V rounded), accumulation is fp32. It is a plain pipeline, not tuned like the
// 16-bit kernels: fp32 activations are what tests and debugging runs use, not what training streams.
//
// One CTA owns 128 query rows of one (batch, head) and walks the key tiles of 64 keys:
//   warps 0-3  softmax (thread = query row): scores from TMEM, online softmax in base 2 with the lazy rescale of the
//              16-bit kernel, P written back to TMEM as TF32, output stage
//   warp 4     one thread loads (TMA, two-stage K / V ring with the key-norm bias slabs) and issues the MMAs:
//              S = Q K_j^T (8 steps of K = 8, smem x smem) + one bias-slab step, O += P V_j (TMEM x smem)
// kind::tf32 takes K-major operands only (an N-major V descriptor is accepted and multiplies by zero, measured), so
// the softmax threads also transpose every V tile in shared memory ([key][d] as the load leaves it -> [d][key]).
// S(j+1) is issued right after O += P V_j, so it runs under the exponentials of tile j + 1.
// TMEM columns: S [0, 64), P [64, 128), O [128, 192).
#include "common.cuh"
#include "launch.h"

namespace rbf {

namespace fwd32 {

static constexpr int D = 64;
static constexpr int kKeys = 64;                        // keys per streamed tile
static constexpr int kThreads = 160;
static constexpr int kIssueWarp = 4;
static constexpr int kStages = 2;
static constexpr float kRescaleThreshold = 8.0f;
static constexpr int kBoxBytes = kTile * 128;           // 16 KB: 128 rows x 32 floats
static constexpr int kQBytes = 2 * kBoxBytes;           // query / output tile: two boxes
static constexpr int kKvBoxBytes = kKeys * 128;         // 8 KB: 64 rows x 32 floats
static constexpr int kKvBytes = 2 * kKvBoxBytes;
static constexpr int kSlabBytes = kKeys * 32;           // 64 rows x 8 floats

struct Smem {
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kQBytes;
  static constexpr int kV = kK + kStages * kKvBytes;
  static constexpr int kVt = kV + kStages * kKvBytes;       // one transposed V tile: [64 d][64 keys] as two boxes
  static constexpr int kKSlab = kVt + kKvBytes;
  static constexpr int kOnes = kKSlab + kStages * kSlabBytes;
  static constexpr int kBars = kOnes + kTile * 32;
  static constexpr int kNumBars = 1 + 3 * kStages + 4;
  static constexpr int kMisc = kBars + kNumBars * 8;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

enum Site : uint32_t {
  kSiteQFull = 160, kSiteKvFull, kSiteStageFree, kSiteSFull, kSitePFull, kSiteODone, kSiteGroup, kSiteVFull
};

// Instruction descriptor for kind::tf32: D format f32 (1) at [4,6), A and B formats tf32 (2) at [7,10) and [10,13),
// major-ness bits 15 / 16, N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ void umma_ss_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t y;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y) : "f"(x));
  return y;
}

template <bool kSoftmax>
__global__ void __launch_bounds__(kThreads, 1)
rbf_fwd_tf32_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                    const __grid_constant__ CUtensorMap tm_kslab, const float* __restrict__ qsq,
                    float* __restrict__ lse, DeviceStatus* status, int H, int N, int n_pad, int causal, float scale2) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem + Smem::kQ;
  uint8_t* s_k = smem + Smem::kK;
  uint8_t* s_v = smem + Smem::kV;
  uint8_t* s_vt = smem + Smem::kVt;
  uint8_t* s_kslab = smem + Smem::kKSlab;
  uint8_t* s_ones = smem + Smem::kOnes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                   // [kStages] K tile + slab landed
  uint64_t* v_full = k_full + kStages;           // [kStages]
  uint64_t* stage_free = v_full + kStages;       // [kStages] the MMAs that read the stage have completed
  uint64_t* s_full = stage_free + kStages;
  uint64_t* p_full = s_full + 1;                 // 4 arrivals: the softmax warps have written P (and read S)
  uint64_t* o_done = p_full + 1;
  uint64_t* grp_sync = o_done + 1;               // 4 arrivals
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + Smem::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::kMisc + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int bh = blockIdx.y;
  const int b = bh / H, h = bh % H;
  const int mb = causal ? (static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)) : static_cast<int>(blockIdx.x);
  const int r0 = mb * kTile;
  const int n_key_tiles_all = (N + kKeys - 1) / kKeys;
  const int nkt = causal ? min(n_key_tiles_all, (r0 + kTile) / kKeys) : n_key_tiles_all;

  auto load_stage = [&](int j) {
    const int st = j % kStages;
    mbar_arrive_expect_tx(&k_full[st], kKvBytes + kSlabBytes);
    for (int x = 0; x < 2; ++x)
      tma_load_4d(s_k + st * kKvBytes + x * kKvBoxBytes, &tm_k, &k_full[st], x * 32, j * kKeys, h, b);
    tma_load_3d(s_kslab + st * kSlabBytes, &tm_kslab, &k_full[st], 0, j * kKeys, bh);
    mbar_arrive_expect_tx(&v_full[st], kKvBytes);
    for (int x = 0; x < 2; ++x)
      tma_load_4d(s_v + st * kKvBytes + x * kKvBoxBytes, &tm_v, &v_full[st], x * 32, j * kKeys, h, b);
  };
  if (tid == kIssueWarp * 32) {
    const unsigned int earlier = *reinterpret_cast<volatile unsigned int*>(&status->code);
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&stage_free[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    mbar_init(grp_sync, 4);
    fence_mbar_init();
    *abort_flag = earlier != 0u ? 1 : 0;
    if (earlier == 0u) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_kslab);
      mbar_arrive_expect_tx(q_full, kQBytes);
      for (int x = 0; x < 2; ++x) tma_load_4d(s_q + x * kBoxBytes, &tm_q, q_full, x * 32, r0, h, b);
      for (int j = 0; j < nkt && j < kStages; ++j) load_stage(j);
    }
  }
  if (warp == 0) {
    tmem_alloc(tmem_base_s, 256);
    tmem_relinquish();
  }
  if (tid < kTile) {
    // slab of constants: every row [1, 1, 1, 0 | 1, 1, 1, 0] (fp32); both 16-byte halves are equal, so the 32-byte
    // swizzle leaves it unchanged, and the key slabs hold zeros in elements 3-7
    *reinterpret_cast<float4*>(s_ones + tid * 32) = make_float4(1.f, 1.f, 1.f, 0.f);
    *reinterpret_cast<float4*>(s_ones + tid * 32 + 16) = make_float4(1.f, 1.f, 1.f, 0.f);
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_base_s;
  if (*abort_flag) {
    if (warp == 0) tmem_dealloc(tmem, 256);
    return;
  }
  const uint32_t tmem_s = tmem, tmem_p = tmem + 64, tmem_o = tmem + 128;

  if (warp == kIssueWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_tf32(kTile, kKeys, false, false);   // S = Q K^T, both K-major
      constexpr uint32_t idesc_o = make_idesc_tf32(kTile, D, false, false);       // O += P V^T^T: V^T is K-major
      const SmemDesc q_desc = make_sdesc_parts(smem_u32(s_q), 16, 1024);
      const SmemDesc k_desc0 = make_sdesc_parts(smem_u32(s_k), 16, 1024);
      const SmemDesc vt_desc = make_sdesc_parts(smem_u32(s_vt), 16, 1024);
      const SmemDesc ones_desc = make_sdesc_slab32(smem_u32(s_ones));
      const SmemDesc kslab_desc0 = make_sdesc_slab32(smem_u32(s_kslab));
      auto issue_s = [&](int st) {
        SmemDesc k_desc = k_desc0;
        k_desc.lo += static_cast<uint32_t>(st) * (kKvBytes >> 4);
        SmemDesc slab = kslab_desc0;
        slab.lo += static_cast<uint32_t>(st) * (kSlabBytes >> 4);
        // 64 fp32 columns = two boxes of 128-byte rows; a K step of 8 elements is 32 bytes
#pragma unroll
        for (int kk = 0; kk < D / 8; ++kk)
          umma_ss_tf32(tmem_s, sdesc_at(q_desc, (kk >> 2) * kBoxBytes + (kk & 3) * 32),
                       sdesc_at(k_desc, (kk >> 2) * kKvBoxBytes + (kk & 3) * 32), idesc_s, kk > 0);
        umma_ss_tf32(tmem_s, sdesc_at(ones_desc, 0), sdesc_at(slab, 0), idesc_s, 1u);   // + key-norm bias
        umma_commit(s_full);
      };
      bool ok = nkt > 0 && mbar_wait(q_full, 0, abort_flag, status, kSiteQFull) &&
                mbar_wait(&k_full[0], 0, abort_flag, status, kSiteKvFull);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0);
      }
      for (int j = 0; j < nkt && ok; ++j) {
        const int st = j % kStages;
        // p_full: P of tile j is in TMEM and the transposed V tile in shared memory
        ok = mbar_wait(p_full, j & 1, abort_flag, status, kSitePFull);
        if (!ok) break;
        tc_fence_after_sync();
        // a K step is 8 keys: 8 TMEM columns of P, 32 bytes of the K-major V^T rows (two boxes of 32 keys)
#pragma unroll
        for (int kk = 0; kk < kKeys / 8; ++kk)
          umma_ts_tf32(tmem_o, tmem_p + kk * 8, sdesc_at(vt_desc, (kk >> 2) * kKvBoxBytes + (kk & 3) * 32), idesc_o,
                       (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(o_done);
        umma_commit(&stage_free[st]);
        if (j + 1 < nkt) {
          // the scores were read before P was written, so S may be overwritten now
          ok = mbar_wait(&k_full[(j + 1) % kStages], ((j + 1) / kStages) & 1, abort_flag, status, kSiteKvFull);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s((j + 1) % kStages);
        }
        if (j + kStages < nkt) {
          ok = mbar_wait(&stage_free[st], (j / kStages) & 1, abort_flag, status, kSiteStageFree);
          if (!ok) break;
          load_stage(j + kStages);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax (thread = query row)
    const int r = tid;
    const int row = r0 + r;
    const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
    float m_used = -INFINITY;
    float l_sum = 0.f;
    float row_bias = 0.f;
    if (!kSoftmax && nkt > 0) row_bias = qsq[static_cast<int64_t>(bh) * n_pad + row];
    bool ok = true;
    for (int j = 0; j < nkt; ++j) {
      ok = mbar_wait(s_full, j & 1, abort_flag, status, kSiteSFull);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t raw[kKeys];
      tmem_ld_x32(tmem_s + lane_sel, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
      tmem_ld_x32(tmem_s + lane_sel + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
      tmem_ld_wait();
      if (causal && (j + 1) * kKeys > r0 + 1) {
        const int c_max = r0 + r - j * kKeys;   // last visible column of this row
#pragma unroll
        for (int c = 0; c < kKeys; ++c)
          if (c > c_max) raw[c] = 0xff800000u;   // -inf
      }
      float sub;
      if constexpr (kSoftmax) {
        float mx = __uint_as_float(raw[0]);
#pragma unroll
        for (int c = 1; c < kKeys; ++c) mx = fmaxf(mx, __uint_as_float(raw[c]));
        const float m_new = fmaxf(m_used, mx * scale2);
        const bool need = (m_new - m_used) > kRescaleThreshold;
        float alpha = 1.f;
        if (need) {
          alpha = ex2_approx(m_used - m_new);
          m_used = m_new;
          l_sum *= alpha;
        }
        if (j > 0 && __any_sync(0xffffffffu, need)) {
          ok = mbar_wait(o_done, (j - 1) & 1, abort_flag, status, kSiteODone);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_x32(tmem_o + lane_sel + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(tmem_o + lane_sel + c * 32, o);
          }
        }
        sub = m_used;
      } else {
        sub = row_bias;
      }
      float ps = 0.f;
#pragma unroll
      for (int c = 0; c < kKeys; ++c) {
        const float p = ex2_approx(fmaf(__uint_as_float(raw[c]), scale2, -sub));
        ps += p;
        raw[c] = to_tf32(p);
      }
      l_sum += ps;
      // P's columns are free once O += P V of the previous tile has completed
      if (j > 0) {
        ok = mbar_wait(o_done, (j - 1) & 1, abort_flag, status, kSiteODone);
        if (!ok) break;
        tc_fence_after_sync();
      }
      tmem_st_x32(tmem_p + lane_sel, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));
      tmem_st_x32(tmem_p + lane_sel + 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[32]));
      // transpose the V tile: V[key][d] (two boxes of 32 d) -> V^T[d][key] (two boxes of 32 keys), both in the
      // 128-byte swizzle; thread = (key, half of the d chunks); the previous tile's MMAs have released V^T (o_done)
      {
        const int st = j % kStages;
        ok = mbar_wait(&v_full[st], (j / kStages) & 1, abort_flag, status, kSiteVFull);
        if (!ok) break;
        const int key = tid & 63, half = tid >> 6;
        const uint8_t* src = s_v + st * kKvBytes;
        // element (d, key) of V^T: box key / 32, row d, 16-byte chunk (key mod 32) / 4 XOR-ed with d mod 8
        uint8_t* dst_box = s_vt + (key >> 5) * kKvBoxBytes + (key & 3) * 4;
        const uint32_t dst_chunk = (key & 31) >> 2;
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          const int c = half * 8 + cc;                      // 16-byte chunk of the V row: d = 4c .. 4c + 3
          const float4 x = *reinterpret_cast<const float4*>(src + (c >> 3) * kKvBoxBytes + sw128_offset(key, c & 7));
          const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int i = 0; i < 4; ++i)      // rounded to TF32 here (the tensor core would truncate)
            *reinterpret_cast<uint32_t*>(dst_box + sw128_offset(4 * c + i, dst_chunk)) = to_tf32(xs[i]);
        }
        fence_proxy_async_smem();
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive_warp(p_full);
    }
    if (ok && nkt > 0) ok = mbar_wait(o_done, (nkt - 1) & 1, abort_flag, status, kSiteODone);
    if (ok && nkt > 0) {
      tc_fence_after_sync();
      const float inv = kSoftmax ? (1.0f / l_sum) : 1.0f;
      uint8_t* stage = s_q;                       // Q is dead once the last S MMA has completed
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_x32(tmem_o + lane_sel + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g)                // box c, 16-byte chunk g of row r
          *reinterpret_cast<float4*>(stage + c * kBoxBytes + sw128_offset(r, g)) =
              make_float4(__uint_as_float(o[4 * g]) * inv, __uint_as_float(o[4 * g + 1]) * inv,
                          __uint_as_float(o[4 * g + 2]) * inv, __uint_as_float(o[4 * g + 3]) * inv);
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(grp_sync);
      ok = mbar_wait(grp_sync, 0, abort_flag, status, kSiteGroup);
      if (ok && r == 0) {
        for (int x = 0; x < 2; ++x) tma_store_4d(&tm_o, stage + x * kBoxBytes, x * 32, r0, h, b);
        tma_store_commit();
        tma_store_wait_read();
      }
      if (kSoftmax && row < N) lse[static_cast<int64_t>(bh) * N + row] = m_used + log2f(l_sum);
    }
  }

  if (*abort_flag) {
    // give copies and MMAs still in flight time to land before shared memory and TMEM are released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace fwd32

template <bool kSoftmax>
static cudaError_t launch_fwd_tf32_t(const FwdArgs& a, cudaStream_t stream) {
  auto kernel = fwd32::rbf_fwd_tf32_kernel<kSoftmax>;
  constexpr int smem = fwd32::Smem::kDynamic;
  static PerDeviceFlags configured{};
  {
    const cudaError_t ce = ensure_dynamic_smem(kernel, smem, configured);
    if (ce != cudaSuccess) return ce;
  }
  dim3 grid((a.N + kTile - 1) / kTile, a.B * a.H);
  kernel<<<grid, fwd32::kThreads, smem, stream>>>(a.tm_q, a.tm_k, a.tm_v, a.tm_o, a.tm_kslab, a.qsq, a.lse, a.status,
                                                 a.H, a.N, a.n_pad, a.causal, a.scale2);
  return cudaGetLastError();
}

cudaError_t launch_fwd_tf32(const FwdArgs& a, bool softmax, cudaStream_t stream) {
  return softmax ? launch_fwd_tf32_t<true>(a, stream) : launch_fwd_tf32_t<false>(a, stream);
}

}  // namespace rbf
