// Single-kernel backward of the softmax RBF attention for head dim 128 (sm_100a).
//
// Same data flow as the head-dim-64 kernel (rbf_bwd_fused.cu): a CTA owns 128 keys (K, V resident in shared
// memory), streams the queries past them, issues the five algorithmic MMAs per step and evaluates every
// exponential once. With D = 128 the two resident accumulators dV and dK already take half of TMEM, so the
// queries are streamed in steps of 64 and dQ is produced transposed:
//   S^T  [128 keys x 64 q] = K Q^T  (+ bias slab: -L[query] / scale)      smem x smem
//   dP^T [128 keys x 64 q] = V dO^T (+ bias slab: -delta[query])          smem x smem
//   P^T = exp2(S^T * 2c - ksq[key]),  dS^T = P^T * dP^T                   (registers; thread = key row)
//   dV  [128 x 128] += P^T dO          TMEM x smem (P^T: 32 TMEM columns of 16-bit pairs)
//   dK  [128 x 128] += dS^T Q          TMEM x smem (dS^T: 32 TMEM columns of 16-bit pairs)
//   dQ^T[128 d x 64 q] = K^T dS^T      smem x smem (K read M-major; dS^T a second time, as a [key][query]
//                                      shared-memory tile of 128-byte rows read N-major)
// dQ^T leaves the CTA straight from registers: a drain thread owns one head-dim index, so for every query of the
// step the 32 lanes of a warp hold 32 consecutive floats of the (B, H, N, D) fp32 accumulator and one scalar
// red.global.add per query is a coalesced 128-byte line. No shared-memory staging: shared-memory bandwidth is
// what bounds this kernel (the MMA operand fetch alone runs at about 120 of the 128 bytes per clock). A small
// kernel scales and converts the accumulator afterwards. (Every SM can push about 25 bytes per clock of
// reduce-adds into L2, measured; a step's 32 KB of dQ therefore takes as long as its MMAs and must overlap them.)
//
// TMEM columns: S^T [0,64), dP^T [64,128), P^T [128,160), dQ^T [160,224), dS^T [224,256), dV [256,384), dK [384,512).
// Roles: warps 0, 1, 3 MMA issuers (A: S^T(n+1), dV(n); B: dP^T(n+1), dK(n); C: dQ^T(n)), warp 2 TMA producer,
// warps 4-19 compute (thread = key row, group g owns query columns [16g, 16g+16) of the step), warps 20-23 drain
// dQ^T (thread = head-dim index).
#include "common.cuh"
#include "launch.h"

namespace rbf {

namespace bwdf128 {


static constexpr int D = 128;
static constexpr int kQStep = 64;                   // queries per step
static constexpr int kThreads = 768;
static constexpr int kNumComputeWarps = 16;
static constexpr int kMmaWarpA = 0;
static constexpr int kMmaWarpB = 1;
static constexpr int kLoadWarp = 2;
static constexpr int kMmaWarpC = 3;
static constexpr int kComputeWarp0 = 4;
static constexpr int kDrainWarp0 = 20;
// setmaxnreg only redistributes the launch allocation (80 per thread): 512 * 96 + 128 * 40 + 128 * 56 = 768 * 80.
static constexpr int kComputeRegs = 96;
static constexpr int kOtherRegs = 40;
static constexpr int kDrainRegs = 56;
static_assert(512 * kComputeRegs + 128 * kOtherRegs + 128 * kDrainRegs <= 768 * 80, "setmaxnreg budget");

static constexpr int kBoxBytes = kTile * 128;             // 16 KB: 128 rows x 64 16-bit columns
static constexpr int kKvBytes = 2 * kBoxBytes;            // K or V tile: two 64-column boxes
static constexpr int kQBoxBytes = kQStep * 128;           // 8 KB: 64 rows x 64 columns
static constexpr int kQTileBytes = 2 * kQBoxBytes;        // Q or dO step tile
static constexpr int kSlabBytes = kQStep * 32;            // 2 KB: 64 rows x 16 x 16-bit
static constexpr int kOnesBytes = kTile * 32;
static constexpr int kQStages = 3;
static constexpr int kDoStages = 3;
static constexpr int kDsBytes = kTile * 128;              // 16 KB: dS^T as [128 keys][64 queries]; two buffers
static constexpr int kDsStages = 2;

struct Smem {
  static constexpr int kK = 0;
  static constexpr int kV = kK + kKvBytes;
  static constexpr int kQ = kV + kKvBytes;
  static constexpr int kDo = kQ + kQStages * kQTileBytes;
  static constexpr int kDs = kDo + kDoStages * kQTileBytes;
  static constexpr int kLSlab = kDs + kDsStages * kDsBytes;
  static constexpr int kDSlab = kLSlab + kQStages * kSlabBytes;
  static constexpr int kOnes = kDSlab + kDoStages * kSlabBytes;
  static constexpr int kRowsum = kOnes + kOnesBytes;         // [4 groups][128] floats
  static constexpr int kBars = kRowsum + 4 * kTile * 4;
  static constexpr int kNumBars = 1 + 2 * kQStages + 2 * kDoStages + 2 * kDsStages + 11;
  static constexpr int kMisc = kBars + kNumBars * 8;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};
static_assert(Smem::kDynamic <= 232448, "shared memory budget");

static constexpr int kColS = 0, kColDP = 64, kColPT = 128, kColDQ = 160, kColDST = 224, kColDV = 256, kColDK = 384;

enum Site : uint32_t {
  kSiteKV = 96, kSiteQFull, kSiteDoFull, kSiteQEmpty, kSiteDoEmpty, kSiteSFull, kSiteDPFull, kSitePFull, kSiteDSFull,
  kSiteDQFull, kSiteDQDrained, kSiteAccDone, kSiteGroup, kSiteSConsumed, kSiteDPConsumed, kSiteDVDone, kSiteDsFree,
  kSiteDrain
};

struct Params {
  float* dq_acc;         // fp32 (B, H, N, 128), zero-initialised
  DeviceStatus* status;
  int H, N, n_pad, causal;
  float scale2, grad_scale, slab_w;
};

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
rbf_bwd_fused128_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                        const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                        const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                        const __grid_constant__ CUtensorMap tm_lslab, const __grid_constant__ CUtensorMap tm_dslab,
                        const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_k = smem + Smem::kK;
  uint8_t* s_v = smem + Smem::kV;
  uint8_t* s_q = smem + Smem::kQ;
  uint8_t* s_do = smem + Smem::kDo;
  uint8_t* s_ds = smem + Smem::kDs;
  uint8_t* s_lslab = smem + Smem::kLSlab;
  uint8_t* s_dslab = smem + Smem::kDSlab;
  uint8_t* s_ones = smem + Smem::kOnes;
  float* s_rowsum = reinterpret_cast<float*>(smem + Smem::kRowsum);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint64_t* kv_full = bars;
  uint64_t* q_full = kv_full + 1;            // [kQStages] Q step tile + L slab landed
  uint64_t* q_empty = q_full + kQStages;     // two arrivals: S^T (issuer A) and dK (issuer B) have completed
  uint64_t* do_full = q_empty + kQStages;    // [kDoStages] dO step tile + delta slab landed
  uint64_t* do_empty = do_full + kDoStages;  // two arrivals: dV (issuer A) and dP^T (issuer B)
  uint64_t* s_full = do_empty + kDoStages;
  uint64_t* s_consumed = s_full + 1;
  uint64_t* dp_full = s_consumed + 1;
  uint64_t* dp_consumed = dp_full + 1;
  uint64_t* p_full = dp_consumed + 1;
  uint64_t* dv_done = p_full + 1;
  uint64_t* ds_full = dv_done + 1;           // [kDsStages] the dS^T tile of a step is written
  uint64_t* ds_free = ds_full + kDsStages;   // [kDsStages] dQ^T (issuer C) has read the shared-memory tile
  uint64_t* dq_full = ds_free + kDsStages;   // dQ^T of the step is complete in TMEM
  uint64_t* dq_drained = dq_full + 1;
  uint64_t* acc_done = dq_drained + 1;       // three arrivals
  uint64_t* grp_sync = acc_done + 1;
  uint64_t* dk_done = grp_sync + 1;          // dK (issuer B) has read the TMEM copy of dS^T
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + Smem::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::kMisc + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int kt = blockIdx.x;                       // key tile; tile 0 is the heaviest under the causal mask
  const int k_row0 = kt * kTile;
  const int n_steps_all = (p.N + kQStep - 1) / kQStep;
  const int first = p.causal ? 2 * kt : 0;         // first 64-query step that sees these keys
  const int cnt = n_steps_all - first;

  // A wait that ran out in an earlier CTA of this launch ends the whole launch quickly: later CTAs leave at once.
  if (tid == 0) *abort_flag = (*reinterpret_cast<volatile unsigned int*>(&p.status->code) != 0u) ? 1 : 0;
  __syncthreads();
  if (*abort_flag) return;

  if (tid == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < kQStages; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 2); }
    for (int s = 0; s < kDoStages; ++s) { mbar_init(&do_full[s], 1); mbar_init(&do_empty[s], 2); }
    mbar_init(s_full, 1);
    mbar_init(s_consumed, kNumComputeWarps);   // one arrival per warp
    mbar_init(dp_full, 1);
    mbar_init(dp_consumed, kNumComputeWarps);
    mbar_init(p_full, kNumComputeWarps);
    mbar_init(dv_done, 1);
    for (int s = 0; s < kDsStages; ++s) { mbar_init(&ds_full[s], kNumComputeWarps); mbar_init(&ds_free[s], 1); }
    mbar_init(dk_done, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 4);
    mbar_init(acc_done, 3);
    mbar_init(grp_sync, kNumComputeWarps);
    fence_mbar_init();
  }
  if (warp == kMmaWarpA) {
    tmem_alloc(tmem_base_s, 512);
    tmem_relinquish();
  }
  if (tid < kTile) {
    // slab of constants (A operand of the bias-slab MMA steps): rows [w, w, w, 0 x5 | w, w, w, 0 x5]
    const uint4 v = make_uint4(pack2<kBf16>(p.slab_w, p.slab_w), pack2<kBf16>(p.slab_w, 0.f), 0u, 0u);
    *reinterpret_cast<uint4*>(s_ones + tid * 32) = v;
    *reinterpret_cast<uint4*>(s_ones + tid * 32 + 16) = v;
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_base_s;

  if (warp < kComputeWarp0) {
    setmaxnreg_dec<kOtherRegs>();
  }
  if (warp == kLoadWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_lslab);
      tma_prefetch_desc(&tm_dslab);
      mbar_arrive_expect_tx(kv_full, 2 * kKvBytes);
      for (int x = 0; x < 2; ++x) {
        tma_load_4d(s_k + x * kBoxBytes, &tm_k, kv_full, x * 64, k_row0, h, b);
        tma_load_4d(s_v + x * kBoxBytes, &tm_v, kv_full, x * 64, k_row0, h, b);
      }
      for (int n = 0; n < cnt; ++n) {
        const int row0 = (first + n) * kQStep;
        const int sq = n % kQStages, sd = n % kDoStages;
        if (n >= kQStages && !mbar_wait(&q_empty[sq], ((n / kQStages) - 1) & 1, abort_flag, p.status, kSiteQEmpty)) break;
        mbar_arrive_expect_tx(&q_full[sq], kQTileBytes + kSlabBytes);
        for (int x = 0; x < 2; ++x)
          tma_load_4d(s_q + sq * kQTileBytes + x * kQBoxBytes, &tm_q, &q_full[sq], x * 64, row0, h, b);
        tma_load_3d(s_lslab + sq * kSlabBytes, &tm_lslab, &q_full[sq], 0, row0, bh);
        if (n >= kDoStages && !mbar_wait(&do_empty[sd], ((n / kDoStages) - 1) & 1, abort_flag, p.status, kSiteDoEmpty)) break;
        mbar_arrive_expect_tx(&do_full[sd], kQTileBytes + kSlabBytes);
        for (int x = 0; x < 2; ++x)
          tma_load_4d(s_do + sd * kQTileBytes + x * kQBoxBytes, &tm_do, &do_full[sd], x * 64, row0, h, b);
        tma_load_3d(s_dslab + sd * kSlabBytes, &tm_dslab, &do_full[sd], 0, row0, bh);
      }
    }
  } else if (warp == kMmaWarpA || warp == kMmaWarpB || warp == kMmaWarpC) {
    // ------------------------------------------------------------------ MMA issuers
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(kTile, kQStep, kBf16, false, false);  // 128 keys x 64 queries, K-major both
      constexpr uint32_t idesc_acc = make_idesc(kTile, D, kBf16, false, true);      // dV, dK: B read N-major
      constexpr uint32_t idesc_dq = make_idesc(D, kQStep, kBf16, true, true);       // dQ^T: A M-major, B N-major
      const SmemDesc ones_desc = make_sdesc_slab32(smem_u32(s_ones));
      auto stage_of = [](SmemDesc d, int stage, uint32_t stage_bytes) {
        d.lo += static_cast<uint32_t>(stage) * (stage_bytes >> 4);
        return d;
      };
      // dst[128 x 64] = A B^T over D = 128 (A: two 16 KB boxes, B: two 8 KB boxes) plus the bias-slab step
      auto issue_scores = [&](uint32_t dst, const SmemDesc& a_desc, const SmemDesc& b_desc, const SmemDesc& slab) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_ss(dst, sdesc_at(a_desc, (kk >> 2) * kBoxBytes + (kk & 3) * 32),
                  sdesc_at(b_desc, (kk >> 2) * kQBoxBytes + (kk & 3) * 32), idesc_s, kk > 0);
        umma_ss(dst, sdesc_at(ones_desc, 0), sdesc_at(slab, 0), idesc_s, 1u);
      };
      auto wait_q = [&](int n) {
        return mbar_wait(&q_full[n % kQStages], (n / kQStages) & 1, abort_flag, p.status, kSiteQFull);
      };
      auto wait_do = [&](int n) {
        return mbar_wait(&do_full[n % kDoStages], (n / kDoStages) & 1, abort_flag, p.status, kSiteDoFull);
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kSiteKV);

      if (warp == kMmaWarpA) {
        const SmemDesc k_kmaj = make_sdesc_parts(smem_u32(s_k), 16, 1024);
        const SmemDesc q_kmaj0 = make_sdesc_parts(smem_u32(s_q), 16, 1024);
        const SmemDesc lslab0 = make_sdesc_slab32(smem_u32(s_lslab));
        const SmemDesc do_nmaj0 = make_sdesc_parts(smem_u32(s_do), kQBoxBytes, 1024);   // 64-column groups 8 KB apart
        if (ok) ok = wait_q(0);
        if (ok) {
          tc_fence_after_sync();
          issue_scores(tmem + kColS, k_kmaj, q_kmaj0, lslab0);
          umma_commit(s_full);
          umma_commit(&q_empty[0]);
        }
        for (int n = 0; n < cnt && ok; ++n) {
          if (n + 1 < cnt) {
            const int st = (n + 1) % kQStages;
            ok = wait_q(n + 1) && mbar_wait(s_consumed, n & 1, abort_flag, p.status, kSiteSConsumed);
            if (!ok) break;
            tc_fence_after_sync();
            issue_scores(tmem + kColS, k_kmaj, stage_of(q_kmaj0, st, kQTileBytes), stage_of(lslab0, st, kSlabBytes));
            umma_commit(s_full);
            umma_commit(&q_empty[st]);
          }
          // dV += P^T dO
          ok = mbar_wait(p_full, n & 1, abort_flag, p.status, kSitePFull);
          if (!ok) break;
          tc_fence_after_sync();
          const SmemDesc do_n = stage_of(do_nmaj0, n % kDoStages, kQTileBytes);
#pragma unroll
          for (int kk = 0; kk < kQStep / 16; ++kk)
            umma_ts(tmem + kColDV, tmem + kColPT + kk * 8, sdesc_at(do_n, kk * 2048), idesc_acc,
                    (n > 0 || kk > 0) ? 1u : 0u);
          umma_commit(dv_done);
          umma_commit(&do_empty[n % kDoStages]);
        }
      } else if (warp == kMmaWarpB) {
        const SmemDesc v_kmaj = make_sdesc_parts(smem_u32(s_v), 16, 1024);
        const SmemDesc do_kmaj0 = make_sdesc_parts(smem_u32(s_do), 16, 1024);
        const SmemDesc dslab0 = make_sdesc_slab32(smem_u32(s_dslab));
        const SmemDesc q_nmaj0 = make_sdesc_parts(smem_u32(s_q), kQBoxBytes, 1024);
        if (ok) ok = wait_do(0);
        if (ok) {
          tc_fence_after_sync();
          issue_scores(tmem + kColDP, v_kmaj, do_kmaj0, dslab0);
          umma_commit(dp_full);
          umma_commit(&do_empty[0]);
        }
        for (int n = 0; n < cnt && ok; ++n) {
          if (n + 1 < cnt) {
            const int st = (n + 1) % kDoStages;
            ok = wait_do(n + 1) && mbar_wait(dp_consumed, n & 1, abort_flag, p.status, kSiteDPConsumed);
            if (!ok) break;
            tc_fence_after_sync();
            issue_scores(tmem + kColDP, v_kmaj, stage_of(do_kmaj0, st, kQTileBytes), stage_of(dslab0, st, kSlabBytes));
            umma_commit(dp_full);
            umma_commit(&do_empty[st]);
          }
          // dK += dS^T Q
          ok = mbar_wait(&ds_full[n % kDsStages], (n / kDsStages) & 1, abort_flag, p.status, kSiteDSFull);
          if (!ok) break;
          tc_fence_after_sync();
          // A = the TMEM copy of dS^T (16-bit pairs, 32 columns): only Q is fetched from shared memory
          const SmemDesc q_n = stage_of(q_nmaj0, n % kQStages, kQTileBytes);
#pragma unroll
          for (int kk = 0; kk < kQStep / 16; ++kk)
            umma_ts(tmem + kColDK, tmem + kColDST + kk * 8, sdesc_at(q_n, kk * 2048), idesc_acc,
                    (n > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&q_empty[n % kQStages]);
          umma_commit(dk_done);
        }
      } else {
        // dQ^T = K^T dS^T : A = K tile read M-major (rows = keys = reduction index, 64-wide d groups 16 KB apart),
        // B = the dS^T tile read N-major
        const SmemDesc k_mmaj = make_sdesc_parts(smem_u32(s_k), kBoxBytes, 1024);
        const SmemDesc ds_nmaj = make_sdesc_parts(smem_u32(s_ds), kBoxBytes, 1024);
        for (int n = 0; n < cnt && ok; ++n) {
          ok = mbar_wait(&ds_full[n % kDsStages], (n / kDsStages) & 1, abort_flag, p.status, kSiteDSFull);
          if (ok && n > 0) ok = mbar_wait(dq_drained, (n - 1) & 1, abort_flag, p.status, kSiteDQDrained);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ss(tmem + kColDQ, sdesc_at(k_mmaj, kk * 2048),
                    sdesc_at(ds_nmaj, (n % kDsStages) * kDsBytes + kk * 2048), idesc_dq, kk > 0);
          umma_commit(dq_full);                    // dQ^T readable
          umma_commit(&ds_free[n % kDsStages]);    // the shared-memory tile's reader is done
        }
      }
      if (ok) umma_commit(acc_done);
    }
  } else if (warp >= kDrainWarp0) {
    // ------------------------------------------------------------------ dQ^T drain (thread = head-dim index)
    setmaxnreg_dec<kDrainRegs>();
    const int wq = warp & 3;                                // TMEM lane quadrant = 32 head-dim rows
    const uint32_t lane_sel = static_cast<uint32_t>(wq * 32) << 16;
    float* acc_col = p.dq_acc + static_cast<int64_t>(bh) * p.N * D + wq * 32 + lane;
    bool ok = true;
    for (int n = 0; n < cnt; ++n) {
      ok = mbar_wait(dq_full, n & 1, abort_flag, p.status, kSiteDQFull);
      if (!ok) break;
      tc_fence_after_sync();
      const int q0 = (first + n) * kQStep;
      const int valid = p.N - q0;                           // queries of this step inside the sequence
      float* dst = acc_col + static_cast<int64_t>(q0) * D;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t v[32];
        tmem_ld_x32(tmem + kColDQ + lane_sel + hh * 32, v);
        tmem_ld_wait();
        if (hh == 1) {
          tc_fence_before_sync();
          mbar_arrive_warp(dq_drained);   // the next dQ^T MMA may overwrite TMEM
        }
        if (valid >= kQStep) {
#pragma unroll
          for (int i = 0; i < 32; ++i) red_add_f32(dst + (hh * 32 + i) * D, __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (hh * 32 + i < valid) red_add_f32(dst + (hh * 32 + i) * D, __uint_as_float(v[i]));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute groups (thread = key row)
    setmaxnreg_inc<kComputeRegs>();
    const int g = (warp - kComputeWarp0) >> 2;             // 16-column slice of the query step
    const int r = tid & (kTile - 1);
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float ds_rowsum = 0.f;
    // c |k_r|^2 of this thread's key row, from the resident K tile; rows past N (zero-filled by the load) get
    // +infinity, i.e. weight exp2(-inf) = 0
    float neg_ksq = -INFINITY;
    bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kSiteKV);
    if (ok && k_row0 + r < p.N) {
      float acc = 0.f;
#pragma unroll 1
      for (int c16 = 0; c16 < D / 8; ++c16) {      // once per key tile: kept rolled, registers are scarce here
        const uint4 kv = *reinterpret_cast<const uint4*>(s_k + (c16 >> 3) * kBoxBytes + sw128_offset(r, c16 & 7));
        const uint32_t w[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 x = unpack2<kBf16>(w[i]);
          acc = fmaf(x.x, x.x, acc);
          acc = fmaf(x.y, x.y, acc);
        }
      }
      neg_ksq = -acc * (0.5f * p.scale2);
    }

    for (int n = 0; n < cnt && ok; ++n) {
      ok = mbar_wait(s_full, n & 1, abort_flag, p.status, kSiteSFull);
      if (!ok) break;
      tc_fence_after_sync();
      float pr[16];
      {
        uint32_t raw[16];
        tmem_ld_x16(tmem + kColS + lane_sel + g * 16, raw);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(s_consumed);
        // acc = k.q - L / scale2 ; P = exp2(acc * scale2 - ksq)
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          float a0, a1;
          ffma2_bcast(a0, a1, __uint_as_float(raw[i]), __uint_as_float(raw[i + 1]), p.scale2, neg_ksq);
          pr[i] = ex2_approx(a0);
          pr[i + 1] = ex2_approx(a1);
        }
      }
      const int q0 = (first + n) * kQStep;
      if (p.causal && q0 < k_row0 + kTile) {
        // steps that straddle the diagonal: query (q0 + 16g + c) sees key (k_row0 + r) iff query >= key
#pragma unroll
        for (int c = 0; c < 16; ++c)
          if (q0 + g * 16 + c < k_row0 + r) pr[c] = 0.f;
      }
      {
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) packed[i] = pack2<kBf16>(pr[2 * i], pr[2 * i + 1]);
        if (n > 0) {   // the P^T columns are free once dV of the previous step has completed
          ok = mbar_wait(dv_done, (n - 1) & 1, abort_flag, p.status, kSiteDVDone);
          if (!ok) break;
          tc_fence_after_sync();
        }
        tmem_st_x8(tmem + kColPT + lane_sel + g * 8, packed);
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(p_full);
      }

      ok = mbar_wait(dp_full, n & 1, abort_flag, p.status, kSiteDPFull);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t ds_packed[8];
      {
        uint32_t raw[16];
        tmem_ld_x16(tmem + kColDP + lane_sel + g * 16, raw);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(dp_consumed);
        // acc = v.dO - delta ; dS = P * acc
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float d0, d1;
          fmul2(d0, d1, pr[2 * i], pr[2 * i + 1], __uint_as_float(raw[2 * i]), __uint_as_float(raw[2 * i + 1]));
          fadd2(rs0, rs1, rs0, rs1, d0, d1);
          ds_packed[i] = pack2<kBf16>(d0, d1);
        }
        ds_rowsum += rs0 + rs1;
      }
      if (n >= kDsStages) {   // the dS^T buffer is free once dK and dQ^T of its previous step have completed
        ok = mbar_wait(&ds_free[n % kDsStages], ((n / kDsStages) - 1) & 1, abort_flag, p.status, kSiteDsFree);
        if (!ok) break;
      }
      // row r of the [key][query] tile: 16-byte chunks 2g and 2g + 1
#pragma unroll
      for (int ch = 0; ch < 2; ++ch)
        *reinterpret_cast<uint4*>(s_ds + (n % kDsStages) * kDsBytes + sw128_offset(r, g * 2 + ch)) =
            make_uint4(ds_packed[ch * 4 + 0], ds_packed[ch * 4 + 1], ds_packed[ch * 4 + 2], ds_packed[ch * 4 + 3]);
      fence_proxy_async_smem();
      // second copy for dK = dS^T Q, which takes its A operand from TMEM; free once dK of the previous step is done
      if (n > 0) {
        ok = mbar_wait(dk_done, (n - 1) & 1, abort_flag, p.status, kSiteDsFree);
        if (!ok) break;
        tc_fence_after_sync();
      }
      tmem_st_x8(tmem + kColDST + lane_sel + g * 8, ds_packed);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive_warp(&ds_full[n % kDsStages]);
    }

    uint32_t grp_phase = 0;
    auto group_sync = [&]() -> bool {
      mbar_arrive_warp(grp_sync);
      const bool done = mbar_wait(grp_sync, grp_phase & 1, abort_flag, p.status, kSiteGroup);
      ++grp_phase;
      return done;
    };
    if (ok) ok = mbar_wait(acc_done, 0, abort_flag, p.status, kSiteAccDone);
    if (ok) {
      tc_fence_after_sync();
      s_rowsum[g * kTile + r] = ds_rowsum;      // every group holds a quarter of rowsum(dS^T)
      ok = group_sync();
    }
    if (ok) {
      // groups 0, 1 finish dK (columns [64(g%2), +64)), groups 2, 3 store dV; the Q and dO rings are dead by now
      const bool is_dk = g < 2;
      const int half = g & 1;
      uint8_t* stage = s_q + ((is_dk ? 0 : 2) + half) * kBoxBytes;
      const float w = is_dk ? (s_rowsum[r] + s_rowsum[kTile + r]) + (s_rowsum[2 * kTile + r] + s_rowsum[3 * kTile + r])
                            : 0.f;
      const float out_scale = is_dk ? p.grad_scale : 1.0f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t acc[32];
        tmem_ld_x32(tmem + (is_dk ? kColDK : kColDV) + lane_sel + half * 64 + c * 32, acc);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t off = sw128_offset(r, c * 4 + q4);
          const uint4 k_raw = *reinterpret_cast<const uint4*>(s_k + half * kBoxBytes + off);
          const uint32_t kw[4] = {k_raw.x, k_raw.y, k_raw.z, k_raw.w};
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 kv = unpack2<kBf16>(kw[i]);
            const float x0 = out_scale * fmaf(-w, kv.x, __uint_as_float(acc[q4 * 8 + 2 * i]));
            const float x1 = out_scale * fmaf(-w, kv.y, __uint_as_float(acc[q4 * 8 + 2 * i + 1]));
            o[i] = pack2<kBf16>(x0, x1);
          }
          *reinterpret_cast<uint4*>(stage + off) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      fence_proxy_async_smem();
      ok = group_sync();
      if (ok && r == 0) {
        tma_store_4d(is_dk ? &tm_dk : &tm_dv, stage, half * 64, k_row0, h, b);
        tma_store_commit();
        tma_store_wait_all();
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarpA) tmem_dealloc(tmem, 512);
}

// dq[b,h,n,:] = scale * acc[b,h,n,:]  (acc fp32 contiguous, dq 16-bit with strides); one thread per 8 elements
template <bool kBf16>
__global__ void __launch_bounds__(256) dq_convert128_kernel(const float* __restrict__ acc, void* __restrict__ dq,
                                                            int H, int N, int64_t sb, int64_t sh, int64_t sn,
                                                            float scale, int64_t total_chunks,
                                                            const void* __restrict__ q, int64_t qsb, int64_t qsh,
                                                            int64_t qsn, const float* __restrict__ delta, int n_pad) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total_chunks) return;
  const int64_t row = i >> 4;
  const int ch = static_cast<int>(i & 15);
  const int64_t n = row % N;
  const int64_t bh = row / N;
  const int64_t b = bh / H, h = bh % H;
  const float4* src = reinterpret_cast<const float4*>(acc + row * D + ch * 8);
  float4 a = src[0], c = src[1];
  if (q != nullptr) {
    // non-softmax variant: subtract delta[row] * q[row, :]
    const float w = delta[bh * n_pad + n];
    const uint4 qv = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(q) + b * qsb + h * qsh +
                                                     n * qsn + ch * 8);
    const float2 q0 = unpack2<kBf16>(qv.x), q1 = unpack2<kBf16>(qv.y), q2 = unpack2<kBf16>(qv.z),
                 q3 = unpack2<kBf16>(qv.w);
    a.x = fmaf(-w, q0.x, a.x); a.y = fmaf(-w, q0.y, a.y); a.z = fmaf(-w, q1.x, a.z); a.w = fmaf(-w, q1.y, a.w);
    c.x = fmaf(-w, q2.x, c.x); c.y = fmaf(-w, q2.y, c.y); c.z = fmaf(-w, q3.x, c.z); c.w = fmaf(-w, q3.y, c.w);
  }
  uint4 o;
  o.x = pack2<kBf16>(a.x * scale, a.y * scale);
  o.y = pack2<kBf16>(a.z * scale, a.w * scale);
  o.z = pack2<kBf16>(c.x * scale, c.y * scale);
  o.w = pack2<kBf16>(c.z * scale, c.w * scale);
  uint16_t* dst = reinterpret_cast<uint16_t*>(dq) + b * sb + h * sh + n * sn + ch * 8;
  *reinterpret_cast<uint4*>(dst) = o;
}

template <bool kBf16>
static cudaError_t launch_t(const BwdFusedArgs& a, cudaStream_t stream) {
  auto kernel = rbf_bwd_fused128_kernel<kBf16>;
  constexpr int smem = Smem::kDynamic;
  static PerDeviceFlags configured{};
  {
    const cudaError_t ce = ensure_dynamic_smem(kernel, smem, configured);
    if (ce != cudaSuccess) return ce;
  }
  // the pre-pass has cleared the dQ accumulator
  cudaError_t e = cudaSuccess;
  Params p{};
  p.dq_acc = a.dq_acc; p.status = a.status;
  p.H = a.H; p.N = a.N; p.n_pad = a.n_pad; p.causal = a.causal;
  p.scale2 = a.scale2; p.grad_scale = a.grad_scale; p.slab_w = a.slab_w;
  dim3 grid((a.N + kTile - 1) / kTile, a.B * a.H);
  kernel<<<grid, kThreads, smem, stream>>>(a.tm_k, a.tm_v, a.tm_q, a.tm_do, a.tm_dk, a.tm_dv, a.tm_lslab, a.tm_dslab,
                                           p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int64_t chunks = static_cast<int64_t>(a.B) * a.H * a.N * (D / 8);
  dq_convert128_kernel<kBf16><<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, stream>>>(
      a.dq_acc, a.dq, a.H, a.N, a.dq_strides[0], a.dq_strides[1], a.dq_strides[2], a.grad_scale, chunks, a.q_rows,
      a.q_strides[0], a.q_strides[1], a.q_strides[2], a.delta, a.n_pad);
  return cudaGetLastError();
}

}  // namespace bwdf128


cudaError_t launch_bwd_fused128(const BwdFusedArgs& a, bool bf16, cudaStream_t stream) {
  return bf16 ? bwdf128::launch_t<true>(a, stream) : bwdf128::launch_t<false>(a, stream);
}

}  // namespace rbf
