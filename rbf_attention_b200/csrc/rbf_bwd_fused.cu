// Single-kernel backward of the softmax RBF attention for head dim 64 (sm_100a).
//
// A CTA owns 128 keys (K, V resident in shared memory) and streams the query tiles (Q, dO) past them. Per
// query tile it issues five MMAs - the algorithmic minimum - and evaluates every exponential once:
//   S^T  = K Q^T  (+ bias slab: -L[query] / scale)        smem x smem -> TMEM
//   dP^T = V dO^T (+ bias slab: -delta[query])            smem x smem -> TMEM
//   P^T  = exp2(S^T * 2c - ksq[key]),   dS^T = P^T * dP^T                        (registers)
//   dV  += P^T  dO               TMEM x smem   (P^T written to TMEM as 16-bit pairs)
//   dK  += dS^T Q                smem x smem   (dS^T stored to shared memory as a [key][query] tile)
//   dQ_partial = dS K            smem x smem   (the same tile read as an M-major A operand)
// The per-query statistics L and delta never pass through registers: the pre-pass stores them as three 16-bit
// parts per query ("bias slabs") and S^T / dP^T get one extra K = 16 MMA step against a slab of constants.
// dQ_partial leaves the CTA as fp32 reduce-adds into an accumulator in global memory; a small kernel converts it
// to the output type (times 2g) afterwards. dK gets the norm-gradient term in the epilogue:
// dK = 2g (acc - rowsum(dS^T)[key] * k).
//
// Roles: warps 0, 1, 3 MMA issuers (one thread sustains one MMA per ~60 cycles, the tensor pipe retires an N = 64
// product in 32; five issuers, one per product, measured slower than three), warp 2 TMA producer, warps 4-19 compute (thread = key row; group g owns query columns [32g, 32g+32) of the
// tile), warps 20-23 drain dQ_partial (thread = query row). Compute warpgroups take registers from the others.
//   issuer A: S^T(n+1) as soon as the compute warps have read S^T(n); dV(n) when P^T(n) is in TMEM
//   issuer B: dP^T(n+1) as soon as dP^T(n) has been read; dK(n) when dS^T(n) is in shared memory
//   issuer C: dQ_partial(n) when dS^T(n) is in shared memory and the drain warps have read dQ_partial(n-1)
// so the compute warps never wait for an MMA that was not issued a full step ahead.
// TMEM columns: S^T [0,128), dP^T [128,256), P^T [256,320), dV [320,384), dK [384,448), dQ_partial [448,512).
#include "common.cuh"
#include "launch.h"

namespace rbf {

namespace bwdf {


static constexpr int D = 64;
static constexpr int kThreads = 768;
static constexpr int kNumComputeWarps = 16;
static constexpr int kMmaWarpA = 0;
static constexpr int kMmaWarpB = 1;
static constexpr int kLoadWarp = 2;
static constexpr int kMmaWarpC = 3;
static constexpr int kComputeWarp0 = 4;
static constexpr int kDrainWarp0 = 20;
// Register budget: the launch allocates 80 per thread (768 threads); setmaxnreg may only redistribute that
// total: 512 * 96 + 128 * 40 + 128 * 56 = 768 * 80. (An increase beyond what the decreases released blocks
// forever, with no timeout.)
static constexpr int kComputeRegs = 96;
static constexpr int kOtherRegs = 40;
static constexpr int kDrainRegs = 56;
static_assert(512 * kComputeRegs + 128 * kOtherRegs + 128 * kDrainRegs <= 768 * 80, "setmaxnreg budget");
static constexpr int kDqBoxBytes = 32 * 128;        // 4 KB: fp32 [32 queries][32 columns] of one drain warp

static constexpr int kTileBytes = kTile * D * 2;    // 16 KB: one 128 x 64 16-bit tile
static constexpr int kSlabBytes = kTile * 32;       // 4 KB: 128 rows x 16 x 16-bit
static constexpr int kStages = 3;                   // Q (+ L slab) and dO (+ delta slab) rings
static constexpr int kDsBytes = kTile * kTile * 2;  // 32 KB: dS^T as [key][query], two 64-query boxes

struct Smem {
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTileBytes;
  static constexpr int kQ = kV + kTileBytes;
  static constexpr int kDo = kQ + kStages * kTileBytes;
  static constexpr int kDs = kDo + kStages * kTileBytes;
  static constexpr int kLSlab = kDs + kDsBytes;
  static constexpr int kDSlab = kLSlab + kStages * kSlabBytes;
  static constexpr int kOnes = kDSlab + kStages * kSlabBytes;
  static constexpr int kDqStage = kOnes + kSlabBytes;          // 32 KB fp32 dQ_partial staging: four warps, two boxes each
  static constexpr int kRowsum = kDqStage + kTile * D * 4;     // [4 groups][128] floats: partial row sums
  static constexpr int kBars = kRowsum + 4 * kTile * 4;
  static constexpr int kNumBars = 1 + 4 * kStages + 12;
  static constexpr int kMisc = kBars + kNumBars * 8;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

static constexpr int kColS = 0, kColDP = 128, kColPT = 256, kColDV = 320, kColDK = 384, kColDQ = 448;

enum Site : uint32_t {
  kSiteKV = 64, kSiteQFull, kSiteDoFull, kSiteQEmpty, kSiteDoEmpty, kSiteSFull, kSiteDPFull, kSitePFull, kSiteDSFull,
  kSiteDQFull, kSiteDQDrained, kSiteAccDone, kSiteGroup, kSiteSConsumed, kSiteDPConsumed, kSiteDVDone, kSiteDsFree, kSiteStageFree
};

struct Params {
  const float* ksq;      // (B*H, n_pad), +inf on padding rows
  float* dq_acc;         // fp32 (B, H, N, 64), zero-initialised
  DeviceStatus* status;
  unsigned int* work;    // [0] next work item, [1] CTAs that have left; both zero at launch, and zero again at its end
  int total_items;       // key tiles x (batch, head) pairs
  int H, N, n_pad, causal;
  float scale2, grad_scale, slab_w;
};

// The launch is persistent: as many CTAs as SMs, each taking (key tile, batch-head) items from a global counter in the
// order a plain grid would run them (key tile fastest, heaviest causal tile first). Between items a CTA keeps its
// TMEM allocation and its barriers (their phases run on), which saves the launch gap and most of the set-up of a
// CTA (about 1.5 of the 6.5 microseconds that an item spent outside its step loop).
template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
rbf_bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                     const __grid_constant__ CUtensorMap tm_lslab, const __grid_constant__ CUtensorMap tm_dslab,
                     const __grid_constant__ CUtensorMap tm_dq_acc, const Params p) {
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
  uint8_t* s_dq = smem + Smem::kDqStage;
  float* s_rowsum = reinterpret_cast<float*>(smem + Smem::kRowsum);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint64_t* kv_full = bars;
  uint64_t* q_full = kv_full + 1;            // [kStages] Q tile + L slab landed
  uint64_t* q_empty = q_full + kStages;      // two arrivals: S^T (issuer A) and dK (issuer B) have completed
  uint64_t* do_full = q_empty + kStages;     // dO tile + delta slab landed
  uint64_t* do_empty = do_full + kStages;    // two arrivals: dV (issuer A) and dP^T (issuer B)
  uint64_t* s_full = do_empty + kStages;     // S^T(n) complete
  uint64_t* s_consumed = s_full + 1;         // compute warps hold S^T(n) in registers
  uint64_t* dp_full = s_consumed + 1;
  uint64_t* dp_consumed = dp_full + 1;
  uint64_t* p_full = dp_consumed + 1;        // P^T(n) stored to TMEM
  uint64_t* dv_done = p_full + 1;            // dV(n) complete: the P^T columns may be overwritten
  uint64_t* ds_full = dv_done + 1;           // dS^T(n) stored to shared memory
  uint64_t* dq_full = ds_full + 1;           // dK(n) and dQ_partial(n) complete: dS^T tile free, dQ_partial readable
  uint64_t* dq_drained = dq_full + 1;        // drain warps have read dQ_partial(n) out of TMEM
  uint64_t* acc_done = dq_drained + 1;       // two arrivals: all MMAs of both issuers complete
  uint64_t* grp_sync = acc_done + 1;         // compute warps (16 arrivals)
  uint64_t* stage_free = grp_sync + 1;       // the previous item's dK and dV stores have read their staging tiles
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + Smem::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::kMisc + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_tiles = (p.N + kTile - 1) / kTile;
  volatile int* s_item = reinterpret_cast<volatile int*>(smem + Smem::kMisc + 8);
  // Barriers are initialised once per CTA and run on across its items: T counts the steps of the CTA's earlier items
  // (step n of the item is global step T + n: ring stage (T + n) % kStages, phase ((T + n) / kStages) & 1; per-step
  // barriers are in phase (T + n) & 1), I counts the earlier items (per-item barriers are in phase I & 1). Every role
  // advances both at the item's closing synchronisation.
  uint32_t T = 0, I = 0;
  // the current work item
  int bh = 0, b = 0, h = 0;
  int kt = 0;                                      // key tile; tile 0 is the heaviest under the causal mask
  int k_row0 = 0;
  int first = 0;                                   // first query tile that sees these keys
  int cnt = 0;
  auto set_item = [&](int item) {
    kt = item % n_tiles;
    bh = item / n_tiles;
    b = bh / p.H;
    h = bh % p.H;
    k_row0 = kt * kTile;
    first = p.causal ? kt : 0;
    cnt = n_tiles - first;
  };

  // One thread (the TMA producer) sets the CTA up: it reads the launch's status word (a wait that ran out in an
  // earlier CTA ends the whole launch quickly: later CTAs leave at once), initialises the barriers while that load
  // is in flight, and issues the first loads before the CTA-wide synchronisation so that K, V and the first query
  // tiles travel while TMEM is allocated and the constant slab is written.
  auto load_step = [&](int n) {
    const int row0 = (first + n) * kTile;
    const int st = (T + n) % kStages;
    mbar_arrive_expect_tx(&q_full[st], kTileBytes + kSlabBytes);
    tma_load_4d(s_q + st * kTileBytes, &tm_q, &q_full[st], 0, row0, h, b);
    tma_load_3d(s_lslab + st * kSlabBytes, &tm_lslab, &q_full[st], 0, row0, bh);
    mbar_arrive_expect_tx(&do_full[st], kTileBytes + kSlabBytes);
    tma_load_4d(s_do + st * kTileBytes, &tm_do, &do_full[st], 0, row0, h, b);
    tma_load_3d(s_dslab + st * kSlabBytes, &tm_dslab, &do_full[st], 0, row0, bh);
  };
  // Executed by the producer warp before every item's opening synchronisation (nothing of the previous item is in
  // flight any more): lane 0 takes the next item and reads the launch's status word, then issues the item's first
  // loads. The barriers are initialised by the first call only, one per lane, and run on across the CTA's items (T, I
  // above). An earlier form invalidated and re-initialised all of them here for every item; it worked as long as the
  // work counter's round trip (about 2000 clocks) lay between that and the loads, and ran into bounded waits that
  // never completed - a load whose completion was lost - as soon as the loads followed within a few hundred clocks,
  // with or without a proxy fence in between. Without re-initialisation the loads may follow at once (measured with
  // the item number taken under the previous item's last steps: correct, and no faster, because what an item waits
  // for at its start is the arrival of its first 70 KB, about 4000 clocks however early the request is made after
  // the closing synchronisation).
  auto prepare_item = [&](bool first_time) {
    int item = 0;
    unsigned int earlier = 0u;
    if (lane == 0) {
      item = static_cast<int>(atomicAdd(&p.work[0], 1u));
      earlier = *reinterpret_cast<volatile unsigned int*>(&p.status->code);
    }
    if (lane < Smem::kNumBars) {
      // arrival counts in the order of the barrier block: kv_full; q_full, q_empty, do_full, do_empty (kStages
      // each); s_full, s_consumed, dp_full, dp_consumed, p_full, dv_done, ds_full, dq_full, dq_drained, acc_done,
      // grp_sync, stage_free
      uint32_t count;
      if (lane == 0) {
        count = 1;
      } else if (lane < 1 + 4 * kStages) {
        const int ring = (lane - 1) / kStages;               // 0 q_full, 1 q_empty, 2 do_full, 3 do_empty
        count = (ring & 1) ? 2 : 1;
      } else {
        constexpr uint32_t tail[12] = {1, kNumComputeWarps, 1, kNumComputeWarps, kNumComputeWarps, 1,
                                       kNumComputeWarps, 2, 4, 3, kNumComputeWarps, 2};
        count = tail[lane - (1 + 4 * kStages)];
      }
      if (first_time) mbar_init(&bars[lane], count);
    }
    if (first_time) fence_mbar_init();
    __syncwarp();
    if (lane != 0) return;
    // first call: the loads below complete on barriers that other lanes have just initialised; besides the warp-level
    // synchronisation, order those generic-proxy writes before this thread's async-proxy operations
    fence_proxy_async_smem();
    *s_item = item;
    if (first_time) *abort_flag = 0;
    if (earlier != 0u) *abort_flag = 1;
    if (earlier == 0u && item < p.total_items) {
      set_item(item);
      mbar_arrive_expect_tx(kv_full, 2 * kTileBytes);
      tma_load_4d(s_k, &tm_k, kv_full, 0, k_row0, h, b);
      tma_load_4d(s_v, &tm_v, kv_full, 0, k_row0, h, b);
      for (int n = 0; n < cnt && n < kStages; ++n) load_step(n);
    }
  };
  // opening synchronisation of an item; false when there is no item left (or the launch is being abandoned)
  auto open_item = [&]() -> bool {
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const int item = *s_item;
    if (item >= p.total_items || *abort_flag) return false;
    set_item(item);
    return true;
  };
  if (warp == kLoadWarp) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_lslab);
      tma_prefetch_desc(&tm_dslab);
    }
    prepare_item(true);
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
  uint32_t tmem = 0;   // read after the first opening synchronisation

  if (warp < kComputeWarp0) {
    setmaxnreg_dec<kOtherRegs>();
  }
  if (warp == kLoadWarp) {
    // ------------------------------------------------------------------ TMA producer
    while (open_item()) {
      if (lane == 0) {
        for (int n = kStages; n < cnt; ++n) {
          const int st = (T + n) % kStages;
          const uint32_t par = (((T + n) / kStages) - 1) & 1;
          // the ring slot is free once the MMAs that read it have completed (both rings, in the order the loads go)
          if (!mbar_wait(&q_empty[st], par, abort_flag, p.status, kSiteQEmpty, s_item)) break;
          if (!mbar_wait(&do_empty[st], par, abort_flag, p.status, kSiteDoEmpty, s_item)) break;
          load_step(n);
        }
      }
      __syncthreads();                       // closing synchronisation: every role is done with the item
      T += cnt;
      ++I;
      prepare_item(false);
    }
  } else if (warp == kMmaWarpA || warp == kMmaWarpB || warp == kMmaWarpC) {
    // ------------------------------------------------------------------ MMA issuers
    while (open_item()) {
    tmem = *tmem_base_s;
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(kTile, kTile, kBf16, false, false);  // keys x queries, both K-major
      constexpr uint32_t idesc_acc = make_idesc(kTile, D, kBf16, false, true);     // A K-major (or TMEM), B N-major
      constexpr uint32_t idesc_dq = make_idesc(kTile, D, kBf16, true, true);       // A M-major (dS^T tile), B N-major
      const SmemDesc ones_desc = make_sdesc_slab32(smem_u32(s_ones));
      auto stage_of = [](SmemDesc d, int stage, uint32_t stage_bytes) {
        d.lo += static_cast<uint32_t>(stage) * (stage_bytes >> 4);
        return d;
      };
      // dst = A B^T over D (both K-major) plus the bias-slab step: dst[m][n] += w * (slab[n] hi + mid + lo)
      auto issue_scores = [&](uint32_t dst, const SmemDesc& a_desc, const SmemDesc& b_desc, const SmemDesc& slab) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_ss(dst, sdesc_at(a_desc, kk * 32), sdesc_at(b_desc, kk * 32), idesc_s, kk > 0);
        umma_ss(dst, sdesc_at(ones_desc, 0), sdesc_at(slab, 0), idesc_s, 1u);
      };
      auto wait_q = [&](int n) {
        return mbar_wait(&q_full[(T + n) % kStages], ((T + n) / kStages) & 1, abort_flag, p.status, kSiteQFull, s_item);
      };
      auto wait_do = [&](int n) {
        return mbar_wait(&do_full[(T + n) % kStages], ((T + n) / kStages) & 1, abort_flag, p.status, kSiteDoFull, s_item);
      };
      bool ok = mbar_wait(kv_full, I & 1, abort_flag, p.status, kSiteKV, s_item);

      if (warp == kMmaWarpA) {
        const SmemDesc k_kmaj = make_sdesc_parts(smem_u32(s_k), 16, 1024);
        const SmemDesc q_kmaj0 = make_sdesc_parts(smem_u32(s_q), 16, 1024);
        const SmemDesc lslab0 = make_sdesc_slab32(smem_u32(s_lslab));
        const SmemDesc do_nmaj0 = make_sdesc_parts(smem_u32(s_do), kTile * 128, 1024);
        if (ok) ok = wait_q(0);
        if (ok) {
          tc_fence_after_sync();
          issue_scores(tmem + kColS, k_kmaj, stage_of(q_kmaj0, T % kStages, kTileBytes),
                       stage_of(lslab0, T % kStages, kSlabBytes));
          umma_commit(s_full);
          umma_commit(&q_empty[T % kStages]);
        }
        for (int n = 0; n < cnt && ok; ++n) {
          if (n + 1 < cnt) {
            // S^T(n+1) may overwrite S^T(n) as soon as every compute warp holds it in registers
            const int st = (T + n + 1) % kStages;
            ok = wait_q(n + 1) && mbar_wait(s_consumed, (T + n) & 1, abort_flag, p.status, kSiteSConsumed, s_item);
            if (!ok) break;
            tc_fence_after_sync();
            issue_scores(tmem + kColS, k_kmaj, stage_of(q_kmaj0, st, kTileBytes), stage_of(lslab0, st, kSlabBytes));
            umma_commit(s_full);
            umma_commit(&q_empty[st]);
          }
          // dV += P^T dO
          ok = mbar_wait(p_full, (T + n) & 1, abort_flag, p.status, kSitePFull, s_item);
          if (!ok) break;
          tc_fence_after_sync();
          const SmemDesc do_n = stage_of(do_nmaj0, (T + n) % kStages, kTileBytes);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ts(tmem + kColDV, tmem + kColPT + kk * 8, sdesc_at(do_n, kk * 2048), idesc_acc,
                    (n > 0 || kk > 0) ? 1u : 0u);
          umma_commit(dv_done);
          umma_commit(&do_empty[(T + n) % kStages]);
        }
      } else if (warp == kMmaWarpC) {
        // dQ_partial = dS K : A = the dS^T tile read M-major (rows = keys = reduction index), B = K read N-major
        const SmemDesc k_nmaj = make_sdesc_parts(smem_u32(s_k), kTile * 128, 1024);
        const SmemDesc ds_mmaj = make_sdesc_parts(smem_u32(s_ds), kTile * 128, 1024);   // rows = reduction (keys)
        for (int n = 0; n < cnt && ok; ++n) {
          ok = mbar_wait(ds_full, (T + n) & 1, abort_flag, p.status, kSiteDSFull, s_item);
          if (ok && n > 0) ok = mbar_wait(dq_drained, (T + n - 1) & 1, abort_flag, p.status, kSiteDQDrained, s_item);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ss(tmem + kColDQ, sdesc_at(ds_mmaj, kk * 2048), sdesc_at(k_nmaj, kk * 2048), idesc_dq, kk > 0);
          umma_commit(dq_full);                    // second arrival: dQ_partial readable, M-major reader done
        }
      } else {
        const SmemDesc v_kmaj = make_sdesc_parts(smem_u32(s_v), 16, 1024);
        const SmemDesc do_kmaj0 = make_sdesc_parts(smem_u32(s_do), 16, 1024);
        const SmemDesc dslab0 = make_sdesc_slab32(smem_u32(s_dslab));
        const SmemDesc q_nmaj0 = make_sdesc_parts(smem_u32(s_q), kTile * 128, 1024);
        const SmemDesc ds_kmaj = make_sdesc_parts(smem_u32(s_ds), 16, 1024);            // rows = keys, K = queries
        if (ok) ok = wait_do(0);
        if (ok) {
          tc_fence_after_sync();
          issue_scores(tmem + kColDP, v_kmaj, stage_of(do_kmaj0, T % kStages, kTileBytes),
                       stage_of(dslab0, T % kStages, kSlabBytes));
          umma_commit(dp_full);
          umma_commit(&do_empty[T % kStages]);
        }
        for (int n = 0; n < cnt && ok; ++n) {
          if (n + 1 < cnt) {
            const int st = (T + n + 1) % kStages;
            ok = wait_do(n + 1) && mbar_wait(dp_consumed, (T + n) & 1, abort_flag, p.status, kSiteDPConsumed, s_item);
            if (!ok) break;
            tc_fence_after_sync();
            issue_scores(tmem + kColDP, v_kmaj, stage_of(do_kmaj0, st, kTileBytes), stage_of(dslab0, st, kSlabBytes));
            umma_commit(dp_full);
            umma_commit(&do_empty[st]);
          }
          // dK += dS^T Q : A = dS^T tile (K-major: 64-query boxes of 128-byte rows), B = Q read N-major
          ok = mbar_wait(ds_full, (T + n) & 1, abort_flag, p.status, kSiteDSFull, s_item);
          if (!ok) break;
          tc_fence_after_sync();
          const SmemDesc q_n = stage_of(q_nmaj0, (T + n) % kStages, kTileBytes);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            umma_ss(tmem + kColDK, sdesc_at(ds_kmaj, (kk >> 2) * (kTile * 128) + (kk & 3) * 32), sdesc_at(q_n, kk * 2048),
                    idesc_acc, (n > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&q_empty[(T + n) % kStages]);
          umma_commit(dq_full);                    // first of two arrivals: the dS^T tile's K-major reader is done
        }
      }
      if (ok) umma_commit(acc_done);   // every issuer arrives: the barrier counts three
    }
    __syncthreads();                         // closing synchronisation
    T += cnt;
    ++I;
    }
  } else if (warp >= kDrainWarp0) {
    // ------------------------------------------------------------------ dQ_partial drain (thread = query row)
    // Every warp stages and reduces its own 32 query rows: a [32 rows][32 floats] box per half of the head dim, two
    // boxes in flight, one TMA bulk reduce-add each, no synchronisation between the warps. (An SM pushes about 25
    // bytes per clock of reduce-adds into L2, measured: the 32 KB of a step take as long as its MMAs and must
    // overlap them.)
    setmaxnreg_dec<kDrainRegs>();
    const int wq = warp & 3;
    const uint32_t lane_sel = static_cast<uint32_t>(wq * 32) << 16;
    uint8_t* my_boxes = s_dq + wq * (2 * kDqBoxBytes);
    while (open_item()) {
    tmem = *tmem_base_s;
    bool ok = true;
    for (int n = 0; n < cnt; ++n) {
      ok = mbar_wait(dq_full, (T + n) & 1, abort_flag, p.status, kSiteDQFull, s_item);
      if (!ok) break;
      tc_fence_after_sync();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        // the box written two halves ago must have been read by the bulk engine
        if (lane == 0) tma_store_wait_read1();
        __syncwarp();
        uint32_t v[32];
        tmem_ld_x32(tmem + kColDQ + lane_sel + hh * 32, v);
        tmem_ld_wait();
        if (hh == 1) {
          tc_fence_before_sync();
          mbar_arrive_warp(dq_drained);   // the next dQ_partial MMA may overwrite TMEM
        }
        uint8_t* row = my_boxes + hh * kDqBoxBytes + lane * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(row + ((c ^ (lane & 7)) << 4)) =
              make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_4d(&tm_dq_acc, my_boxes + hh * kDqBoxBytes, hh * 32, (first + n) * kTile + wq * 32, h, b);
          tma_store_commit();
        }
      }
    }
    if (lane == 0) tma_store_wait_all();
    __syncthreads();                         // closing synchronisation
    T += cnt;
    ++I;
    }
  } else {
    // ------------------------------------------------------------------ compute groups (thread = key row)
    setmaxnreg_inc<kComputeRegs>();
    const int g = (warp - kComputeWarp0) >> 2;             // 32-column slice of the query tile
    const int r = tid & (kTile - 1);
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t grp_phase = 0;                       // two rendezvous per item, counted across items
    const bool storer = r == 0 && (g & 1) == 0;   // issues the item's dK (g = 0) or dV (g = 2) store
    bool store_pending = false;
    while (open_item()) {
    tmem = *tmem_base_s;
    const float neg_ksq = -p.ksq[static_cast<int64_t>(bh) * p.n_pad + k_row0 + r];
    float ds_rowsum = 0.f;
    bool ok = true;
    if (storer) {
      // dK and dV leave through the dS^T tile, which the previous item's stores may still be reading: they were
      // issued a set-up and a load latency ago, so this wait is over at once; the compute warps check `stage_free`
      // before the item's first dS^T store
      if (store_pending) tma_store_wait_read();
      store_pending = false;
      mbar_arrive(stage_free);
    }

    for (int n = 0; n < cnt; ++n) {
      ok = mbar_wait(s_full, (T + n) & 1, abort_flag, p.status, kSiteSFull, s_item);
      if (!ok) break;
      tc_fence_after_sync();
      float pr[32];
      {
        uint32_t raw[32];
        tmem_ld_x32(tmem + kColS + lane_sel + g * 32, raw);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(s_consumed);
        // acc = k.q - L / scale2 ; P = exp2(acc * scale2 - ksq)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a0, a1;
          ffma2_bcast(a0, a1, __uint_as_float(raw[i]), __uint_as_float(raw[i + 1]), p.scale2, neg_ksq);
          pr[i] = ex2_approx(a0);
          pr[i + 1] = ex2_approx(a1);
        }
      }
      if (p.causal && n == 0) {
        // diagonal tile: query column (32g + c) sees key row r iff column >= row
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (g * 32 + c < r) pr[c] = 0.f;
      }
      {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) packed[i] = pack2<kBf16>(pr[2 * i], pr[2 * i + 1]);
        // the P^T columns are free once dV of the previous step has completed
        if (n > 0) {
          ok = mbar_wait(dv_done, (T + n - 1) & 1, abort_flag, p.status, kSiteDVDone, s_item);
          if (!ok) break;
          tc_fence_after_sync();
        }
        tmem_st_x16(tmem + kColPT + lane_sel + g * 16, packed);
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(p_full);
      }

      ok = mbar_wait(dp_full, (T + n) & 1, abort_flag, p.status, kSiteDPFull, s_item);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t ds_packed[16];
      {
        uint32_t raw[32];
        tmem_ld_x32(tmem + kColDP + lane_sel + g * 32, raw);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(dp_consumed);
        // acc = v.dO - delta ; dS = P * acc
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float d0, d1;
          fmul2(d0, d1, pr[2 * i], pr[2 * i + 1], __uint_as_float(raw[2 * i]), __uint_as_float(raw[2 * i + 1]));
          fadd2(rs0, rs1, rs0, rs1, d0, d1);
          ds_packed[i] = pack2<kBf16>(d0, d1);
        }
        ds_rowsum += rs0 + rs1;
      }
      // the dS^T tile is free once dK and dQ_partial of the previous step have completed (first step: once the
      // previous item's output stores have read it)
      ok = n > 0 ? mbar_wait(dq_full, (T + n - 1) & 1, abort_flag, p.status, kSiteDsFree, s_item)
                 : mbar_wait(stage_free, I & 1, abort_flag, p.status, kSiteStageFree, s_item);
      if (!ok) break;
      // row r of the [key][query] tile, box g/2, 16-byte chunks 4(g%2) .. +3
#pragma unroll
      for (int ch = 0; ch < 4; ++ch)
        *reinterpret_cast<uint4*>(s_ds + (g >> 1) * (kTile * 128) + sw128_offset(r, (g & 1) * 4 + ch)) =
            make_uint4(ds_packed[ch * 4 + 0], ds_packed[ch * 4 + 1], ds_packed[ch * 4 + 2], ds_packed[ch * 4 + 3]);
      fence_proxy_async_smem();
      mbar_arrive_warp(ds_full);
    }

    auto group_sync = [&]() -> bool {
      mbar_arrive_warp(grp_sync);
      const bool done = mbar_wait(grp_sync, grp_phase & 1, abort_flag, p.status, kSiteGroup, s_item);
      ++grp_phase;
      return done;
    };
    if (ok) ok = mbar_wait(acc_done, I & 1, abort_flag, p.status, kSiteAccDone, s_item);
    if (ok) {
      tc_fence_after_sync();
      s_rowsum[g * kTile + r] = ds_rowsum;      // every group holds a quarter of rowsum(dS^T)
      ok = group_sync();
    }
    if (ok) {
      // groups 0, 1 finish dK (columns [32(g%2), +32)), groups 2, 3 store dV; the dS^T tile is dead by now (all MMAs
      // have completed) and is not written again before the next item's first step
      const bool is_dk = g < 2;
      uint8_t* stage = s_ds + (is_dk ? 0 : kTileBytes);
      const float w = is_dk ? (s_rowsum[r] + s_rowsum[kTile + r]) + (s_rowsum[2 * kTile + r] + s_rowsum[3 * kTile + r])
                            : 0.f;
      const float out_scale = is_dk ? p.grad_scale : 1.0f;
      uint32_t acc[32];
      tmem_ld_x32(tmem + (is_dk ? kColDK : kColDV) + lane_sel + (g & 1) * 32, acc);
      tmem_ld_wait();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint32_t off = sw128_offset(r, (g & 1) * 4 + q4);
        const uint4 k_raw = *reinterpret_cast<const uint4*>(s_k + off);
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
      fence_proxy_async_smem();
      ok = group_sync();
      if (ok && storer) {
        tma_store_4d(is_dk ? &tm_dk : &tm_dv, stage, 0, k_row0, h, b);
        tma_store_commit();
        store_pending = true;    // read-wait deferred to the next item (or to the end of the kernel)
      }
    }
    __syncthreads();                         // closing synchronisation
    T += cnt;
    ++I;
    }
    if (storer && store_pending) tma_store_wait_read();
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarpA) tmem_dealloc(*tmem_base_s, 512);
  if (tid == 0) {
    // the last CTA to leave puts the work counters back to zero for the next launch on this workspace
    __threadfence();
    if (atomicAdd(&p.work[1], 1u) == gridDim.x - 1) {
      p.work[0] = 0u;
      p.work[1] = 0u;
    }
  }
}

// dq[b,h,n,:] = scale * acc[b,h,n,:]  (acc fp32 contiguous, dq 16-bit with strides)
template <bool kBf16>
__global__ void __launch_bounds__(256) dq_convert_kernel(const float* __restrict__ acc, void* __restrict__ dq, int H,
                                                         int N, int64_t sb, int64_t sh, int64_t sn, float scale,
                                                         int64_t total_chunks, const void* __restrict__ q,
                                                         int64_t qsb, int64_t qsh, int64_t qsn,
                                                         const float* __restrict__ delta, int n_pad) {
  // one thread per 8 consecutive elements of a row (D = 64: 8 chunks per row)
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total_chunks) return;
  const int64_t row = i >> 3;
  const int ch = static_cast<int>(i & 7);
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
  auto kernel = rbf_bwd_fused_kernel<kBf16>;
  constexpr int smem = Smem::kDynamic;
  static PerDeviceFlags configured{};
  {
    const cudaError_t ce = ensure_dynamic_smem(kernel, smem, configured);
    if (ce != cudaSuccess) return ce;
  }
  // the pre-pass has cleared the dQ accumulator
  cudaError_t e = cudaSuccess;
  Params p{};
  p.ksq = a.ksq; p.dq_acc = a.dq_acc; p.status = a.status;
  p.H = a.H; p.N = a.N; p.n_pad = a.n_pad; p.causal = a.causal;
  p.scale2 = a.scale2; p.grad_scale = a.grad_scale; p.slab_w = a.slab_w;
  p.work = a.work;
  p.total_items = ((a.N + kTile - 1) / kTile) * a.B * a.H;
  dim3 grid(p.total_items < a.sm_count ? p.total_items : a.sm_count);
  kernel<<<grid, kThreads, smem, stream>>>(a.tm_k, a.tm_v, a.tm_q, a.tm_do, a.tm_dk, a.tm_dv, a.tm_lslab, a.tm_dslab, a.tm_dq_acc, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int64_t chunks = static_cast<int64_t>(a.B) * a.H * a.N * 8;
  dq_convert_kernel<kBf16><<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, stream>>>(
      a.dq_acc, a.dq, a.H, a.N, a.dq_strides[0], a.dq_strides[1], a.dq_strides[2], a.grad_scale, chunks, a.q_rows,
      a.q_strides[0], a.q_strides[1], a.q_strides[2], a.delta, a.n_pad);
  return cudaGetLastError();
}

}  // namespace bwdf


cudaError_t launch_bwd_fused(const BwdFusedArgs& a, bool bf16, cudaStream_t stream) {
  return bf16 ? bwdf::launch_t<true>(a, stream) : bwdf::launch_t<false>(a, stream);
}

}  // namespace rbf
