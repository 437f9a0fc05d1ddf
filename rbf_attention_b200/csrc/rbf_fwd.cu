// Fused RBF attention forward for sm_100a.
//
//   softmax variant      O = softmax_j(2g q_i.k_j - g|k_j|^2) V,  L_i = log2 sum_j 2^(log2e * logit_ij)
//   non-softmax variant  O = exp(-g|q_i - k_j|^2) V
//
// One CTA owns 256 consecutive query rows of one (batch, head) as two 128-row tiles and walks the
// key tiles (128 keys at D = 64, 64 keys at D = 128) once for both. Roles:
//   softmax warps    one warpgroup per query tile, one thread per query row (the non-softmax variant at D = 64: two
//                    warpgroups per tile, two threads per row, see Roles below)
//   next warp        TMA producer: Q tiles once, then a ring of K (+ its key-norm bias slab) and V tiles
//   next two warps   tcgen05.mma issuers, one per query tile: S_t = Q_t K_j^T (smem x smem), O_t += P_t V_j
//                    (TMEM x smem). One thread sustains one MMA per ~58 cycles, slower than the tensor pipe retires
//                    the N = 64 products, hence two issuing threads.
// TMEM columns: S_0, S_1 (one key tile wide each), O_0 and O_1 (D columns each), P_0 and P_1 (16-bit pairs, half a key
// tile wide each): P_t has columns of its own and is consumed from there as the A operand of the second MMA, so the
// next scores are issued as soon as the current ones are in registers.
//
// The key-norm bias never passes through registers or shared-memory loads: the pre-pass stores
// -|k_j|^2 / 2 as three 16-bit parts per key ("bias slab"), and S_t gets one extra K = 16 MMA step against a
// slab of constants, so the fp32 accumulator already holds q.k - |k|^2/2 and the logit is acc * 2 g log2e.
// (Reading the bias per column from shared memory costs four wavefronts per warp instruction and made the
// shared-memory pipe, which also feeds the MMA operands, the bottleneck.)
// The running maximum is only raised (and O rescaled in TMEM) when it grew by more than 2^8, so the
// rescale is rare; L and the final 1/l normalisation use the maximum actually applied. With bf16 operands the tile
// maxima are not even computed once the applied maximum is close enough to the row's upper bound g |q|^2 (kSkipMax).
#include "common.cuh"
#include "launch.h"

namespace rbf {

namespace fwd {



static constexpr float kRescaleThreshold = 8.0f;
// Keys per streamed tile: 128 at D = 64; 64 at D = 128, where the narrower score tile leaves TMEM columns for P of
// its own (2 x 64 S + 2 x 32 P + 2 x 128 O), so that the next scores run under the current tile's exponentials.
template <int D>
struct KeyTile {
  static constexpr int kKeys = (D == 64) ? 128 : 64;
};
// Warp roles and register budget. At D = 64 the exponentials (MUFU, 16 per clock per SM) outweigh the MMAs. The
// non-softmax variant, whose rows need no statistics, shares a query row between kSplit = 2 threads of two warpgroups
// (64 of the tile's 128 key columns each): sixteen softmax warps, four per scheduler, keep the MUFU pipe busier
// than eight (measured 8 % on the kernel). For the softmax variant the two halves would have to agree on the row
// maximum and sum; with that hand-over the split measured slower than one thread per row and is not used.
// setmaxnreg only redistributes the launch allocation: softmax * kSoftmaxRegs + 128 * kOtherRegs <= threads * launch.
template <int D, bool kSoftmax, bool kBf16>
struct Roles {
  static constexpr int kSplit = (D == 64 && !kSoftmax) ? 2 : 1;
  // The logits of a row are bounded: 2 g q.k - g |k|^2 = g |q|^2 - g |q - k|^2 <= g |q|^2. Once the maximum applied
  // so far is within 2^64 of that bound no later tile can overflow (P is kept in fp32 / bf16, whose range is 2^127),
  // and the tile maxima - a third of the softmax warps' work outside the exponentials - are not computed any more
  // (measured 5-6 % on the kernel at both head dims). fp16's range (2^16) is too small for that.
  static constexpr bool kSkipMax = kSoftmax && kBf16;
  static constexpr int kSoftmaxWarps = 8 * kSplit;
  static constexpr int kLoadWarp = kSoftmaxWarps;
  static constexpr int kMmaWarp0 = kLoadWarp + 1;          // issuer of query tile t is warp kMmaWarp0 + t
  static constexpr int kThreads = (kSoftmaxWarps + 4) * 32;
  static constexpr int kLaunchRegs = kSplit == 2 ? 96 : 168;
  static constexpr int kSoftmaxRegs = kSplit == 2 ? 104 : 216;
  static constexpr int kOtherRegs = kSplit == 2 ? 64 : 72;
  static_assert(kSoftmaxWarps * 32 * kSoftmaxRegs + 128 * kOtherRegs <= kThreads * kLaunchRegs, "setmaxnreg budget");
};
static constexpr float kSafeGap = 64.0f;

template <int D>
struct Smem {
  static constexpr int kKeys = KeyTile<D>::kKeys;
  static constexpr int kTileBytes = kTile * D * 2;          // one 128-row query tile
  static constexpr int kKvBytes = kKeys * D * 2;            // one key / value tile
  static constexpr int kSlabBytes = kKeys * 32;             // kKeys rows x 16 x 16-bit
  static constexpr int kStages = (D == 64) ? 3 : 4;
  static constexpr int kQ = 0;                              // 2 tiles
  static constexpr int kK = kQ + 2 * kTileBytes;            // kStages tiles
  static constexpr int kV = kK + kStages * kKvBytes;        // kStages tiles
  static constexpr int kKSlab = kV + kStages * kKvBytes;    // kStages bias slabs
  static constexpr int kOnes = kKSlab + kStages * kSlabBytes;
  static constexpr int kBars = kOnes + kTile * 32;
  static constexpr int kNumBars = 2 + 4 * kStages + 10;
  static constexpr int kMisc = kBars + kNumBars * 8;        // tmem base, abort flag
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;            // slack for 1024-byte alignment
};

enum Site : uint32_t {
  kSiteQFull = 1, kSiteKFull, kSiteVFull, kSiteKEmpty, kSiteVEmpty, kSiteSFull, kSitePFull, kSiteODone,
  kSiteODoneFinal, kSiteGroup, kSiteSConsumed, kSitePFree
};

template <int D, bool kSoftmax, bool kBf16>
__global__ void __launch_bounds__(Roles<D, kSoftmax, kBf16>::kThreads, 1)
rbf_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               const __grid_constant__ CUtensorMap tm_kslab, const float* __restrict__ qsq,
               float* __restrict__ lse, DeviceStatus* status, int H, int N, int n_pad, int causal, float scale2,
               float slab_w) {
  using L = Smem<D>;
  using R = Roles<D, kSoftmax, kBf16>;
  constexpr int kSplit = R::kSplit;
  constexpr int kLoadWarp = R::kLoadWarp;
  constexpr int kMmaWarp0 = R::kMmaWarp0;
  constexpr int kStages = L::kStages;
  constexpr int kKeys = L::kKeys;                // keys per streamed tile
  constexpr int kBoxes = D / 64;                 // 64-column TMA boxes per tile row
  constexpr int kBoxBytes = kTile * 128;         // one query / output box: 128 rows x 128 bytes
  constexpr int kKvBoxBytes = kKeys * 128;       // one key / value box
  constexpr uint32_t kTileBytes = L::kTileBytes;
  constexpr uint32_t kKvBytes = L::kKvBytes;
  constexpr int kSlabBytes = L::kSlabBytes;
  // P has TMEM columns of its own (D = 64: 2 x 128 S + 2 x 64 O + 2 x 64 P; D = 128: 2 x 64 S + 2 x 32 P + 2 x 128 O):
  // S_t(j+1) is issued as soon as the softmax group holds S_t(j) in registers and runs under the exponentials.
  constexpr bool kSeparateP = true;   // (the issuers below rely on it)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem + L::kQ;
  uint8_t* s_k = smem + L::kK;
  uint8_t* s_v = smem + L::kV;
  uint8_t* s_kslab = smem + L::kKSlab;
  uint8_t* s_ones = smem + L::kOnes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* q_full = bars;                       // [2]
  uint64_t* k_full = bars + 2;                   // [kStages]
  uint64_t* k_empty = k_full + kStages;          // two arrivals: one per issuer
  uint64_t* v_full = k_empty + kStages;
  uint64_t* v_empty = v_full + kStages;          // two arrivals
  uint64_t* s_full = v_empty + kStages;          // [2]
  uint64_t* p_full = s_full + 2;                 // [2]
  uint64_t* o_done = p_full + 2;                 // [2]
  uint64_t* grp_sync = o_done + 2;               // [2] rendezvous of the 4 warps of a softmax group
  uint64_t* s_consumed = grp_sync + 2;           // [2] the softmax group holds S_t(j) in registers
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // Blocks are dispatched x-fastest. Causal: x = (batch, head), y = query block, heaviest block first, so that all
  // heads work on equally long blocks at any time and the tail of the launch is short (measured 6 % faster).
  // Non-causal: x = query block, y = (batch, head), which keeps one head's K/V hot in L2 (measured 20 % faster).
  const int bh = causal ? blockIdx.x : blockIdx.y;
  const int b = bh / H, h = bh % H;
  const int num_blocks = causal ? gridDim.y : gridDim.x;
  // heaviest causal blocks first
  const int mb = causal ? (num_blocks - 1 - static_cast<int>(blockIdx.y)) : static_cast<int>(blockIdx.x);
  const int m0 = mb * 2 * kTile;
  const int n_key_tiles_all = (N + kKeys - 1) / kKeys;
  int nkt[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = m0 + t * kTile;
    nkt[t] = (r0 >= N) ? 0 : (causal ? min(n_key_tiles_all, (r0 + kTile) / kKeys) : n_key_tiles_all);
  }
  const int nkt_max = max(nkt[0], nkt[1]);

  // One thread (the TMA producer) sets the CTA up: it reads the launch's status word (a wait that ran out in an
  // earlier CTA ends the whole launch quickly: later CTAs leave at once), initialises the barriers while that load
  // is in flight, and issues the first loads before the CTA-wide synchronisation, so that Q and the first key tiles
  // travel while TMEM is allocated and the constant slab is written.
  auto load_keys = [&](int j) {
    const int st = j % kStages;
    mbar_arrive_expect_tx(&k_full[st], kKvBytes + kSlabBytes);
    for (int x = 0; x < kBoxes; ++x)
      tma_load_4d(s_k + st * kKvBytes + x * kKvBoxBytes, &tm_k, &k_full[st], x * 64, j * kKeys, h, b);
    tma_load_3d(s_kslab + st * kSlabBytes, &tm_kslab, &k_full[st], 0, j * kKeys, bh);
  };
  auto load_values = [&](int j) {
    const int st = j % kStages;
    mbar_arrive_expect_tx(&v_full[st], kKvBytes);
    for (int x = 0; x < kBoxes; ++x)
      tma_load_4d(s_v + st * kKvBytes + x * kKvBoxBytes, &tm_v, &v_full[st], x * 64, j * kKeys, h, b);
  };
  if (tid == kLoadWarp * 32) {
    const unsigned int earlier = *reinterpret_cast<volatile unsigned int*>(&status->code);
    mbar_init(&q_full[0], 1);
    mbar_init(&q_full[1], 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 2);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 2);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4 * kSplit);     // one arrival per softmax warp of the tile
      mbar_init(&o_done[t], 1);
      mbar_init(&grp_sync[t], 4 * kSplit);
      mbar_init(&s_consumed[t], 4 * kSplit);
    }
    fence_mbar_init();
    *abort_flag = earlier != 0u ? 1 : 0;
    if (earlier == 0u) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_kslab);
      for (int t = 0; t < 2; ++t) {
        if (nkt[t] == 0) continue;
        mbar_arrive_expect_tx(&q_full[t], kTileBytes);
        for (int x = 0; x < kBoxes; ++x)
          tma_load_4d(s_q + t * kTileBytes + x * kBoxBytes, &tm_q, &q_full[t], x * 64, m0 + t * kTile, h, b);
      }
      for (int j = 0; j < nkt_max && j < kStages; ++j) {
        load_keys(j);
        load_values(j);
      }
    }
  }
  if (warp == kMmaWarp0) {
    tmem_alloc(tmem_base_s, 512);
    tmem_relinquish();
  }
  if (tid < kTile) {
    // slab of constants: every row [w, w, w, 0 x5 | w, w, w, 0 x5]; both 16-byte halves are equal, so the
    // 32-byte swizzle leaves it unchanged
    const uint4 v = make_uint4(pack2<kBf16>(slab_w, slab_w), pack2<kBf16>(slab_w, 0.f), 0u, 0u);
    *reinterpret_cast<uint4*>(s_ones + tid * 32) = v;
    *reinterpret_cast<uint4*>(s_ones + tid * 32 + 16) = v;
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_base_s;
  if (*abort_flag) {
    if (warp == kMmaWarp0) tmem_dealloc(tmem, 512);
    return;
  }
  const uint32_t tmem_s[2] = {tmem, tmem + kKeys};
  const uint32_t tmem_o[2] = {tmem + 256, tmem + 256 + D};
  const uint32_t tmem_p[2] = {D == 64 ? tmem + 384 : tmem + 128, D == 64 ? tmem + 448 : tmem + 160};

  if (warp == kLoadWarp) {
    // ------------------------------------------------------------------ TMA producer
    setmaxnreg_dec<R::kOtherRegs>();
    if (lane == 0) {
      for (int j = kStages; j < nkt_max; ++j) {
        const int st = j % kStages;
        const uint32_t par = ((j / kStages) - 1) & 1;
        if (!mbar_wait(&k_empty[st], par, abort_flag, status, kSiteKEmpty)) break;
        load_keys(j);
        if (!mbar_wait(&v_empty[st], par, abort_flag, status, kSiteVEmpty)) break;
        load_values(j);
      }
    }
  } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
    // ------------------------------------------------------------------ MMA issuer of query tile t
    setmaxnreg_dec<R::kOtherRegs>();
    if (lane == 0) {
      const int t = warp - kMmaWarp0;
      const int my_nkt = nkt[t];
      constexpr uint32_t idesc_s = make_idesc(kTile, kKeys, kBf16, false, false);   // S = Q K^T
      constexpr uint32_t idesc_o = make_idesc(kTile, D, kBf16, false, true);        // O += P V (V is N-major)
      const SmemDesc q_desc = make_sdesc_parts(smem_u32(s_q) + t * kTileBytes, 16, 1024);
      const SmemDesc k_desc0 = make_sdesc_parts(smem_u32(s_k), 16, 1024);
      const SmemDesc v_desc0 = make_sdesc_parts(smem_u32(s_v), kKvBoxBytes, 1024);
      const SmemDesc ones_desc = make_sdesc_slab32(smem_u32(s_ones));
      const SmemDesc kslab_desc0 = make_sdesc_slab32(smem_u32(s_kslab));
      auto issue_s = [&](int st) {
        SmemDesc k_desc = k_desc0;
        k_desc.lo += static_cast<uint32_t>(st) * (kKvBytes >> 4);
        SmemDesc slab = kslab_desc0;
        slab.lo += static_cast<uint32_t>(st) * (kSlabBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          umma_ss(tmem_s[t], sdesc_at(q_desc, (kk >> 2) * kBoxBytes + (kk & 3) * 32),
                  sdesc_at(k_desc, (kk >> 2) * kKvBoxBytes + (kk & 3) * 32), idesc_s, kk > 0);
        }
        umma_ss(tmem_s[t], sdesc_at(ones_desc, 0), sdesc_at(slab, 0), idesc_s, 1u);   // + key-norm bias
        umma_commit(&s_full[t]);
      };
      auto issue_o = [&](int st, uint32_t accumulate) {
        SmemDesc v_desc = v_desc0;
        v_desc.lo += static_cast<uint32_t>(st) * (kKvBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < kKeys / 16; ++kk)
          umma_ts(tmem_o[t], tmem_p[t] + kk * 8, sdesc_at(v_desc, kk * 2048), idesc_o, kk > 0 ? 1u : accumulate);
        umma_commit(&o_done[t]);
      };
      bool ok = true;
      if (my_nkt > 0) {
        ok = mbar_wait(&q_full[t], 0, abort_flag, status, kSiteQFull) &&
             mbar_wait(&k_full[0], 0, abort_flag, status, kSiteKFull);
        if (ok) {
          tc_fence_after_sync();
          issue_s(0);
        }
      }
      // Every stage is released by both issuers: by a commit after this tile's last MMA that reads it, or - when this
      // tile has nothing (left) to do with it - by a plain arrival made only after the stage has been filled, so that
      // an idle issuer can never arrive twice within one phase.
      auto wait_k = [&](int jj) {
        return mbar_wait(&k_full[jj % kStages], (jj / kStages) & 1, abort_flag, status, kSiteKFull);
      };
      auto wait_v = [&](int jj) {
        return mbar_wait(&v_full[jj % kStages], (jj / kStages) & 1, abort_flag, status, kSiteVFull);
      };
      if (ok && nkt_max > 0) {
        if (my_nkt > 0) {
          umma_commit(&k_empty[0]);
        } else {
          ok = wait_k(0);
          if (ok) mbar_arrive(&k_empty[0]);
        }
      }
      for (int j = 0; j < nkt_max && ok; ++j) {
        const int st = j % kStages;
        const int st_next = (j + 1) % kStages;
        bool used_k_next = false;
        if (j < my_nkt) {
          if (kSeparateP && j + 1 < my_nkt) {
            // next scores first: they only need S_t(j) to have been read
            ok = wait_k(j + 1) && mbar_wait(&s_consumed[t], j & 1, abort_flag, status, kSiteSConsumed);
            if (!ok) break;
            tc_fence_after_sync();
            issue_s(st_next);
            used_k_next = true;
          }
          ok = wait_v(j);
          ok = ok && mbar_wait(&p_full[t], j & 1, abort_flag, status, kSitePFull);
          if (!ok) break;
          tc_fence_after_sync();
          issue_o(st, j > 0 ? 1u : 0u);
          if (!kSeparateP && j + 1 < my_nkt) {
            ok = wait_k(j + 1);
            if (!ok) break;
            tc_fence_after_sync();
            issue_s(st_next);
            used_k_next = true;
          }
          umma_commit(&v_empty[st]);
        } else {
          ok = wait_v(j);
          if (!ok) break;
          mbar_arrive(&v_empty[st]);
        }
        if (j + 1 < nkt_max) {
          if (used_k_next) {
            umma_commit(&k_empty[st_next]);
          } else {
            ok = wait_k(j + 1);
            if (!ok) break;
            mbar_arrive(&k_empty[st_next]);
          }
        }
      }
    }
  } else if (warp < kLoadWarp) {
    // ------------------------------------------------------------------ softmax groups
    setmaxnreg_inc<R::kSoftmaxRegs>();
    constexpr int kCols = kKeys / kSplit;            // key columns of a tile handled by one thread
    constexpr int kChunk = kCols >= 64 && kSplit == 1 ? 64 : 32;   // columns converted and stored to TMEM at a time
    constexpr int kOCols = D / kSplit;               // output columns rescaled / written by one thread
    const int grp = warp >> 2;                       // warpgroup
    const int t = grp / kSplit;                      // query tile of this group
    const int hf = grp % kSplit;                     // which part of the tile's key columns (and of the output columns)
    const int r = tid & (kTile - 1);                 // row within the tile == TMEM lane
    const int r0 = m0 + t * kTile;
    const int row = r0 + r;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int my_nkt = nkt[t];
    const int col0 = hf * kCols;
    float m_used = -INFINITY;                        // maximum applied so far, in accumulator units times scale2
    float l_sum = 0.f;
    float row_bias = 0.f;
    if (!kSoftmax && my_nkt > 0) row_bias = qsq[static_cast<int64_t>(bh) * n_pad + row];
    bool ok = true;
    constexpr bool kSkipMax = R::kSkipMax;
    static_assert(kSplit == 1 || !kSoftmax, "threads that share a row would have to agree on its maximum and sum");
    // upper bound of this row's logits in base-2 units, c |q_row|^2, from the row's Q tile (rows past N are zero)
    float ub = INFINITY;
    bool safe = false;                               // warp-wide: no row of this warp can overflow any more
    if (kSkipMax && my_nkt > 0) {
      ok = mbar_wait(&q_full[t], 0, abort_flag, status, kSiteQFull);
      if (ok) {
        float acc = 0.f;
#pragma unroll
        for (int c16 = 0; c16 < D / 8; ++c16) {
          const uint4 qv = *reinterpret_cast<const uint4*>(s_q + t * kTileBytes + (c16 >> 3) * kBoxBytes +
                                                           sw128_offset(r, c16 & 7));
          const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 x = unpack2<kBf16>(w[i]);
            acc = fmaf(x.x, x.x, acc);
            acc = fmaf(x.y, x.y, acc);
          }
        }
        ub = acc * (0.5f * scale2);
      }
    }
    if (D == 64 && kSplit == 1 && t == 1) {
      // The two softmax groups share the MUFU pipe. Started a few hundred cycles apart, one group's exponentials
      // overlap the other group's loads and stores more often than they collide (measured: 3 % at D = 64; making
      // the groups take strict turns was slower).
      const long long t_start = clock64();
      while (clock64() - t_start < 800) {
      }
    }
    for (int j = 0; j < my_nkt; ++j) {
      ok = ok && mbar_wait(&s_full[t], j & 1, abort_flag, status, kSiteSFull);
      if (!ok) break;
      tc_fence_after_sync();

      // acc = q.k - |k|^2 / 2 for this thread's keys of the tile; the logit in base-2 units is acc * scale2
      uint32_t raw[kCols];
      {
#pragma unroll
        for (int c = 0; c < kCols / 32; ++c)
          tmem_ld_x32(tmem_s[t] + lane_sel + col0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[c * 32]));
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(&s_consumed[t]);
      }
      if (causal && (j + 1) * kKeys > r0 + 1) {
        // tiles that reach past the block's first row: key (j * kKeys + col0 + c) is visible to query (r0 + r) iff it
        // is not larger
        const int c_max = r0 + r - j * kKeys - col0;   // last visible column of this thread
#pragma unroll
        for (int c = 0; c < kCols; ++c)
          if (c > c_max) raw[c] = 0xff800000u;   // -inf
      }

      float sub;   // p = exp2(acc * scale2 - sub)
      if constexpr (kSoftmax) {
        if (!(kSkipMax && safe)) {
          // four independent three-input maxima: short dependency chains, half the instructions
          float mx0 = __uint_as_float(raw[0]), mx1 = __uint_as_float(raw[1]), mx2 = __uint_as_float(raw[2]),
                mx3 = __uint_as_float(raw[3]);
#pragma unroll
          for (int c = 4; c + 8 <= kCols; c += 8) {
            mx0 = fmax3(mx0, __uint_as_float(raw[c + 0]), __uint_as_float(raw[c + 1]));
            mx1 = fmax3(mx1, __uint_as_float(raw[c + 2]), __uint_as_float(raw[c + 3]));
            mx2 = fmax3(mx2, __uint_as_float(raw[c + 4]), __uint_as_float(raw[c + 5]));
            mx3 = fmax3(mx3, __uint_as_float(raw[c + 6]), __uint_as_float(raw[c + 7]));
          }
          mx0 = fmax3(mx0, __uint_as_float(raw[kCols - 4]), __uint_as_float(raw[kCols - 3]));
          mx1 = fmax3(mx1, __uint_as_float(raw[kCols - 2]), __uint_as_float(raw[kCols - 1]));
          const float tile_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
          const float m_new = fmaxf(m_used, tile_max * scale2);
          const bool need = (m_new - m_used) > kRescaleThreshold;
          float alpha = 1.f;
          if (need) {
            alpha = ex2_approx(m_used - m_new);
            m_used = m_new;
            l_sum *= alpha;
          }
          if (j > 0 && __any_sync(0xffffffffu, need)) {
            // O_t holds the sum over key tiles < j; wait until the last P V has landed, then rescale this thread's
            // share of the row.
            ok = mbar_wait(&o_done[t], (j - 1) & 1, abort_flag, status, kSiteODone);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < kOCols / 32; ++c) {
              uint32_t o[32];
              tmem_ld_x32(tmem_o[t] + lane_sel + hf * kOCols + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_x32(tmem_o[t] + lane_sel + hf * kOCols + c * 32, o);
            }
          }
          if constexpr (kSkipMax) safe = __all_sync(0xffffffffu, ub - m_used <= kSafeGap);
        }
        sub = m_used;
      } else {
        sub = row_bias;
      }

      bool waited_o = j == 0;   // P's own columns are free once O_t += P_t V_(j-1) has completed
      const float neg_sub = -sub;
      float ps0 = 0.f, ps1 = 0.f, ps2 = 0.f, ps3 = 0.f;
#pragma unroll
      for (int c = 0; c < kCols / kChunk; ++c) {
        uint32_t packed[kChunk / 2];
#pragma unroll
        for (int i = 0; i < kChunk / 2; i += 2) {
          float a0, a1, a2, a3;
          ffma2_bcast(a0, a1, __uint_as_float(raw[c * kChunk + 2 * i + 0]), __uint_as_float(raw[c * kChunk + 2 * i + 1]),
                      scale2, neg_sub);
          ffma2_bcast(a2, a3, __uint_as_float(raw[c * kChunk + 2 * i + 2]), __uint_as_float(raw[c * kChunk + 2 * i + 3]),
                      scale2, neg_sub);
          const float p0 = ex2_approx(a0), p1 = ex2_approx(a1), p2 = ex2_approx(a2), p3 = ex2_approx(a3);
          fadd2(ps0, ps1, ps0, ps1, p0, p1);
          fadd2(ps2, ps3, ps2, ps3, p2, p3);
          packed[i] = pack2<kBf16>(p0, p1);
          packed[i + 1] = pack2<kBf16>(p2, p3);
        }
        if (!waited_o) {
          ok = mbar_wait(&o_done[t], (j - 1) & 1, abort_flag, status, kSitePFree);
          if (!ok) break;
          tc_fence_after_sync();
          waited_o = true;
        }
        // key column c holds its 16-bit P in column c / 2 of the tile's P block
        if constexpr (kChunk == 64) {
          tmem_st_x32(tmem_p[t] + lane_sel + (col0 + c * kChunk) / 2, packed);
        } else {
          tmem_st_x16(tmem_p[t] + lane_sel + (col0 + c * kChunk) / 2, packed);
        }
      }
      if (!ok) break;
      l_sum += (ps0 + ps1) + (ps2 + ps3);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive_warp(&p_full[t]);
    }

    if (ok && my_nkt > 0) ok = mbar_wait(&o_done[t], (my_nkt - 1) & 1, abort_flag, status, kSiteODoneFinal);
    if (ok && my_nkt > 0) {
      tc_fence_after_sync();
      const float inv = kSoftmax ? (1.0f / l_sum) : 1.0f;
      uint8_t* stage = s_q + t * kTileBytes;       // Q_t is dead once the last S_t MMA has completed
#pragma unroll
      for (int c = 0; c < kOCols / 32; ++c) {
        uint32_t o[32];
        tmem_ld_x32(tmem_o[t] + lane_sel + hf * kOCols + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            w[i] = pack2<kBf16>(__uint_as_float(o[g * 8 + 2 * i]) * inv, __uint_as_float(o[g * 8 + 2 * i + 1]) * inv);
          const int col16 = (hf * kOCols) / 8 + c * 4 + g;             // 16-byte chunk index along D
          *reinterpret_cast<uint4*>(stage + (col16 >> 3) * kBoxBytes + sw128_offset(r, col16 & 7)) =
              make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(&grp_sync[t]);
      ok = mbar_wait(&grp_sync[t], 0, abort_flag, status, kSiteGroup);
      if (ok && r == 0 && hf == 0) {
        for (int x = 0; x < kBoxes; ++x) tma_store_4d(&tm_o, stage + x * kBoxBytes, x * 64, r0, h, b);
        tma_store_commit();
        tma_store_wait_read();   // the CTA may exit once the staging tile has been read
      }
      if (kSoftmax && hf == 0 && row < N) lse[static_cast<int64_t>(bh) * N + row] = m_used + log2f(l_sum);
    }
  } else {
    setmaxnreg_dec<R::kOtherRegs>();   // idle warp of the producer / issuer warpgroup
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // give copies and MMAs still in flight time to land before shared memory and TMEM are released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp0) tmem_dealloc(tmem, 512);
}

}  // namespace fwd

template <int D, bool kSoftmax, bool kBf16>
static cudaError_t launch_fwd_t(const FwdArgs& a, cudaStream_t stream) {
  auto kernel = fwd::rbf_fwd_kernel<D, kSoftmax, kBf16>;
  constexpr int smem = fwd::Smem<D>::kDynamic;
  static PerDeviceFlags configured{};
  {
    const cudaError_t ce = ensure_dynamic_smem(kernel, smem, configured);
    if (ce != cudaSuccess) return ce;
  }
  const unsigned blocks = (a.N + 2 * kTile - 1) / (2 * kTile), heads = a.B * a.H;
  dim3 grid(a.causal ? heads : blocks, a.causal ? blocks : heads);
  kernel<<<grid, fwd::Roles<D, kSoftmax, kBf16>::kThreads, smem, stream>>>(a.tm_q, a.tm_k, a.tm_v, a.tm_o, a.tm_kslab, a.qsq, a.lse, a.status,
                                                a.H, a.N, a.n_pad, a.causal, a.scale2, a.slab_w);
  return cudaGetLastError();
}

cudaError_t launch_fwd(const FwdArgs& a, bool bf16, int D, bool softmax, cudaStream_t stream) {
#define RBF_FWD_CASE(DD, SM, BF) \
  if (D == DD && softmax == SM && bf16 == BF) return launch_fwd_t<DD, SM, BF>(a, stream);
  RBF_FWD_CASE(64, true, true)
  RBF_FWD_CASE(64, false, true)
  RBF_FWD_CASE(128, true, true)
  RBF_FWD_CASE(128, false, true)
  RBF_FWD_CASE(64, true, false)
  RBF_FWD_CASE(64, false, false)
  RBF_FWD_CASE(128, true, false)
  RBF_FWD_CASE(128, false, false)
#undef RBF_FWD_CASE
  return cudaErrorInvalidValue;
}


}  // namespace rbf
