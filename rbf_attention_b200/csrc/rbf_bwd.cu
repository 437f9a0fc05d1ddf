// Fused RBF attention backward for sm_100a: one kernel template, instantiated in two modes.
//
//   mode kKeyStationary   (dK, dV): a CTA owns 128 keys and streams the query / dO tiles past them.
//   mode kQueryStationary (dQ)    : a CTA owns 128 queries and streams the key / value tiles.
//
// With A1, A2 the stationary tiles and B1, B2 the streamed ones (K, V, Q, dO resp. Q, dO, K, V) both modes run
//   S  = A1 B1^T,  dP = A2 B2^T                          (smem x smem MMAs into TMEM)
//   P  = exp2(S * 2g log2e - row_stat[r] - col_stat[c])  (one thread per stationary row r, in registers)
//   dS = P * (dP - delta)
//   accS += dS B1            (dK resp. dQ;  dS is written back to TMEM as the 16-bit A operand)
//   accP += P  B2            (dV; key-stationary mode only)
// and finish with out_S = 2g (accS - w * rowsum_c(dS)[r] * A1[r]): the second term is the gradient through
// the squared-norm bias (|k|^2 for dK, always; |q|^2 for dQ in the non-softmax variant only).
//
// For the softmax variant row/col statistics are the key norms c|k|^2 and the forward's base-2 LSE, and
// delta = rowsum(O * dO); for the non-softmax variant the LSE is replaced by c|q|^2 and delta is zero.
//
// Roles: warps 0-3 compute (one thread per stationary row), warp 4 TMA producer, warp 5 MMA issuer.
#include "common.cuh"
#include "launch.h"

namespace rbf {

namespace bwd {

static constexpr int kThreads = 192;
static constexpr int kLoadWarp = 4;
static constexpr int kMmaWarp = 5;

enum Mode : int { kKeyStationary = 0, kQueryStationary = 1 };

template <int D, int kMode>
struct Cfg {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kSBufs = (D == 64) ? 2 : 1;            // S accumulators in TMEM
  static constexpr int kB1Stages = (D == 64) ? 3 : 2;
  static constexpr int kB2Stages = (D == 64) ? 3 : 2;
  // TMEM columns
  static constexpr int kColS = 0;
  static constexpr int kColDP = kSBufs * kTile;
  static constexpr int kColAccS = kColDP + kTile;
  static constexpr int kColAccP = kColAccS + D;               // key-stationary mode only
  static constexpr int kColsUsed = kColAccP + (kMode == kKeyStationary ? D : 0);
  static_assert(kColsUsed <= 512, "TMEM budget");
  // shared memory
  static constexpr int kA1 = 0;
  static constexpr int kA2 = kA1 + kTileBytes;
  static constexpr int kB1 = kA2 + kTileBytes;
  static constexpr int kB2 = kB1 + kB1Stages * kTileBytes;
  static constexpr int kVec = kB2 + kB2Stages * kTileBytes;  // [2 buffers][2 vectors][128] floats
  static constexpr int kBars = kVec + 2 * 2 * kTile * 4;
  static constexpr int kNumBars = 1 + 2 * kB1Stages + 2 * kB2Stages + 2 + 1 + 2 + 1 + 1 + 1;
  static constexpr int kMisc = kBars + kNumBars * 8;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

enum Site : uint32_t {
  kSiteAFull = 32, kSiteB1Full, kSiteB2Full, kSiteB1Empty, kSiteB2Empty, kSiteSFull, kSiteDPFull, kSitePFull,
  kSiteDSFull, kSiteAccDone, kSiteGroup
};

struct Params {
  const float* row_stat;   // indexed by stationary row
  int row_stat_pitch, row_stat_limit;
  const float* col_stat;   // indexed by streamed row
  int col_stat_pitch, col_stat_limit;
  const float* delta;      // (B*H, n_pad), zero padded
  DeviceStatus* status;
  int H, N, n_pad, causal;
  float scale2, grad_scale;
  int norm_term;           // 1: subtract rowsum(dS) * A1 row in the epilogue
};

template <int D, int kMode, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
rbf_bwd_kernel(const __grid_constant__ CUtensorMap tm_a1, const __grid_constant__ CUtensorMap tm_a2,
               const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_b2,
               const __grid_constant__ CUtensorMap tm_out_s, const __grid_constant__ CUtensorMap tm_out_p,
               const Params p) {
  using C = Cfg<D, kMode>;
  constexpr int kBoxes = D / 64;
  constexpr int kBoxBytes = kTile * 128;
  constexpr uint32_t kTileBytes = C::kTileBytes;
  constexpr bool kHasAccP = (kMode == kKeyStationary);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_a1 = smem + C::kA1;
  uint8_t* s_a2 = smem + C::kA2;
  uint8_t* s_b1 = smem + C::kB1;
  uint8_t* s_b2 = smem + C::kB2;
  float* s_vec = reinterpret_cast<float*>(smem + C::kVec);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBars);
  uint64_t* a_full = bars;
  uint64_t* b1_full = a_full + 1;
  uint64_t* b1_empty = b1_full + C::kB1Stages;
  uint64_t* b2_full = b1_empty + C::kB1Stages;
  uint64_t* b2_empty = b2_full + C::kB2Stages;
  uint64_t* s_full = b2_empty + C::kB2Stages;   // [2]
  uint64_t* dp_full = s_full + 2;
  uint64_t* p_full = dp_full + 1;            // [2], one per S buffer
  uint64_t* ds_full = p_full + 2;
  uint64_t* acc_done = ds_full + 1;
  uint64_t* grp_sync = acc_done + 1;
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + C::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::kMisc + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int n_tiles = (p.N + kTile - 1) / kTile;
  // Key-stationary: tile 0 sees every query tile (heaviest) so natural order is heaviest-first.
  // Query-stationary: the last tile sees every key tile, so reverse.
  const int at = (kMode == kQueryStationary && p.causal) ? (n_tiles - 1 - static_cast<int>(blockIdx.x))
                                                         : static_cast<int>(blockIdx.x);
  const int a_row0 = at * kTile;
  int first, cnt;   // streamed tiles first .. first + cnt - 1
  if (!p.causal) {
    first = 0;
    cnt = n_tiles;
  } else if (kMode == kKeyStationary) {
    first = at;
    cnt = n_tiles - at;
  } else {
    first = 0;
    cnt = at + 1;
  }
  const int diag = p.causal ? at : -1;   // streamed tile index that straddles the diagonal

  // A wait that ran out in an earlier CTA of this launch ends the whole launch quickly: later CTAs leave at once.
  if (tid == 0) *abort_flag = (*reinterpret_cast<volatile unsigned int*>(&p.status->code) != 0u) ? 1 : 0;
  __syncthreads();
  if (*abort_flag) return;

  if (tid == 0) {
    mbar_init(a_full, 1);
    for (int s = 0; s < C::kB1Stages; ++s) { mbar_init(&b1_full[s], 1); mbar_init(&b1_empty[s], 1); }
    for (int s = 0; s < C::kB2Stages; ++s) { mbar_init(&b2_full[s], 1); mbar_init(&b2_empty[s], 1); }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(dp_full, 1);
    mbar_init(&p_full[0], 4);                 // one arrival per compute warp
    mbar_init(&p_full[1], 4);
    mbar_init(ds_full, 4);
    mbar_init(acc_done, 1);
    mbar_init(grp_sync, 4);
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_base_s;

  if (warp == kLoadWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_a1);
      tma_prefetch_desc(&tm_a2);
      tma_prefetch_desc(&tm_b1);
      tma_prefetch_desc(&tm_b2);
      mbar_arrive_expect_tx(a_full, 2 * kTileBytes);
      for (int x = 0; x < kBoxes; ++x) {
        tma_load_4d(s_a1 + x * kBoxBytes, &tm_a1, a_full, x * 64, a_row0, h, b);
        tma_load_4d(s_a2 + x * kBoxBytes, &tm_a2, a_full, x * 64, a_row0, h, b);
      }
      for (int n = 0; n < cnt; ++n) {
        const int row0 = (first + n) * kTile;
        const int s1 = n % C::kB1Stages, s2 = n % C::kB2Stages;
        if (n >= C::kB1Stages &&
            !mbar_wait(&b1_empty[s1], ((n / C::kB1Stages) - 1) & 1, abort_flag, p.status, kSiteB1Empty))
          break;
        mbar_arrive_expect_tx(&b1_full[s1], kTileBytes);
        for (int x = 0; x < kBoxes; ++x)
          tma_load_4d(s_b1 + s1 * kTileBytes + x * kBoxBytes, &tm_b1, &b1_full[s1], x * 64, row0, h, b);
        if (n >= C::kB2Stages &&
            !mbar_wait(&b2_empty[s2], ((n / C::kB2Stages) - 1) & 1, abort_flag, p.status, kSiteB2Empty))
          break;
        mbar_arrive_expect_tx(&b2_full[s2], kTileBytes);
        for (int x = 0; x < kBoxes; ++x)
          tma_load_4d(s_b2 + s2 * kTileBytes + x * kBoxBytes, &tm_b2, &b2_full[s2], x * 64, row0, h, b);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(kTile, kTile, kBf16, false, false);   // A K-major, B K-major
      constexpr uint32_t idesc_acc = make_idesc(kTile, D, kBf16, false, true);      // A from TMEM, B N-major
      const uint32_t a1 = smem_u32(s_a1), a2 = smem_u32(s_a2), b1 = smem_u32(s_b1), b2 = smem_u32(s_b2);
      // S-like product: tmem_dst = A (stationary tile at a_addr) * B^T (streamed tile at b_addr)
      auto issue_qk = [&](uint32_t dst, uint32_t a_addr, uint32_t b_addr) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
          umma_ss(dst, make_sdesc_sw128(a_addr + off, 16, 1024), make_sdesc_sw128(b_addr + off, 16, 1024), idesc_s,
                  kk > 0);
        }
      };
      // accumulator product: tmem_dst (+)= A (16-bit in TMEM at a_tmem) * B (streamed tile, rows = reduction index)
      auto issue_acc = [&](uint32_t dst, uint32_t a_tmem, uint32_t b_addr, bool accumulate) {
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          umma_ts(dst, a_tmem + kk * 8, make_sdesc_sw128(b_addr + kk * 2048, kBoxBytes, 1024), idesc_acc,
                  (accumulate || kk > 0) ? 1u : 0u);
        }
      };
      auto wait_b1 = [&](int n) {
        return mbar_wait(&b1_full[n % C::kB1Stages], (n / C::kB1Stages) & 1, abort_flag, p.status, kSiteB1Full);
      };
      auto wait_b2 = [&](int n) {
        return mbar_wait(&b2_full[n % C::kB2Stages], (n / C::kB2Stages) & 1, abort_flag, p.status, kSiteB2Full);
      };
      auto issue_s = [&](int n) {
        const int sb = n % C::kSBufs;
        issue_qk(tmem + C::kColS + sb * kTile, a1, b1 + (n % C::kB1Stages) * kTileBytes);
        umma_commit(&s_full[sb]);
      };
      auto issue_dp = [&](int n) {
        issue_qk(tmem + C::kColDP, a2, b2 + (n % C::kB2Stages) * kTileBytes);
        umma_commit(dp_full);
      };

      bool ok = mbar_wait(a_full, 0, abort_flag, p.status, kSiteAFull);
      if (ok) ok = wait_b1(0);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0);
        ok = wait_b2(0);
      }
      if (ok) {
        tc_fence_after_sync();
        issue_dp(0);
        if (C::kSBufs == 2 && cnt > 1) {
          ok = wait_b1(1);
          if (ok) {
            tc_fence_after_sync();
            issue_s(1);
          }
        }
      }
      for (int n = 0; n < cnt && ok; ++n) {
        const int sb = n % C::kSBufs;
        if (kHasAccP) {
          ok = mbar_wait(&p_full[sb], (n / C::kSBufs) & 1, abort_flag, p.status, kSitePFull);
          if (!ok) break;
          tc_fence_after_sync();
          issue_acc(tmem + C::kColAccP, tmem + C::kColS + sb * kTile, b2 + (n % C::kB2Stages) * kTileBytes, n > 0);
        }
        ok = mbar_wait(ds_full, n & 1, abort_flag, p.status, kSiteDSFull);
        if (!ok) break;
        tc_fence_after_sync();
        issue_acc(tmem + C::kColAccS, tmem + C::kColDP, b1 + (n % C::kB1Stages) * kTileBytes, n > 0);
        umma_commit(&b1_empty[n % C::kB1Stages]);
        umma_commit(&b2_empty[n % C::kB2Stages]);
        if (n + 1 < cnt) {
          if (C::kSBufs == 1) {
            ok = wait_b1(n + 1);
            if (!ok) break;
            tc_fence_after_sync();
            issue_s(n + 1);
          }
          ok = wait_b2(n + 1);
          if (!ok) break;
          tc_fence_after_sync();
          issue_dp(n + 1);
          if (C::kSBufs == 2 && n + 2 < cnt) {
            ok = wait_b1(n + 2);
            if (!ok) break;
            tc_fence_after_sync();
            issue_s(n + 2);
          }
        }
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int r = tid;                                   // stationary row within the tile == TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
    const int a_row = a_row0 + r;
    const int64_t bh64 = bh;
    float row_stat = INFINITY;
    if (a_row < p.row_stat_limit) row_stat = p.row_stat[bh64 * p.row_stat_pitch + a_row];
    float row_delta = 0.f;
    if (kMode == kQueryStationary) row_delta = p.delta[bh64 * p.n_pad + a_row];
    const float neg_row_stat = -row_stat;
    float ds_rowsum = 0.f;
    bool ok = true;
    uint32_t grp_phase = 0;
    auto group_sync = [&]() -> bool {
      mbar_arrive_warp(grp_sync);
      const bool done = mbar_wait(grp_sync, grp_phase & 1, abort_flag, p.status, kSiteGroup);
      ++grp_phase;
      return done;
    };
    // column statistics of streamed tile n: thread r fetches entry r; buffers alternate
    auto fetch_col = [&](int n, float& cs, float& cd) {
      const int idx = (first + n) * kTile + r;
      cs = (idx < p.col_stat_limit) ? p.col_stat[bh64 * p.col_stat_pitch + idx] : INFINITY;
      cd = 0.f;
      if (kMode == kKeyStationary) cd = p.delta[bh64 * p.n_pad + idx];
    };
    {
      float cs, cd;
      fetch_col(0, cs, cd);
      s_vec[r] = cs;
      s_vec[kTile + r] = cd;
    }

    for (int n = 0; n < cnt; ++n) {
      const int sb = n % C::kSBufs;
      float cs_next = 0.f, cd_next = 0.f;
      if (n + 1 < cnt) fetch_col(n + 1, cs_next, cd_next);
      ok = group_sync() && mbar_wait(&s_full[sb], (n / C::kSBufs) & 1, abort_flag, p.status, kSiteSFull);
      if (!ok) break;
      tc_fence_after_sync();
      const float* vbuf = s_vec + (n & 1) * 2 * kTile;
      const float4* cs4 = reinterpret_cast<const float4*>(vbuf);
      const float4* cd4 = reinterpret_cast<const float4*>(vbuf + kTile);

      float pr[kTile];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_ld_x32(tmem + C::kColS + sb * kTile + lane_sel + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 cs = cs4[c * 8 + i];
          pr[c * 32 + i * 4 + 0] = ex2_approx(fmaf(__uint_as_float(raw[i * 4 + 0]), p.scale2, neg_row_stat) - cs.x);
          pr[c * 32 + i * 4 + 1] = ex2_approx(fmaf(__uint_as_float(raw[i * 4 + 1]), p.scale2, neg_row_stat) - cs.y);
          pr[c * 32 + i * 4 + 2] = ex2_approx(fmaf(__uint_as_float(raw[i * 4 + 2]), p.scale2, neg_row_stat) - cs.z);
          pr[c * 32 + i * 4 + 3] = ex2_approx(fmaf(__uint_as_float(raw[i * 4 + 3]), p.scale2, neg_row_stat) - cs.w);
        }
      }
      if (first + n == diag) {
        // key-stationary: row = key, column = query, visible iff column >= row; query-stationary: column <= row
#pragma unroll
        for (int c = 0; c < kTile; ++c) {
          const bool hidden = (kMode == kKeyStationary) ? (c < r) : (c > r);
          if (hidden) pr[c] = 0.f;
        }
      }
      if (kHasAccP) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t packed[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) packed[i] = pack2<kBf16>(pr[c * 64 + 2 * i], pr[c * 64 + 2 * i + 1]);
          tmem_st_x32(tmem + C::kColS + sb * kTile + lane_sel + c * 32, packed);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(&p_full[sb]);
      }

      ok = mbar_wait(dp_full, n & 1, abort_flag, p.status, kSiteDPFull);
      if (!ok) break;
      tc_fence_after_sync();
      // dS = P * (dP - delta): read dP in four 32-column chunks, then write the packed dS over dP's columns
      uint32_t ds_packed[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_ld_x32(tmem + C::kColDP + lane_sel + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float4 cd = make_float4(row_delta, row_delta, row_delta, row_delta);
          if (kMode == kKeyStationary) cd = cd4[c * 8 + i];
          const float d0 = pr[c * 32 + i * 4 + 0] * (__uint_as_float(raw[i * 4 + 0]) - cd.x);
          const float d1 = pr[c * 32 + i * 4 + 1] * (__uint_as_float(raw[i * 4 + 1]) - cd.y);
          const float d2 = pr[c * 32 + i * 4 + 2] * (__uint_as_float(raw[i * 4 + 2]) - cd.z);
          const float d3 = pr[c * 32 + i * 4 + 3] * (__uint_as_float(raw[i * 4 + 3]) - cd.w);
          ds_rowsum += (d0 + d1) + (d2 + d3);
          ds_packed[c * 16 + i * 2 + 0] = pack2<kBf16>(d0, d1);
          ds_packed[c * 16 + i * 2 + 1] = pack2<kBf16>(d2, d3);
        }
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t chunk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) chunk[i] = ds_packed[c * 32 + i];
        tmem_st_x32(tmem + C::kColDP + lane_sel + c * 32, chunk);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive_warp(ds_full);
      if (n + 1 < cnt) {
        float* nbuf = s_vec + ((n + 1) & 1) * 2 * kTile;
        nbuf[r] = cs_next;
        nbuf[kTile + r] = cd_next;
      }
    }

    if (ok) ok = mbar_wait(acc_done, 0, abort_flag, p.status, kSiteAccDone);
    if (ok) {
      tc_fence_after_sync();
      // All MMAs are complete: the B1 ring is free and serves as staging for the TMA stores.
      uint8_t* stage_s = s_b1;
      uint8_t* stage_p = s_b1 + kTileBytes;
      const float w = p.norm_term ? ds_rowsum : 0.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t acc[32];
        tmem_ld_x32(tmem + C::kColAccS + lane_sel + c * 32, acc);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int col16 = c * 4 + g;                 // 16-byte chunk along D
          const uint32_t off = (col16 >> 3) * kBoxBytes + sw128_offset(r, col16 & 7);
          const uint4 a_raw = *reinterpret_cast<const uint4*>(s_a1 + off);
          const uint32_t aw[4] = {a_raw.x, a_raw.y, a_raw.z, a_raw.w};
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 av = unpack2<kBf16>(aw[i]);
            const float x0 = p.grad_scale * fmaf(-w, av.x, __uint_as_float(acc[g * 8 + 2 * i]));
            const float x1 = p.grad_scale * fmaf(-w, av.y, __uint_as_float(acc[g * 8 + 2 * i + 1]));
            o[i] = pack2<kBf16>(x0, x1);
          }
          *reinterpret_cast<uint4*>(stage_s + off) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      if (kHasAccP) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t acc[32];
          tmem_ld_x32(tmem + C::kColAccP + lane_sel + c * 32, acc);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col16 = c * 4 + g;
            const uint32_t off = (col16 >> 3) * kBoxBytes + sw128_offset(r, col16 & 7);
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              o[i] = pack2<kBf16>(__uint_as_float(acc[g * 8 + 2 * i]), __uint_as_float(acc[g * 8 + 2 * i + 1]));
            *reinterpret_cast<uint4*>(stage_p + off) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
      fence_proxy_async_smem();
      ok = group_sync();
      if (ok && r == 0) {
        for (int x = 0; x < kBoxes; ++x) tma_store_4d(&tm_out_s, stage_s + x * kBoxBytes, x * 64, a_row0, h, b);
        if (kHasAccP)
          for (int x = 0; x < kBoxes; ++x) tma_store_4d(&tm_out_p, stage_p + x * kBoxBytes, x * 64, a_row0, h, b);
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
  if (warp == kMmaWarp) tmem_dealloc(tmem, 512);
}

template <int D, int kMode, bool kBf16>
static cudaError_t launch_t(const BwdArgs& a, bool softmax, cudaStream_t stream) {
  auto kernel = rbf_bwd_kernel<D, kMode, kBf16>;
  constexpr int smem = Cfg<D, kMode>::kDynamic;
  static PerDeviceFlags configured{};
  {
    const cudaError_t ce = ensure_dynamic_smem(kernel, smem, configured);
    if (ce != cudaSuccess) return ce;
  }
  Params p{};
  p.delta = a.delta;
  p.status = a.status;
  p.H = a.H; p.N = a.N; p.n_pad = a.n_pad; p.causal = a.causal;
  p.scale2 = a.scale2; p.grad_scale = a.grad_scale;
  dim3 grid((a.N + kTile - 1) / kTile, a.B * a.H);
  if (kMode == kKeyStationary) {
    p.row_stat = a.ksq; p.row_stat_pitch = a.n_pad; p.row_stat_limit = a.n_pad;
    p.col_stat = a.row_bias; p.col_stat_pitch = a.row_bias_pitch; p.col_stat_limit = a.N;
    p.norm_term = 1;
    kernel<<<grid, kThreads, smem, stream>>>(a.tm_k, a.tm_v, a.tm_q, a.tm_do, a.tm_dk, a.tm_dv, p);
  } else {
    p.row_stat = a.row_bias; p.row_stat_pitch = a.row_bias_pitch; p.row_stat_limit = a.N;
    p.col_stat = a.ksq; p.col_stat_pitch = a.n_pad; p.col_stat_limit = a.n_pad;
    p.norm_term = softmax ? 0 : 1;
    kernel<<<grid, kThreads, smem, stream>>>(a.tm_q, a.tm_do, a.tm_k, a.tm_v, a.tm_dq, a.tm_dq, p);
  }
  return cudaGetLastError();
}

}  // namespace bwd

cudaError_t launch_bwd_dkdv(const BwdArgs& a, bool bf16, int D, bool softmax, cudaStream_t stream) {
  if (D == 64) return bf16 ? bwd::launch_t<64, bwd::kKeyStationary, true>(a, softmax, stream)
                           : bwd::launch_t<64, bwd::kKeyStationary, false>(a, softmax, stream);
  if (D == 128) return bf16 ? bwd::launch_t<128, bwd::kKeyStationary, true>(a, softmax, stream)
                            : bwd::launch_t<128, bwd::kKeyStationary, false>(a, softmax, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_bwd_dq(const BwdArgs& a, bool bf16, int D, bool softmax, cudaStream_t stream) {
  if (D == 64) return bf16 ? bwd::launch_t<64, bwd::kQueryStationary, true>(a, softmax, stream)
                           : bwd::launch_t<64, bwd::kQueryStationary, false>(a, softmax, stream);
  if (D == 128) return bf16 ? bwd::launch_t<128, bwd::kQueryStationary, true>(a, softmax, stream)
                            : bwd::launch_t<128, bwd::kQueryStationary, false>(a, softmax, stream);
  return cudaErrorInvalidValue;
}

}  // namespace rbf
