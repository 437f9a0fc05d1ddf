// Fused RBF attention forward for sm_100a.
//
//   softmax variant      O = softmax_j(2g q_i.k_j - g|k_j|^2) V,  L_i = log2 sum_j 2^(log2e * logit_ij)
//   non-softmax variant  O = exp(-g|q_i - k_j|^2) V
//
// A work item is 256 consecutive query rows of one (batch, head) as two 128-row tiles; a CTA walks the item's
// key tiles (128 keys at D = 64, 64 keys at D = 128) once for both. At D = 64 the launch is persistent: one CTA per
// SM takes items from a launch-wide counter (heaviest causal items first), all barriers and the
// K/V ring run on across items, the next item's Q and first K/V tiles travel and its first scores are issued while
// the current item's output is normalised and stored, so that set-up, first loads and pipeline fill are paid once per
// CTA and not once per item (an item is 2 to 32 key tiles long at N = 4096, 1 to 9 at N = 1028). At D = 128 (items
// of 64+ key tiles at the sizes it is used at; shared memory has no room for an output staging tile beside Q) every
// CTA has one item. Roles:
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
  // output staging of the two query tiles: tiles of its own in the persistent launch (the next item's Q is loaded
  // while the previous output is still being stored), else the dead Q tiles
  static constexpr bool kPersistent = (D == 64);
  static constexpr int kStage = kPersistent ? kOnes + kTile * 32 : kQ;
  static constexpr int kBars = kOnes + kTile * 32 + (kPersistent ? 2 * kTileBytes : 0);
  static constexpr int kItemSlots = 4;                     // ring of work item numbers, producer -> all other roles
  static constexpr int kNumBars = 2 + 4 * kStages + 10 + 4 + 2 * kItemSlots;
  static constexpr int kMisc = kBars + kNumBars * 8;        // tmem base, abort flag
  static constexpr int kTotal = kMisc + 16 + 16 * kItemSlots;
  static constexpr int kDynamic = kTotal + 1024;            // slack for 1024-byte alignment
};

enum Site : uint32_t {
  kSiteQFull = 1, kSiteKFull, kSiteVFull, kSiteKEmpty, kSiteVEmpty, kSiteSFull, kSitePFull, kSiteODone,
  kSiteODoneFinal, kSiteGroup, kSiteSConsumed, kSitePFree, kSiteQFree, kSiteStageFree, kSiteItemFull, kSiteItemEmpty
};

// Work item w of a launch: causal launches run the heaviest query blocks first, (batch, head) fastest, so that all
// heads work on equally long items at any time and the tail of the launch is short (measured 6 % faster); non-causal
// launches run a head's query blocks one after the other, which keeps its K/V hot in L2 (measured 20 % faster).
struct Item {
  int bh, b, h, m0;
  int nkt0, nkt1;  // key tiles of the two query tiles (0: the tile lies past N); scalars: no indexed local array
  int nkt_max;
  __device__ __forceinline__ int nkt(int t) const { return t == 0 ? nkt0 : nkt1; }
};
// key tiles of the item's two query tiles from its first row (shifts only: the producer thread decodes an item number -
// four integer divisions - once and hands bh, b, h, m0 to the other roles)
template <int kKeys>
__device__ __forceinline__ void count_key_tiles(Item& it, int N, int causal) {
  const int all = (N + kKeys - 1) / kKeys;
  const int r1 = it.m0 + kTile;
  it.nkt0 = (it.m0 < 0 || it.m0 >= N) ? 0 : (causal ? min(all, (it.m0 + kTile) / kKeys) : all);
  it.nkt1 = (r1 >= N) ? 0 : (causal ? min(all, (r1 + kTile) / kKeys) : all);
  it.nkt_max = max(it.nkt0, it.nkt1);
}
template <int kKeys>
__device__ __forceinline__ Item get_item(int w, int heads, int blocks, int H, int N, int causal) {
  Item it;
  int mb;
  if (causal) {
    it.bh = w % heads;
    mb = blocks - 1 - w / heads;
  } else {
    it.bh = w / blocks;
    mb = w % blocks;
  }
  it.b = it.bh / H;
  it.h = it.bh % H;
  // An odd number of query tiles leaves one item with a single tile. Under the causal mask the pairs are counted from
  // the last tile down - (T-1, T-2), ..., (2, 1) and tile 0 alone, m0 = -kTile - so that the lone tile is the cheapest
  // one (one key tile) and not the dearest: at N = 1028 an item sequence of 9 + 7 + 5 + 3 + 1 key-tile steps per head
  // instead of 9 + 8 + 6 + 4 + 2.
  const int odd_shift = (causal && (((N + kTile - 1) / kTile) & 1)) ? kTile : 0;
  it.m0 = mb * 2 * kTile - odd_shift;
  count_key_tiles<kKeys>(it, N, causal);
  return it;
}

template <int D, bool kSoftmax, bool kBf16>
__global__ void __launch_bounds__(Roles<D, kSoftmax, kBf16>::kThreads, 1)
rbf_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               const __grid_constant__ CUtensorMap tm_kslab, const float* __restrict__ qsq,
               float* __restrict__ lse, DeviceStatus* status, int H, int N, int n_pad, int causal, float scale2,
               float slab_w, int heads, int blocks, unsigned int* work) {
  using L = Smem<D>;
  using R = Roles<D, kSoftmax, kBf16>;
  constexpr bool kPersistent = L::kPersistent;
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

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem + L::kQ;
  uint8_t* s_k = smem + L::kK;
  uint8_t* s_v = smem + L::kV;
  uint8_t* s_kslab = smem + L::kKSlab;
  uint8_t* s_ones = smem + L::kOnes;
  uint8_t* s_stage = smem + L::kStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* q_full = bars;                       // [2]
  uint64_t* k_full = bars + 2;                   // [kStages]
  uint64_t* k_empty = k_full + kStages;          // two arrivals: one per issuer
  uint64_t* v_full = k_empty + kStages;
  uint64_t* v_empty = v_full + kStages;          // two arrivals
  uint64_t* s_full = v_empty + kStages;          // [2]
  uint64_t* p_full = s_full + 2;                 // [2]
  uint64_t* o_done = p_full + 2;                 // [2]
  uint64_t* grp_sync = o_done + 2;               // [2] rendezvous of the warps of a query tile
  uint64_t* s_consumed = grp_sync + 2;           // [2] the softmax group holds S_t(j) in registers
  uint64_t* q_free = s_consumed + 2;             // [2] persistent: Q_t may be overwritten (issuer + softmax warps)
  uint64_t* stage_free = q_free + 2;             // [2] persistent: the previous output store has read its staging tile
  uint64_t* item_full = stage_free + 2;          // [kItemSlots] the producer has published the CTA's n-th item number
  uint64_t* item_empty = item_full + L::kItemSlots;   // [kItemSlots] every other role has read it
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);
  volatile int4* s_items = reinterpret_cast<volatile int4*>(smem + L::kMisc + 16);   // {bh (< 0: end), b, h, m0}
  // work item the CTA's producer is loading (the status word of a wait that runs out names it, not the block index)
  volatile int* s_unit = reinterpret_cast<volatile int*>(smem + L::kMisc + 8);
  constexpr int kItemSlots = L::kItemSlots;
  constexpr int kItemReaders = 2 + 8 * kSplit;   // two issuing threads, one arrival per softmax warp

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int total = heads * blocks;
  // Items of this CTA: its first one is its block index (the launch never has more CTAs than items); in the
  // persistent launch the producer thread then takes further items from a launch-wide counter (work[0], zero at
  // launch) once it has issued the current item's loads, and hands each number to the other roles through a small ring in
  // shared memory. Causal items come sorted by length, so the CTAs finish within one of the shortest items of each
  // other (a fixed assignment - items w, w + G, ... - left the first CTAs 7 % above the average at B4 H16 N8192).
  // -1 ends the sequence.
  const Item first_item = get_item<kKeys>(blockIdx.x, heads, blocks, H, N, causal);
  const bool queue = kPersistent && static_cast<int>(gridDim.x) < total;   // else: one item per CTA, no counter traffic
  auto take_item = [&]() -> int {
    if (!queue) return -1;
    const long long w = static_cast<long long>(gridDim.x) + atomicAdd(&work[0], 1u);
    return w < total ? static_cast<int>(w) : -1;
  };
  // n-th item of the CTA as seen by the issuers and the softmax warps (whole warps call this together); false at the
  // end of the sequence
  auto read_item = [&](uint32_t n, bool whole_warp, bool& ok_ref, Item& it) -> bool {
    if (n == 0) {
      it = first_item;
      if (!kPersistent) return true;
    } else if (!kPersistent) {
      return false;
    }
    const int slot = n % kItemSlots;
    if (!mbar_wait(&item_full[slot], (n / kItemSlots) & 1, abort_flag, status, kSiteItemFull, s_unit)) {
      ok_ref = false;
      return false;
    }
    if (n != 0) {
      it.bh = s_items[slot].x;
      it.b = s_items[slot].y;
      it.h = s_items[slot].z;
      it.m0 = s_items[slot].w;
    }
    if (whole_warp) mbar_arrive_warp(&item_empty[slot]);
    else mbar_arrive(&item_empty[slot]);
    if (it.bh < 0) return false;
    if (n != 0) count_key_tiles<kKeys>(it, N, causal);
    return true;
  };

  auto load_q = [&](const Item& it, int t) {
    mbar_arrive_expect_tx(&q_full[t], kTileBytes);
    for (int x = 0; x < kBoxes; ++x)
      tma_load_4d(s_q + t * kTileBytes + x * kBoxBytes, &tm_q, &q_full[t], x * 64, it.m0 + t * kTile, it.h, it.b);
  };
  auto load_keys = [&](const Item& it, int j, int st) {
    mbar_arrive_expect_tx(&k_full[st], kKvBytes + kSlabBytes);
    for (int x = 0; x < kBoxes; ++x)
      tma_load_4d(s_k + st * kKvBytes + x * kKvBoxBytes, &tm_k, &k_full[st], x * 64, j * kKeys, it.h, it.b);
    tma_load_3d(s_kslab + st * kSlabBytes, &tm_kslab, &k_full[st], 0, j * kKeys, it.bh);
  };
  auto load_values = [&](const Item& it, int j, int st) {
    mbar_arrive_expect_tx(&v_full[st], kKvBytes);
    for (int x = 0; x < kBoxes; ++x)
      tma_load_4d(s_v + st * kKvBytes + x * kKvBoxBytes, &tm_v, &v_full[st], x * 64, j * kKeys, it.h, it.b);
  };
  // One thread (the TMA producer) sets the CTA up: it reads the launch's status word (a wait that ran out in an
  // earlier CTA ends the whole launch quickly: later CTAs leave at once), initialises the barriers while that load
  // is in flight, and issues the first loads before the CTA-wide synchronisation, so that Q and the first key tiles
  // travel while TMEM is allocated and the constant slab is written.
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
      mbar_init(&q_free[t], 1 + 4 * kSplit);
      mbar_init(&stage_free[t], 1);
    }
    for (int i = 0; i < kItemSlots; ++i) {
      mbar_init(&item_full[i], 1);
      mbar_init(&item_empty[i], kItemReaders);
    }
    fence_mbar_init();
    s_items[0].x = first_item.bh;
    *s_unit = static_cast<int>(blockIdx.x);
    mbar_arrive(&item_full[0]);
    *abort_flag = earlier != 0u ? 1 : 0;
    if (earlier == 0u) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_kslab);
      for (int t = 0; t < 2; ++t)
        if (first_item.nkt(t) > 0) load_q(first_item, t);
      for (int j = 0; j < first_item.nkt_max && j < kStages; ++j) {
        load_keys(first_item, j, j);
        load_values(first_item, j, j);
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

  // Counters that run on across a CTA's items, kept identically by every role that needs them:
  //   G      K/V tiles put through the ring by earlier items (tile j of the item uses stage (G + j) % kStages in
  //          round (G + j) / kStages)
  //   ct     key tiles query tile t has processed in earlier items (phase of s_full, s_consumed, p_full, o_done)
  //   qn     loads of Q_t by earlier items (phase of q_full, q_free; also of grp_sync and stage_free: one output
  //          store per load)
  if (warp == kLoadWarp) {
    // ------------------------------------------------------------------ TMA producer
    setmaxnreg_dec<R::kOtherRegs>();
    if (lane == 0) {
      uint32_t G = 0, qn[2] = {0, 0};
      bool ok = true;
      Item it = first_item;
      bool more = true;
      for (uint32_t n = 0; more && ok && (kPersistent || n == 0); ++n) {
        if (n != 0) {
          for (int t = 0; t < 2 && ok; ++t) {
            if (it.nkt(t) == 0) continue;
            if (qn[t] > 0) ok = mbar_wait(&q_free[t], (qn[t] - 1) & 1, abort_flag, status, kSiteQFree, s_unit);
            if (ok) load_q(it, t);
          }
        }
        for (int j = 0; j < it.nkt_max && ok; ++j) {
          const uint32_t g = G + j;
          if (n == 0 && j < kStages) continue;       // issued before the CTA-wide synchronisation
          const int st = g % kStages;
          const uint32_t par = ((g / kStages) - 1) & 1;
          if (g >= kStages && !mbar_wait(&k_empty[st], par, abort_flag, status, kSiteKEmpty, s_unit)) {
            ok = false;
            break;
          }
          load_keys(it, j, st);
          if (g >= kStages && !mbar_wait(&v_empty[st], par, abort_flag, status, kSiteVEmpty, s_unit)) {
            ok = false;
            break;
          }
          load_values(it, j, st);
        }
        if (!ok) break;
        G += it.nkt_max;
        for (int t = 0; t < 2; ++t) qn[t] += it.nkt(t) > 0 ? 1 : 0;
        // Take and publish the next item number (or the end of the sequence) only now: all loads of this item are
        // issued, the other roles still have up to kStages key tiles of it ahead of them, which hides the counter's
        // round trip; taking items earlier leaves the launch's last items reserved by CTAs that are still busy.
        const int w = take_item();
        more = w >= 0;
        if (more) {
          it = get_item<kKeys>(w, heads, blocks, H, N, causal);
          *s_unit = w;
        }
        const int slot = (n + 1) % kItemSlots;
        if (n + 1 >= kItemSlots &&
            !mbar_wait(&item_empty[slot], (((n + 1) / kItemSlots) - 1) & 1, abort_flag, status, kSiteItemEmpty, s_unit))
          break;
        s_items[slot].x = more ? it.bh : -1;
        s_items[slot].y = it.b;
        s_items[slot].z = it.h;
        s_items[slot].w = it.m0;
        mbar_arrive(&item_full[slot]);
      }
    }
  } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
    // ------------------------------------------------------------------ MMA issuer of query tile t
    setmaxnreg_dec<R::kOtherRegs>();
    if (lane == 0) {
      const int t = warp - kMmaWarp0;
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
      auto wait_k = [&](uint32_t g) {
        return mbar_wait(&k_full[g % kStages], (g / kStages) & 1, abort_flag, status, kSiteKFull, s_unit);
      };
      auto wait_v = [&](uint32_t g) {
        return mbar_wait(&v_full[g % kStages], (g / kStages) & 1, abort_flag, status, kSiteVFull, s_unit);
      };
      uint32_t G = 0, ct = 0, qn = 0;
      bool ok = true;
      for (uint32_t n = 0; ok && (kPersistent || n == 0); ++n) {
        Item it;
        if (!read_item(n, false, ok, it)) break;
        const int my_nkt = it.nkt(t), nkt_max = it.nkt_max;
        // Every stage is released by both issuers: by a commit after this tile's last MMA that reads it, or - when
        // this tile has nothing (left) to do with it - by a plain arrival made only after the stage has been filled,
        // so that an idle issuer can never arrive twice within one phase.
        if (my_nkt > 0) {
          // first scores of the item: Q_t has landed, the first key tile has landed, and the group holds the last
          // scores of the previous item in registers (it is then busy with their exponentials and its output)
          ok = mbar_wait(&q_full[t], qn & 1, abort_flag, status, kSiteQFull, s_unit) && wait_k(G);
          if (ok && ct > 0) ok = mbar_wait(&s_consumed[t], (ct - 1) & 1, abort_flag, status, kSiteSConsumed, s_unit);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s(G % kStages);
          if (kPersistent && my_nkt == 1) umma_commit(&q_free[t]);
          umma_commit(&k_empty[G % kStages]);
        } else {
          ok = wait_k(G);
          if (!ok) break;
          mbar_arrive(&k_empty[G % kStages]);
        }
        for (int j = 0; j < nkt_max && ok; ++j) {
          const uint32_t g = G + j;
          const int st = g % kStages;
          const int st_next = (g + 1) % kStages;
          bool used_k_next = false;
          if (j < my_nkt) {
            if (j + 1 < my_nkt) {
              // next scores first: they only need S_t(j) to have been read
              ok = wait_k(g + 1) && mbar_wait(&s_consumed[t], (ct + j) & 1, abort_flag, status, kSiteSConsumed, s_unit);
              if (!ok) break;
              tc_fence_after_sync();
              issue_s(st_next);
              if (kPersistent && j + 2 == my_nkt) umma_commit(&q_free[t]);   // the item's last read of Q_t
              used_k_next = true;
            }
            ok = wait_v(g);
            ok = ok && mbar_wait(&p_full[t], (ct + j) & 1, abort_flag, status, kSitePFull, s_unit);
            if (!ok) break;
            tc_fence_after_sync();
            issue_o(st, j > 0 ? 1u : 0u);
            umma_commit(&v_empty[st]);
          } else {
            ok = wait_v(g);
            if (!ok) break;
            mbar_arrive(&v_empty[st]);
          }
          if (j + 1 < nkt_max) {
            if (used_k_next) {
              umma_commit(&k_empty[st_next]);
            } else {
              ok = wait_k(g + 1);
              if (!ok) break;
              mbar_arrive(&k_empty[st_next]);
            }
          }
        }
        G += nkt_max;
        ct += my_nkt;
        qn += my_nkt > 0 ? 1 : 0;
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
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int col0 = hf * kCols;
    const bool storer = r == 0 && hf == 0;           // issues the tile's output stores
    constexpr bool kSkipMax = R::kSkipMax;
    static_assert(kSplit == 1 || !kSoftmax, "threads that share a row would have to agree on its maximum and sum");
    uint32_t ct = 0, qn = 0;
    bool ok = true;
    bool store_pending = false;                      // storer: a store whose staging tile has not been released yet
    if (D == 64 && kSplit == 1 && t == 1) {
      // The two softmax groups share the MUFU pipe. Started a few hundred cycles apart, one group's exponentials
      // overlap the other group's loads and stores more often than they collide (measured: 3 % at D = 64; making
      // the groups take strict turns was slower).
      const long long t_start = clock64();
      while (clock64() - t_start < 800) {
      }
    }
    for (uint32_t n = 0; ok && (kPersistent || n == 0); ++n) {
      Item it;
      if (!read_item(n, true, ok, it)) break;
      const int my_nkt = it.nkt(t);
      if (my_nkt == 0) continue;
      const int r0 = it.m0 + t * kTile;
      const int row = r0 + r;
      float m_used = -INFINITY;                      // maximum applied so far, in accumulator units times scale2
      float l_sum = 0.f;
      float row_bias = 0.f;
      if (!kSoftmax) row_bias = qsq[static_cast<int64_t>(it.bh) * n_pad + row];
      // upper bound of this row's logits in base-2 units, c |q_row|^2, from the row's Q tile (rows past N are zero)
      float ub = INFINITY;
      bool safe = false;                             // warp-wide: no row of this warp can overflow any more
      if (kSkipMax) {
        ok = mbar_wait(&q_full[t], qn & 1, abort_flag, status, kSiteQFull, s_unit);
        if (!ok) break;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};         // independent sums: the chain is on every item's critical path
#pragma unroll
        for (int c16 = 0; c16 < D / 8; ++c16) {
          const uint4 qv = *reinterpret_cast<const uint4*>(s_q + t * kTileBytes + (c16 >> 3) * kBoxBytes +
                                                           sw128_offset(r, c16 & 7));
          const uint32_t wv[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 x = unpack2<kBf16>(wv[i]);
            acc[i] = fmaf(x.x, x.x, acc[i]);
            acc[i] = fmaf(x.y, x.y, acc[i]);
          }
        }
        ub = ((acc[0] + acc[1]) + (acc[2] + acc[3])) * (0.5f * scale2);
      }
      if (kPersistent) mbar_arrive_warp(&q_free[t]);   // this warp will not read Q_t of this item (again)
      for (int j = 0; j < my_nkt; ++j) {
        ok = ok && mbar_wait(&s_full[t], (ct + j) & 1, abort_flag, status, kSiteSFull, s_unit);
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
          // tiles that reach past the block's first row: key (j * kKeys + col0 + c) is visible to query (r0 + r) iff
          // it is not larger
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
              ok = mbar_wait(&o_done[t], (ct + j - 1) & 1, abort_flag, status, kSiteODone, s_unit);
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

        // P's own columns are free once O_t += P_t V_(j-1) has completed (for the item's first tile: the output of
        // the previous item has been read, which waited for its last P V)
        bool waited_o = j == 0;
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
            ok = mbar_wait(&o_done[t], (ct + j - 1) & 1, abort_flag, status, kSitePFree, s_unit);
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
        if (kPersistent && j == 0 && storer && store_pending) {
          // the previous item's output store was issued a whole tile ago: its staging tile has been read by now
          tma_store_wait_read();
          mbar_arrive(&stage_free[t]);
          store_pending = false;
        }
      }
      if (!ok) break;

      ok = mbar_wait(&o_done[t], (ct + my_nkt - 1) & 1, abort_flag, status, kSiteODoneFinal, s_unit);
      if (ok && kPersistent && qn > 0) ok = mbar_wait(&stage_free[t], (qn - 1) & 1, abort_flag, status, kSiteStageFree, s_unit);
      if (!ok) break;
      tc_fence_after_sync();
      const float inv = kSoftmax ? (1.0f / l_sum) : 1.0f;
      uint8_t* stage = s_stage + t * kTileBytes;     // not persistent: Q_t, dead once the last S_t MMA has completed
#pragma unroll
      for (int c = 0; c < kOCols / 32; ++c) {
        uint32_t o[32];
        tmem_ld_x32(tmem_o[t] + lane_sel + hf * kOCols + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t wv[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            wv[i] = pack2<kBf16>(__uint_as_float(o[g * 8 + 2 * i]) * inv, __uint_as_float(o[g * 8 + 2 * i + 1]) * inv);
          const int col16 = (hf * kOCols) / 8 + c * 4 + g;             // 16-byte chunk index along D
          *reinterpret_cast<uint4*>(stage + (col16 >> 3) * kBoxBytes + sw128_offset(r, col16 & 7)) =
              make_uint4(wv[0], wv[1], wv[2], wv[3]);
        }
      }
      tc_fence_before_sync();                        // the output has been read: the next item may accumulate into O_t
      fence_proxy_async_smem();
      mbar_arrive_warp(&grp_sync[t]);
      ok = mbar_wait(&grp_sync[t], qn & 1, abort_flag, status, kSiteGroup, s_unit);
      if (!ok) break;
      if (storer) {
        for (int x = 0; x < kBoxes; ++x) tma_store_4d(&tm_o, stage + x * kBoxBytes, x * 64, r0, it.h, it.b);
        tma_store_commit();
        store_pending = true;
      }
      if (kSoftmax && hf == 0 && row < N) lse[static_cast<int64_t>(it.bh) * N + row] = m_used + log2f(l_sum);
      ct += my_nkt;
      ++qn;
    }
    if (storer && store_pending) tma_store_wait_read();   // the CTA may exit once the staging tile has been read
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
  if (queue && tid == 0) {
    // the last CTA to leave puts the work counters back to zero for the next launch on this workspace
    __threadfence();
    if (atomicAdd(&work[1], 1u) == gridDim.x - 1) {
      work[0] = 0u;
      work[1] = 0u;
    }
  }
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
  const int blocks = (a.N + 2 * kTile - 1) / (2 * kTile), heads = a.B * a.H;
  int grid = blocks * heads;                       // one CTA per item, dispatched in item order
  if (fwd::Smem<D>::kPersistent) {
    const int sms = device_sm_count();
    if (sms <= 0) return cudaErrorInvalidDevice;
    if (grid > sms) grid = sms;                    // one CTA per SM walks the items w, w + grid, ...
  }
  kernel<<<grid, fwd::Roles<D, kSoftmax, kBf16>::kThreads, smem, stream>>>(a.tm_q, a.tm_k, a.tm_v, a.tm_o, a.tm_kslab, a.qsq, a.lse, a.status,
                                                a.H, a.N, a.n_pad, a.causal, a.scale2, a.slab_w, heads, blocks,
                                                // forward work counters: words 18, 19 of the status block (zeroed with it)
                                                reinterpret_cast<unsigned int*>(a.status) + 18);
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
