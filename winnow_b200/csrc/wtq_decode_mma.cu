// Split-K decode attention over paged packed K/V: the sm_100a tensor-core path
// for head_dim 128, key/value widths of 4, 6 or 8 bits (4/4, 4/6, 6/6, 8/8),
// pages of 16, 32, 64, ... tokens and a GQA group of at most 8 query heads.
//
// One persistent CTA per SM, up to 12 warps.  A warp is an independent worker:
// it takes (sequence, kv head, chunk of tokens) items round-robin, streams the
// chunk's 16-token tiles from HBM into its private shared-memory ring with
// 16-byte cp.async copies (the next 32 tokens are in flight while the current
// 32 are consumed), and keeps the whole flash-decoding state in registers.
//
// Per 16-token tile, with the packed bytes never leaving registers/smem:
//   scores   S^T[16 tok x 8 heads] = C_K[16 x 128] . Qrot^T   8 x mma.m16n8k16
//   softmax  online, fp32, exp2 domain, against a reference value that is only
//            raised (and the state rescaled) when a score exceeds it: the
//            common window costs one vote, no shuffles
//   values   O^T[128 d x 8 heads] += C_V^T[128 x 16 tok] . P'^T   8 x mma
// The fp16 operands C_K / C_V come from shared-memory tables replicated per
// lane (every lookup of a warp is bank-conflict free) that start at shared
// address 0x10000, so that the address of an entry is
// 0x10000 | index << 8 | side << 7 | lane << 2 and needs no addition.  The
// tables are built once per call by the query-rotation kernel (into the
// workspace) and pulled into shared memory by one bulk copy.
//   4-bit: ONE lookup per packed byte (= two codes) into a 256-entry table of
//     half2 {centroid[lo nibble], centroid[hi nibble]}; one byte-permute builds
//     the address.  Keys: a byte holds two adjacent coordinates of one token,
//     which is the pair an A-fragment register of the score MMA wants (the
//     contraction runs over coordinates, whose order is free: q is permuted to
//     match).  Values: the contraction runs over tokens, so a register must
//     hold one coordinate of two tokens; the low (high) nibbles of the same
//     byte of two tokens are merged by one shift and one bit-select into a byte
//     that indexes the same table.
//   6- and 8-bit: one lookup per code into a table of half2 {c, c}; a shift
//     and a mask (8-bit: a byte-permute) build the address and one
//     byte-permute joins two results into an operand register.
// mma.sync is the right tensor instruction here: the operands are born in
// registers; tcgen05 would need them written back to shared memory first.
//
// Reference schedule being reproduced: turboquant_kv/packed_attention.py:
// 260-334 (tiled online softmax), split merge :328-334.
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "wtq_decode.cuh"
#include "wtq_lut.cuh"

#include <atomic>

namespace wtq {

namespace mma {

constexpr int kTileTokens = 16;
constexpr int kTilesPerIter = 2;                       // 32 tokens per iteration
constexpr int kIterTokens = kTileTokens * kTilesPerIter;
constexpr uint32_t kPrefixAddr = 2048;                 // chunk prefix copy (>= dynamic smem base)
constexpr int kPrefixMax = 1024;                       // entries (sequences + 1) it can hold
constexpr uint32_t kLutBar = kPrefixAddr + 4 * kPrefixMax;    // mbarrier of the tables' copy
constexpr uint32_t kFifoAddr = kLutBar + 64;           // per warp: four decoded items of 32 bytes
constexpr uint32_t kRingLow = kFifoAddr + 16 * 128;    // rings start here
constexpr uint32_t kSmemLimit = 227 * 1024;
constexpr float kPreciseAbove = 8.0f;   // |score| (log2 units) that triggers fp32 rescoring
constexpr float kSlack = 4.0f;          // the softmax reference is set this far above a new maximum
constexpr int kWaitTries = 1 << 18;     // bound of the mbarrier wait (each try suspends for a while)
// Worker warps per CTA.  Twelve warps of 168 registers beat sixteen of 128 on
// every benchmark shape: the lookups of a warp overlap better than more warps do.
constexpr int kMaxWarps = 12;

constexpr int cmax(int a, int b) { return a > b ? a : b; }
constexpr int cmin(int a, int b) { return a < b ? a : b; }

// Shared-memory plan of one (key width, value width) instantiation.
template <int BWK, int BWV> struct Cfg {
  static constexpr int NBK = 16 * BWK, NBV = 16 * BWV;          // bytes per packed row
  static constexpr int kVRow = BWV == 4 ? 80 : NBV;             // 4-bit value rows are padded
  static constexpr int kOffV = kTileTokens * NBK;               // tile slot: K | V | nK | nV
  static constexpr int kOffNK = kOffV + kTileTokens * kVRow;
  static constexpr int kOffNV = kOffNK + 32;
  static constexpr int kSlot = kOffNV + 32;
  static constexpr int kRing = 2 * kTilesPerIter * kSlot;       // two windows per warp
  static constexpr uint32_t kLutBytes = cmax(lut_entries(BWK), lut_entries(BWV)) * 256u;
  static constexpr int kRingsBelow = (int)((kLutAddr - kRingLow) / kRing);
  static constexpr int kRingsAbove = (int)((kSmemLimit - kLutAddr - kLutBytes) / kRing);
  static constexpr int kWarps = cmin(kMaxWarps, kRingsBelow + kRingsAbove);
  static constexpr int kThreads = kWarps * 32;
  static constexpr size_t kDynamicSmem =
      kLutAddr + kLutBytes + (size_t)cmax(kWarps - kRingsBelow, 0) * kRing;
  static_assert(kWarps >= 8, "too few warps fit");
  static_assert(kDynamicSmem <= kSmemLimit, "shared memory budget");
  __device__ static uint32_t ring_address(int w) {
    return w < kRingsBelow ? kRingLow + (uint32_t)w * kRing
                           : kLutAddr + kLutBytes + (uint32_t)(w - kRingsBelow) * kRing;
  }
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;\n" ::: "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
// ---- asynchronous copies and their barriers -----------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded: false when the phase did not complete within kWaitTries tries.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < kWaitTries; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// `bytes` (a multiple of 16) from global `src` to this CTA's shared `dst`, both
// 16-byte aligned; completion is counted on the mbarrier at `bar`.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void griddep_wait() {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
}
__device__ __forceinline__ void griddep_launch() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

}  // namespace mma

using namespace mma;

// Value side of one tile: the lane holds coordinates 16g..16g+15 of tokens
// 2t, 2t+1 (A, B) and 2t+8, 2t+9 (C, D); `at` = address of its 16 codes of
// token 2t.  MMA j (0..7) takes coordinates 16g+2j (row g) and 16g+2j+1 (row
// g+8) of the output tile.
template <int BW, int VROW>
__device__ __forceinline__ void value_mmas(uint32_t at, uint32_t sel, uint32_t pb0, uint32_t pb1,
                                           float (&acc)[8][4]) {
  constexpr int NB8 = 2 * BW;                       // bytes of 16 codes
  if constexpr (BW == 4) {
    const uint2 wa = lds64(at), wb = lds64(at + VROW);
    const uint2 wc = lds64(at + 8 * VROW), wd = lds64(at + 9 * VROW);
    // byte j of lo_* : low nibbles of tokens (A | B << 4) at coordinate 16g+2j
    // byte j of hi_* : high nibbles, coordinate 16g+2j+1
    auto up4 = [](uint32_t x) { return x << 4; };
    auto down4 = [](uint32_t x) { return x >> 4; };
    const uint32_t lo_ab[2] = {(wa.x & 0x0F0F0F0Fu) | (up4(wb.x) & 0xF0F0F0F0u),
                               (wa.y & 0x0F0F0F0Fu) | (up4(wb.y) & 0xF0F0F0F0u)};
    const uint32_t hi_ab[2] = {(down4(wa.x) & 0x0F0F0F0Fu) | (wb.x & 0xF0F0F0F0u),
                               (down4(wa.y) & 0x0F0F0F0Fu) | (wb.y & 0xF0F0F0F0u)};
    const uint32_t lo_cd[2] = {(wc.x & 0x0F0F0F0Fu) | (up4(wd.x) & 0xF0F0F0F0u),
                               (wc.y & 0x0F0F0F0Fu) | (up4(wd.y) & 0xF0F0F0F0u)};
    const uint32_t hi_cd[2] = {(down4(wc.x) & 0x0F0F0F0Fu) | (wd.x & 0xF0F0F0F0u),
                               (down4(wc.y) & 0x0F0F0F0Fu) | (wd.y & 0xF0F0F0F0u)};
    // The sixteen table addresses of a half are formed first, then the sixteen
    // lookups are issued, then the four MMAs: a lookup never waits for the
    // byte-permute that builds its own address.
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t ad[4][4], f[4][4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t src = q == 0 ? lo_ab[h] : q == 1 ? hi_ab[h] : q == 2 ? lo_cd[h] : hi_cd[h];
        ad[0][q] = lut_addr<0>(src, sel); ad[1][q] = lut_addr<1>(src, sel);
        ad[2][q] = lut_addr<2>(src, sel); ad[3][q] = lut_addr<3>(src, sel);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int q = 0; q < 4; ++q) f[j][q] = lds32(ad[j][q]);
#pragma unroll
      for (int j = 0; j < 4; ++j) mma16816(acc[4 * h + j], f[j][0], f[j][1], f[j][2], f[j][3], pb0, pb1);
    }
  } else {
    constexpr int NW = NB8 / 4;
    uint32_t wa[NW], wb[NW], wc[NW], wd[NW];
    load_words<NB8>(at, wa);
    load_words<NB8>(at + VROW, wb);
    load_words<NB8>(at + 8 * VROW, wc);
    load_words<NB8>(at + 9 * VROW, wd);
    auto one = [&](auto jc) {
      constexpr int j = decltype(jc)::value;
      mma16816(acc[j],
               join(lut_code<BW, 2 * j>(wa, sel), lut_code<BW, 2 * j>(wb, sel)),
               join(lut_code<BW, 2 * j + 1>(wa, sel), lut_code<BW, 2 * j + 1>(wb, sel)),
               join(lut_code<BW, 2 * j>(wc, sel), lut_code<BW, 2 * j>(wd, sel)),
               join(lut_code<BW, 2 * j + 1>(wc, sel), lut_code<BW, 2 * j + 1>(wd, sel)), pb0, pb1);
    };
    one(std::integral_constant<int, 0>{}); one(std::integral_constant<int, 1>{});
    one(std::integral_constant<int, 2>{}); one(std::integral_constant<int, 3>{});
    one(std::integral_constant<int, 4>{}); one(std::integral_constant<int, 5>{});
    one(std::integral_constant<int, 6>{}); one(std::integral_constant<int, 7>{});
  }
}

// Scores of one tile: S^T fragment (rows g, g+8; heads 2t, 2t+1), unscaled.
// `at` = address of the lane's 32 codes of token row g.  Even and odd
// contraction steps accumulate separately (two chains of four dependent MMAs
// instead of one of eight).
template <int BW>
__device__ __forceinline__ void key_mmas(uint32_t at, uint32_t sel, const uint32_t (&qf)[8][2],
                                         float (&c)[4]) {
  constexpr int NB4 = 4 * BW;                       // bytes of 32 codes
  constexpr int NW = NB4 / 4, NB = 16 * BW;
  uint32_t w0[NW], w1[NW];
  load_words<NB4>(at, w0);
  load_words<NB4>(at + 8 * NB, w1);
  constexpr int kChains = 2;
  float cc[kChains][4];
#pragma unroll
  for (int i = 0; i < kChains; ++i) cc[i][0] = cc[i][1] = cc[i][2] = cc[i][3] = 0.f;
  if constexpr (BW == 4) {
    // per word of the two rows: eight addresses, eight lookups, two MMAs
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t ad[8], f[8];
      ad[0] = lut_addr<0>(w0[j], sel); ad[1] = lut_addr<0>(w1[j], sel);
      ad[2] = lut_addr<1>(w0[j], sel); ad[3] = lut_addr<1>(w1[j], sel);
      ad[4] = lut_addr<2>(w0[j], sel); ad[5] = lut_addr<2>(w1[j], sel);
      ad[6] = lut_addr<3>(w0[j], sel); ad[7] = lut_addr<3>(w1[j], sel);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = lds32(ad[i]);
      mma16816(cc[0], f[0], f[1], f[2], f[3], qf[2 * j][0], qf[2 * j][1]);
      mma16816(cc[1], f[4], f[5], f[6], f[7], qf[2 * j + 1][0], qf[2 * j + 1][1]);
    }
  } else {
    auto one = [&](auto ksc) {
      constexpr int ks = decltype(ksc)::value;
      uint32_t a[4];
      key_fragment<BW, ks>(w0, w1, sel, a);
      mma16816(cc[ks % kChains], a[0], a[1], a[2], a[3], qf[ks][0], qf[ks][1]);
    };
    one(std::integral_constant<int, 0>{}); one(std::integral_constant<int, 1>{});
    one(std::integral_constant<int, 2>{}); one(std::integral_constant<int, 3>{});
    one(std::integral_constant<int, 4>{}); one(std::integral_constant<int, 5>{});
    one(std::integral_constant<int, 6>{}); one(std::integral_constant<int, 7>{});
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float v = cc[0][e];
#pragma unroll
    for (int i = 1; i < kChains; ++i) v += cc[i][e];
    c[e] = v;
  }
}

// fp32 scores of tile rows g and g+8 against two query rows (already rotated
// and scaled, read through L1), times the key norms: {row g . qa, row g . qb,
// row g+8 . qa, row g+8 . qb}.  Kept out of line: it runs only for windows
// whose fp16 scores came out large, and must not cost the common path
// registers.
template <int BW>
__device__ __noinline__ float4 precise_scores(uint32_t kbase, uint32_t nk_addr, int g,
                                              const float *qa, const float *qb,
                                              const float *centroids) {
  constexpr int NB = 16 * BW;
  float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
  const uint32_t r0 = kbase + g * NB, r1 = kbase + (g + 8) * NB;
#pragma unroll 1
  for (int d = 0; d < 128; ++d) {
    const int bit = d * BW, b0 = bit >> 3, sh = bit & 7;
    uint32_t x0 = lds_u8(r0 + b0), x1 = lds_u8(r1 + b0);
    if (sh + BW > 8) {
      x0 |= lds_u8(r0 + b0 + 1) << 8;
      x1 |= lds_u8(r1 + b0 + 1) << 8;
    }
    const float c0 = __ldg(centroids + ((x0 >> sh) & ((1u << BW) - 1u)));
    const float c1 = __ldg(centroids + ((x1 >> sh) & ((1u << BW) - 1u)));
    const float fa = __ldg(qa + d), fb = __ldg(qb + d);
    d0 = fmaf(fa, c0, d0); d1 = fmaf(fb, c0, d1);
    d2 = fmaf(fa, c1, d2); d3 = fmaf(fb, c1, d3);
  }
  const float nk0 = lds_half(nk_addr + g * 2), nk1 = lds_half(nk_addr + (g + 8) * 2);
  return make_float4(d0 * nk0, d1 * nk0, d2 * nk1, d3 * nk1);
}

template <int BWK, int BWV, bool S16>
__global__ void __launch_bounds__(Cfg<BWK, BWV>::kThreads, 1)
decode_mma_kernel(DecodeParams p, int chunk_tokens) {
  using C = Cfg<BWK, BWV>;
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  const uint32_t dyn_base = (uint32_t)__cvta_generic_to_shared(dyn_smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  if (dyn_base > kPrefixAddr) {          // layout assumption broken: refuse, do not touch memory
    if (p.status && tid == 0) atomicOr(p.status, WTQ_STATUS_LAYOUT);
    return;
  }
  constexpr uint32_t kFull = 0xffffffffu;
  if (tid == 0) {
    mbar_init(kLutBar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }

  const uint32_t ring = C::ring_address(warp);
  const uint32_t sel_k = 0x10000u | (uint32_t)(lane << 2);
  const uint32_t sel_v = sel_k | 0x80u;
  // tiles per page (a power of two) as a shift and a mask; both are constants
  // for 16-token pages, the common case
  const int S = S16 ? 16 : p.S;
  const int ts = S16 ? 0 : 27 - __clz(S);
  const int tmask = S16 ? 0 : (S >> 4) - 1;
  const int chunks = p.num_splits;

  // Exclusive prefix of chunks per sequence, in shared memory when the batch
  // fits (it only needs seq_lens, so it too overlaps the previous kernel).
  const bool prefix_local = p.B < kPrefixMax - 1;
  if (prefix_local && warp == 0) {
    int running = 0, least = 0x7fffffff, most = 0;
    for (int b0 = 0; b0 < p.B; b0 += 32) {
      const int bb = b0 + lane;
      int n = 0;
      if (bb < p.B) {
        int Lb = p.seq_lens[bb];
        Lb = Lb < 0 ? 0 : (Lb > p.max_pages * p.S ? p.max_pages * p.S : Lb);
        n = (Lb + chunk_tokens - 1) / chunk_tokens;
        least = min(least, n);
        most = max(most, n);
      }
      int incl = n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(kFull, incl, o);
        if (lane >= o) incl += up;
      }
      if (bb < p.B) sts32(kPrefixAddr + 4 * bb, (uint32_t)(running + incl - n));
      running += __shfl_sync(kFull, incl, 31);
    }
    if (lane == 0) sts32(kPrefixAddr + 4 * p.B, (uint32_t)running);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      least = min(least, __shfl_xor_sync(kFull, least, o));
      most = max(most, __shfl_xor_sync(kFull, most, o));
    }
    // all sequences have the same number of chunks: items are equal, a fixed
    // round-robin balances them and the queue is not needed
    if (lane == 0) sts32(kPrefixAddr + 4 * (kPrefixMax - 1), least == most ? 1u : 0u);
  }
  __syncthreads();
  auto prefix_at = [&](int i) -> int {
    return prefix_local ? (int)lds32(kPrefixAddr + 4 * i) : p.chunk_prefix[i];
  };
  // The prefix in global memory, q_rot and the tables are written by the
  // rotation kernel launched just before this one; pages, page table and
  // lengths are older than that kernel's start (it is launched without the
  // programmatic attribute), so the first window may be requested before the
  // wait whenever the prefix is local.
  if (!prefix_local) griddep_wait();

  // Items (one chunk of one kv head of one sequence; only chunks that exist are
  // numbered) are dealt round-robin, consecutive items to different CTAs; when
  // the sequences differ in length the last rounds come from a queue in global
  // memory instead, so that the warps finish together.
  const int64_t items_live = (int64_t)prefix_at(p.B) * p.Hkv;
  const int workers = gridDim.x * C::kWarps;
  const bool fixed_rounds = prefix_local && lds32(kPrefixAddr + 4 * (kPrefixMax - 1)) != 0u;
  // Ragged batches: items differ only in each sequence's last chunk, so all
  // rounds but the last two are dealt round-robin as well (no queue traffic,
  // no round trip); the queue hands out the rest and evens out the end.
  const int static_rounds =
      fixed_rounds ? 0x7fffffff : max(1, (int)min(items_live / workers, (int64_t)0x7fffffff) - 1);
  const int queue_base = fixed_rounds ? 0 : static_rounds * workers;
  int taken = 1;                                      // items this warp has been dealt
  int next_item = warp * gridDim.x + blockIdx.x;

  // ---- the copies -------------------------------------------------------------
  // They run one window (two tiles) ahead of the arithmetic, through item
  // boundaries, along their own stream of items: an item is decoded when the
  // stream reaches it and handed to the arithmetic through a small queue in
  // shared memory; the item after it is asked for at once (from the static deal
  // or the global queue), so that round trip hides behind a whole item of copies.
  // Every instruction here competes with the table lookups for the integer
  // pipe, which is what bounds this kernel, so the per-tile work is kept to a
  // page-id shuffle, one range check and three multiply-adds for addresses:
  //   src_*      the lane's share of the key rows, value rows and (lanes 0..3)
  //              norm rows of (kv head, page 0);
  //   ids0/ids1  entries first_page + lane and first_page + 32 + lane of the
  //              sequence's page-table row (a chunk spans at most 64 pages; longer
  //              ones reload);
  //   cs_tile    tiles of the item requested so far, cs_tiles its tile count,
  //              cs_t0 the tile of the chunk's first token inside its page.
  const uint8_t *src_k = nullptr, *src_v = nullptr, *src_n = nullptr;
  const bool n_is_v = lane >= 2;
  const uint32_t n_page = 2u * (uint32_t)(n_is_v ? p.v.norm_page_stride : p.k.norm_page_stride);
  const uint32_t n_dst = n_is_v ? C::kOffNV + (lane - 2) * 16 : C::kOffNK + lane * 16;
  const uint32_t k_page = (uint32_t)p.k.page_stride, v_page = (uint32_t)p.v.page_stride;
  int ids0 = -1, ids1 = -1, ids_first = 0;
  const int32_t *table_row = p.page_table;
  int cs_tile = 0, cs_tiles = 0, cs_t0 = 0;
  bool cs_valid = false;
  const uint32_t fifo = kFifoAddr + (uint32_t)warp * 128;
  int fifo_w = 0, fifo_r = 0;
  uint32_t bad = 0;                   // tiles whose page id was refused: bit 2 * half + tile
  auto load_ids = [&]() {
    ids0 = ids_first + lane < p.max_pages ? table_row[ids_first + lane] : -1;
    ids1 = ids_first + 32 + lane < p.max_pages ? table_row[ids_first + 32 + lane] : -1;
  };
  auto next_stream_item = [&]() {
    const int64_t item = __shfl_sync(kFull, next_item, 0);
    cs_valid = false;
    if (item >= items_live) return;
    const int kvh = (int)(item % p.Hkv);
    const int flat = (int)(item / p.Hkv);                   // chunk number over all sequences
    int lo = 0, hi = p.B;                                   // last b with prefix[b] <= flat
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (prefix_at(mid) <= flat) lo = mid;
      else hi = mid;
    }
    const int chunk = flat - prefix_at(lo);
    int L = p.seq_lens[lo];
    if (L > p.max_pages * S) {
      L = p.max_pages * S;
      if (p.status && lane == 0) atomicOr(p.status, WTQ_STATUS_BAD_POSITION);
    }
    const int tok0 = chunk * chunk_tokens, tok1 = min(L, tok0 + chunk_tokens);
    if (tok0 >= tok1) {
      // (an empty chunk cannot be numbered by a consistent prefix; if it happens
      // the warp stops and says so rather than guess)
      if (p.status && lane == 0) atomicOr(p.status, WTQ_STATUS_BAD_POSITION);
      return;
    }
    cs_valid = true;
    cs_tile = 0;
    cs_tiles = (tok1 - tok0 + kTileTokens - 1) / kTileTokens;
    cs_t0 = (tok0 & (S - 1)) >> 4;
    src_k = p.k.pages + (int64_t)kvh * p.k.head_stride + lane * 16;
    src_v = p.v.pages + (int64_t)kvh * p.v.head_stride + lane * 16;
    src_n = n_is_v ? reinterpret_cast<const uint8_t *>(p.v.norms + (int64_t)kvh * p.v.norm_head_stride) + (lane - 2) * 16
                   : reinterpret_cast<const uint8_t *>(p.k.norms + (int64_t)kvh * p.k.norm_head_stride) + lane * 16;
    table_row = p.page_table + (int64_t)lo * p.table_stride;
    ids_first = tok0 >> (ts + 4);
    load_ids();
    if (lane == 0) {
      const uint32_t e = fifo + (uint32_t)(fifo_w & 3) * 32;
      sts32(e, (uint32_t)lo); sts32(e + 4, (uint32_t)kvh); sts32(e + 8, (uint32_t)chunk);
      sts32(e + 12, (uint32_t)tok0); sts32(e + 16, (uint32_t)tok1);
      next_item = taken++ < static_rounds ? next_item + workers
                                          : queue_base + atomicAdd(p.work_counter, 1);
    }
    ++fifo_w;
  };
  // Requests the next window of the stream into the ring half at `ibase`
  // (`ihalf` = 0 or 1 names it in `bad`).  Always commits one group.
  uint32_t ibase = ring;
  int ihalf = 0;
  auto issue_one = [&]() {
    if (bad) bad &= ~(3u << (2 * ihalf));
    if (cs_valid) {
#pragma unroll
      for (int u = 0; u < kTilesPerIter; ++u) {
        const int n = cs_tile + u;
        if (n < cs_tiles) {
          const int q = cs_t0 + n;
          int rel = S16 ? q : q >> ts;                      // page of the tile, from the item's first
          const uint32_t sub = S16 ? 0u : (uint32_t)(q & tmask) << 4;
          if (rel >= 64) {                                  // beyond the ids held (very long chunks)
            ids_first += rel & ~31;
            cs_t0 -= (rel & ~31) << ts;
            rel &= 31;
            load_ids();
          }
          const int pid = __shfl_sync(kFull, rel < 32 ? ids0 : ids1, rel);
          if ((uint32_t)pid < (uint32_t)p.P) {
            const uint32_t dst = ibase + u * C::kSlot;
            const uint8_t *ks = src_k + (uint64_t)(uint32_t)pid * k_page + sub * C::NBK;
            const uint8_t *vs = src_v + (uint64_t)(uint32_t)pid * v_page + sub * C::NBV;
#pragma unroll
            for (int i = 0; i < C::NBK / 32; ++i) cp_async16(dst + lane * 16 + i * 512, ks + i * 512);
#pragma unroll
            for (int i = 0; i < C::NBV / 32; ++i) {
              if constexpr (BWV == 4)      // chunk c -> padded row c/4, quarter c%4
                cp_async16(dst + C::kOffV + (g + 8 * i) * C::kVRow + t * 16, vs + i * 512);
              else
                cp_async16(dst + C::kOffV + lane * 16 + i * 512, vs + i * 512);
            }
            if (lane < 4)
              cp_async16(dst + n_dst, src_n + (uint64_t)(uint32_t)pid * n_page + sub * 2);
          } else {
            bad |= 1u << (2 * ihalf + u);
            if (p.status && lane == 0) atomicOr(p.status, WTQ_STATUS_BAD_PAGE);
          }
        }
      }
      cs_tile += kTilesPerIter;
      if (cs_tile >= cs_tiles) next_stream_item();
    }
    cp_async_commit();
    ibase = 2 * ring + kTilesPerIter * C::kSlot - ibase;     // the other half
    ihalf ^= 1;
  };
  next_stream_item();
  issue_one();
  if (prefix_local) griddep_wait();
  // The merge that follows may be scheduled as soon as SMs free up.
  griddep_launch();
  if (tid == 0) {
    mbar_expect_tx(kLutBar, C::kLutBytes);
    bulk_g2s(kLutAddr, p.lut, C::kLutBytes, kLutBar);
  }
  const bool tables_ok = mbar_wait(kLutBar, 0);
  if (!tables_ok && p.status && lane == 0) atomicOr(p.status, WTQ_STATUS_SCAN_TIMEOUT);

  uint32_t cbase = ring;              // ring half consumed next
  int chalf = 0;
  for (int guard = 0; guard < (1 << 24) && fifo_r < fifo_w && tables_ok; ++guard) {   // bounded
    __syncwarp();
    const uint32_t entry = fifo + (uint32_t)(fifo_r & 3) * 32;
    const int b = (int)lds32(entry), kvh = (int)lds32(entry + 4), chunk = (int)lds32(entry + 8);
    const int tok0 = (int)lds32(entry + 12), tok1 = (int)lds32(entry + 16);
    ++fifo_r;

    // ---- query fragments: head g, coordinates 32t .. 32t+31 ----------------
    uint32_t qf[8][2];
    {
      const bool live = g < p.n_rep;
      const float4 *src = reinterpret_cast<const float4 *>(
          p.q_rot + ((int64_t)b * p.Hq + kvh * p.n_rep + (live ? g : 0)) * 128 + 32 * t);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        float4 v = live ? src[ks] : make_float4(0.f, 0.f, 0.f, 0.f);
        qf[ks][0] = pack_half2(v.x, v.y);
        qf[ks][1] = pack_half2(v.z, v.w);
      }
    }
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    // Softmax state of heads 2t, 2t+1: reference M (the probabilities are
    // 2^(s - M), M >= every score seen), -M with -inf replaced by 0, the bound
    // a window's scores (relative to M) must stay under to take the short path,
    // and the sum of the probabilities.
    float M0 = -INFINITY, M1 = -INFINITY, neg0 = 0.f, neg1 = 0.f;
    float hi0 = -INFINITY, hi1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // A window whose 32 tokens all exist on pages that were found needs no
    // masks; only the last window of a chunk (or a refused page id) takes the
    // masked form of the same code.
    const int n_full = (tok1 - tok0) / kIterTokens;            // windows without a ragged end
    const int n_iter = (tok1 - tok0 + kIterTokens - 1) / kIterTokens;
    int wtok = tok0;                                           // first token of the window
    uint32_t loaded = 3u;
      auto window = [&](auto masked_c) {
        constexpr bool MASKED = decltype(masked_c)::value;
        const uint32_t slot0 = cbase;
        // ---- scores of the tiles --------------------------------------------
        float c[kTilesPerIter][4], a[kTilesPerIter][4], nk[kTilesPerIter][2];
        bool ok[kTilesPerIter][2];
#pragma unroll
        for (int u = 0; u < kTilesPerIter; ++u) {
          const uint32_t slot = slot0 + u * C::kSlot;
          key_mmas<BWK>(slot + g * C::NBK + t * (4 * BWK), sel_k, qf, c[u]);
          nk[u][0] = lds_half(slot + C::kOffNK + g * 2);
          nk[u][1] = lds_half(slot + C::kOffNK + (g + 8) * 2);
          ok[u][0] = ok[u][1] = true;
        }
        bool slow = true;
        if constexpr (!MASKED) {
          float top0 = -INFINITY, top1 = -INFINITY;
#pragma unroll
          for (int u = 0; u < kTilesPerIter; ++u) {
            a[u][0] = fmaf(c[u][0], nk[u][0], neg0); a[u][1] = fmaf(c[u][1], nk[u][0], neg1);
            a[u][2] = fmaf(c[u][2], nk[u][1], neg0); a[u][3] = fmaf(c[u][3], nk[u][1], neg1);
            top0 = max3(top0, a[u][0], a[u][2]);
            top1 = max3(top1, a[u][1], a[u][3]);
          }
          slow = __any_sync(kFull, top0 > hi0 || top1 > hi1);
        }
        if (slow) {
          // A score above the reference (or the first window, a large score, a
          // partly filled window): exact scores, fp32 rescoring when they are
          // large, new reference, state rescaled.
          float s[kTilesPerIter][4];
          float big = 0.f;
#pragma unroll
          for (int u = 0; u < kTilesPerIter; ++u) {
            s[u][0] = c[u][0] * nk[u][0]; s[u][1] = c[u][1] * nk[u][0];
            s[u][2] = c[u][2] * nk[u][1]; s[u][3] = c[u][3] * nk[u][1];
            if constexpr (MASKED) {
              const int tok = wtok + u * kTileTokens;
              const bool page_ok = (loaded >> u) & 1u;
              ok[u][0] = page_ok && tok + g < tok1;
              ok[u][1] = page_ok && tok + g + 8 < tok1;
            }
            if (ok[u][0]) big = fmaxf(big, fmaxf(fabsf(s[u][0]), fabsf(s[u][1])));
            if (ok[u][1]) big = fmaxf(big, fmaxf(fabsf(s[u][2]), fabsf(s[u][3])));
          }
          // fp16 operands carry about 2^-11.5 of the score scale as error; when
          // any score of this window is large (|s| > 8 in log2 units) its tiles
          // are scored again in fp32 on the CUDA cores, so that large logits
          // cost time, not accuracy.
          if (__any_sync(kFull, big > kPreciseAbove)) {
            const float *q0 = p.q_rot + ((int64_t)b * p.Hq + kvh * p.n_rep) * 128;
            const bool h0 = 2 * t < p.n_rep, h1 = 2 * t + 1 < p.n_rep;
            const float *qa = q0 + (h0 ? 2 * t : 0) * 128, *qb = q0 + (h1 ? 2 * t + 1 : 0) * 128;
#pragma unroll
            for (int u = 0; u < kTilesPerIter; ++u) {
              const uint32_t slot = slot0 + u * C::kSlot;
              const float4 d = precise_scores<BWK>(slot, slot + C::kOffNK, g, qa, qb, p.k.centroids);
              s[u][0] = h0 ? d.x : 0.f; s[u][1] = h1 ? d.y : 0.f;
              s[u][2] = h0 ? d.z : 0.f; s[u][3] = h1 ? d.w : 0.f;
            }
          }
          float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
          for (int u = 0; u < kTilesPerIter; ++u) {
            if (!ok[u][0]) s[u][0] = s[u][1] = -INFINITY;
            if (!ok[u][1]) s[u][2] = s[u][3] = -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[u][0], s[u][2]));
            mx1 = fmaxf(mx1, fmaxf(s[u][1], s[u][3]));
          }
#pragma unroll
          for (int o = 4; o < 32; o <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, o));
            mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, o));
          }
          const float n0 = mx0 > M0 ? mx0 + kSlack : M0;
          const float n1 = mx1 > M1 ? mx1 + kSlack : M1;
          if (__any_sync(kFull, n0 != M0 || n1 != M1)) {
            // 2^(-inf - x) = 0 for the first window; an unchanged reference keeps 1
            const float alpha0 = n0 != M0 ? ex2(M0 - n0) : 1.f;
            const float alpha1 = n1 != M1 ? ex2(M1 - n1) : 1.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              acc[j][0] *= alpha0; acc[j][1] *= alpha1; acc[j][2] *= alpha0; acc[j][3] *= alpha1;
            }
            l0 *= alpha0;
            l1 *= alpha1;
            M0 = n0;
            M1 = n1;
          }
          // exp2(-inf - -inf) is defined as 0: with nothing seen the base is 0
          neg0 = M0 == -INFINITY ? 0.f : -M0;
          neg1 = M1 == -INFINITY ? 0.f : -M1;
          // short path while every score stays under the reference and under the
          // rescoring threshold; never when the running maximum is a large
          // negative number (all scores are large then)
          hi0 = (M0 == -INFINITY || M0 - kSlack < -kPreciseAbove) ? -INFINITY
                                                                 : fminf(0.f, kPreciseAbove - M0);
          hi1 = (M1 == -INFINITY || M1 - kSlack < -kPreciseAbove) ? -INFINITY
                                                                 : fminf(0.f, kPreciseAbove - M1);
#pragma unroll
          for (int u = 0; u < kTilesPerIter; ++u) {
            a[u][0] = s[u][0] + neg0; a[u][1] = s[u][1] + neg1;
            a[u][2] = s[u][2] + neg0; a[u][3] = s[u][3] + neg1;
          }
        }

        // ---- values of the tiles --------------------------------------------
#pragma unroll
        for (int u = 0; u < kTilesPerIter; ++u) {
          const uint32_t slot = slot0 + u * C::kSlot;
          const float nv0 = lds_half(slot + C::kOffNV + g * 2);
          const float nv1 = lds_half(slot + C::kOffNV + (g + 8) * 2);
          const float p0 = ex2(a[u][0]), p1 = ex2(a[u][1]);
          const float p2 = ex2(a[u][2]), p3 = ex2(a[u][3]);
          l0 += p0 + p2;
          l1 += p1 + p3;
          // rows g / g+8 of P' (token x head) -> B fragment (token pairs of head g)
          uint32_t r0 = pack_half2(p0 * nv0, p1 * nv0), r1 = pack_half2(p2 * nv1, p3 * nv1);
          if constexpr (MASKED) {
            r0 = ok[u][0] ? r0 : 0u;
            r1 = ok[u][1] ? r1 : 0u;
          }
          const uint32_t pb0 = movmatrix_trans(r0), pb1 = movmatrix_trans(r1);
          value_mmas<BWV, C::kVRow>(slot + C::kOffV + g * (2 * BWV) + (2 * t) * C::kVRow, sel_v, pb0,
                                    pb1, acc);
        }
      };
    for (int it = 0; it < n_iter; ++it) {
      issue_one();
      cp_async_wait<1>();
      __syncwarp();
      if (it < n_full && bad == 0u) {
        window(std::false_type{});
      } else {
        loaded = ~(bad >> (2 * chalf)) & 3u;
        window(std::true_type{});
      }
      __syncwarp();       // every lane is done with this half of the ring before it is refilled
      cbase = 2 * ring + kTilesPerIter * C::kSlot - cbase;
      chalf ^= 1;
      wtok += kIterTokens;
    }

    // ---- partial state of this chunk ---------------------------------------
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l0 += __shfl_xor_sync(kFull, l0, o);
      l1 += __shfl_xor_sync(kFull, l1, o);
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int h = 2 * t + e;
      if (h < p.n_rep) {
        const int64_t row = ((int64_t)b * p.Hq + kvh * p.n_rep + h) * chunks + chunk;
        float2 *dst = reinterpret_cast<float2 *>(p.part_acc + row * 128 + 16 * g);
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j] = make_float2(acc[j][e], acc[j][2 + e]);
        if (g == 0) {
          p.part_m[row] = e ? M1 : M0;
          p.part_l[row] = e ? l1 : l0;
        }
      }
    }
  }
  cp_async_wait<0>();
}

// End of a merge block in the exchange form.  The block's rows are on their way
// to every rank's buffer; after a barrier (which makes the block's stores
// visible to thread 0) and a system-scope fence (which orders them before what
// follows), thread 0 counts the block on a local counter.  The last block to
// arrive has, through that counter, seen every other block's fence; it fences
// once more and adds ONE arrival to slot `rank` of every rank's flag array
// (one remote operation per peer and call: an arrival per block, measured on
// two GPUs, cost 5 us more).  A rank's rows of call number s are complete in a
// buffer when that slot has reached s x state[2] (arrivals per call, 1 here).
// The last block also advances the call counter (state[0]).
__device__ __forceinline__ void publish_rows(const MergeParams &p, uint32_t step, unsigned blocks) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(p.done_counter, 1u) == blocks - 1) {
      *p.done_counter = 0;
      p.step_counter[2] = 1u;
      p.step_counter[0] = step;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;\n" ::"l"(p.peer_flags[r] + p.rank) : "memory");
    }
  }
}

// Merge of the chunk states of `hpb` query heads of one (sequence, kv head)
// group and rotation of their output rows back to the model basis:
// out = (sum_c w_c acc_c / sum_c w_c l_c) Pi_V with w_c = 2^(m_c - max m).  Only
// the chunks that exist for the sequence's length are read.  grid = (groups,
// n_rep / hpb): few groups with many chunks (one long sequence) are spread over
// more blocks by giving each block fewer heads.  512 threads: one warp per head
// computes the weights; the chunk sum of a (head, coordinate) is split over
// 512 / (hpb * 128) threads; thread (column, quarter) accumulates its quarter of
// the rows of Pi_V for every head, and the quarters are added through shared
// memory.
constexpr int kMergeThreads = 512;
__global__ void __launch_bounds__(kMergeThreads, 1) merge_group_kernel(
    MergeParams p, const int32_t *seq_lens, int num_groups, int Hkv, int n_rep, int hpb,
    int chunk_tokens, int max_tokens) {
  __shared__ float a_s[8][128];           // [way * hpb + head][coordinate] partial chunk sums
  __shared__ __align__(16) float at_s[128][8];   // [coordinate][head] normalised sums, for the rotation
  __shared__ float w_s[8][kMaxSplits];    // chunk weights; reused for the rotation's partial sums
  __shared__ float inv_s[8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Pi_V does not depend on the scan: stage it in shared memory while the scan
  // kernel is still draining; it serves every group this block merges.
  extern __shared__ __align__(16) float pi_s[];            // [128][128]
  const int col = tid & 127, part = tid >> 7;
  {
    const float4 *src = reinterpret_cast<const float4 *>(p.Pi_v);
    float4 *dst = reinterpret_cast<float4 *>(pi_s);
    const int shift = (int)((blockIdx.x * 37u + blockIdx.y * 11u) & 7u) * 512;   // spread the blocks
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = (tid + i * kMergeThreads + shift) & 4095;
      dst[e] = __ldg(src + e);
    }
  }
  asm volatile("griddepcontrol.wait;\n" ::: "memory");      // partial states are complete
  // (the exchange's wait kernel, if it follows, may be scheduled now: it waits
  // for this grid to finish before it reads anything)
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  if (p.work_counter != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0)
    *p.work_counter = 0;
  // The first 32 chunk states of a thread's (head, coordinate) are requested one
  // group ahead: for the first group before its weights, for every later group
  // during the previous group's rotation, so their round trip is hidden.
  const int ways = hpb <= 1 ? 4 : hpb <= 2 ? 2 : 1;        // threads sharing one (head, coordinate)
  const bool e0_on = tid < hpb * 128 * ways;               // element `tid` exists
  const int way0 = tid / (hpb * 128), hd0 = tid - way0 * hpb * 128;
  float v0[32];
  auto preload = [&](int grp) {
    const int gb = grp / Hkv, gk = grp - gb * Hkv;
    int gl = seq_lens[gb];
    gl = gl < 0 ? 0 : (gl > max_tokens ? max_tokens : gl);
    const int gchunks = (gl + chunk_tokens - 1) / chunk_tokens;
    const float *src0 = p.part_acc +
        (((int64_t)gb * p.Hq + gk * n_rep + blockIdx.y * hpb + (hd0 >> 7)) * p.num_splits) * 128 +
        (hd0 & 127);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int c = way0 + i * ways;
      v0[i] = e0_on && c < gchunks ? __ldcg(src0 + (int64_t)c * 128) : 0.f;
    }
  };
  if ((int)blockIdx.x < num_groups) preload(blockIdx.x);
  // number of this call in the exchange protocol (the counter is advanced by
  // the last block, after every block has read it: see the end of the kernel)
  const uint32_t exchange_step = p.world > 0 ? *p.step_counter + 1u : 0u;
  for (int group = blockIdx.x; group < num_groups; group += gridDim.x) {
  const int b = group / Hkv, kvh = group - b * Hkv;
  const int head0 = kvh * n_rep + blockIdx.y * hpb;          // first query head of this pass
  int L = seq_lens[b];
  L = L < 0 ? 0 : (L > max_tokens ? max_tokens : L);
  const int chunks = (L + chunk_tokens - 1) / chunk_tokens;
  const int64_t row0 = ((int64_t)b * p.Hq + head0) * p.num_splits;
  if (warp < hpb) {                                    // weights of head `warp`
    const int64_t base = row0 + (int64_t)warp * p.num_splits;
    float gmax = -INFINITY, denom = 0.f;
    if (chunks <= 256) {                               // one round trip: 8 chunks per lane
      float mv[8], lv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        mv[i] = c < chunks ? __ldcg(p.part_m + base + c) : -INFINITY;
        lv[i] = c < chunks ? __ldcg(p.part_l + base + c) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) gmax = fmaxf(gmax, mv[i]);
      gmax = warp_max(gmax);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        const float w = mv[i] == -INFINITY ? 0.f : exp2f(mv[i] - gmax);
        if (c < chunks) w_s[warp][c] = w;
        denom += w * lv[i];
      }
    } else {
      for (int c0 = 0; c0 < chunks; c0 += 256) {       // 8 loads per lane in flight
        float mv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = c0 + lane + 32 * i;
          mv[i] = c < chunks ? __ldcg(p.part_m + base + c) : -INFINITY;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) gmax = fmaxf(gmax, mv[i]);
      }
      gmax = warp_max(gmax);
      for (int c0 = 0; c0 < chunks; c0 += 256) {
        float mv[8], lv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = c0 + lane + 32 * i;
          mv[i] = c < chunks ? __ldcg(p.part_m + base + c) : -INFINITY;
          lv[i] = c < chunks ? __ldcg(p.part_l + base + c) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = c0 + lane + 32 * i;
          const float w = mv[i] == -INFINITY ? 0.f : exp2f(mv[i] - gmax);
          if (c < chunks) w_s[warp][c] = w;
          denom += w * lv[i];
        }
      }
    }
    denom = warp_sum(denom);
    if (lane == 0) inv_s[warp] = denom > 0.f ? 1.f / fmaxf(denom, 1e-30f) : 0.f;
  }
  __syncthreads();
  // chunk sums: element `tid` starts from the states requested above; a group of
  // 8 heads has a second element per thread
  for (int e = tid; e < hpb * 128 * ways; e += kMergeThreads) {
    const int way = e / (hpb * 128), hd = e - way * hpb * 128;
    const int h = hd >> 7, d = hd & 127;
    const float *src = p.part_acc + (row0 + (int64_t)h * p.num_splits) * 128 + d;
    float a = 0.f;
    for (int c0 = way; c0 < chunks; c0 += 32 * ways) {      // 32 loads in flight
      if (e != tid || c0 != way) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int c = c0 + i * ways;
          v0[i] = c < chunks ? __ldcg(src + (int64_t)c * 128) : 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int c = c0 + i * ways;
        a = fmaf(c < chunks ? w_s[h][c] : 0.f, v0[i], a);
      }
    }
    a_s[way * hpb + h][d] = a;
  }
  __syncthreads();
  for (int e = tid; e < hpb * 128; e += kMergeThreads) {
    const int h = e >> 7, d = e & 127;
    float a = a_s[h][d];
    for (int w = 1; w < ways; ++w) a += a_s[w * hpb + h][d];
    at_s[d][h] = a * inv_s[h];
  }
  __syncthreads();
  if (group + (int)gridDim.x < num_groups) preload(group + gridDim.x);   // next group's states
  float o[8];
#pragma unroll
  for (int h = 0; h < 8; ++h) o[h] = 0.f;
  // (heads hpb .. 7 of at_s are never written and the sums made of them are
  // never stored; a group of at most four heads skips the second half)
  const bool wide = hpb > 4;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int d = part * 32 + i;
    const float w = pi_s[d * 128 + col];
    const float4 x = *reinterpret_cast<const float4 *>(&at_s[d][0]);
    o[0] = fmaf(x.x, w, o[0]); o[1] = fmaf(x.y, w, o[1]);
    o[2] = fmaf(x.z, w, o[2]); o[3] = fmaf(x.w, w, o[3]);
    if (wide) {
      const float4 y = *reinterpret_cast<const float4 *>(&at_s[d][4]);
      o[4] = fmaf(y.x, w, o[4]); o[5] = fmaf(y.y, w, o[5]);
      o[6] = fmaf(y.z, w, o[6]); o[7] = fmaf(y.w, w, o[7]);
    }
  }
  // the weights are consumed (second barrier above): their storage now holds the
  // partial outputs of quarters 1..3; quarter 0 stays in registers
  float (*o_s)[8][128] = reinterpret_cast<float (*)[8][128]>(&w_s[0][0]);
  if (part > 0) {
#pragma unroll
    for (int h = 0; h < 8; ++h)
      if (h < hpb) o_s[part][h][col] = o[h];
  }
  __syncthreads();
  if (part == 0) {
#pragma unroll
    for (int h = 0; h < 8; ++h) {
      if (h < hpb) {
        const float v = (o[h] + o_s[1][h][col]) + (o_s[2][h][col] + o_s[3][h][col]);
        if (p.world == 0) {
          store_from_float(p.out, (int64_t)b * p.osb + (int64_t)(head0 + h) * p.osh + col, v,
                           p.dtype);
        } else {                          // the row goes to every rank's full buffer
          const int64_t at = (int64_t)b * p.osb + (int64_t)(p.head_offset + head0 + h) * p.osh + col;
          void *const *dests = p.peer_out[exchange_step & 1u];
          for (int r = 0; r < p.world; ++r) store_from_float(dests[r], at, v, p.dtype);
        }
      }
    }
  }
  __syncthreads();                        // shared arrays are reused by the next group
  }
  if (p.world > 0) publish_rows(p, exchange_step, gridDim.x * gridDim.y);
}

// The same merge with many small blocks: one 128-thread block per `hpb` query
// heads of a (sequence, kv head) group (grid = groups x n_rep / hpb), so that an
// SM holds many blocks at once and their round trips to L2 overlap (the
// persistent kernel above walks its groups one after the other).  Thread =
// output coordinate.  Warp w computes the chunk weights of heads w and w + 4 of
// the block's heads; every thread then sums its coordinate over the chunks,
// sixteen states in flight; the rotation reads Pi_V through L1, which this
// kernel leaves large (it holds the 64 KB of Pi_V for every block of the SM).
// At most kSmallMergeChunks chunks per sequence.
constexpr int kSmallMergeChunks = 256;
__global__ void __launch_bounds__(128, 8) merge_small_kernel(MergeParams p, const int32_t *seq_lens,
                                                          int Hkv, int group_heads, int n_rep,
                                                          int chunk_tokens, int max_tokens) {
  __shared__ float w_s[8][kSmallMergeChunks];
  __shared__ __align__(16) float a_s[128][8];           // [coordinate][head]
  __shared__ float inv_s[8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = blockIdx.x;
  const int b = group / Hkv, kvh = group - b * Hkv;
  const int head0 = kvh * group_heads + blockIdx.y * n_rep;   // n_rep: heads of this block
  int L = seq_lens[b];
  L = L < 0 ? 0 : (L > max_tokens ? max_tokens : L);
  const int chunks = (L + chunk_tokens - 1) / chunk_tokens;
  asm volatile("griddepcontrol.wait;\n" ::: "memory");      // partial states are complete
  // (the exchange's wait kernel, if it follows, may be scheduled now: it waits
  // for this grid to finish before it reads anything)
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  if (p.work_counter != nullptr && group == 0 && blockIdx.y == 0 && tid == 0) *p.work_counter = 0;
  const uint32_t exchange_step = p.world > 0 ? *p.step_counter + 1u : 0u;
  const int64_t row0 = ((int64_t)b * p.Hq + head0) * p.num_splits;
  for (int h = warp; h < n_rep; h += 4) {              // weights of head h
    const int64_t base = row0 + (int64_t)h * p.num_splits;
    float mv[kSmallMergeChunks / 32], lv[kSmallMergeChunks / 32];
    float gmax = -INFINITY, denom = 0.f;
#pragma unroll
    for (int i = 0; i < kSmallMergeChunks / 32; ++i) {
      const int c = lane + 32 * i;
      mv[i] = c < chunks ? __ldcg(p.part_m + base + c) : -INFINITY;
      lv[i] = c < chunks ? __ldcg(p.part_l + base + c) : 0.f;
      gmax = fmaxf(gmax, mv[i]);
    }
    gmax = warp_max(gmax);
#pragma unroll
    for (int i = 0; i < kSmallMergeChunks / 32; ++i) {
      const int c = lane + 32 * i;
      const float w = mv[i] == -INFINITY ? 0.f : exp2f(mv[i] - gmax);
      if (c < chunks) w_s[h][c] = w;
      denom += w * lv[i];
    }
    denom = warp_sum(denom);
    if (lane == 0) inv_s[h] = denom > 0.f ? 1.f / fmaxf(denom, 1e-30f) : 0.f;
  }
  __syncthreads();
  for (int h = 0; h < n_rep; ++h) {                     // chunk sums of coordinate `tid`
    const float *src = p.part_acc + (row0 + (int64_t)h * p.num_splits) * 128 + tid;
    float a = 0.f;
    for (int c0 = 0; c0 < chunks; c0 += 16) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = c0 + i < chunks ? __ldcg(src + (int64_t)(c0 + i) * 128) : 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) a = fmaf(c0 + i < chunks ? w_s[h][c0 + i] : 0.f, v[i], a);
    }
    a_s[tid][h] = a * inv_s[h];
  }
  for (int h = n_rep; h < 8; ++h) a_s[tid][h] = 0.f;
  __syncthreads();
  float o[8];
#pragma unroll
  for (int h = 0; h < 8; ++h) o[h] = 0.f;
  const float *pi = p.Pi_v + tid;
#pragma unroll 8
  for (int d = 0; d < 128; ++d) {
    const float w = __ldg(pi + d * 128);
    const float4 x = *reinterpret_cast<const float4 *>(&a_s[d][0]);
    const float4 y = *reinterpret_cast<const float4 *>(&a_s[d][4]);
    o[0] = fmaf(x.x, w, o[0]); o[1] = fmaf(x.y, w, o[1]);
    o[2] = fmaf(x.z, w, o[2]); o[3] = fmaf(x.w, w, o[3]);
    o[4] = fmaf(y.x, w, o[4]); o[5] = fmaf(y.y, w, o[5]);
    o[6] = fmaf(y.z, w, o[6]); o[7] = fmaf(y.w, w, o[7]);
  }
#pragma unroll
  for (int h = 0; h < 8; ++h) {
    if (h < n_rep) {
      if (p.world == 0) {
        store_from_float(p.out, (int64_t)b * p.osb + (int64_t)(head0 + h) * p.osh + tid, o[h],
                         p.dtype);
      } else {                            // the row goes to every rank's full buffer
        const int64_t at = (int64_t)b * p.osb + (int64_t)(p.head_offset + head0 + h) * p.osh + tid;
        void *const *dests = p.peer_out[exchange_step & 1u];
        for (int r = 0; r < p.world; ++r) store_from_float(dests[r], at, o[h], p.dtype);
      }
    }
  }
  if (p.world > 0) publish_rows(p, exchange_step, gridDim.x * gridDim.y);
}

// Waits (bounded) until every rank's rows of the call being waited for are in
// the local buffer: slot r of the local flag array counts the arrivals of rank
// r's merge blocks, `state` = {calls completed, waits completed, merge blocks
// per call}.  The kernel numbers its own calls (state[1]), so it does not
// depend on the merge kernel ahead of it and starts polling as soon as it is
// scheduled; the blocks per call are read inside the loop because the local
// merge may not have recorded them yet.
__global__ void exchange_wait_kernel(const uint32_t *flags, int world, uint32_t *state,
                                     long long spin_limit, int32_t *status) {
  const int r = threadIdx.x;
  uint32_t step = 0;
  if (r == 0) step = ++state[1];
  step = __shfl_sync(0xffffffffu, step, 0);
  if (r < world) {
    const volatile uint32_t *slot = flags + r;
    const volatile uint32_t *blocks = state + 2;
    bool arrived = false;
    for (long long i = 0; i < spin_limit; ++i) {
      const uint32_t n = *blocks;
      if (n != 0u && (int32_t)(*slot - step * n) >= 0) {
        arrived = true;
        break;
      }
      __nanosleep(20);
    }
    if (!arrived && status != nullptr) atomicOr(status, WTQ_STATUS_EXCHANGE_TIMEOUT);
  }
  __threadfence_system();
}

int launch_exchange_wait(const uint32_t *flags, int world, uint32_t *state,
                         long long spin_limit, int32_t *status, cudaStream_t stream) {
  cudaLaunchAttribute pdl;
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = stream;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, exchange_wait_kernel, flags, world, state, spin_limit,
                                     status);
  note_launches(1);
  return check_cuda(e, "wtq_exchange_wait launch");
}

// Worker warps per SM of the instantiation serving (bw_k, bw_v); 0 when the
// widths have no tensor-core kernel.
int mma_warps_per_sm(int bw_k, int bw_v) {
  if (bw_k == 4 && bw_v == 4) return Cfg<4, 4>::kWarps;
  if (bw_k == 4 && bw_v == 6) return Cfg<4, 6>::kWarps;
  if (bw_k == 6 && bw_v == 6) return Cfg<6, 6>::kWarps;
  if (bw_k == 8 && bw_v == 8) return Cfg<8, 8>::kWarps;
  return 0;
}

bool mma_eligible(const DecodeParams &p) {
  auto aligned = [](const void *ptr) { return ((uintptr_t)ptr & 15) == 0; };
  return p.D == 128 && mma_warps_per_sm(p.k.bw, p.v.bw) > 0 && p.S >= 16 &&
         (p.S & (p.S - 1)) == 0 && p.n_rep <= 8 &&
         aligned(p.k.pages) && aligned(p.v.pages) && aligned(p.k.norms) && aligned(p.v.norms) &&
         p.k.page_stride % 16 == 0 && p.k.head_stride % 16 == 0 && p.v.page_stride % 16 == 0 &&
         p.v.head_stride % 16 == 0 && p.k.norm_page_stride % 8 == 0 &&
         p.k.norm_head_stride % 8 == 0 && p.v.norm_page_stride % 8 == 0 &&
         p.v.norm_head_stride % 8 == 0 && aligned(p.q_rot) && aligned(p.part_acc) &&
         aligned(p.lut) && p.k.page_stride < (int64_t)1 << 31 && p.v.page_stride < (int64_t)1 << 31 &&
         p.k.norm_page_stride < (int64_t)1 << 30 && p.v.norm_page_stride < (int64_t)1 << 30;
}

int mma_lut_words(int bw_k, int bw_v) {
  if (bw_k == 4 && bw_v == 4) return Cfg<4, 4>::kLutBytes / 4;
  if (bw_k == 4 && bw_v == 6) return Cfg<4, 6>::kLutBytes / 4;
  if (bw_k == 6 && bw_v == 6) return Cfg<6, 6>::kLutBytes / 4;
  if (bw_k == 8 && bw_v == 8) return Cfg<8, 8>::kLutBytes / 4;
  return 0;
}

// Tokens per chunk for `splits` chunks over `max_tokens`, a multiple of 32.
int mma_chunk_tokens(int max_tokens, int splits) {
  constexpr int kGrain = 2 * kTileTokens;
  int per = (max_tokens + splits - 1) / splits;
  per = (per + kGrain - 1) / kGrain * kGrain;
  return per < kGrain ? kGrain : per;
}

// Merge of the chunk states written by a tensor-core scan (decode or prefill):
// `B` rows of `seq_lens`, each with ceil(len / chunk_tokens) chunk states per
// head, m.num_splits slots apart.  Launched so that it may begin while the scan
// drains (it waits before it reads).
int launch_mma_merge(const MergeParams &m, const int32_t *seq_lens, int B, int Hkv, int n_rep,
                     int chunk_tokens, int max_tokens, cudaStream_t stream) {
  const int sms = device_sms();
  static std::atomic<bool> opted_in_dev[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !opted_in_dev[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(merge_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         128 * 128 * (int)sizeof(float));
    if (e != cudaSuccess) return check_cuda(e, "wtq_decode: merge shared memory opt-in");
    opted_in_dev[dev & 63].store(true, std::memory_order_release);
  }
  cudaLaunchAttribute pdl;
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.stream = stream;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cudaError_t e;
  const int num_groups = B * Hkv;
  if (num_groups >= 4 * sms && m.num_splits <= kSmallMergeChunks) {
    // many groups: small blocks, several resident per SM, all heads of a group
    // in one block.  (With fewer groups the persistent kernel below is faster,
    // also against this kernel run with fewer heads per block: measured.)
    const int heads = n_rep;
    cfg.gridDim = dim3((unsigned)num_groups, (unsigned)(n_rep / heads));
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    e = cudaLaunchKernelEx(&cfg, merge_small_kernel, m, seq_lens, Hkv, n_rep, heads, chunk_tokens,
                           max_tokens);
    note_launches(1);
    return check_cuda(e, "wtq_decode merge launch");
  }
  // heads per merge block: all of the group when there are many groups, fewer
  // (down to one) when a handful of long sequences would leave most SMs idle
  int hpb = n_rep;
  while (hpb > 1 && hpb % 2 == 0 && (int64_t)num_groups * (n_rep / hpb) < sms / 2) hpb /= 2;
  // one merge block is resident per SM: no more blocks than SMs, each walks its groups
  const int passes = n_rep / hpb;
  cfg.gridDim = dim3((unsigned)std::min(num_groups, std::max(1, sms / passes)), (unsigned)passes);
  cfg.blockDim = dim3(kMergeThreads);
  cfg.dynamicSmemBytes = 128 * 128 * sizeof(float);
  e = cudaLaunchKernelEx(&cfg, merge_group_kernel, m, seq_lens, num_groups, Hkv, n_rep, hpb,
                         chunk_tokens, max_tokens);
  note_launches(1);
  return check_cuda(e, "wtq_decode merge launch");
}

template <int BWK, int BWV>
static int launch_one(const DecodeParams &p, const MergeParams &m, int sms, cudaStream_t stream) {
  using C = Cfg<BWK, BWV>;
  // function attributes belong to the device the call runs on
  static std::atomic<bool> opted_in_dev[64];
  int dev = 0;
  cudaGetDevice(&dev);
  std::atomic<bool> &opted_in = opted_in_dev[dev & 63];
  if (dev >= 64 || !opted_in.load(std::memory_order_acquire)) {   // setting twice is harmless
    cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<BWK, BWV, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)C::kDynamicSmem);
    if (e != cudaSuccess) return check_cuda(e, "wtq_decode: shared memory opt-in");
    e = cudaFuncSetAttribute(decode_mma_kernel<BWK, BWV, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kDynamicSmem);
    if (e != cudaSuccess) return check_cuda(e, "wtq_decode: shared memory opt-in");
    opted_in.store(true, std::memory_order_release);
  }
  const int max_tokens = p.max_pages * p.S;
  const int chunk_tokens = mma_chunk_tokens(max_tokens, p.num_splits);
  const int64_t items = (int64_t)p.B * p.Hkv * p.num_splits;
  int grid = (int)((items + C::kWarps - 1) / C::kWarps);
  if (grid > sms) grid = sms;
  // Both launches may begin before the kernel ahead of them has drained; each
  // kernel waits (griddepcontrol.wait) before it touches what that kernel wrote.
  cudaLaunchAttribute pdl;
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kDynamicSmem;
  cfg.stream = stream;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  profile_mark_begin(stream);
  cudaError_t e = p.S == 16 ? cudaLaunchKernelEx(&cfg, decode_mma_kernel<BWK, BWV, true>, p, chunk_tokens)
                            : cudaLaunchKernelEx(&cfg, decode_mma_kernel<BWK, BWV, false>, p, chunk_tokens);
  profile_mark_end(stream);
  if (e != cudaSuccess) return check_cuda(e, "wtq_decode mma launch");
  note_launches(1);
  return launch_mma_merge(m, p.seq_lens, p.B, p.Hkv, p.n_rep, chunk_tokens, max_tokens, stream);
}

int launch_decode_mma(const DecodeParams &p, const MergeParams &m, cudaStream_t stream) {
  const int sms = device_sms();
  if (p.k.bw == 4 && p.v.bw == 4) return launch_one<4, 4>(p, m, sms, stream);
  if (p.k.bw == 4 && p.v.bw == 6) return launch_one<4, 6>(p, m, sms, stream);
  if (p.k.bw == 6 && p.v.bw == 6) return launch_one<6, 6>(p, m, sms, stream);
  if (p.k.bw == 8 && p.v.bw == 8) return launch_one<8, 8>(p, m, sms, stream);
  return fail(WTQ_ERR_UNSUPPORTED, "wtq_decode: no tensor-core kernel for widths %d/%d", p.k.bw,
              p.v.bw);
}

}  // namespace wtq
