// Fused dequantisation on the fifth-generation tensor cores (tcgen05): the
// same product as dequant_mma_kernel, out = (C Pi) * norm for head_dim 128 and
// widths 4/6/8, with the 128 x 128 accumulator of a tile in tensor memory
// instead of registers.
//
// A block of sixteen warps takes tiles of 128 packed rows.  Per tile:
//   decode    every warp turns 8 rows into fp16 centroid values through the
//             per-lane lookup tables (wtq_lut.cuh) and stores them as the A
//             operand in shared memory, in the canonical K-major layout without
//             swizzle: 8-row x 16-byte core matrices, 128 bytes each, the 16
//             pieces of a row group one after the other (2 KB per 8 rows);
//   multiply  one thread issues tcgen05.mma (M 128, N 128, K 16, fp16 in, fp32
//             out) for the eight K steps of each product term; B is Pi with one
//             row per output coordinate in the same layout, resident in shared
//             memory; tcgen05.commit signals an mbarrier when they are done;
//   store     every warp reads its 32 lanes x 32 columns of the accumulator with
//             tcgen05.ld, scales by the row norm, converts, and passes the rows
//             through a staging area so that they leave as whole row segments.
// The accumulator is double-buffered: while the tensor cores work on tile i the
// warps store tile i - 1, and the packed rows of tile i + 1 are already on their
// way into registers.
// TERMS = 1: single fp16 operands.  TERMS = 3: centroids and Pi as fp16 high and
// low parts (times 2^8), the three significant products accumulated in the same
// tensor-memory tile.  Every wait is bounded; a wait that runs out marks the
// status word and the block leaves after freeing its tensor memory.
#include <atomic>
#include <mutex>

#include "wtq_common.cuh"
#include "wtq_lut.cuh"
#include "wtq_dequant.cuh"

namespace wtq {
namespace dq5 {

// Eight warps decode and feed the tensor cores, eight warps drain the accumulators.
constexpr int kFeedWarps = 8, kDrainWarps = 8, kWarps = kFeedWarps + kDrainWarps, kThreads = 32 * kWarps;
constexpr int kLaneRows = 16 / kFeedWarps;         // rows a lane decodes per tile (8 per warp each)
constexpr int kWarpCols = 128 / (kDrainWarps / 4); // accumulator columns a warp stores
constexpr uint32_t kBase = 1024;                  // dynamic shared memory is assumed to start at or below this
constexpr uint32_t kBarDone = kBase;              // 2 mbarriers: the products into accumulator b are complete
constexpr uint32_t kBarFree = kBase + 16;         // 2 mbarriers: accumulator b has been read out
constexpr uint32_t kTmemSlot = kBase + 32;        // tensor-memory address written by tcgen05.alloc
constexpr uint32_t kNorms = kBase + 64;           // 3 x 128 floats: the norms of three tiles in flight
constexpr uint32_t kCent = kBase + 2048;          // 256 floats: the codebook while the tables are built
constexpr uint32_t kOperand = 128 * 128 * 2;      // one fp16 operand tile
constexpr uint32_t kBHi = 4096;
static_assert(kCent + 1024 <= kBHi, "low region");
constexpr uint32_t kStage = kBHi + kOperand;      // output staging, per warp (see store_tile)
constexpr uint32_t kStageBytes = 16 * (2 * kWarpCols + 16);
static_assert(kStage + kDrainWarps * kStageBytes <= mma::kLutAddr && 8 * (4 * kWarpCols + 16) <= kStageBytes, "staging");
constexpr uint32_t kCols = 256;                   // tensor memory: two accumulators of 128 columns
constexpr float kOperandScale = 256.f, kResultScale = 1.f / (256.f * 256.f);
// instruction descriptor: dense, fp32 accumulator, fp16 A and B, both K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

template <int BW, int TERMS> struct Map {
  static constexpr uint32_t kLutBytes = mma::lut_entries(BW) * 256u;
  static constexpr uint32_t kAHi = mma::kLutAddr + kLutBytes;
  static constexpr uint32_t kALo = kAHi + kOperand;
  static constexpr uint32_t kBLo = kALo + kOperand;
  // the single-term form has room for two operand tiles: tile i + 1 is decoded while the
  // tensor cores still read tile i
  static constexpr int kOperandTiles = TERMS == 3 ? 1 : 2;
  static constexpr uint32_t kDynamic = TERMS == 3 ? kBLo + kOperand : kAHi + 2 * kOperand;
  static_assert(kDynamic <= 227u * 1024u, "shared memory budget");
};

// Element (row, piece) of an operand tile: 16-byte piece `piece` (8 values along K) of row `row`.
__device__ __forceinline__ uint32_t operand_at(uint32_t tile, int row, int piece) {
  return tile + (uint32_t)(row >> 3) * 2048u + (uint32_t)piece * 128u + (uint32_t)(row & 7) * 16u;
}
// Shared-memory descriptor of the two pieces (K = 16) starting at piece 2 * ks of a tile.
__device__ __forceinline__ uint64_t operand_desc(uint32_t tile, int ks) {
  const uint32_t start = tile + (uint32_t)ks * 256u;
  return (uint64_t)((start >> 4) & 0x3fffu) | ((uint64_t)(128u >> 4) << 16) |   // leading offset: next piece
         ((uint64_t)(2048u >> 4) << 32) |                                       // stride offset: next 8 rows
         ((uint64_t)1 << 46);                                                   // descriptor version, no swizzle
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(kIdesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t addr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr));
}

// Eight consecutive centroid values (fp16 pairs) of a lane's share of a packed
// row: codes 8 J .. 8 J + 7 of the 32 the words hold.
template <int BW, int J>
__device__ __forceinline__ void decode_piece(const uint32_t (&w)[BW], uint32_t sel, uint32_t (&f)[4]) {
  if constexpr (BW == 4) {
    f[0] = lut_byte<0>(w[J], sel); f[1] = lut_byte<1>(w[J], sel);
    f[2] = lut_byte<2>(w[J], sel); f[3] = lut_byte<3>(w[J], sel);
  } else {
    f[0] = join(lut_code<BW, 8 * J>(w, sel), lut_code<BW, 8 * J + 1>(w, sel));
    f[1] = join(lut_code<BW, 8 * J + 2>(w, sel), lut_code<BW, 8 * J + 3>(w, sel));
    f[2] = join(lut_code<BW, 8 * J + 4>(w, sel), lut_code<BW, 8 * J + 5>(w, sel));
    f[3] = join(lut_code<BW, 8 * J + 6>(w, sel), lut_code<BW, 8 * J + 7>(w, sel));
  }
}
template <int BW>
__device__ __forceinline__ void decode_row(const uint32_t (&w)[BW], uint32_t sel, uint32_t tile, int row, int t) {
  uint32_t f[4];
  decode_piece<BW, 0>(w, sel, f); sts128(operand_at(tile, row, 4 * t + 0), f[0], f[1], f[2], f[3]);
  decode_piece<BW, 1>(w, sel, f); sts128(operand_at(tile, row, 4 * t + 1), f[0], f[1], f[2], f[3]);
  decode_piece<BW, 2>(w, sel, f); sts128(operand_at(tile, row, 4 * t + 2), f[0], f[1], f[2], f[3]);
  decode_piece<BW, 3>(w, sel, f); sts128(operand_at(tile, row, 4 * t + 3), f[0], f[1], f[2], f[3]);
}
template <int BW>
__device__ __forceinline__ void load_row(const uint8_t *packed, int64_t src, int t, uint32_t (&w)[BW]) {
  const uint8_t *at = packed + src * (16 * BW) + t * (4 * BW);
  if constexpr (BW == 6) {
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const uint2 v = __ldg(reinterpret_cast<const uint2 *>(at) + i);
      w[2 * i] = v.x; w[2 * i + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < BW / 4; ++i) {
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(at) + i);
      w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
    }
  }
}

template <int DT> __device__ __forceinline__ uint32_t pack2(float x, float y) {
  if constexpr (DT == WTQ_BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t *>(&h);
  } else {
    return pack_half2(x, y);
  }
}

// state: word 0 = 1 when the shared-memory layout assumption is broken, word 1 =
// 1 when a wait for the tensor cores ran out.
template <int BW, int TERMS, int DT>
__global__ void __launch_bounds__(kThreads, 1) dequant_umma_kernel(DequantParams p, int32_t *state) {
  using M = Map<BW, TERMS>;
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  // lane = g + 8 t: the eight lanes that store together hold eight different rows of one
  // 16-byte piece, which the operand layout puts in eight different bank groups
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane & 7, t = lane >> 3;
  if ((uint32_t)__cvta_generic_to_shared(dyn_smem) > kBase) {
    if (tid == 0 && blockIdx.x == 0) state[0] = 1;
    return;
  }
  if (p.N == 0) return;                           // the set-up probe: nothing to read
  // ---- one-time: tensor memory, barrier, tables ------------------------------------
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(kTmemSlot),
                 "r"(kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  if (tid == 0) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(kBarDone + 8u * b) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(kBarFree + 8u * b), "r"(kDrainWarps) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  for (int e = tid; e < (1 << BW); e += kThreads)
    sts32(kCent + 4 * e, __float_as_uint(__ldg(p.centroids + e) * kOperandScale));
  // B[c][d] = Pi[d][c]: a lane takes column c = 8 cb + (lane & 7) and the rows d = 2 (4 db +
  // (lane >> 3)), d + 1 (sector-sized reads)
#pragma unroll 8
  for (int it = 0; it < 256 / kWarps; ++it) {
    const int combo = it * kWarps + warp, cb = combo & 15, db = combo >> 4;
    const int c = 8 * cb + (lane & 7), d = 2 * (4 * db + (lane >> 3));
    const float x0 = __ldg(p.Pi + d * 128 + c) * kOperandScale;
    const float x1 = __ldg(p.Pi + (d + 1) * 128 + c) * kOperandScale;
    const __half2 hi = __floats2half2_rn(x0, x1);
    const uint32_t off = operand_at(0, c, d >> 3) + (uint32_t)(d & 7) * 2u;
    sts32(kBHi + off, *reinterpret_cast<const uint32_t *>(&hi));
    if constexpr (TERMS == 3)
      sts32(M::kBLo + off, pack_half2(x0 - __low2float(hi), x1 - __high2float(hi)));
  }
  __syncthreads();
  constexpr int kLutWords = (int)(M::kLutBytes / 8);       // one side: entries x 32 lanes
  for (int idx = tid; idx < kLutWords; idx += kThreads) {
    const int index = idx >> 5;
    float a, b;
    if constexpr (BW == 4) {
      a = __uint_as_float(lds32(kCent + 4 * (index & 15)));
      b = __uint_as_float(lds32(kCent + 4 * (index >> 4)));
    } else {
      a = b = __uint_as_float(lds32(kCent + 4 * index));
    }
    const __half2 hi = __floats2half2_rn(a, b);
    const uint32_t at = mma::kLutAddr | (uint32_t)index << 8 | (uint32_t)(idx & 31) << 2;
    sts32(at, *reinterpret_cast<const uint32_t *>(&hi));
    if constexpr (TERMS == 3)
      sts32(at | 0x80u, pack_half2(a - __low2float(hi), b - __high2float(hi)));
  }
  // what the tensor cores will read was written with ordinary stores
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = lds32(kTmemSlot);

  const uint32_t sel = mma::kLutAddr | (uint32_t)(lane << 2);
  const int64_t tiles = (p.N + 127) >> 7;
  const uint32_t L32 = (uint32_t)p.L;
  constexpr int kEsize = DT == WTQ_F32 ? 4 : 2;

  // packed words and norm of the lane's row(s) of a tile
  const bool dense = p.L == p.MAXLEN;                       // source row = logical row: no plane arithmetic
  auto fetch = [&](int64_t tile, uint32_t (&w)[kLaneRows][BW], float (&nrm)[kLaneRows]) {
    const int64_t row0 = tile << 7;
    const int last = (int)min((int64_t)127, p.N - 1 - row0);   // rows past the end re-read the last one
    int64_t plane0 = 0;
    uint32_t pos0 = 0;
    if (!dense) {
      plane0 = row0 / p.L;
      pos0 = (uint32_t)(row0 - plane0 * p.L);
    }
#pragma unroll
    for (int h = 0; h < kLaneRows; ++h) {
      const int lr = min(8 * kLaneRows * warp + 8 * h + g, last);
      int64_t src = row0 + lr;
      if (!dense) {
        const uint32_t pos = pos0 + (uint32_t)lr, wrap = pos / L32;
        src = (plane0 + wrap) * p.MAXLEN + (pos - wrap * L32);
      }
      load_row<BW>(p.packed, src, t, w[h]);
      nrm[h] = __half2float(p.norms[src]) * kResultScale;
    }
  };
  // this thread's share of a finished accumulator: lane 32 (warp % 4) + lane, columns
  // kWarpCols (warp / 4) ..
  // (a warp may read the tensor-memory lanes 32 (warp % 4) ..; kFeedWarps is a multiple of 4)
  const int dw = warp - kFeedWarps;                         // index among the draining warps
  auto store_tile = [&](int64_t tile, int buf, int slot) {
    const int lr = 32 * (dw & 3) + lane;
    const float nrm = __uint_as_float(lds32(kNorms + 512u * slot + 4u * lr));
    const uint32_t taddr =
        tmem + ((uint32_t)(32 * (dw & 3)) << 16) + (uint32_t)(128 * buf + kWarpCols * (dw >> 2));
    uint32_t v[kWarpCols / 32][32];
#pragma unroll
    for (int i = 0; i < kWarpCols / 32; ++i) tmem_load32(taddr + 32 * i, v[i]);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
    // the accumulator and the norms are in registers: hand the buffer back
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncwarp();
    if (lane == 0)
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(kBarFree + 8u * buf) : "memory");
    // The thread holds consecutive columns of ONE row; stored as they are, every
    // store instruction of the warp would touch 32 rows.  A few rows at a time go
    // through a staging area instead and leave as whole row segments.
    constexpr int kRowBytes = kWarpCols * kEsize;           // this warp's part of a row
    constexpr int kPassRows = kEsize == 2 ? 16 : 8;
    constexpr uint32_t kStride = kRowBytes + 16;            // pad: the rows of a pass land in different banks
    const uint32_t stage = kStage + (uint32_t)dw * kStageBytes;
    uint32_t q[kRowBytes / 4];                              // the row segment, converted
#pragma unroll
    for (int j = 0; j < kWarpCols / 32; ++j) {
      if constexpr (kEsize == 4) {
#pragma unroll
        for (int i = 0; i < 32; ++i) q[32 * j + i] = __float_as_uint(__uint_as_float(v[j][i]) * nrm);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          q[16 * j + i] = pack2<DT>(__uint_as_float(v[j][2 * i]) * nrm, __uint_as_float(v[j][2 * i + 1]) * nrm);
      }
    }
    uint8_t *base = (uint8_t *)p.out + (dw >> 2) * kRowBytes;
    const int64_t n0 = (tile << 7) + 32 * (dw & 3);
#pragma unroll
    for (int ps = 0; ps < 32 / kPassRows; ++ps) {
      if (lane / kPassRows == ps) {
#pragma unroll
        for (int i = 0; i < kRowBytes / 16; ++i)
          sts128(stage + (uint32_t)(lane % kPassRows) * kStride + 16u * i, q[4 * i], q[4 * i + 1], q[4 * i + 2],
                 q[4 * i + 3]);
      }
      __syncwarp();
      constexpr int kPieces = kPassRows * kRowBytes / 16;
      static_assert(kPieces % 32 == 0, "a pass is a whole number of warp-wide copies");
#pragma unroll
      for (int k = 0; k < kPieces / 32; ++k) {
        const int c = lane + 32 * k, r = c / (kRowBytes / 16), piece = c % (kRowBytes / 16);
        const uint4 v = lds128(stage + (uint32_t)r * kStride + 16u * piece);
        const int64_t n = n0 + ps * kPassRows + r;
        if (n < p.N) *reinterpret_cast<uint4 *>(base + n * (128 * kEsize) + 16 * piece) = v;
      }
      __syncwarp();
    }
  };

  // Bounded wait for completion number `use` (0, 1, ...) of an mbarrier; false if it ran out.
  auto wait_for = [&](uint32_t bar, int use) -> bool {
    uint32_t done = 0;
    for (int spin = 0; spin < (1 << 22) && !done; ++spin) {
      asm volatile(
          "{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, q;\n\t}\n"
          : "=r"(done) : "r"(bar), "r"((uint32_t)(use & 1)) : "memory");
    }
    return done != 0;
  };

  // Tile i of this block uses accumulator i & 1 and norm slot i % 3.  What orders the two
  // groups of warps:
  //   done[b]  arrives (tcgen05.commit) when the products of a tile into accumulator b are
  //            complete: the draining warps may read it, the feeding warps may overwrite the
  //            operand tile;
  //   free[b]  arrives (once per draining warp) when accumulator b and its norms are in
  //            registers: the next products into b may be issued.
  // Every wait is bounded; whoever runs out of patience marks the state word and leaves its
  // loop, and the others then run out of patience too.
  if (warp < kFeedWarps) {
    uint32_t w[kLaneRows][BW], w_next[kLaneRows][BW];
    float nrm[kLaneRows], nrm_next[kLaneRows] = {};
    int64_t tile = blockIdx.x;
    if (tile < tiles) fetch(tile, w, nrm);
    for (int i = 0; tile < tiles; tile += gridDim.x, ++i) {
      const int buf = i & 1, slot = i % 3;
      // the next tile's rows are requested now and used a whole iteration later
      const bool more = tile + gridDim.x < tiles;
      if (more) fetch(tile + gridDim.x, w_next, nrm_next);
      // the operand tile this one is decoded into is free once the products of the tile that
      // used it last (the previous tile, or the one before with two operand tiles) are complete
      uint32_t late = 0;
      const uint32_t a_hi = M::kAHi + (M::kOperandTiles == 2 ? (uint32_t)buf * kOperand : 0u);
      if constexpr (M::kOperandTiles == 2) {
        if (i > 1) late = wait_for(kBarDone + 8u * buf, (i - 2) >> 1) ? 0u : 1u;
      } else {
        if (i > 0) late = wait_for(kBarDone + 8u * (buf ^ 1), (i - 1) >> 1) ? 0u : 1u;
      }
      {
        uint32_t any;                                       // the same answer for all feeding warps
        asm volatile(
            "{\n\t.reg .pred q, r;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred r, 1, %2, q;\n\t"
            "selp.u32 %0, 1, 0, r;\n\t}\n"
            : "=r"(any) : "r"(late), "r"(32 * kFeedWarps) : "memory");
        if (any) {
          if (tid == 0) state[1] = 1;
          break;
        }
      }
      // ---- decode: a warp takes 16 consecutive rows, lane (g, t) rows g and g + 8 of them, quarter t
#pragma unroll
      for (int h = 0; h < kLaneRows; ++h) {
        const int row = 8 * kLaneRows * warp + 8 * h + g;
        if (t == 0) sts32(kNorms + 512u * slot + 4u * row, __float_as_uint(nrm[h]));
        decode_row<BW>(w[h], sel, a_hi, row, t);
        if constexpr (TERMS == 3) decode_row<BW>(w[h], sel | 0x80u, M::kALo, row, t);
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      asm volatile("bar.sync 1, %0;\n" ::"r"(32 * kFeedWarps) : "memory");
      // ---- multiply: one thread issues into accumulator buf once it has been read out ------
      if (tid == 0) {
        bool ok = true;
        if (i >= 2) ok = wait_for(kBarFree + 8u * buf, (i - 2) >> 1);
        if (ok) {
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t d = tmem + 128u * buf;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            if constexpr (TERMS == 3) {
              umma(d, operand_desc(M::kALo, ks), operand_desc(kBHi, ks), ks > 0);
              umma(d, operand_desc(M::kAHi, ks), operand_desc(M::kBLo, ks), 1u);
              umma(d, operand_desc(M::kAHi, ks), operand_desc(kBHi, ks), 1u);
            } else {
              umma(d, operand_desc(a_hi, ks), operand_desc(kBHi, ks), ks > 0);
            }
          }
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                       ::"r"(kBarDone + 8u * buf) : "memory");
        } else {
          state[1] = 1;        // nothing is issued: every later wait on done[] runs out as well
        }
      }
      if (more) {
#pragma unroll
        for (int h = 0; h < kLaneRows; ++h) {
#pragma unroll
          for (int k = 0; k < BW; ++k) w[h][k] = w_next[h][k];
          nrm[h] = nrm_next[h];
        }
      }
    }
  } else {
    int64_t tile = blockIdx.x;
    for (int i = 0; tile < tiles; tile += gridDim.x, ++i) {
      const int buf = i & 1;
      const bool ok = wait_for(kBarDone + 8u * buf, i >> 1);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) state[1] = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      store_tile(tile, buf, i % 3);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kCols) : "memory");
}

}  // namespace dq5

namespace {

__device__ int32_t g_umma_state[2];

template <int BW, int TERMS, int DT> std::atomic<int> &variant_state(int dev) {
  static std::atomic<int> state[64];
  return state[dev & 63];
}

}  // namespace

// Runs the tcgen05 kernel.  `*usable` comes back false (and nothing was
// launched for the call) when the kernel cannot be used here: the stream is
// capturing and the variant has not been set up yet, or the device places
// dynamic shared memory where the fixed addresses do not work.
template <int BW, int TERMS, int DT>
static int launch_variant(const DequantParams &p, cudaStream_t stream, bool *usable) {
  using M = dq5::Map<BW, TERMS>;
  *usable = false;
  int dev = 0;
  cudaGetDevice(&dev);
  std::atomic<int> &state = variant_state<BW, TERMS, DT>(dev);
  int32_t *flag = nullptr;
  if (cudaGetSymbolAddress((void **)&flag, g_umma_state) != cudaSuccess)
    return check_cuda(cudaGetLastError(), "wtq_dequant: tensor-memory kernel set-up");
  auto kernel = dq5::dequant_umma_kernel<BW, TERMS, DT>;
  int s = state.load(std::memory_order_acquire);
  if (s == 0) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)
      return WTQ_OK;
    static std::mutex gate;
    std::lock_guard<std::mutex> hold(gate);
    if ((s = state.load(std::memory_order_acquire)) == 0) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)M::kDynamic);
      int32_t seen[2] = {0, 0};
      if (e == cudaSuccess) e = cudaMemsetAsync(flag, 0, sizeof(seen), stream);
      if (e == cudaSuccess) {
        DequantParams none = {};
        none.L = none.MAXLEN = 1;
        kernel<<<1, dq5::kThreads, M::kDynamic, stream>>>(none, flag);
        note_launches(1);
        e = cudaGetLastError();
      }
      if (e == cudaSuccess) e = cudaMemcpyAsync(seen, flag, sizeof(seen), cudaMemcpyDeviceToHost, stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
      if (e != cudaSuccess) return check_cuda(e, "wtq_dequant: tensor-memory kernel set-up");
      s = seen[0] ? 2 : 1;
      state.store(s, std::memory_order_release);
    }
  }
  if (s != 1) return WTQ_OK;
  const int64_t tiles = (p.N + 127) / 128;
  const int grid = (int)std::min<int64_t>(tiles, device_sms());
  kernel<<<grid, dq5::kThreads, M::kDynamic, stream>>>(p, flag);
  note_launches(1);
  *usable = true;
  return check_cuda(cudaGetLastError(), "wtq_dequant tensor-memory launch");
}

template <int BW, int TERMS>
static int launch_dtype(const DequantParams &p, cudaStream_t stream, bool *usable) {
  if (p.out_dtype == WTQ_F32) return launch_variant<BW, TERMS, WTQ_F32>(p, stream, usable);
  if (p.out_dtype == WTQ_F16) return launch_variant<BW, TERMS, WTQ_F16>(p, stream, usable);
  return launch_variant<BW, TERMS, WTQ_BF16>(p, stream, usable);
}

int launch_dequant_umma(const DequantParams &p, int terms, cudaStream_t stream, bool *usable) {
  if (terms == 3) {
    if (p.bw == 4) return launch_dtype<4, 3>(p, stream, usable);
    if (p.bw == 6) return launch_dtype<6, 3>(p, stream, usable);
    return launch_dtype<8, 3>(p, stream, usable);
  }
  if (p.bw == 4) return launch_dtype<4, 1>(p, stream, usable);
  if (p.bw == 6) return launch_dtype<6, 1>(p, stream, usable);
  return launch_dtype<8, 1>(p, stream, usable);
}

// 1 if a wait for the tensor cores ran out in a tcgen05 dequantisation kernel
// since the library was loaded (synchronises the device; a diagnostic).
int dequant_umma_gave_up() {
  int32_t seen[2] = {0, 0};
  if (cudaMemcpyFromSymbol(seen, g_umma_state, sizeof(seen)) != cudaSuccess) return -1;
  return seen[1];
}

}  // namespace wtq
