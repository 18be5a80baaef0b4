// Chunked prefill straight from the packed pages: causal attention of a chunk
// of Q query tokens per sequence over that sequence's packed history, every
// page read and decoded once for all the query rows that share it.  Replaces
// the reference's prefill fallback, which dequantizes the whole history of
// each sequence to the model dtype and calls SDPA
// (turboquant_kv/packed_backend.py:192-226), and this library's own earlier
// form of it (B * Q one-token rows through the decode kernels, the history
// read Q times).
//
// Work is cut into items (sequence b, kv head, block of 256 query rows, chunk
// of the history); the query rows of a kv head are (token i, head r) pairs in
// token-major order, so the causal length never decreases along them.  A block
// of eight warps takes items from a counter.  Per item it loads its 256 rotated
// query rows as fp16 into shared memory once, then walks the chunk in tiles of
// 64 tokens:
//
//   copy     cp.async brings the tile's packed K and V rows and their fp16 norms
//            into a landing buffer, one tile ahead of the arithmetic;
//   decode   each warp turns one 16-token group of one side into fp16 centroid
//            values through the per-lane lookup tables (wtq_lut.cuh) and stores
//            them as a [token][coordinate] tile, 16-byte pieces XOR-swizzled by
//            the row so that ldmatrix reads it without bank conflicts;
//   scores   each warp owns 32 query rows: S = Q K^T with mma.m16n8k16 (A: query
//            fragments by ldmatrix, B: key tile by ldmatrix; the tile holds
//            centroid x norm), causal mask where the tile reaches a row's limit;
//   softmax  online, in the exp2 domain, on the score fragments in registers;
//   values   O += P V (V tile = centroid x norm), the probability fragments
//            feeding the MMA as A operands directly, V by ldmatrix.trans.
//
// fp16 scores are exact enough while they are small; a warp whose tile holds a
// score beyond 8 (log2 domain) recomputes that tile's scores in fp32 from the
// packed codes.  At the end of the chunk every row that sees the chunk writes
// its state (reference maximum, sum, un-normalised accumulator in the value
// basis) in the layout of the decode scan, and the decode path's merge kernels
// combine the chunks, rotate back and store.
#include <algorithm>
#include <atomic>

#include "wtq_decode.cuh"
#include "wtq_lut.cuh"

namespace wtq {
namespace pf {

constexpr int kWarps = 8, kThreads = 32 * kWarps;
constexpr int kRows = 32 * kWarps;              // query rows per item
constexpr int kTile = 64;                       // tokens per tile
constexpr uint32_t kBase = 1024;                // dynamic shared memory is assumed to start at or below this
constexpr uint32_t kKTile = kBase;              // [64][128] fp16
constexpr uint32_t kVTile = kKTile + kTile * 256;
constexpr uint32_t kNormK = kVTile + kTile * 256;   // 64 floats each
constexpr uint32_t kNormV = kNormK + kTile * 4;
constexpr uint32_t kItem = kNormV + kTile * 4;      // the item being worked on (8 words)
constexpr uint32_t kWalk = kItem + 32;              // balanced schedule: where this block stands (10 words)
constexpr uint32_t kPlan = kWalk + 64;              // balanced schedule: tiles of every (sequence, row block)
constexpr int kMaxPairs = 4096;                     // (sequence, row block) pairs the plan has room for
constexpr int kBalancedSlots = 3;                   // a group is cut by at most two block boundaries
static_assert(kPlan + 4 * kMaxPairs <= mma::kLutAddr, "tiles and the plan must end below the lookup tables");
constexpr float kPreciseAbove = 8.f;            // |score| (log2 domain) beyond which fp16 is not trusted

struct Params {
  DecodeSideDev k, v;
  const float *q_rot;        // (B * Q, Hq, 128) fp32, times scale * log2(e)
  const int32_t *page_table;
  int64_t table_stride;
  const int32_t *seq_lens;   // (B)
  int32_t *row_lens;         // (B * Q) causal lengths, written here for the merge
  int B, Hq, Hkv, n_rep, Q, S, P, max_pages, max_tokens;
  int num_splits, chunk_tokens, row_blocks;
  int balanced;              // 1: tiles dealt evenly to the blocks (chunk_tokens unused), 0: equal chunks
  float *part_acc, *part_m, *part_l;
  int32_t *status, *work_counter;
  const uint32_t *lut;
};

template <int BWK, int BWV> struct Map {
  static constexpr int kNBK = 16 * BWK, kNBV = 16 * BWV;
  static constexpr uint32_t kLutBytes =
      (uint32_t)(mma::lut_entries(BWK) > mma::lut_entries(BWV) ? mma::lut_entries(BWK)
                                                                : mma::lut_entries(BWV)) * 256u;
  static constexpr uint32_t kQTile = mma::kLutAddr + kLutBytes;        // [256][128] fp16
  static constexpr uint32_t kRaw = kQTile + kRows * 256;
  // landing buffer of one tile: K rows, V rows, K norms, V norms
  static constexpr uint32_t kRawV = kTile * kNBK;
  static constexpr uint32_t kRawNK = kRawV + kTile * kNBV;
  static constexpr uint32_t kRawNV = kRawNK + kTile * 2;
  static constexpr uint32_t kRawBytes = kRawNV + kTile * 2;
  static constexpr uint32_t kDynamic = kRaw + 2 * kRawBytes;
  static_assert(kDynamic <= 227u * 1024u, "shared memory budget");
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t a, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t a, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void sts64u(uint32_t a, uint32_t x, uint32_t y) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ float2 lds_f2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
// 16 bytes global -> shared; `bytes` = 16, or 0 to fill the piece with zeros
__device__ __forceinline__ void copy16(uint32_t dst, const void *src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes)
               : "memory");
}

// Address of 16-byte piece `piece` (0..15) of row `row` in a [rows][128] fp16 tile.
__device__ __forceinline__ uint32_t tile_at(uint32_t tile, int row, int piece) {
  return tile + (uint32_t)row * 256u + (uint32_t)((piece ^ (row & 7)) << 4);
}

// Eight consecutive centroid values (fp16) of a lane's share of a packed row:
// codes 8 J .. 8 J + 7 of the 32 the words hold.
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

// One warp decodes tokens 16 u .. 16 u + 15 of one side: the lane (g, t) takes
// rows g and g + 8 and coordinates 32 t .. 32 t + 31 of each.
// The values stored are centroid x row norm, rounded to fp16 (`norms` = address of the
// tile's fp16 norms; rows from `valid` on get norm 0): the scores and the value sums then
// need no per-token scaling.
template <int BW>
__device__ __forceinline__ void decode_group(uint32_t raw, uint32_t norms, int valid, uint32_t tile,
                                             uint32_t sel, int u, int g, int t) {
  constexpr int NB = 16 * BW;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = 16 * u + g + 8 * h;
    uint32_t w[BW];
    load_words<4 * BW>(raw + (uint32_t)row * NB + (uint32_t)t * (4 * BW), w);
    unsigned short nh;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(nh) : "r"(norms + 2u * row));
    if (row >= valid) nh = 0;
    const __half2 n2 = __half2half2(__ushort_as_half(nh));
    auto scaled = [&](uint32_t x) {
      const __half2 y = __hmul2(*reinterpret_cast<const __half2 *>(&x), n2);
      return *reinterpret_cast<const uint32_t *>(&y);
    };
    uint32_t f[4];
    decode_piece<BW, 0>(w, sel, f);
    sts128(tile_at(tile, row, 4 * t + 0), scaled(f[0]), scaled(f[1]), scaled(f[2]), scaled(f[3]));
    decode_piece<BW, 1>(w, sel, f);
    sts128(tile_at(tile, row, 4 * t + 1), scaled(f[0]), scaled(f[1]), scaled(f[2]), scaled(f[3]));
    decode_piece<BW, 2>(w, sel, f);
    sts128(tile_at(tile, row, 4 * t + 2), scaled(f[0]), scaled(f[1]), scaled(f[2]), scaled(f[3]));
    decode_piece<BW, 3>(w, sel, f);
    sts128(tile_at(tile, row, 4 * t + 3), scaled(f[0]), scaled(f[1]), scaled(f[2]), scaled(f[3]));
  }
}

// fp32 dot products of one token's key centroids (row `at` of the landing
// buffer) with four rotated query rows (null: the row does not exist), without
// the key norm.  Out of line and returning its result in registers: it runs only
// for tiles whose fp16 scores came out large and must cost the common path
// neither registers nor stack.
template <int BW>
__device__ __noinline__ float4 precise_token(uint32_t at, const float *q0, const float *q1,
                                             const float *q2, const float *q3,
                                             const float *centroids) {
  float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int d = 0; d < 128; ++d) {
    const int bit = d * BW, b0 = bit >> 3, sh = bit & 7;
    uint32_t x = lds_u8(at + b0);
    if (sh + BW > 8) x |= lds_u8(at + b0 + 1) << 8;
    const float cv = __ldg(centroids + ((x >> sh) & ((1u << BW) - 1u)));
    r.x = fmaf(q0 ? __ldg(q0 + d) : 0.f, cv, r.x);
    r.y = fmaf(q1 ? __ldg(q1 + d) : 0.f, cv, r.y);
    r.z = fmaf(q2 ? __ldg(q2 + d) : 0.f, cv, r.z);
    r.w = fmaf(q3 ? __ldg(q3 + d) : 0.f, cv, r.w);
  }
  return r;
}

template <int BWK, int BWV>
__global__ void __launch_bounds__(kThreads, 1) prefill_kernel(Params p) {
  using M = Map<BWK, BWV>;
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  if ((uint32_t)__cvta_generic_to_shared(dyn_smem) > kBase) {   // layout assumption broken
    if (p.status && tid == 0) atomicOr(p.status, WTQ_STATUS_LAYOUT);
    return;
  }
  constexpr uint32_t kFull = 0xffffffffu;
  // causal length of every query row, for the merge
  for (int i = blockIdx.x * kThreads + tid; i < p.B * p.Q; i += gridDim.x * kThreads) {
    int L = p.seq_lens[i / p.Q];
    L = L < 0 ? 0 : (L > p.max_tokens ? p.max_tokens : L);
    const int len = L - p.Q + 1 + i % p.Q;
    p.row_lens[i] = len < 0 ? 0 : len;
  }
  // lookup tables (built by the rotation launch)
  for (int i = tid; i < (int)(M::kLutBytes / 16); i += kThreads) {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p.lut) + i);
    sts128(mma::kLutAddr + 16u * i, v.x, v.y, v.z, v.w);
  }
  const uint32_t sel_k = mma::kLutAddr | (uint32_t)(lane << 2), sel_v = sel_k | 0x80u;
  // ldmatrix row addresses of this lane.  A piece index is 2 * step + (0 or 1) and
  // the swizzle XORs it with the row's low bits, so the step enters as one XOR of
  // step << 5 with these bases; steps over rows of 16 leave the low bits alone.
  const uint32_t q_at = tile_at(M::kQTile, 32 * warp + (lane & 7) + 8 * ((lane >> 3) & 1), lane >> 4);
  const uint32_t k_at = tile_at(kKTile, (lane & 7) + 8 * (lane >> 4), (lane >> 3) & 1);
  const uint32_t v_at = tile_at(kVTile, (lane & 7) + 8 * ((lane >> 3) & 1), lane >> 4);
  const int R = p.Q * p.n_rep;                              // query rows per (sequence, kv head)
  const int items = p.B * p.Hkv * p.row_blocks * p.num_splits;
  const int page_shift = 31 - __clz(p.S);

  // ---- balanced schedule ---------------------------------------------------------------
  // The 64-token tiles of all groups, laid end to end (sequence, row block, kv head), are
  // cut into one equal run per block, so every multiprocessor gets the same number of
  // tiles whatever the number of groups.  A run is at least half the longest group, hence a
  // group is cut at most twice and its pieces take chunk slots 0..2; the slot of a piece is
  // its block's distance from the block that holds the group's first tile.
  if (p.balanced) {
    const int pairs = p.B * p.row_blocks;
    for (int i = tid; i < pairs; i += kThreads) {
      const int b = i / p.row_blocks, rb = i - b * p.row_blocks;
      int L = p.seq_lens[b];
      L = L < 0 ? 0 : (L > p.max_tokens ? p.max_tokens : L);
      const int last = min(R, (rb + 1) * kRows) - 1;          // last row of the block
      const int len = L - p.Q + 1 + last / p.n_rep;
      sts32(kPlan + 4u * i, len > 0 ? (uint32_t)((len + kTile - 1) / kTile) : 0u);
    }
    __syncthreads();
    if (warp == 0) {
      long long total = 0;
      int longest = 0;
      for (int i = lane; i < pairs; i += 32) {
        const int n = (int)lds32(kPlan + 4u * i);
        total += n;
        longest = max(longest, n);
      }
#pragma unroll
      for (int d = 16; d; d >>= 1) {
        total += __shfl_xor_sync(kFull, total, d);
        longest = max(longest, __shfl_xor_sync(kFull, longest, d));
      }
      if (lane == 0) {
        total *= p.Hkv;
        long long share = (total + gridDim.x - 1) / gridDim.x;
        share = max(share, (long long)((longest + 1) / 2));
        share = max(share, 1LL);
        const long long lo = min(total, share * blockIdx.x), hi = min(total, lo + share);
        sts32(kWalk + 0, 0u);                                             // pair the walk stands in
        sts32(kWalk + 4, 0u); sts32(kWalk + 8, 0u);                       // tiles before that pair
        sts32(kWalk + 12, (uint32_t)lo); sts32(kWalk + 16, (uint32_t)(lo >> 32));   // next tile
        sts32(kWalk + 20, (uint32_t)hi); sts32(kWalk + 24, (uint32_t)(hi >> 32));   // end of the run
        sts32(kWalk + 28, (uint32_t)share); sts32(kWalk + 32, (uint32_t)(share >> 32));
      }
    }
  }
  auto walk64 = [&](uint32_t at) -> long long {
    return (long long)(((unsigned long long)lds32(at + 4) << 32) | lds32(at));
  };

  for (;;) {
    __syncthreads();                                        // everyone is done with the previous item
    if (tid == 0) {
      if (!p.balanced) {
        sts32(kItem, (uint32_t)atomicAdd(p.work_counter, 1));
      } else {
        int i = (int)lds32(kWalk);
        long long pre = walk64(kWalk + 4), x = walk64(kWalk + 12);
        const long long hi = walk64(kWalk + 20), share = walk64(kWalk + 28);
        if (x >= hi) {
          sts32(kItem, 0xffffffffu);
        } else {
          int n = (int)lds32(kPlan + 4u * i);
          // ends before the last pair: x < hi <= all tiles (the bound on i only guards the plan)
          while (x >= pre + (long long)p.Hkv * n && i + 1 < p.B * p.row_blocks) {
            pre += (long long)p.Hkv * n;
            n = (int)lds32(kPlan + 4u * ++i);
          }
          const long long rel = x - pre;
          const int kvh = n > 0 ? (int)(rel / n) : p.Hkv, off = (int)(rel - (long long)kvh * n);
          const int take = (int)min(hi - x, (long long)(n - off));
          const long long slot = (long long)blockIdx.x - (pre + (long long)kvh * n) / share;
          if (slot < 0 || slot >= p.num_splits || kvh >= p.Hkv || take < 1) {   // cannot happen; never
            x = hi - take;                                                      // write outside the states
            if (p.status) atomicOr(p.status, WTQ_STATUS_LAYOUT);
            sts32(kItem, 0xffffffffu);
          } else {
            sts32(kItem, (uint32_t)i);
            sts32(kItem + 4, (uint32_t)kvh);
            sts32(kItem + 8, (uint32_t)off);
            sts32(kItem + 12, (uint32_t)(off + take));
            sts32(kItem + 16, (uint32_t)slot);
          }
          x += take;
          sts32(kWalk, (uint32_t)i);
          sts32(kWalk + 4, (uint32_t)pre); sts32(kWalk + 8, (uint32_t)(pre >> 32));
          sts32(kWalk + 12, (uint32_t)x); sts32(kWalk + 16, (uint32_t)(x >> 32));
        }
      }
    }
    __syncthreads();
    const int item = (int)lds32(kItem);
    int chunk, rb, kvh, b, start, cap;                       // cap: end of the item's token range
    if (!p.balanced) {
      if (item >= items) break;
      // chunks vary fastest, so blocks working at the same time share the query rows in L2
      chunk = item % p.num_splits;
      rb = (item / p.num_splits) % p.row_blocks;
      kvh = (item / (p.num_splits * p.row_blocks)) % p.Hkv;
      b = item / (p.num_splits * p.row_blocks * p.Hkv);
      start = chunk * p.chunk_tokens;
      cap = start + p.chunk_tokens;
    } else {
      if (item < 0) break;
      b = item / p.row_blocks;
      rb = item - b * p.row_blocks;
      kvh = (int)lds32(kItem + 4);
      start = (int)lds32(kItem + 8) * kTile;
      cap = (int)lds32(kItem + 12) * kTile;
      chunk = (int)lds32(kItem + 16);
    }
    int L = p.seq_lens[b];
    L = L < 0 ? 0 : (L > p.max_tokens ? p.max_tokens : L);
    const int row_lo = rb * kRows;
    const int row_hi = min(R, row_lo + kRows);             // rows [row_lo, row_hi) exist
    auto length_of = [&](int row) {                         // causal length of a row of this group
      const int len = L - p.Q + 1 + row / p.n_rep;
      return len < 0 ? 0 : len;
    };
    const int len_last = length_of(row_hi - 1);
    if (row_lo >= R || start >= len_last) continue;         // no row of the block sees this chunk
    const int end = min(cap, len_last);
    const int ntiles = (end - start + kTile - 1) / kTile;

    // ---- this lane's four rows ------------------------------------------------
    const int wrow0 = row_lo + 32 * warp;
    int limit[2][2];                                        // first token a row does NOT see, within the chunk
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = wrow0 + 16 * m + 8 * h + g;
        limit[m][h] = min(row < row_hi ? length_of(row) : 0, cap);
      }
    // index of a row's rotated query (and, times num_splits, of its chunk states); -1: no such row
    auto query_row = [&](int m, int h) -> int64_t {
      const int row = wrow0 + 16 * m + 8 * h + g;
      if (row >= row_hi) return -1;
      const int i = row / p.n_rep, r = row - i * p.n_rep;
      return ((int64_t)b * p.Q + i) * p.Hq + kvh * p.n_rep + r;
    };
    // rows are in causal order: the warp's first and last existing rows bound its limits
    const int warp_hi = wrow0 < row_hi ? min(length_of(min(wrow0 + 31, row_hi - 1)), cap) : 0;
    const int warp_lo = wrow0 < row_hi ? min(length_of(wrow0), cap) : 0;
    const bool warp_on = warp_hi > start;

    // ---- copy of one tile into a landing buffer ----------------------------------
    // Done in two steps so that the page-table reads are not in front of the
    // copies: `lookup(j)` fetches the page id of each of this thread's pieces of
    // tile j into registers (at the top of tile j - 1's turn), `copy(j)` issues
    // the copies after that tile has been decoded.
    const int32_t *table = p.page_table + (int64_t)b * p.table_stride;
    constexpr int kPiecesK = kTile * M::kNBK / 16, kPiecesV = kTile * M::kNBV / 16;
    constexpr int kPieces = kPiecesK + kPiecesV + 16;       // + 8 + 8 pieces of norms
    constexpr int kTurns = (kPieces + kThreads - 1) / kThreads;
    // piece c: side 0/1 = K/V codes, 2/3 = K/V norms; first token; byte offset in the row
    auto piece = [&](int c, int &side, int &tok, int &off, uint32_t &dst) {
      if (c < kPiecesK) {
        side = 0; tok = c / (M::kNBK / 16); off = (c - tok * (M::kNBK / 16)) * 16; dst = 16u * c;
      } else if (c < kPiecesK + kPiecesV) {
        const int cc = c - kPiecesK;
        side = 1; tok = cc / (M::kNBV / 16); off = (cc - tok * (M::kNBV / 16)) * 16;
        dst = M::kRawV + 16u * cc;
      } else {
        const int cc = c - kPiecesK - kPiecesV;              // eight tokens of norms per piece
        side = 2 + (cc >> 3); tok = (cc & 7) * 8; off = 0;
        dst = (side == 2 ? M::kRawNK : M::kRawNV) + 16u * (cc & 7);
      }
    };
    int page_of[kTurns];                                     // -2: the piece lies past the end
    auto lookup = [&](int j) {
#pragma unroll
      for (int i = 0; i < kTurns; ++i) {
        const int c = tid + i * kThreads;
        int side, tok, off;
        uint32_t dst;
        piece(c < kPieces ? c : 0, side, tok, off, dst);
        const int token = start + j * kTile + tok;
        page_of[i] = c < kPieces && token < end ? table[token >> page_shift] : -2;
      }
    };
    auto copy = [&](int j) {
      const uint32_t raw = M::kRaw + (uint32_t)(j & 1) * M::kRawBytes;
#pragma unroll
      for (int i = 0; i < kTurns; ++i) {
        const int c = tid + i * kThreads;
        if (c >= kPieces) break;
        int side, tok, off;
        uint32_t dst;
        piece(c, side, tok, off, dst);
        const int page = page_of[i], pos = (start + j * kTile + tok) & (p.S - 1);
        int bytes = 16;
        const void *src = p.k.pages;                         // any valid address when nothing is read
        if (page < 0 || page >= p.P) {
          if (page != -2 && p.status) atomicOr(p.status, WTQ_STATUS_BAD_PAGE);
          bytes = 0;
        } else if (side < 2) {
          const DecodeSideDev &sd = side ? p.v : p.k;
          src = sd.pages + (int64_t)page * sd.page_stride + (int64_t)kvh * sd.head_stride +
                (int64_t)pos * sd.nb + off;
        } else {
          const DecodeSideDev &sd = side == 3 ? p.v : p.k;
          src = sd.norms + (int64_t)page * sd.norm_page_stride + (int64_t)kvh * sd.norm_head_stride + pos;
        }
        copy16(raw + dst, src, bytes);
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    lookup(0);
    copy(0);
    if (ntiles > 1) lookup(1);

    // ---- query rows -> fp16 tile (behind the first copy, eight loads in flight per thread) ----
    for (int e0 = tid; e0 < kRows * 32; e0 += 8 * kThreads) {  // 32 float4 per row
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int e = e0 + u * kThreads, lr = e >> 5, c4 = e & 31, row = row_lo + lr;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < row_hi) {
          const int i = row / p.n_rep, r = row - i * p.n_rep;
          const int64_t qrow = ((int64_t)b * p.Q + i) * p.Hq + kvh * p.n_rep + r;
          v[u] = __ldg(reinterpret_cast<const float4 *>(p.q_rot + qrow * 128) + c4);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int e = e0 + u * kThreads, lr = e >> 5, c4 = e & 31;
        sts64u(tile_at(M::kQTile, lr, c4 >> 1) + (uint32_t)(c4 & 1) * 8u, pack_half2(v[u].x, v[u].y),
               pack_half2(v[u].z, v[u].w));
      }
    }

    float o[2][16][4];                                      // rows x coordinates of the value basis
    float mx[2][2], sum[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
      for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[m][n][e] = 0.f;
      mx[m][0] = mx[m][1] = -INFINITY;
      sum[m][0] = sum[m][1] = 0.f;
    }

    for (int j = 0; j < ntiles; ++j) {
      const uint32_t raw = M::kRaw + (uint32_t)(j & 1) * M::kRawBytes;
      const int tok0 = start + j * kTile;
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      __syncthreads();       // the tile has landed for everyone; everyone is done with the previous tiles
      // ---- decode: warps 0..3 the four key groups, warps 4..7 the value groups ------
      // (norms are copied eight tokens at a time: those of tokens past the end of
      // the tile's range are whatever the page holds and become 0 here)
      if (warp < 4) {
        decode_group<BWK>(raw, raw + M::kRawNK, end - tok0, kKTile, sel_k, warp, g, t);
        if (lane < 16) {                                     // fp32 norms, for the fp32 re-scoring only
          const int tk = 16 * warp + lane;
          const float v = tok0 + tk < end ? lds_half(raw + M::kRawNK + 2u * tk) : 0.f;
          sts32(kNormK + 4u * tk, __float_as_uint(v));
        }
      } else {
        decode_group<BWV>(raw + M::kRawV, raw + M::kRawNV, end - tok0, kVTile, sel_v, warp - 4, g, t);
      }
      __syncthreads();
      if (j + 1 < ntiles) copy(j + 1);
      if (j + 2 < ntiles) lookup(j + 2);                    // ids for the tile after: a whole tile ahead
      if (!warp_on || tok0 >= warp_hi) continue;            // no row of this warp sees the tile

      // ---- scores -------------------------------------------------------------------
      float s[2][8][4];
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[m][n][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[2][4];
#pragma unroll
        for (int m = 0; m < 2; ++m) ldmatrix_x4((q_at + m * 16 * 256) ^ (uint32_t)(ks << 5), a[m]);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t kb[4];
          ldmatrix_x4((k_at + np * 16 * 256) ^ (uint32_t)(ks << 5), kb);
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            mma16816_free(s[m][2 * np], a[m][0], a[m][1], a[m][2], a[m][3], kb[0], kb[1]);
            mma16816_free(s[m][2 * np + 1], a[m][0], a[m][1], a[m][2], a[m][3], kb[2], kb[3]);
          }
        }
      }
      const bool masked = tok0 + kTile > warp_lo;            // some row of the warp stops inside the tile
      if (masked) {
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (tok0 + 8 * n + 2 * t + (e & 1) >= limit[m][e >> 1]) s[m][n][e] = -INFINITY;
      }
      float ref[2][2];                                       // maxima of the tile's rows
      auto row_maxima = [&]() {
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n) v = max3(v, s[m][n][2 * h], s[m][n][2 * h + 1]);
            v = fmaxf(v, __shfl_xor_sync(kFull, v, 1));
            ref[m][h] = fmaxf(v, __shfl_xor_sync(kFull, v, 2));
          }
      };
      row_maxima();
      // The fp16 error of a score grows with its size, and only scores near their
      // row's maximum carry weight: a tile is re-scored in fp32 when a row maximum
      // lies beyond +-8 (or is not a number).
      bool large = false;
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) large |= !(fabsf(ref[m][h]) <= kPreciseAbove) && ref[m][h] != -INFINITY;
      if (__any_sync(kFull, large)) {
        const float *qp[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int64_t qr = query_row(i >> 1, i & 1);
          qp[i] = qr < 0 ? nullptr : p.q_rot + qr * 128;
        }
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int tk = 8 * n + 2 * t + c;
            const float4 r = precise_token<BWK>(raw + (uint32_t)tk * M::kNBK, qp[0], qp[1], qp[2], qp[3],
                                                p.k.centroids);
            const float nk_tk = __uint_as_float(lds32(kNormK + 4u * tk));
            const float x[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
              for (int h = 0; h < 2; ++h)
                s[m][n][2 * h + c] = masked && tok0 + tk >= limit[m][h] ? -INFINITY
                                                                        : x[2 * m + h] * nk_tk;
          }
        row_maxima();
      }

      // ---- online softmax -------------------------------------------------------------
      bool grew = false;
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) grew |= ref[m][h] > mx[m][h];
      if (__any_sync(kFull, grew)) {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          float scale[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float now = fmaxf(mx[m][h], ref[m][h]);
            scale[h] = now == -INFINITY ? 1.f : ex2(mx[m][h] - now);   // ex2(-inf) = 0 on the first tile
            mx[m][h] = now;
            sum[m][h] *= scale[h];
          }
#pragma unroll
          for (int n = 0; n < 16; ++n) {
            o[m][n][0] *= scale[0]; o[m][n][1] *= scale[0];
            o[m][n][2] *= scale[1]; o[m][n][3] *= scale[1];
          }
        }
      }
      uint32_t pa[2][8][2];                                  // P * value norm as fp16 pairs
      float base[2][2];
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) base[m][h] = mx[m][h] == -INFINITY ? 0.f : mx[m][h];
      auto probabilities = [&](int n) {                      // of tokens 8 n .. 8 n + 7
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const float p0 = ex2(s[m][n][0] - base[m][0]), p1 = ex2(s[m][n][1] - base[m][0]);
          const float p2 = ex2(s[m][n][2] - base[m][1]), p3 = ex2(s[m][n][3] - base[m][1]);
          sum[m][0] += p0 + p1;
          sum[m][1] += p2 + p3;
          pa[m][n][0] = pack_half2(p0, p1);
          pa[m][n][1] = pack_half2(p2, p3);
        }
      };

      // ---- values: in source order the probabilities of the next 16 tokens sit
      // between the MMAs of the current 16 (the compiler is free to schedule the
      // exponentials under the tensor pipe's work; measured, it made no difference)
      probabilities(0);
      probabilities(1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          uint32_t vb[4];
          ldmatrix_x4_trans((v_at + kk * 16 * 256) ^ (uint32_t)(dp << 5), vb);
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            mma16816_free(o[m][2 * dp], pa[m][2 * kk][0], pa[m][2 * kk][1], pa[m][2 * kk + 1][0],
                     pa[m][2 * kk + 1][1], vb[0], vb[1]);
            mma16816_free(o[m][2 * dp + 1], pa[m][2 * kk][0], pa[m][2 * kk][1], pa[m][2 * kk + 1][0],
                     pa[m][2 * kk + 1][1], vb[2], vb[3]);
          }
          if (kk < 3 && dp == 1) probabilities(2 * kk + 2);
          if (kk < 3 && dp == 5) probabilities(2 * kk + 3);
        }
      }
    }

    // ---- chunk states ---------------------------------------------------------------------
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float l = sum[m][h];
        l += __shfl_xor_sync(kFull, l, 1);
        l += __shfl_xor_sync(kFull, l, 2);
        const int64_t qr = query_row(m, h);
        if (qr < 0 || limit[m][h] <= start) continue;          // the row does not exist or sees none of the chunk
        const int64_t state = qr * p.num_splits + chunk;
        float2 *dst = reinterpret_cast<float2 *>(p.part_acc + state * 128 + 2 * t);
#pragma unroll
        for (int n = 0; n < 16; ++n) dst[4 * n] = make_float2(o[m][n][2 * h], o[m][n][2 * h + 1]);
        if (t == 0) {
          p.part_m[state] = mx[m][h];
          p.part_l[state] = l;
        }
      }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

template <int BWK, int BWV>
int launch(const Params &p, cudaStream_t stream) {
  using M = Map<BWK, BWV>;
  static std::atomic<bool> opted_in_dev[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !opted_in_dev[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel<BWK, BWV>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)M::kDynamic);
    if (e != cudaSuccess) return check_cuda(e, "wtq_prefill: shared memory opt-in");
    opted_in_dev[dev & 63].store(true, std::memory_order_release);
  }
  const int64_t items = (int64_t)p.B * p.Hkv * p.row_blocks * p.num_splits;
  const int grid = p.balanced ? device_sms() : (int)std::min<int64_t>(items, device_sms());
  prefill_kernel<BWK, BWV><<<grid, kThreads, M::kDynamic, stream>>>(p);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_prefill launch");
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Tokens per chunk: a multiple of the tile, at least 256.
int chunk_tokens_for(int max_tokens, int splits) {
  int tokens = (max_tokens + splits - 1) / splits;
  tokens = (tokens + kTile - 1) / kTile * kTile;
  return tokens < 256 ? 256 : tokens;
}

// Shapes the balanced schedule serves: enough query rows for the tensor-core merge, at
// least half as many groups as multiprocessors (a run is never shorter than half a
// group, so fewer groups would leave blocks idle), and a plan that fits.
bool balanced_shape(int B, int Hq, int Hkv, int Q) {
  const int row_blocks = (Q * (Hq / Hkv) + kRows - 1) / kRows;
  const int64_t groups = (int64_t)B * Hkv * row_blocks;
  return (int64_t)B * Q * Hq >= 4096 && 2 * groups >= device_sms() &&
         (int64_t)B * row_blocks <= kMaxPairs;
}

// Equal chunks: items = groups x chunks run in waves of one per multiprocessor; every chunk
// beyond the first adds about 5 % (states to write and merge, queries to reload).  Both
// effects were measured at 16 x 8 kv heads x 8k tokens: 64 query tokens (128 groups) 690 /
// 726 / 769 us with 1 / 2 / 3 chunks, 256 query tokens (512 groups) 2549 / 2388 / 2633 us.
// Takes the count with the lowest modelled cost; chunks of at least 256 tokens.
int equal_chunks(int B, int Hq, int Hkv, int Q, int64_t max_tokens) {
  const int row_blocks = (Q * (Hq / Hkv) + kRows - 1) / kRows;
  const int64_t groups = (int64_t)B * Hkv * row_blocks;
  const int64_t sms = device_sms();
  const int64_t most = std::max<int64_t>(1, std::min<int64_t>(max_tokens / 256, 32));
  int64_t splits = 1;
  double best = 0.0;
  for (int64_t s = 1; s <= most; ++s) {
    const int64_t items = groups * s, waves = (items + sms - 1) / sms;
    const double cost = (1.0 + 0.05 * (double)(s - 1)) * (double)(waves * sms) / (double)items;
    if (s == 1 || cost < best - 1e-9) {
      best = cost;
      splits = s;
    }
  }
  // chunk sizes round up to whole tiles: drop chunks that would stay empty
  const int tokens = chunk_tokens_for((int)max_tokens, (int)splits);
  return (int)((max_tokens + tokens - 1) / tokens);
}

}  // namespace pf
}  // namespace wtq

using namespace wtq;

extern "C" int wtq_prefill_auto_splits(int B, int Hq, int Hkv, int Q, int max_pages, int S) {
  if (B < 1 || Hq < 1 || Hkv < 1 || Q < 1 || max_pages < 1 || S < 1 || Hq % Hkv) return 1;
  if (pf::balanced_shape(B, Hq, Hkv, Q)) return pf::kBalancedSlots;
  return pf::equal_chunks(B, Hq, Hkv, Q, (int64_t)max_pages * S);
}

static thread_local int g_last_schedule = -1;
extern "C" int wtq_prefill_last_schedule(void) { return g_last_schedule; }

extern "C" size_t wtq_prefill_workspace_bytes(int B, int Hq, int Hkv, int Q, int D, int num_splits) {
  if (B < 1 || Hq < 1 || Hkv < 1 || Q < 1 || D < 1 || num_splits < 1) return 0;
  const size_t rows = (size_t)B * Q * Hq;
  return 256 + pf::round_up((size_t)B * Q * sizeof(int32_t), 256) +
         pf::round_up(rows * D * sizeof(float), 256) +
         pf::round_up(rows * num_splits * D * sizeof(float), 256) +
         2 * pf::round_up(rows * num_splits * sizeof(float), 256) + 256 * 256;
}

extern "C" int wtq_prefill(const void *q, int dtype, const int64_t q_strides[2], void *out,
                           const int64_t out_strides[2], const wtq_side_t *k_side,
                           const wtq_side_t *v_side, const int32_t *page_table,
                           int64_t table_stride, const int32_t *seq_lens, float scale, int B, int Hq,
                           int Hkv, int Q, int D, int S, int P, int max_pages, int num_splits,
                           void *workspace, size_t workspace_bytes, int32_t *status, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (Q < 1) return fail(WTQ_ERR_ARG, "wtq_prefill: need Q >= 1");
  if (B > 0 && (int64_t)B * Q > (int64_t)1 << 24)
    return fail(WTQ_ERR_ARG, "wtq_prefill: B * Q is limited to 2^24 query tokens");
  // the rows of the call are the B * Q query tokens; everything the decode entry
  // checks about buffers, strides and shapes holds for them as for B sequences
  if (int rc = decode_validate(q, dtype, q_strides, out, out_strides, false, k_side, v_side,
                               page_table, seq_lens, B * Q, Hq, Hkv, D, S, P, max_pages))
    return rc;
  if (B == 0) return WTQ_OK;
  if (!workspace) return fail(WTQ_ERR_ARG, "wtq_prefill: null workspace");
  const int max_tokens = max_pages * S;
  const int64_t total_rows = (int64_t)B * Q * Hq;
  // Schedule.  An explicit num_splits cuts every history into that many equal chunks.
  // Left to the library (num_splits <= 0), shapes with enough groups and rows take the
  // balanced schedule (tiles dealt evenly to the blocks, three chunk slots per row) when
  // the output layout lets the tensor-core merge run; everything else takes equal chunks,
  // never more than wtq_prefill_auto_splits promised the caller's workspace.
  bool balanced = false;
  int splits = num_splits;
  if (num_splits <= 0) {
    splits = pf::equal_chunks(B, Hq, Hkv, Q, max_tokens);
    if (Hq % Hkv == 0 && pf::balanced_shape(B, Hq, Hkv, Q)) {
      MergeParams fit = {};
      fit.D = D; fit.Hq = Hq; fit.num_splits = pf::kBalancedSlots; fit.out = out;
      fit.osb = out_strides[0]; fit.osh = out_strides[1]; fit.Pi_v = v_side->Pi;
      fit.part_acc = (float *)workspace;                 // states start at a multiple of 256 bytes from here
      balanced = rows_mma_merge_eligible(fit, total_rows);
      splits = std::min(splits, pf::kBalancedSlots);
    }
  }
  splits = std::min(splits, std::max(1, max_tokens / pf::kTile));
  splits = std::min(splits, 256);
  const int chunk_tokens = pf::chunk_tokens_for(max_tokens, splits);
  splits = balanced ? pf::kBalancedSlots : (max_tokens + chunk_tokens - 1) / chunk_tokens;
  const size_t need = wtq_prefill_workspace_bytes(B, Hq, Hkv, Q, D, splits);
  if (workspace_bytes < need)
    return fail(WTQ_ERR_WORKSPACE, "wtq_prefill: workspace %zu < %zu bytes", workspace_bytes, need);

  pf::Params p;
  auto fill = [&](DecodeSideDev &d, const wtq_side_t &s) {
    d.pages = (const uint8_t *)s.pages; d.norms = (const __half *)s.norms;
    d.page_stride = s.page_stride; d.head_stride = s.head_stride;
    d.norm_page_stride = s.norm_page_stride; d.norm_head_stride = s.norm_head_stride;
    d.Pi = s.Pi; d.centroids = s.centroids; d.bw = s.bw; d.nb = D * s.bw / 8;
  };
  fill(p.k, *k_side);
  fill(p.v, *v_side);
  const size_t rows = (size_t)B * Q * Hq;
  char *ws = (char *)workspace;
  p.work_counter = (int32_t *)ws;
  ws += 256;
  p.row_lens = (int32_t *)ws;
  ws += pf::round_up((size_t)B * Q * sizeof(int32_t), 256);
  float *q_rot = (float *)ws;
  ws += pf::round_up(rows * D * sizeof(float), 256);
  p.part_acc = (float *)ws;
  ws += pf::round_up(rows * splits * D * sizeof(float), 256);
  p.part_m = (float *)ws;
  ws += pf::round_up(rows * splits * sizeof(float), 256);
  p.part_l = (float *)ws;
  ws += pf::round_up(rows * splits * sizeof(float), 256);
  p.lut = (const uint32_t *)ws;
  p.q_rot = q_rot;
  p.page_table = page_table; p.table_stride = table_stride; p.seq_lens = seq_lens;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.n_rep = Hq / Hkv; p.Q = Q; p.S = S; p.P = P;
  p.max_pages = max_pages; p.max_tokens = max_tokens; p.num_splits = splits;
  p.chunk_tokens = chunk_tokens;
  p.balanced = balanced ? 1 : 0;
  g_last_schedule = p.balanced;
  p.row_blocks = (Q * p.n_rep + pf::kRows - 1) / pf::kRows;
  p.status = status;
  if ((int64_t)B * Hkv * p.row_blocks * splits > (int64_t)1 << 30)
    return fail(WTQ_ERR_ARG, "wtq_prefill: too many work items; lower num_splits");

  // what the tensor-core kernels need of the layout (the same as the decode scan)
  DecodeParams probe = {};
  probe.k = p.k; probe.v = p.v; probe.D = D; probe.S = S; probe.n_rep = p.n_rep;
  probe.q_rot = q_rot; probe.part_acc = p.part_acc; probe.lut = p.lut;
  if (!mma_eligible(probe) || D != 128)
    return fail(WTQ_ERR_UNSUPPORTED, "wtq_prefill: needs head_dim 128, widths 4/4, 4/6, 6/6 or 8/8, "
                "a power-of-two page size >= 16, at most 8 query heads per kv head and 16-byte "
                "aligned pages");
  if (cudaMemsetAsync(p.work_counter, 0, 256, stream) != cudaSuccess)
    return check_cuda(cudaGetLastError(), "wtq_prefill: counter reset");
  // balanced schedule: a row's slots that no piece writes must read as empty (l = 0)
  if (balanced && cudaMemsetAsync(p.part_l, 0, rows * splits * sizeof(float), stream) != cudaSuccess)
    return check_cuda(cudaGetLastError(), "wtq_prefill: chunk state reset");
  // rotation of the B * Q * Hq query rows (exp2 domain) and the lookup tables
  ScanSetup setup = {nullptr, (uint32_t *)p.lut, k_side->centroids, v_side->centroids, k_side->bw,
                     v_side->bw, mma_lut_words(k_side->bw, v_side->bw)};
  const float q_scale = scale * 1.4426950408889634f;
  if (rows_mma_rotate_eligible(q, q_strides[0], q_strides[1], Hq, D, total_rows, k_side->Pi, q_rot)) {
    if (int rc = launch_rotate_rows_mma(q, dtype, k_side->Pi, q_scale, total_rows, q_rot, setup, status,
                                        stream))
      return rc;
  } else if (int rc = launch_rotate_q(q, dtype, q_strides, k_side->Pi, q_scale, B * Q, Hq, D, q_rot,
                                      nullptr, chunk_tokens, max_tokens, setup, stream)) {
    return rc;
  }
  int rc = WTQ_ERR_UNSUPPORTED;
  if (p.k.bw == 4 && p.v.bw == 4) rc = pf::launch<4, 4>(p, stream);
  else if (p.k.bw == 4 && p.v.bw == 6) rc = pf::launch<4, 6>(p, stream);
  else if (p.k.bw == 6 && p.v.bw == 6) rc = pf::launch<6, 6>(p, stream);
  else if (p.k.bw == 8 && p.v.bw == 8) rc = pf::launch<8, 8>(p, stream);
  if (rc) return rc;
  MergeParams m = {};
  m.part_acc = p.part_acc; m.part_m = p.part_m; m.part_l = p.part_l;
  m.Pi_v = v_side->Pi; m.out = out; m.osb = out_strides[0]; m.osh = out_strides[1];
  m.dtype = dtype; m.Hq = Hq; m.D = D; m.num_splits = splits;
  m.work_counter = nullptr;
  // (balanced: slot c of a row is read when the row sees more than c tokens; a piece in
  // slot c starts at tile c or later, so no filled slot goes unread)
  if (balanced || rows_mma_merge_eligible(m, total_rows))
    return launch_merge_rows_mma(m, p.row_lens, total_rows, balanced ? 1 : chunk_tokens, max_tokens, status,
                                 stream);
  return launch_mma_merge(m, p.row_lens, B * Q, Hkv, p.n_rep, chunk_tokens, max_tokens, stream);
}
