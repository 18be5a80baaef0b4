// Fused dequantisation of packed rows: unpack -> centroid gather -> rotation
// by Pi -> norm rescale -> one store in the output dtype.  Serves the prefill
// fallback and the contiguous legacy cache, which hand over a
// (planes, MAXLEN, NB) buffer viewed through its first L positions
// (turboquant_kv/kernel.py:47-53).
//
// Two kernels here, and the tcgen05 kernel of wtq_dequant_umma.cu, which the
// tensor-core modes try first:
//
// dequant_kernel (any D <= 256, any width): fp32 on the CUDA cores.  A block
// takes kRows rows; their centroid values sit in shared memory; thread c owns
// output column c and walks Pi[:, c] once for all kRows rows, so every Pi
// element fetched (coalesced across the block) feeds kRows FMAs.
//
// dequant_mma_kernel (D = 128, widths 4/6/8): out = (C Pi) * norm as a
// (rows x 128)(128 x 128) product on the tensor cores.  A warp takes 32 rows;
// the A fragments of mma.m16n8k16 come straight out of the packed words through
// the per-lane lookup tables of wtq_lut.cuh (no decoded tile is ever written),
// Pi sits in shared memory as fp16 in the order the fragments consume it and is
// fetched with ldmatrix, the accumulators hold the whole 32 x 128 result, and
// the epilogue scales by the row norm, converts, and turns the fragment layout
// into full 256-byte row segments through a small per-warp staging area.  With
// TERMS = 1 the operands are single fp16 values (the accuracy class of the
// reference's allow_tf32 path, turboquant_kv/kernel.py:69); with TERMS = 3
// centroids and Pi are split into fp16 high and low parts and the three
// significant products are accumulated in fp32.
#include "wtq_common.cuh"
#include "wtq_lut.cuh"
#include "wtq_dequant.cuh"

#include <atomic>
#include <mutex>

namespace wtq {

constexpr int kRows = 16;

__global__ void dequant_kernel(DequantParams p) {
  __shared__ float y[kRows][256];
  __shared__ float nrm[kRows];
  __shared__ float cent[256];
  const int tid = threadIdx.x;
  for (int e = tid; e < (1 << p.bw); e += blockDim.x) cent[e] = p.centroids[e];
  __syncthreads();
  for (int64_t r0 = (int64_t)blockIdx.x * kRows; r0 < p.N; r0 += (int64_t)gridDim.x * kRows) {
    const int rows = (int)min((int64_t)kRows, p.N - r0);
    for (int e = tid; e < rows * p.D; e += blockDim.x) {
      const int r = e / p.D, d = e - r * p.D;
      const int64_t row = r0 + r;
      const int64_t src = (row / p.L) * p.MAXLEN + row % p.L;
      y[r][d] = cent[extract_code(p.packed + src * p.nb, d, p.bw, p.nb)];
      if (d == 0) nrm[r] = __half2float(p.norms[src]);
    }
    __syncthreads();
    for (int c = tid; c < p.D; c += blockDim.x) {
      float acc[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r) acc[r] = 0.0f;
      for (int d = 0; d < p.D; ++d) {
        const float w = p.Pi[(int64_t)d * p.D + c];
#pragma unroll
        for (int r = 0; r < kRows; ++r) acc[r] = fmaf(y[r][d], w, acc[r]);
      }
#pragma unroll
      for (int r = 0; r < kRows; ++r)
        if (r < rows) store_from_float(p.out, (r0 + r) * p.D + c, acc[r] * nrm[r], p.out_dtype);
    }
    __syncthreads();
  }
}


// ---- tensor-core kernel ------------------------------------------------------
namespace dq {

constexpr int kWarps = 8, kThreads = 32 * kWarps;
constexpr uint32_t kPiRow = 272;                  // bytes per row of a Pi table (256 + 16: ldmatrix conflict-free)
constexpr uint32_t kPiBytes = 128 * kPiRow;
constexpr uint32_t kPiHi = 1024;                  // shared address of Pi (high parts)
// Bytes per staged output row, 256 of payload plus a pad that keeps the
// fragment-layout stores conflict-free: 32-bit stores (16-bit outputs) want the
// eight row groups 4 banks apart, 64-bit stores (fp32 outputs) 8 banks apart.
constexpr uint32_t kStageBytes = 16 * 288;        // per warp: 16 rows
// Centroids and Pi are held as fp16 multiplied by 2^8 each (exact), which lifts
// the low parts of the split, about 2^-12 of a value, out of fp16's subnormal
// range; the epilogue takes the 2^-16 back together with the row norm.
constexpr float kOperandScale = 256.f, kResultScale = 1.f / (256.f * 256.f);
static_assert(kPiHi + kPiBytes <= mma::kLutAddr, "Pi must end below the lookup tables");

template <int BW, int TERMS> struct Map {
  static constexpr uint32_t kLutBytes = mma::lut_entries(BW) * 256u;
  static constexpr uint32_t kPiLo = mma::kLutAddr + kLutBytes;
  static constexpr uint32_t kStage = kPiLo + (TERMS == 3 ? kPiBytes : 0u);
  static constexpr uint32_t kStageEnd = kStage + kWarps * kStageBytes;
  // Landing slots of the packed rows copied ahead (one tile per warp and slot):
  // the first goes below the lookup tables if it fits there, the rest above the
  // staging area; as many of two as the 227 KB allow (none: rows are loaded
  // straight into registers at the top of each tile).
  static constexpr uint32_t kSlotBytes = kWarps * 32u * 16u * BW;
  static constexpr uint32_t kLowFree = mma::kLutAddr - (kPiHi + kPiBytes);
  static constexpr bool kLowSlot = kSlotBytes <= kLowFree;
  static constexpr uint32_t kLimit = 227u * 1024u;
  static constexpr int kHighSlots = (int)((kLimit - kStageEnd) / kSlotBytes);
  static constexpr int kSlots = (kLowSlot ? 1 : 0) + kHighSlots >= 2 ? 2 : (kLowSlot ? 1 : 0) + kHighSlots;
  static constexpr uint32_t kSlot0 = kLowSlot ? kPiHi + kPiBytes : kStageEnd;
  static constexpr uint32_t kSlot1 = kLowSlot ? kStageEnd : kStageEnd + kSlotBytes;
  static constexpr uint32_t kDynamic =
      kStageEnd + (uint32_t)(kSlots - (kLowSlot && kSlots > 0 ? 1 : 0)) * kSlotBytes;
  static_assert(kDynamic <= kLimit, "shared memory budget");
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t a, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void sts64(uint32_t a, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(a), "f"(x), "f"(y) : "memory");
}
__device__ __forceinline__ void sts16(uint32_t a, __half h) {
  asm volatile("st.shared.u16 [%0], %1;\n" ::"r"(a), "h"(__half_as_ushort(h)) : "memory");
}

// The lane's quarter of packed row `src`: NW 32-bit words.
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

// The same quarter row, copied asynchronously to this lane's place in a slot
// (16-byte pieces; 8-byte ones for the 24-byte quarters of 6-bit rows), and
// read back by the lane that copied it.  Piece j of the lane's row i sits at
// (i * pieces + j) * 32 + lane, so a warp's reads are contiguous.
template <int BW>
__device__ __forceinline__ void copy_row(uint32_t slot, int i, int lane, const uint8_t *packed,
                                         int64_t src, int t) {
  const uint8_t *at = packed + src * (16 * BW) + t * (4 * BW);
  if constexpr (BW == 6) {
#pragma unroll
    for (int j = 0; j < 3; ++j)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(slot + (uint32_t)((i * 3 + j) * 32 + lane) * 8),
                   "l"(at + 8 * j) : "memory");
  } else {
#pragma unroll
    for (int j = 0; j < BW / 4; ++j)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(slot + (uint32_t)((i * (BW / 4) + j) * 32 + lane) * 16),
                   "l"(at + 16 * j) : "memory");
  }
}
template <int BW>
__device__ __forceinline__ void read_row(uint32_t slot, int i, int lane, uint32_t (&w)[BW]) {
  if constexpr (BW == 6) {
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const uint2 v = lds64(slot + (uint32_t)((i * 3 + j) * 32 + lane) * 8);
      w[2 * j] = v.x; w[2 * j + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < BW / 4; ++j) {
      const uint4 v = lds128(slot + (uint32_t)((i * (BW / 4) + j) * 32 + lane) * 16);
      w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
    }
  }
}

// Contraction steps KS..7 for the warp's two 16-row tiles.  Step KS covers, for
// the lane group t, the coordinates 32t + 4KS .. 32t + 4KS + 3 (the order in
// which key_fragment hands out codes); the Pi tables are stored to match.
template <int BW, int TERMS, int KS>
__device__ __forceinline__ void contract(const uint32_t (&w)[2][2][BW], uint32_t sel, uint32_t pi_hi,
                                         uint32_t pi_lo, float (&acc)[2][16][4]) {
  uint32_t ah[2][4], al[2][4];
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    key_fragment<BW, KS>(w[m][0], w[m][1], sel, ah[m]);
    if constexpr (TERMS == 3) key_fragment<BW, KS>(w[m][0], w[m][1], sel | 0x80u, al[m]);
  }
#pragma unroll
  for (int np = 0; np < 8; ++np) {
    uint32_t bh[4], bl[4];
    ldmatrix_x4(pi_hi + np * 16 * kPiRow + KS * 32, bh);
    if constexpr (TERMS == 3) ldmatrix_x4(pi_lo + np * 16 * kPiRow + KS * 32, bl);
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      if constexpr (TERMS == 3) {                 // small products first
        mma16816(acc[m][2 * np], al[m][0], al[m][1], al[m][2], al[m][3], bh[0], bh[1]);
        mma16816(acc[m][2 * np + 1], al[m][0], al[m][1], al[m][2], al[m][3], bh[2], bh[3]);
        mma16816(acc[m][2 * np], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bl[0], bl[1]);
        mma16816(acc[m][2 * np + 1], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bl[2], bl[3]);
      }
      mma16816(acc[m][2 * np], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bh[0], bh[1]);
      mma16816(acc[m][2 * np + 1], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bh[2], bh[3]);
    }
  }
  if constexpr (KS < 7) contract<BW, TERMS, KS + 1>(w, sel, pi_hi, pi_lo, acc);
}

template <int DT> __device__ __forceinline__ uint32_t pack2(float x, float y);
template <> __device__ __forceinline__ uint32_t pack2<WTQ_F16>(float x, float y) {
  return pack_half2(x, y);
}
template <> __device__ __forceinline__ uint32_t pack2<WTQ_BF16>(float x, float y) {
  __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<uint32_t *>(&h);
}

template <int BW, int TERMS, int DT>
__global__ void __launch_bounds__(kThreads, 1) dequant_mma_kernel(DequantParams p, int32_t *refused) {
  using M = Map<BW, TERMS>;
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  if ((uint32_t)__cvta_generic_to_shared(dyn_smem) > kPiHi) {   // layout assumption broken
    if (tid == 0 && blockIdx.x == 0) *refused = 1;
    return;
  }
  if (p.N == 0) return;                           // the set-up probe: nothing to read
  // ---- one-time tables ---------------------------------------------------------
  // Codebook first (it is read 32 times per entry below).
  constexpr uint32_t kCent = M::kStage;             // the staging area is idle until the first epilogue
  for (int e = tid; e < (1 << BW); e += kThreads)
    sts32(kCent + 4 * e, __float_as_uint(__ldg(p.centroids + e) * kOperandScale));
  // A lane takes column c = 8 cb + (lane & 7) and the pair of contraction
  // positions 2 (4 kb + (lane >> 3)), + 1: its two loads share a 32-byte sector
  // with seven other lanes, and the 32 stores of a warp fall into 32 banks.
#pragma unroll 8
  for (int it = 0; it < 32; ++it) {
    const int combo = it * kWarps + warp, cb = combo & 15, kb = combo >> 4;
    const int c = 8 * cb + (lane & 7), kpos = 2 * (4 * kb + (lane >> 3));
    const int ks = kpos >> 4, kappa = kpos & 15;
    const int d = 32 * ((kappa & 7) >> 1) + 4 * ks + 2 * (kappa >> 3);     // kappa is even: d, d + 1
    const float x0 = __ldg(p.Pi + d * 128 + c) * kOperandScale;
    const float x1 = __ldg(p.Pi + (d + 1) * 128 + c) * kOperandScale;
    const __half2 hi = __floats2half2_rn(x0, x1);
    const uint32_t off = (uint32_t)c * kPiRow + (uint32_t)kpos * 2;
    sts32(kPiHi + off, *reinterpret_cast<const uint32_t *>(&hi));
    if constexpr (TERMS == 3)
      sts32(M::kPiLo + off, pack_half2(x0 - __low2float(hi), x1 - __high2float(hi)));
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
  __syncthreads();

  const uint32_t sel = mma::kLutAddr | (uint32_t)(lane << 2);
  const uint32_t lane_off = (uint32_t)(((lane >> 4) * 8 + (lane & 7)) * kPiRow + ((lane >> 3) & 1) * 16);
  const uint32_t stage = M::kStage + (uint32_t)warp * kStageBytes;
  const int64_t tiles = (p.N + 31) >> 5;
  const uint32_t L32 = (uint32_t)p.L;
  constexpr int kEsize = DT == WTQ_F32 ? 4 : 2;
  constexpr uint32_t kStageRow = kEsize == 4 ? 288u : 272u;

  // Source row and norm of the lane's row i (0..3: rows g, g + 8, g + 16, g + 24)
  // of a tile; rows past the end re-read the last row.
  auto source = [&](int64_t tile, int i) -> int64_t {
    const int64_t row0 = tile << 5;
    const int64_t plane0 = row0 / p.L;
    const uint32_t pos0 = (uint32_t)(row0 - plane0 * p.L);
    const int last = (int)min((int64_t)31, p.N - 1 - row0);
    const uint32_t pos = pos0 + (uint32_t)min(8 * i + g, last);
    const uint32_t wrap = pos / L32;
    return (plane0 + wrap) * p.MAXLEN + (pos - wrap * L32);
  };
  const int64_t stride = (int64_t)gridDim.x * kWarps;
  int64_t tile = (int64_t)blockIdx.x * kWarps + warp;
  const uint32_t slot_a = M::kSlot0 + (uint32_t)warp * (32u * 16u * BW);
  const uint32_t slot_b = M::kSlots == 2 ? M::kSlot1 + (uint32_t)warp * (32u * 16u * BW) : slot_a;
  float ahead[4] = {0.f, 0.f, 0.f, 0.f};          // norms of the tile being copied
  int parity = 0;
  if constexpr (M::kSlots > 0) {
    if (tile < tiles) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t src = source(tile, i);
        copy_row<BW>(slot_a, i, lane, p.packed, src, t);
        ahead[i] = __half2float(p.norms[src]) * kResultScale;
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }

  for (; tile < tiles; tile += stride) {
    const int64_t row0 = tile << 5;
    uint32_t w[2][2][BW];
    float nrm[2][2];
    if constexpr (M::kSlots > 0) {
      // A lane reads back only what it copied itself, so its own wait is enough.
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      const uint32_t slot = parity ? slot_b : slot_a;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        read_row<BW>(slot, i, lane, w[i >> 1][i & 1]);
        nrm[i >> 1][i & 1] = ahead[i];
      }
      // Next tile: into the other slot, or, with a single slot, into the one just
      // read (the reads above were issued first through the same load/store unit
      // and the copies land a global-memory round trip later).
      const int64_t next = tile + stride;
      parity ^= 1;
      if (next < tiles) {
        const uint32_t into = parity ? slot_b : slot_a;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int64_t src = source(next, i);
          copy_row<BW>(into, i, lane, p.packed, src, t);
          ahead[i] = __half2float(p.norms[src]) * kResultScale;
        }
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int64_t src = source(tile, i);
        load_row<BW>(p.packed, src, t, w[i >> 1][i & 1]);
        nrm[i >> 1][i & 1] = __half2float(p.norms[src]) * kResultScale;
      }
    }
    float acc[2][16][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int j = 0; j < 16; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][j][i] = 0.f;
    contract<BW, TERMS, 0>(w, sel, kPiHi + lane_off, M::kPiLo + lane_off, acc);

    // ---- epilogue: 16 rows x 256 payload bytes per pass through the staging area
    constexpr int kPasses = kEsize == 4 ? 2 : 1;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
      for (int ps = 0; ps < kPasses; ++ps) {
        if constexpr (kEsize == 4) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float(&a)[4] = acc[m][8 * ps + j];
            sts64(stage + g * kStageRow + j * 32 + t * 8, a[0] * nrm[m][0], a[1] * nrm[m][0]);
            sts64(stage + (g + 8) * kStageRow + j * 32 + t * 8, a[2] * nrm[m][1], a[3] * nrm[m][1]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float(&a)[4] = acc[m][j];
            sts32(stage + g * kStageRow + j * 16 + t * 4, pack2<DT>(a[0] * nrm[m][0], a[1] * nrm[m][0]));
            sts32(stage + (g + 8) * kStageRow + j * 16 + t * 4,
                  pack2<DT>(a[2] * nrm[m][1], a[3] * nrm[m][1]));
          }
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = (lane >> 4) + 2 * i;
          const uint4 v = lds128(stage + r * kStageRow + (lane & 15) * 16);
          const int64_t n = row0 + 16 * m + r;
          if (n < p.N)
            *reinterpret_cast<uint4 *>((uint8_t *)p.out + n * (128 * kEsize) + ps * 256 + (lane & 15) * 16) = v;
        }
        __syncwarp();
      }
    }
  }
}

}  // namespace dq

}  // namespace wtq

using namespace wtq;

namespace {

// Set by dequant_mma_kernel when its shared-memory window does not start where
// the fixed table addresses assume; read back once per kernel variant and device.
__device__ int32_t g_layout_refused;

// 0: not probed, 1: usable, 2: refused
template <int BW, int TERMS, int DT> std::atomic<int> &variant_state(int dev) {
  static std::atomic<int> state[64];
  return state[dev & 63];
}

// First use of a variant on a device: opt in to its shared memory and run it
// over zero rows to learn whether the layout assumption holds.  That needs one
// synchronisation, which a capturing stream cannot give: the caller then gets
// `false` with *busy set and decides.
template <int BW, int TERMS, int DT>
bool variant_ready(cudaStream_t stream, bool *busy, int *err) {
  using M = dq::Map<BW, TERMS>;
  int dev = 0;
  cudaGetDevice(&dev);
  std::atomic<int> &state = variant_state<BW, TERMS, DT>(dev);
  int s = state.load(std::memory_order_acquire);
  if (s) return s == 1;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    *busy = true;
    return false;
  }
  static std::mutex gate;
  std::lock_guard<std::mutex> hold(gate);
  if ((s = state.load(std::memory_order_acquire))) return s == 1;
  auto kernel = dq::dequant_mma_kernel<BW, TERMS, DT>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)M::kDynamic);
  int32_t *flag = nullptr, refused = 0;
  if (e == cudaSuccess) e = cudaGetSymbolAddress((void **)&flag, g_layout_refused);
  if (e == cudaSuccess) e = cudaMemsetAsync(flag, 0, sizeof(int32_t), stream);
  if (e == cudaSuccess) {
    DequantParams none = {};
    none.L = none.MAXLEN = 1;
    kernel<<<1, dq::kThreads, M::kDynamic, stream>>>(none, flag);
    note_launches(1);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(&refused, flag, sizeof(int32_t), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    *err = check_cuda(e, "wtq_dequant: tensor-core kernel set-up");
    return false;
  }
  state.store(refused ? 2 : 1, std::memory_order_release);
  return refused == 0;
}

template <int BW, int TERMS, int DT>
int launch_mma(const DequantParams &p, cudaStream_t stream, bool *unavailable) {
  using M = dq::Map<BW, TERMS>;
  bool busy = false;
  int err = WTQ_OK;
  if (!variant_ready<BW, TERMS, DT>(stream, &busy, &err)) {
    if (err != WTQ_OK) return err;                // a CUDA error: nothing else should run
    *unavailable = true;
    return busy ? fail(WTQ_ERR_UNSUPPORTED,
                       "wtq_dequant: the first tensor-core call of a kind must be made outside "
                       "stream capture")
                : fail(WTQ_ERR_UNSUPPORTED,
                       "wtq_dequant: this device places dynamic shared memory where the "
                       "tensor-core kernel's fixed table addresses cannot be used");
  }
  int32_t *flag = nullptr;
  cudaGetSymbolAddress((void **)&flag, g_layout_refused);
  const int64_t tiles = (p.N + 31) / 32;
  int64_t blocks = (tiles + dq::kWarps - 1) / dq::kWarps;
  const int sms = device_sms();
  if (blocks > sms) blocks = sms;
  dq::dequant_mma_kernel<BW, TERMS, DT><<<(unsigned)blocks, dq::kThreads, M::kDynamic, stream>>>(p, flag);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_dequant tensor-core launch");
}

template <int BW, int TERMS>
int launch_mma_dtype(const DequantParams &p, cudaStream_t stream, bool *unavailable) {
  if (p.out_dtype == WTQ_F32) return launch_mma<BW, TERMS, WTQ_F32>(p, stream, unavailable);
  if (p.out_dtype == WTQ_F16) return launch_mma<BW, TERMS, WTQ_F16>(p, stream, unavailable);
  return launch_mma<BW, TERMS, WTQ_BF16>(p, stream, unavailable);
}

template <int TERMS>
int launch_mma_width(const DequantParams &p, cudaStream_t stream, bool *unavailable) {
  if (p.bw == 4) return launch_mma_dtype<4, TERMS>(p, stream, unavailable);
  if (p.bw == 6) return launch_mma_dtype<6, TERMS>(p, stream, unavailable);
  return launch_mma_dtype<8, TERMS>(p, stream, unavailable);
}

// What the tensor-core kernel needs of a call; `why` names the first miss.
bool mma_eligible(const DequantParams &p, const char **why) {
  *why = nullptr;
  if (p.D != 128) *why = "head_dim must be 128";
  else if (p.bw != 4 && p.bw != 6 && p.bw != 8) *why = "bit width must be 4, 6 or 8";
  else if (p.MAXLEN >= (int64_t)1 << 31) *why = "MAXLEN must be below 2^31";
  else if ((uintptr_t)p.packed % (p.bw == 6 ? 8 : 16)) *why = "packed rows must be 16-byte aligned (8 for 6-bit)";
  else if ((uintptr_t)p.out % 16 || (uintptr_t)p.Pi % 16) *why = "out and Pi must be 16-byte aligned";
  return *why == nullptr;
}

int launch_exact(const DequantParams &p, cudaStream_t stream) {
  int64_t blocks = (p.N + kRows - 1) / kRows;
  const int64_t cap = (int64_t)device_sms() * 8;
  if (blocks > cap) blocks = cap;
  const int threads = p.D <= 32 ? 32 : p.D <= 64 ? 64 : 128;
  dequant_kernel<<<(unsigned)blocks, threads, 0, stream>>>(p);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_dequant launch");
}

}  // namespace

extern "C" int wtq_dequant_mode(const uint8_t *packed, const void *norms_f16, const float *centroids,
                                const float *Pi, void *out, int out_dtype, int bw, int D, int64_t N,
                                int64_t L, int64_t MAXLEN, int mode, void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (N < 0 || D < 1 || D > 256) return fail(WTQ_ERR_ARG, "wtq_dequant: need 1 <= D <= 256");
  if (!width_supported(bw) || (D * bw) % 8)
    return fail(WTQ_ERR_ARG, "wtq_dequant: bit width %d unsupported for D=%d", bw, D);
  if (out_dtype < WTQ_F32 || out_dtype > WTQ_BF16)
    return fail(WTQ_ERR_ARG, "wtq_dequant: bad output dtype");
  if (mode < WTQ_DEQUANT_AUTO || mode > WTQ_DEQUANT_TC_FAST_MMA)
    return fail(WTQ_ERR_ARG, "wtq_dequant: bad mode %d", mode);
  if (N == 0) return WTQ_OK;
  if (L < 1 || MAXLEN < L) return fail(WTQ_ERR_ARG, "wtq_dequant: need 1 <= L <= MAXLEN");
  if (!packed || !norms_f16 || !centroids || !Pi || !out)
    return fail(WTQ_ERR_ARG, "wtq_dequant: null buffer");
  DequantParams p;
  p.packed = packed; p.norms = (const __half *)norms_f16; p.centroids = centroids; p.Pi = Pi;
  p.out = out; p.out_dtype = out_dtype; p.bw = bw; p.D = D; p.nb = D * bw / 8;
  p.N = N; p.L = L; p.MAXLEN = MAXLEN;
  const char *why = nullptr;
  const bool can = mma_eligible(p, &why);
  // Tensor-core modes: the tcgen05 kernel where it can run, the mma.sync kernel
  // otherwise (or when asked for by name).
  auto tensor_cores = [&](int terms, bool legacy_only, bool *unavailable) -> int {
    if (!legacy_only) {
      bool usable = false;
      if (int rc = launch_dequant_umma(p, terms, stream, &usable)) return rc;
      if (usable) return WTQ_OK;
    }
    return terms == 3 ? launch_mma_width<3>(p, stream, unavailable)
                      : launch_mma_width<1>(p, stream, unavailable);
  };
  if (mode == WTQ_DEQUANT_AUTO) {
    // 16-bit outputs take the split tensor-core form where it applies; fp32
    // outputs keep the fp32 contraction.
    if (!can || out_dtype == WTQ_F32) return launch_exact(p, stream);
    bool unavailable = false;
    const int rc = tensor_cores(3, false, &unavailable);
    return unavailable ? launch_exact(p, stream) : rc;
  }
  if (mode == WTQ_DEQUANT_EXACT) return launch_exact(p, stream);
  if (!can) return fail(WTQ_ERR_UNSUPPORTED, "wtq_dequant: tensor-core kernel: %s", why);
  bool unavailable = false;
  const bool split = mode == WTQ_DEQUANT_TC || mode == WTQ_DEQUANT_TC_MMA;
  const bool legacy = mode == WTQ_DEQUANT_TC_MMA || mode == WTQ_DEQUANT_TC_FAST_MMA;
  return tensor_cores(split ? 3 : 1, legacy, &unavailable);
}

extern "C" int wtq_dequant(const uint8_t *packed, const void *norms_f16, const float *centroids,
                           const float *Pi, void *out, int out_dtype, int bw, int D, int64_t N,
                           int64_t L, int64_t MAXLEN, void *stream) {
  return wtq_dequant_mode(packed, norms_f16, centroids, Pi, out, out_dtype, bw, D, N, L, MAXLEN,
                          WTQ_DEQUANT_AUTO, stream);
}
