// (rows x 128) times a 128 x 128 rotation on the tensor cores, for calls with
// thousands of rows: the query rotation and the chunk merge of chunked prefill
// (wtq_prefill), whose 32k+ rows made the CUDA-core kernels of the decode step
// (one block per few rows, Pi through L1/L2 for every block) a fifth of the call.
//
//   rotate  q_rot[r][c] = mult * sum_d q[r][d] Pi[c][d]        (fp32 out)
//   merge   out[r][c]   = sum_d a[r][d] Pi[d][c],  a = merged and normalised
//           chunk states of row r (the arithmetic of merge_small_kernel)
//
// A warp takes 32 rows.  The A fragments of mma.m16n8k16 are made in registers
// from global loads (two adjacent coordinates per register), each value split
// into fp16 high and low parts; the rotation sits in shared memory as fp16 high
// and low parts times 2^8, one row per output coordinate, fetched with
// ldmatrix; the three significant products accumulate in fp32 (the dropped
// low x low term is 2^-22 of a product).  The epilogue turns the fragment layout
// into whole 256-byte row segments through a per-warp staging area, as the
// dequantisation kernel does.
#include <algorithm>
#include <atomic>

#include "wtq_decode.cuh"
#include "wtq_lut.cuh"

namespace wtq {
namespace rows {

constexpr int kWarps = 8, kThreads = 32 * kWarps;
constexpr uint32_t kBase = 1024;                  // dynamic shared memory is assumed to start at or below this
constexpr uint32_t kPiRow = 272;                  // 256 + 16: ldmatrix conflict-free
constexpr uint32_t kPiBytes = 128 * kPiRow;
constexpr uint32_t kPiHi = kBase, kPiLo = kPiHi + kPiBytes;
constexpr uint32_t kStage = kPiLo + kPiBytes;
constexpr uint32_t kStageBytes = 16 * 288;        // per warp: 16 rows x 256 payload bytes (+ pad)
constexpr uint32_t kWeights = kStage + kWarps * kStageBytes;   // merge: 32 rows x kMaxChunks weights per warp
constexpr int kMaxChunks = 8;
constexpr uint32_t kDynamic = kWeights + kWarps * 32 * kMaxChunks * 4;
constexpr float kPiScale = 256.f;

struct Params {
  // rotate
  const void *q;             // (rows, 128) contiguous, `in_dtype`
  int in_dtype;
  float mult;
  // merge
  const float *part_acc, *part_m, *part_l;
  const int32_t *row_lens;   // (rows / Hq) causal lengths
  int Hq, num_splits, chunk_tokens, max_tokens;
  // both
  const float *Pi;           // rotate: out coordinate c = row c of Pi; merge: c = column c
  void *out;                 // (rows, 128) contiguous
  int out_dtype;
  int64_t rows;
  // rotate also builds the lookup tables of the scan (all blocks share the words)
  uint32_t *lut;
  const float *cent_k, *cent_v;
  int bw_k, bw_v, lut_words;
  int32_t *status;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t a, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void sts64f(uint32_t a, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(a), "f"(x), "f"(y) : "memory");
}
template <int DT> __device__ __forceinline__ uint32_t pack2(float x, float y) {
  if constexpr (DT == WTQ_BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t *>(&h);
  } else {
    return pack_half2(x, y);
  }
}

// value pair (x, y) -> fp16 high parts and the fp16 of what they leave
__device__ __forceinline__ void split(float x, float y, uint32_t &hi, uint32_t &lo) {
  const __half2 h = __floats2half2_rn(x, y);
  hi = *reinterpret_cast<const uint32_t *>(&h);
  lo = pack_half2(x - __low2float(h), y - __high2float(h));
}

template <bool MERGE, int DT>
__global__ void __launch_bounds__(kThreads, 1) rows_kernel(Params p) {
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  if ((uint32_t)__cvta_generic_to_shared(dyn_smem) > kBase) {   // layout assumption broken
    if (p.status && tid == 0) atomicOr(p.status, WTQ_STATUS_LAYOUT);
    return;
  }
  if constexpr (!MERGE) {
    if (p.lut != nullptr)
      for (int e = blockIdx.x * kThreads + tid; e < p.lut_words; e += gridDim.x * kThreads)
        p.lut[e] = mma::lut_word(e, p.bw_k, p.bw_v, p.cent_k, p.cent_v);
  }
  // ---- the rotation, one shared-memory row per output coordinate c, contraction
  // index d along the row
  if constexpr (!MERGE) {
    // T[c][d] = Pi[c][d]: a lane takes the pair (d, d + 1) of row c
#pragma unroll 8
    for (int it = 0; it < 32; ++it) {
      const int e = it * kThreads + tid, c = e >> 6, d = (e & 63) * 2;
      const float2 v = __ldg(reinterpret_cast<const float2 *>(p.Pi + c * 128 + d));
      uint32_t hi, lo;
      split(v.x * kPiScale, v.y * kPiScale, hi, lo);
      sts32(kPiHi + (uint32_t)c * kPiRow + 2u * d, hi);
      sts32(kPiLo + (uint32_t)c * kPiRow + 2u * d, lo);
    }
  } else {
    // T[c][d] = Pi[d][c]: a lane takes column c = 8 cb + (lane & 7) and the pair of
    // rows d = 2 (4 db + (lane >> 3)), d + 1 (sector-sized reads, conflict-free writes)
#pragma unroll 8
    for (int it = 0; it < 32; ++it) {
      const int combo = it * kWarps + warp, cb = combo & 15, db = combo >> 4;
      const int c = 8 * cb + (lane & 7), d = 2 * (4 * db + (lane >> 3));
      uint32_t hi, lo;
      split(__ldg(p.Pi + d * 128 + c) * kPiScale, __ldg(p.Pi + (d + 1) * 128 + c) * kPiScale, hi, lo);
      sts32(kPiHi + (uint32_t)c * kPiRow + 2u * d, hi);
      sts32(kPiLo + (uint32_t)c * kPiRow + 2u * d, lo);
    }
  }
  __syncthreads();
  if constexpr (MERGE) asm volatile("griddepcontrol.wait;\n" ::: "memory");   // chunk states are complete

  const uint32_t lane_off = (uint32_t)(((lane >> 4) * 8 + (lane & 7)) * kPiRow + ((lane >> 3) & 1) * 16);
  const uint32_t stage = kStage + (uint32_t)warp * kStageBytes;
  const uint32_t weights = kWeights + (uint32_t)warp * (32 * kMaxChunks * 4);
  const int64_t tiles = (p.rows + 31) >> 5;
  constexpr int kEsize = DT == WTQ_F32 ? 4 : 2;
  constexpr uint32_t kStageRow = kEsize == 4 ? 288u : 272u;

  for (int64_t tile = (int64_t)blockIdx.x * kWarps + warp; tile < tiles; tile += (int64_t)gridDim.x * kWarps) {
    const int64_t row0 = tile << 5;
    // ---- merge: lane l computes the chunk weights of row row0 + l -----------------
    int chunks_of[2][2] = {{0, 0}, {0, 0}};
    if constexpr (MERGE) {
      const int64_t row = row0 + lane;
      int chunks = 0;
      if (row < p.rows) {
        int L = p.row_lens[row / p.Hq];
        L = L < 0 ? 0 : (L > p.max_tokens ? p.max_tokens : L);
        chunks = min((L + p.chunk_tokens - 1) / p.chunk_tokens, p.num_splits);
      }
      float mv[kMaxChunks], lv[kMaxChunks], gmax = -INFINITY, denom = 0.f;
#pragma unroll
      for (int c = 0; c < kMaxChunks; ++c) {
        // a state with l = 0 is empty (nothing seen, or never written): its m and
        // accumulator are not read
        lv[c] = c < chunks ? __ldcg(p.part_l + row * p.num_splits + c) : 0.f;
        mv[c] = lv[c] > 0.f ? __ldcg(p.part_m + row * p.num_splits + c) : -INFINITY;
        gmax = fmaxf(gmax, mv[c]);
      }
#pragma unroll
      for (int c = 0; c < kMaxChunks; ++c) {
        mv[c] = mv[c] == -INFINITY ? 0.f : exp2f(mv[c] - gmax);
        denom += mv[c] * lv[c];
      }
      const float inv = denom > 0.f ? 1.f / fmaxf(denom, 1e-30f) : 0.f;
#pragma unroll
      for (int c = 0; c < kMaxChunks; ++c) sts32(weights + (uint32_t)(lane * kMaxChunks + c) * 4u, __float_as_uint(mv[c] * inv));
      __syncwarp();
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) chunks_of[m][h] = __shfl_sync(0xffffffffu, chunks, 16 * m + 8 * h + g);
    }
    // values (d, d + 1) of the lane's row (m, h), d even
    auto pair_at = [&](int m, int h, int d) -> float2 {
      const int lr = 16 * m + 8 * h + g;
      const int64_t row = row0 + lr;
      if (row >= p.rows) return make_float2(0.f, 0.f);
      if constexpr (!MERGE) {
        if (p.in_dtype == WTQ_F32) {
          return __ldg(reinterpret_cast<const float2 *>((const float *)p.q + row * 128 + d));
        } else if (p.in_dtype == WTQ_F16) {
          return __half22float2(__ldg(reinterpret_cast<const __half2 *>((const __half *)p.q + row * 128 + d)));
        } else {
          return __bfloat1622float2(
              __ldg(reinterpret_cast<const __nv_bfloat162 *>((const __nv_bfloat16 *)p.q + row * 128 + d)));
        }
      } else {
        float2 a = make_float2(0.f, 0.f);
        const float *src = p.part_acc + row * p.num_splits * 128 + d;
#pragma unroll
        for (int c = 0; c < kMaxChunks; ++c) {
          if (c < chunks_of[m][h]) {
            const float w = __uint_as_float(lds32(weights + (uint32_t)(lr * kMaxChunks + c) * 4u));
            if (w != 0.f) {
              const float2 v = __ldcg(reinterpret_cast<const float2 *>(src + c * 128));
              a.x = fmaf(w, v.x, a.x);
              a.y = fmaf(w, v.y, a.y);
            }
          }
        }
        return a;
      }
    };

    float acc[2][16][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int j = 0; j < 16; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][j][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t ah[2][4], al[2][4];
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const float2 v0 = pair_at(m, 0, 16 * ks + 2 * t), v1 = pair_at(m, 1, 16 * ks + 2 * t);
        const float2 v2 = pair_at(m, 0, 16 * ks + 8 + 2 * t), v3 = pair_at(m, 1, 16 * ks + 8 + 2 * t);
        split(v0.x, v0.y, ah[m][0], al[m][0]);
        split(v1.x, v1.y, ah[m][1], al[m][1]);
        split(v2.x, v2.y, ah[m][2], al[m][2]);
        split(v3.x, v3.y, ah[m][3], al[m][3]);
      }
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t bh[4], bl[4];
        ldmatrix_x4(kPiHi + lane_off + np * 16 * kPiRow + ks * 32, bh);
        ldmatrix_x4(kPiLo + lane_off + np * 16 * kPiRow + ks * 32, bl);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          mma16816_free(acc[m][2 * np], al[m][0], al[m][1], al[m][2], al[m][3], bh[0], bh[1]);
          mma16816_free(acc[m][2 * np + 1], al[m][0], al[m][1], al[m][2], al[m][3], bh[2], bh[3]);
          mma16816_free(acc[m][2 * np], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bl[0], bl[1]);
          mma16816_free(acc[m][2 * np + 1], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bl[2], bl[3]);
          mma16816_free(acc[m][2 * np], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bh[0], bh[1]);
          mma16816_free(acc[m][2 * np + 1], ah[m][0], ah[m][1], ah[m][2], ah[m][3], bh[2], bh[3]);
        }
      }
    }

    // ---- epilogue: 16 rows x 256 payload bytes per pass through the staging area
    const float post = (MERGE ? 1.f : p.mult) / kPiScale;
    constexpr int kPasses = kEsize == 4 ? 2 : 1;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
      for (int ps = 0; ps < kPasses; ++ps) {
        if constexpr (kEsize == 4) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float(&a)[4] = acc[m][8 * ps + j];
            sts64f(stage + g * kStageRow + j * 32 + t * 8, a[0] * post, a[1] * post);
            sts64f(stage + (g + 8) * kStageRow + j * 32 + t * 8, a[2] * post, a[3] * post);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float(&a)[4] = acc[m][j];
            sts32(stage + g * kStageRow + j * 16 + t * 4, pack2<DT>(a[0] * post, a[1] * post));
            sts32(stage + (g + 8) * kStageRow + j * 16 + t * 4, pack2<DT>(a[2] * post, a[3] * post));
          }
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = (lane >> 4) + 2 * i;
          const uint4 v = lds128(stage + r * kStageRow + (lane & 15) * 16);
          const int64_t n = row0 + 16 * m + r;
          if (n < p.rows)
            *reinterpret_cast<uint4 *>((uint8_t *)p.out + n * (128 * kEsize) + ps * 256 + (lane & 15) * 16) = v;
        }
        __syncwarp();
      }
    }
  }
}

template <bool MERGE, int DT>
int launch(const Params &p, bool pdl, cudaStream_t stream) {
  static std::atomic<bool> opted_in_dev[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !opted_in_dev[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(rows_kernel<MERGE, DT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDynamic);
    if (e != cudaSuccess) return check_cuda(e, "wtq_prefill: shared memory opt-in");
    opted_in_dev[dev & 63].store(true, std::memory_order_release);
  }
  const int64_t tiles = (p.rows + 31) / 32;
  const int grid = (int)std::min<int64_t>((tiles + kWarps - 1) / kWarps, device_sms());
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kDynamic;
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, rows_kernel<MERGE, DT>, p);
  note_launches(1);
  return check_cuda(e, MERGE ? "wtq_prefill merge launch" : "wtq_prefill rotation launch");
}

}  // namespace rows

bool rows_mma_rotate_eligible(const void *q, int64_t row_stride, int64_t head_stride, int Hq, int D,
                              int64_t rows, const float *Pi, const float *q_rot) {
  return D == 128 && rows >= 4096 && head_stride == D && row_stride == (int64_t)Hq * D &&
         ((uintptr_t)q & 15) == 0 && ((uintptr_t)Pi & 15) == 0 && ((uintptr_t)q_rot & 15) == 0;
}

int launch_rotate_rows_mma(const void *q, int dtype, const float *Pi, float mult, int64_t rows,
                           float *q_rot, const ScanSetup &setup, int32_t *status, cudaStream_t stream) {
  rows::Params p = {};
  p.q = q; p.in_dtype = dtype; p.mult = mult; p.Pi = Pi; p.out = q_rot; p.out_dtype = WTQ_F32;
  p.rows = rows; p.lut = setup.lut; p.cent_k = setup.cent_k; p.cent_v = setup.cent_v;
  p.bw_k = setup.bw_k; p.bw_v = setup.bw_v; p.lut_words = setup.lut_words; p.status = status;
  return rows::launch<false, WTQ_F32>(p, false, stream);
}

bool rows_mma_merge_eligible(const MergeParams &m, int64_t rows) {
  return m.D == 128 && rows >= 4096 && m.num_splits <= rows::kMaxChunks && m.world == 0 &&
         m.osh == m.D && m.osb == (int64_t)m.Hq * m.D && ((uintptr_t)m.out & 15) == 0 &&
         ((uintptr_t)m.Pi_v & 15) == 0 && ((uintptr_t)m.part_acc & 15) == 0;
}

int launch_merge_rows_mma(const MergeParams &m, const int32_t *row_lens, int64_t rows, int chunk_tokens,
                          int max_tokens, int32_t *status, cudaStream_t stream) {
  rows::Params p = {};
  p.part_acc = m.part_acc; p.part_m = m.part_m; p.part_l = m.part_l; p.row_lens = row_lens;
  p.Hq = m.Hq; p.num_splits = m.num_splits; p.chunk_tokens = chunk_tokens; p.max_tokens = max_tokens;
  p.Pi = m.Pi_v; p.out = m.out; p.out_dtype = m.dtype; p.rows = rows; p.status = status;
  if (m.dtype == WTQ_F32) return rows::launch<true, WTQ_F32>(p, true, stream);
  if (m.dtype == WTQ_F16) return rows::launch<true, WTQ_F16>(p, true, stream);
  return rows::launch<true, WTQ_BF16>(p, true, stream);
}

}  // namespace wtq
