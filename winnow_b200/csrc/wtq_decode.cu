// Split-K decode attention over paged packed K/V: the width- and shape-generic
// CUDA-core path (any head_dim <= 256 that packs to whole bytes, any supported
// bit width, any page size, any GQA ratio).
//
//   rotate_q_kernel        q_rot = scale * q Pi_K^T            (B*Hq blocks)
//   decode_generic_kernel  per (sequence, kv head, split): stream the pages of
//                          the split, scores n_K (q_rot . c_K), online softmax,
//                          accumulate p n_V c_V in the value basis, write the
//                          partial state (m, l, acc)
//   merge_rotate_kernel    stable merge of the split states, normalise,
//                          out = a Pi_V, cast to the query dtype
//
// Follows the schedule of the reference's tiled operator
// (turboquant_kv/packed_attention.py:260-334) and its split merge
// (turboquant_kv/packed_attention_triton.py:137-159); all state is fp32.
#include <algorithm>

#include "wtq_decode.cuh"
#include "wtq_lut.cuh"

namespace wtq {

// Exclusive prefix of chunks per sequence (B + 1 ints), computed by one warp.
__device__ void write_chunk_prefix(const int32_t *seq_lens, int B, int chunk_tokens,
                                   int max_tokens, int32_t *chunk_prefix) {
  int running = 0;
  for (int b0 = 0; b0 < B; b0 += 32) {
    const int b = b0 + (int)threadIdx.x;
    int n = 0;
    if (b < B) {
      int L = seq_lens[b];
      L = L < 0 ? 0 : (L > max_tokens ? max_tokens : L);
      n = (L + chunk_tokens - 1) / chunk_tokens;
    }
    int incl = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if ((int)threadIdx.x >= o) incl += up;
    }
    if (b < B) chunk_prefix[b] = running + incl - n;
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (threadIdx.x == 0) chunk_prefix[B] = running;
}

// Side jobs of the rotation launch for the tensor-core scan: the last block's
// first warp writes the chunk prefix; all blocks share the table words, each a
// half2 of centroids: 4-bit tables are indexed by a packed byte ({c[lo nibble],
// c[hi nibble]}), wider ones by a code ({c, c}); word = [index][key | value][lane].
__device__ void scan_setup(const ScanSetup &s, const int32_t *seq_lens, int B, int chunk_tokens,
                           int max_tokens) {
  if (s.chunk_prefix != nullptr && blockIdx.x == gridDim.x - 1 && threadIdx.x < 32)
    write_chunk_prefix(seq_lens, B, chunk_tokens, max_tokens, s.chunk_prefix);
  if (s.lut == nullptr) return;
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < s.lut_words; e += gridDim.x * blockDim.x) {
    s.lut[e] = mma::lut_word(e, s.bw_k, s.bw_v, s.cent_k, s.cent_v);
  }
}

// q_rot[row][c] = mult * sum_d q[row][d] Pi[c][d] for the `rows` query rows that
// start at row blockIdx.x * NR.  A warp takes output coordinates c = warp,
// warp + 16, ...; its lanes stride over d, so every Pi row is read once per
// block, coalesced, for all NR query rows, and the NR partial sums are reduced
// by shuffles.  Eight Pi rows are in flight per warp to cover L2 latency.
constexpr int kRotThreads = 512;
template <int NR>
__global__ void __launch_bounds__(kRotThreads) rotate_q_kernel(
    const void *q, int dtype, int64_t qsb, int64_t qsh, const float *Pi, float mult, int Hq,
    int D, int total_rows, float *q_rot, const int32_t *seq_lens, int B, int chunk_tokens,
    int max_tokens, ScanSetup setup) {
  __shared__ float qs[NR][256];
  scan_setup(setup, seq_lens, B, chunk_tokens, max_tokens);
  const int row0 = blockIdx.x * NR;
  for (int e = threadIdx.x; e < NR * D; e += kRotThreads) {
    const int r = e / D, d = e - r * D;
    const int row = row0 + r;
    float v = 0.f;
    if (row < total_rows) {
      const int b = row / Hq, h = row - b * Hq;
      v = load_as_float(q, (int64_t)b * qsb + (int64_t)h * qsh + d, dtype);
    }
    qs[r][d] = v;
  }
  __syncthreads();
  // the page scan that follows may start its own prologue now
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarps = kRotThreads / 32, kBatch = 8;
  // Every block needs all of Pi; blocks start at different rows so that at any
  // moment their requests spread over all of Pi's cache lines instead of
  // queueing on the same few.
  const int shift = (int)((blockIdx.x * 37u) % (unsigned)D);
  for (int c0 = warp; c0 < D; c0 += kWarps * kBatch) {
    float part[kBatch][NR];
    int rows[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int c = c0 + i * kWarps;
      rows[i] = c < D ? (c + shift) % D : -1;
#pragma unroll
      for (int r = 0; r < NR; ++r) part[i][r] = 0.f;
    }
#pragma unroll 4
    for (int d = lane; d < D; d += 32) {
      float w[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) w[i] = rows[i] >= 0 ? __ldg(Pi + (int64_t)rows[i] * D + d) : 0.f;
#pragma unroll
      for (int i = 0; i < kBatch; ++i)
#pragma unroll
        for (int r = 0; r < NR; ++r) part[i][r] = fmaf(qs[r][d], w[i], part[i][r]);
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const float v = warp_sum(part[i][r]);
        if (lane == 0 && rows[i] >= 0 && row0 + r < total_rows)
          q_rot[(int64_t)(row0 + r) * D + rows[i]] = v * mult;
      }
    }
  }
}

constexpr int kTile = 128;  // tokens per tile == threads per block

// Sequential reader of the codes of one packed row.
struct CodeReader {
  const uint8_t *row;
  uint64_t buf;
  int have, at, nb;
  __device__ CodeReader(const uint8_t *r, int nbytes) : row(r), buf(0), have(0), at(0), nb(nbytes) {}
  __device__ __forceinline__ unsigned next(int bw, bool words) {
    if (have < bw) {
      if (words) {
        buf |= (uint64_t)(*(const uint32_t *)(row + at)) << have;
        at += 4;
        have += 32;
      } else {
        while (have < bw && at < nb) {
          buf |= (uint64_t)row[at++] << have;
          have += 8;
        }
      }
    }
    const unsigned v = (unsigned)buf & ((1u << bw) - 1u);
    buf >>= bw;
    have -= bw;
    return v;
  }
};

template <int NR>
__global__ void __launch_bounds__(kTile) decode_generic_kernel(DecodeParams p) {
  __shared__ float qs[NR][256];
  __shared__ float cent_k[256], cent_v[256];
  __shared__ float p_s[NR][kTile];
  __shared__ const uint8_t *vrow_s[kTile];
  __shared__ float red[NR][kTile / 32];
  __shared__ float tile_max[NR];

  const int split = blockIdx.x;
  const int groups = (p.n_rep + NR - 1) / NR;
  const int kvh = blockIdx.y / groups, group = blockIdx.y - kvh * groups;
  const int b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int heads = min(NR, p.n_rep - group * NR);
  const int qh0 = kvh * p.n_rep + group * NR;
  const int D = p.D, S = p.S;

  for (int e = tid; e < NR * D; e += kTile) {
    const int h = e / D, d = e - h * D;
    qs[h][d] = h < heads ? p.q_rot[((int64_t)b * p.Hq + qh0 + h) * D + d] : 0.0f;
  }
  for (int e = tid; e < (1 << p.k.bw); e += kTile) cent_k[e] = p.k.centroids[e];
  for (int e = tid; e < (1 << p.v.bw); e += kTile) cent_v[e] = p.v.centroids[e];

  int L = p.seq_lens[b];
  if (L < 0) L = 0;
  if (L > p.max_pages * S) {
    L = p.max_pages * S;
    if (p.status && tid == 0) atomicOr(p.status, WTQ_STATUS_BAD_POSITION);
  }
  const int tiles_total = (L + kTile - 1) / kTile;
  const int tiles_per_split = (tiles_total + p.num_splits - 1) / p.num_splits;
  const int t_begin = split * tiles_per_split * kTile;
  const int t_end = min(L, (split + 1) * tiles_per_split * kTile);

  float m_run[NR], l_part[NR], acc[NR][2];
#pragma unroll
  for (int h = 0; h < NR; ++h) {
    m_run[h] = -INFINITY;
    l_part[h] = 0.0f;
    acc[h][0] = acc[h][1] = 0.0f;
  }
  const bool kwords = (p.k.nb & 3) == 0 && (p.k.page_stride & 3) == 0 &&
                      (p.k.head_stride & 3) == 0 && ((uintptr_t)p.k.pages & 3) == 0;
  __syncthreads();

  for (int base = t_begin; base < t_end; base += kTile) {
    const int tok = base + tid;
    bool ok = tok < t_end;
    float s[NR], nv = 0.0f;
#pragma unroll
    for (int h = 0; h < NR; ++h) s[h] = -INFINITY;
    const uint8_t *vrow = nullptr;
    if (ok) {
      const int slot_page = tok / S, slot = tok - slot_page * S;
      const int pid = p.page_table[(int64_t)b * p.table_stride + slot_page];
      if (pid < 0 || pid >= p.P) {
        ok = false;
        if (p.status) atomicOr(p.status, WTQ_STATUS_BAD_PAGE);
      } else {
        const uint8_t *krow = p.k.pages + (int64_t)pid * p.k.page_stride +
                              (int64_t)kvh * p.k.head_stride + (int64_t)slot * p.k.nb;
        vrow = p.v.pages + (int64_t)pid * p.v.page_stride + (int64_t)kvh * p.v.head_stride +
               (int64_t)slot * p.v.nb;
        const float nk = __half2float(
            p.k.norms[(int64_t)pid * p.k.norm_page_stride + (int64_t)kvh * p.k.norm_head_stride + slot]);
        nv = __half2float(
            p.v.norms[(int64_t)pid * p.v.norm_page_stride + (int64_t)kvh * p.v.norm_head_stride + slot]);
        float dot[NR];
#pragma unroll
        for (int h = 0; h < NR; ++h) dot[h] = 0.0f;
        CodeReader rd(krow, p.k.nb);
        for (int d = 0; d < D; ++d) {
          const float c = cent_k[rd.next(p.k.bw, kwords)];
#pragma unroll
          for (int h = 0; h < NR; ++h) dot[h] = fmaf(qs[h][d], c, dot[h]);
        }
#pragma unroll
        for (int h = 0; h < NR; ++h) s[h] = dot[h] * nk;
      }
    }
    vrow_s[tid] = ok ? vrow : nullptr;
    // block-wide running max per head
#pragma unroll
    for (int h = 0; h < NR; ++h) {
      const float wm = warp_max(s[h]);
      if (lane == 0) red[h][warp] = wm;
    }
    __syncthreads();
    if (tid < NR) {
      float t = red[tid][0];
      for (int w = 1; w < kTile / 32; ++w) t = fmaxf(t, red[tid][w]);
      tile_max[tid] = t;
    }
    __syncthreads();
    float alpha[NR];
#pragma unroll
    for (int h = 0; h < NR; ++h) {
      const float m_new = fmaxf(m_run[h], tile_max[h]);
      // exp(-inf - -inf) is defined as 0: nothing seen yet contributes nothing
      alpha[h] = (m_run[h] == -INFINITY) ? 0.0f : __expf(m_run[h] - m_new);
      const float pr = (ok && m_new != -INFINITY) ? __expf(s[h] - m_new) : 0.0f;
      l_part[h] = alpha[h] * l_part[h] + pr;
      p_s[h][tid] = pr * nv;
      m_run[h] = m_new;
    }
    __syncthreads();
    // value side: this thread owns output coordinates tid and tid + 128
    const int count = min(kTile, t_end - base);
#pragma unroll
    for (int slot2 = 0; slot2 < 2; ++slot2) {
      const int d = tid + slot2 * kTile;
      if (d < D) {
        float a[NR];
#pragma unroll
        for (int h = 0; h < NR; ++h) a[h] = alpha[h] * acc[h][slot2];
        for (int t = 0; t < count; ++t) {
          const uint8_t *row = vrow_s[t];
          if (row == nullptr) continue;
          const float c = cent_v[extract_code(row, d, p.v.bw, p.v.nb)];
#pragma unroll
          for (int h = 0; h < NR; ++h) a[h] = fmaf(p_s[h][t], c, a[h]);
        }
#pragma unroll
        for (int h = 0; h < NR; ++h) acc[h][slot2] = a[h];
      }
    }
    __syncthreads();
  }

  // partial state of this split; an empty split writes (m=-inf, l=0, acc=0)
#pragma unroll
  for (int h = 0; h < NR; ++h) {
    const float wl = warp_sum(l_part[h]);
    if (lane == 0) red[h][warp] = wl;
  }
  __syncthreads();
#pragma unroll
  for (int h = 0; h < NR; ++h) {
    if (h < heads) {
      const int64_t prow = ((int64_t)b * p.Hq + qh0 + h) * p.num_splits + split;
      if (tid < D) p.part_acc[prow * D + tid] = acc[h][0];
      if (tid + kTile < D) p.part_acc[prow * D + tid + kTile] = acc[h][1];
      if (tid == 0) {
        float l = 0.0f;
        for (int w = 0; w < kTile / 32; ++w) l += red[h][w];
        p.part_m[prow] = m_run[h];
        p.part_l[prow] = l;
      }
    }
  }
}

__global__ void __launch_bounds__(128) merge_rotate_kernel(MergeParams p) {
  __shared__ float a_s[256];
  __shared__ float w_s[kMaxSplits];
  __shared__ float denom_s;
  const int row = blockIdx.x;  // b * Hq + h
  const int b = row / p.Hq, h = row - b * p.Hq;
  const int tid = threadIdx.x;
  const int64_t base = (int64_t)row * p.num_splits;
  if (tid == 0) {
    float gmax = -INFINITY;
    for (int s = 0; s < p.num_splits; ++s) gmax = fmaxf(gmax, p.part_m[base + s]);
    float denom = 0.0f;
    for (int s = 0; s < p.num_splits; ++s) {
      const float m = p.part_m[base + s];
      const float w = (m == -INFINITY) ? 0.0f : __expf(m - gmax);
      w_s[s] = w;
      denom += w * p.part_l[base + s];
    }
    denom_s = denom;
  }
  __syncthreads();
  const float denom = denom_s;
  for (int d = tid; d < p.D; d += blockDim.x) {
    float a = 0.0f;
    for (int s = 0; s < p.num_splits; ++s)
      if (w_s[s] != 0.0f) a = fmaf(w_s[s], p.part_acc[(base + s) * p.D + d], a);
    a_s[d] = denom > 0.0f ? a / fmaxf(denom, 1e-30f) : 0.0f;
  }
  __syncthreads();
  for (int c = tid; c < p.D; c += blockDim.x) {
    float o = 0.0f;
    for (int d = 0; d < p.D; ++d) o = fmaf(a_s[d], p.Pi_v[(int64_t)d * p.D + c], o);
    store_from_float(p.out, (int64_t)b * p.osb + (int64_t)h * p.osh + c, o, p.dtype);
  }
}

int generic_group_width(int n_rep) { return n_rep >= 8 ? 8 : n_rep >= 3 ? 4 : n_rep; }

int launch_decode_generic(const DecodeParams &p, cudaStream_t stream) {
  const int nr = generic_group_width(p.n_rep);
  const int groups = (p.n_rep + nr - 1) / nr;
  dim3 grid((unsigned)p.num_splits, (unsigned)(p.Hkv * groups), (unsigned)p.B);
  profile_mark_begin(stream);
  switch (nr) {
    case 1: decode_generic_kernel<1><<<grid, kTile, 0, stream>>>(p); break;
    case 2: decode_generic_kernel<2><<<grid, kTile, 0, stream>>>(p); break;
    case 4: decode_generic_kernel<4><<<grid, kTile, 0, stream>>>(p); break;
    default: decode_generic_kernel<8><<<grid, kTile, 0, stream>>>(p); break;
  }
  profile_mark_end(stream);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_decode generic launch");
}

// Same result as rotate_q_kernel for head_dim a multiple of 16: thread
// (column c, quarter) walks its quarter of row c of Pi with 16-byte loads (a
// thread owns a row, so no cross-lane reduction is needed; the row's sectors
// are reused through L1), the four query rows come from shared memory as one
// 16-byte broadcast per coordinate, and the quarters are added through shared
// memory.  About a seventh of the instructions of the shuffle version.
template <int NR>
__global__ void __launch_bounds__(kRotThreads) rotate_q_rows_kernel(
    const void *q, int dtype, int64_t qsb, int64_t qsh, const float *Pi, float mult, int Hq,
    int D, int total_rows, float *q_rot, const int32_t *seq_lens, int B, int chunk_tokens,
    int max_tokens, ScanSetup setup) {
  __shared__ __align__(16) float qs[256][NR];          // [coordinate][row]
  __shared__ float part_s[3][NR][256];
  scan_setup(setup, seq_lens, B, chunk_tokens, max_tokens);
  const int quarter = threadIdx.x >> 7, dq = D / 4, col = threadIdx.x & 127;
  // For head_dim <= 128 a thread's share of Pi (a quarter of one row, at most 8
  // float4) stays in registers for every group of rows this block processes.
  const bool resident = D <= 128;
  float4 held[8];
  if (resident) {
    const float4 *row = reinterpret_cast<const float4 *>(Pi + (int64_t)(col < D ? col : 0) * D + quarter * dq);
#pragma unroll
    for (int j = 0; j < 8; ++j) held[j] = (col < D && j < dq / 4) ? __ldg(row + j) : make_float4(0, 0, 0, 0);
  }
  const int groups = (total_rows + NR - 1) / NR;
  for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const int row0 = grp * NR;
    for (int e = threadIdx.x; e < NR * D; e += kRotThreads) {
      const int r = e / D, d = e - r * D;
      const int row = row0 + r;
      float v = 0.f;
      if (row < total_rows) {
        const int b = row / Hq, h = row - b * Hq;
        v = load_as_float(q, (int64_t)b * qsb + (int64_t)h * qsh + d, dtype);
      }
      qs[d][r] = v;
    }
    __syncthreads();
    if (grp == (int)blockIdx.x) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    for (int c0 = 0; c0 < D; c0 += 128) {                  // same trip count for every thread
      const int c = c0 + col;
      const bool on = c < D;
      float acc[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) acc[r] = 0.f;
      const float4 *row = reinterpret_cast<const float4 *>(Pi + (int64_t)(on ? c : 0) * D + quarter * dq);
      for (int j0 = 0; on && j0 < dq / 4; j0 += 8) {       // 8 loads in flight
        float4 w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          w[j] = resident ? held[j] : (j0 + j < dq / 4 ? __ldg(row + j0 + j) : make_float4(0, 0, 0, 0));
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j0 + j < dq / 4) {
            const int d = quarter * dq + 4 * (j0 + j);
            const float wv[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
#pragma unroll
              for (int r = 0; r < NR; ++r) acc[r] = fmaf(qs[d + k][r], wv[k], acc[r]);
          }
        }
      }
      if (quarter > 0 && on) {
#pragma unroll
        for (int r = 0; r < NR; ++r) part_s[quarter - 1][r][c] = acc[r];
      }
      __syncthreads();
      if (quarter == 0 && on) {
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          const float v = (acc[r] + part_s[0][r][c]) + (part_s[1][r][c] + part_s[2][r][c]);
          if (row0 + r < total_rows) q_rot[(int64_t)(row0 + r) * D + c] = v * mult;
        }
      }
      __syncthreads();
    }
  }
}

// head_dim 128, the shape of the tensor-core path: the same sums in the same
// order as rotate_q_rows_kernel with everything a compile-time constant, the
// next group's query rows requested before the current group's arithmetic
// (their round trip is hidden) and two barriers per group instead of three
// (the staging buffer alternates).
template <int NR>
__global__ void __launch_bounds__(kRotThreads) rotate_q128_kernel(
    const void *q, int dtype, int64_t qsb, int64_t qsh, const float *Pi, float mult, int Hq,
    int total_rows, float *q_rot, const int32_t *seq_lens, int B, int chunk_tokens,
    int max_tokens, ScanSetup setup) {
  __shared__ __align__(16) float qs[2][128][NR];       // [buffer][coordinate][row]
  __shared__ float part_s[3][NR][128];
  scan_setup(setup, seq_lens, B, chunk_tokens, max_tokens);
  const int tid = threadIdx.x, col = tid & 127, quarter = tid >> 7;
  float4 held[8];                                       // this thread's quarter of row `col` of Pi
  {
    const float4 *row = reinterpret_cast<const float4 *>(Pi + col * 128 + quarter * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j) held[j] = __ldg(row + j);
  }
  constexpr int PER = NR * 128 / kRotThreads;           // query elements a thread stages
  static_assert(PER >= 1, "at least four rows per group");
  float pre[PER];
  auto fetch = [&](int grp) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = tid + i * kRotThreads;
      const int row = grp * NR + (e >> 7);
      float v = 0.f;
      if (row < total_rows) {
        const int b = row / Hq, h = row - b * Hq;
        v = load_as_float(q, (int64_t)b * qsb + (int64_t)h * qsh + (e & 127), dtype);
      }
      pre[i] = v;
    }
  };
  const int groups = (total_rows + NR - 1) / NR;
  int grp = blockIdx.x;
  if (grp < groups) fetch(grp);
  for (int buf = 0; grp < groups; grp += gridDim.x, buf ^= 1) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = tid + i * kRotThreads;
      qs[buf][e & 127][e >> 7] = pre[i];
    }
    __syncthreads();
    if (grp == (int)blockIdx.x) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    if (grp + (int)gridDim.x < groups) fetch(grp + gridDim.x);
    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float wv[4] = {held[j].x, held[j].y, held[j].z, held[j].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int d = quarter * 32 + 4 * j + k;
#pragma unroll
        for (int r4 = 0; r4 < NR; r4 += 4) {
          const float4 x = *reinterpret_cast<const float4 *>(&qs[buf][d][r4]);
          acc[r4 + 0] = fmaf(x.x, wv[k], acc[r4 + 0]);
          acc[r4 + 1] = fmaf(x.y, wv[k], acc[r4 + 1]);
          acc[r4 + 2] = fmaf(x.z, wv[k], acc[r4 + 2]);
          acc[r4 + 3] = fmaf(x.w, wv[k], acc[r4 + 3]);
        }
      }
    }
    if (quarter > 0) {
#pragma unroll
      for (int r = 0; r < NR; ++r) part_s[quarter - 1][r][col] = acc[r];
    }
    __syncthreads();
    if (quarter == 0) {
      const int row0 = grp * NR;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const float v = (acc[r] + part_s[0][r][col]) + (part_s[1][r][col] + part_s[2][r][col]);
        if (row0 + r < total_rows) q_rot[(int64_t)(row0 + r) * 128 + col] = v * mult;
      }
    }
  }
}

int launch_rotate_q(const void *q, int dtype, const int64_t *qs, const float *Pi, float scale,
                    int B, int Hq, int D, float *q_rot, const int32_t *seq_lens, int chunk_tokens,
                    int max_tokens, const ScanSetup &setup, cudaStream_t stream) {
  const int rows = B * Hq;
  // (two 512-thread blocks of the head_dim-128 kernel fit an SM, one of the general kernel)
  if (D == 128 && ((uintptr_t)Pi & 15) == 0 && rows >= 8 * 148)
    rotate_q128_kernel<8><<<std::min((rows + 7) / 8, 2 * 148), kRotThreads, 0, stream>>>(
        q, dtype, qs[0], qs[1], Pi, scale, Hq, rows, q_rot, seq_lens, B, chunk_tokens, max_tokens,
        setup);
  else if (D == 128 && ((uintptr_t)Pi & 15) == 0)
    rotate_q128_kernel<4><<<std::min((rows + 3) / 4, 2 * 148), kRotThreads, 0, stream>>>(
        q, dtype, qs[0], qs[1], Pi, scale, Hq, rows, q_rot, seq_lens, B, chunk_tokens, max_tokens,
        setup);
  else if (D % 16 == 0 && D <= 256 && ((uintptr_t)Pi & 15) == 0 && rows >= 8 * 148)
    // many rows: eight per pass halve the passes of the persistent blocks
    rotate_q_rows_kernel<8><<<std::min((rows + 7) / 8, 148), kRotThreads, 0, stream>>>(
        q, dtype, qs[0], qs[1], Pi, scale, Hq, D, rows, q_rot, seq_lens, B, chunk_tokens,
        max_tokens, setup);
  else if (D % 16 == 0 && D <= 256 && ((uintptr_t)Pi & 15) == 0)
    rotate_q_rows_kernel<4><<<std::min((rows + 3) / 4, 148), kRotThreads, 0, stream>>>(
        q, dtype, qs[0], qs[1], Pi, scale, Hq, D, rows, q_rot, seq_lens, B, chunk_tokens,
        max_tokens, setup);
  else if (rows % 4 == 0)
    rotate_q_kernel<4><<<rows / 4, kRotThreads, 0, stream>>>(
        q, dtype, qs[0], qs[1], Pi, scale, Hq, D, rows, q_rot, seq_lens, B, chunk_tokens,
        max_tokens, setup);
  else
    rotate_q_kernel<1><<<rows, kRotThreads, 0, stream>>>(
        q, dtype, qs[0], qs[1], Pi, scale, Hq, D, rows, q_rot, seq_lens, B, chunk_tokens,
        max_tokens, setup);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_decode rotate launch");
}

int launch_merge(const MergeParams &p, int B, cudaStream_t stream) {
  merge_rotate_kernel<<<B * p.Hq, 128, 0, stream>>>(p);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_decode merge launch");
}

}  // namespace wtq
