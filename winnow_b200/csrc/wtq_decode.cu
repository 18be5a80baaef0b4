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
#include "wtq_decode.cuh"

namespace wtq {

// q_rot[row][c] = mult * sum_d q[row][d] Pi[c][d] for the `rows` query rows that
// start at row blockIdx.x * NR.  A warp takes output coordinates c = warp,
// warp + 16, ...; its lanes stride over d, so every Pi row is read once per
// block, coalesced, for all NR query rows, and the NR partial sums are reduced
// by shuffles.  Eight Pi rows are in flight per warp to cover L2 latency.
constexpr int kRotThreads = 512;
template <int NR>
__global__ void __launch_bounds__(kRotThreads) rotate_q_kernel(
    const void *q, int dtype, int64_t qsb, int64_t qsh, const float *Pi, float mult, int Hq,
    int D, int total_rows, float *q_rot) {
  __shared__ float qs[NR][256];
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
  for (int c0 = warp; c0 < D; c0 += kWarps * kBatch) {
    float part[kBatch][NR];
#pragma unroll
    for (int i = 0; i < kBatch; ++i)
#pragma unroll
      for (int r = 0; r < NR; ++r) part[i][r] = 0.f;
#pragma unroll 4
    for (int d = lane; d < D; d += 32) {
      float w[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        const int c = c0 + i * kWarps;
        w[i] = c < D ? __ldg(Pi + (int64_t)c * D + d) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i)
#pragma unroll
        for (int r = 0; r < NR; ++r) part[i][r] = fmaf(qs[r][d], w[i], part[i][r]);
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int c = c0 + i * kWarps;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const float v = warp_sum(part[i][r]);
        if (lane == 0 && c < D && row0 + r < total_rows)
          q_rot[(int64_t)(row0 + r) * D + c] = v * mult;
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

int launch_rotate_q(const void *q, int dtype, const int64_t *qs, const float *Pi, float scale,
                    int B, int Hq, int D, float *q_rot, cudaStream_t stream) {
  const int rows = B * Hq;
  if (rows % 4 == 0)
    rotate_q_kernel<4><<<rows / 4, kRotThreads, 0, stream>>>(q, dtype, qs[0], qs[1], Pi, scale, Hq,
                                                            D, rows, q_rot);
  else
    rotate_q_kernel<1><<<rows, kRotThreads, 0, stream>>>(q, dtype, qs[0], qs[1], Pi, scale, Hq, D,
                                                        rows, q_rot);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_decode rotate launch");
}

int launch_merge(const MergeParams &p, int B, cudaStream_t stream) {
  merge_rotate_kernel<<<B * p.Hq, 128, 0, stream>>>(p);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_decode merge launch");
}

}  // namespace wtq
