// Decode attention over UNQUANTISED paged K/V: the matched baseline arm of the
// packed operator, same split-K schedule over the same page table
// (reference: turboquant_kv/packed_attention_triton.py:190-201, the `dense`
// branch of its kernel :51-134).  Pages are (P, Hkv, S, D) in fp16, bf16 or
// fp32; nothing is rotated or looked up, so the kernel is a plain
// flash-decoding scan: a block of four warps takes (split, kv head, sequence),
// walks its share of the sequence in tiles of 32 tokens, stages a tile's keys
// (then its values) in shared memory as fp32 with coalesced loads, computes the
// scores with one thread per (token, head group), keeps the online softmax per
// head in the warp that owns the head, and accumulates the output with one
// thread per coordinate.  A second kernel merges the split states.
#include "wtq_common.cuh"

namespace wtq {

namespace dense {

constexpr int kTile = 32;          // tokens per tile (one per lane)
constexpr int kThreads = 128;
constexpr int kMaxHeads = 8;       // query heads per kv head served by one block
constexpr int kMaxD = 256;

struct Params {
  const void *q, *k_pages, *v_pages;
  void *out;
  int q_dtype, page_dtype;
  int64_t qsb, qsh, osb, osh;                 // element strides of q and out {batch, head}
  int64_t k_page_stride, k_head_stride;       // element strides of the pages
  int64_t v_page_stride, v_head_stride;
  const int32_t *page_table;
  int64_t table_stride;
  const int32_t *seq_lens;
  float scale;
  int B, Hq, Hkv, n_rep, D, S, P, max_pages, num_splits;
  float *part_acc, *part_m, *part_l;          // (B, Hq, splits, D), (B, Hq, splits) x 2
  int32_t *status;
};

// grid (splits, Hkv * ceil(n_rep / 8), B)
__global__ void __launch_bounds__(kThreads) decode_kernel(Params p) {
  extern __shared__ float tile_s[];                    // [kTile][D + 1]
  __shared__ float q_s[kMaxHeads][kMaxD];
  __shared__ float p_s[kMaxHeads][kTile];
  __shared__ float alpha_s[kMaxHeads];
  __shared__ int pid_s[kTile];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int D = p.D, S = p.S, row = D + 1;
  const int groups = (p.n_rep + kMaxHeads - 1) / kMaxHeads;
  const int kvh = blockIdx.y / groups, grp = blockIdx.y - kvh * groups;
  const int split = blockIdx.x, b = blockIdx.z;
  const int h0 = grp * kMaxHeads;
  const int heads = min(kMaxHeads, p.n_rep - h0);
  const int qh0 = kvh * p.n_rep + h0;
  for (int e = tid; e < heads * D; e += kThreads) {
    const int h = e / D, d = e - h * D;
    q_s[h][d] = load_as_float(p.q, (int64_t)b * p.qsb + (int64_t)(qh0 + h) * p.qsh + d, p.q_dtype) *
                p.scale;
  }
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

  // the warp that owns head h (h = warp, warp + 4) keeps its running maximum and sum
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float acc[kMaxHeads][2];                               // coordinates tid and tid + 128
#pragma unroll
  for (int h = 0; h < kMaxHeads; ++h) acc[h][0] = acc[h][1] = 0.f;
  __syncthreads();

  for (int base = t_begin; base < t_end; base += kTile) {
    const int count = min(kTile, t_end - base);
    if (tid < kTile) {
      int pid = -1;
      if (tid < count) {
        const int tok = base + tid;
        pid = p.page_table[(int64_t)b * p.table_stride + tok / S];
        if (pid < 0 || pid >= p.P) {
          pid = -1;
          if (p.status) atomicOr(p.status, WTQ_STATUS_BAD_PAGE);
        }
      }
      pid_s[tid] = pid;
    }
    __syncthreads();
    auto stage = [&](const void *pages, int64_t page_stride, int64_t head_stride) {
      for (int e = tid; e < count * D; e += kThreads) {
        const int t = e / D, d = e - t * D;
        const int pid = pid_s[t];
        float v = 0.f;
        if (pid >= 0) {
          const int slot = (base + t) % S;
          v = load_as_float(pages, (int64_t)pid * page_stride + (int64_t)kvh * head_stride +
                                       (int64_t)slot * D + d, p.page_dtype);
        }
        tile_s[t * row + d] = v;
      }
    };
    stage(p.k_pages, p.k_page_stride, p.k_head_stride);
    __syncthreads();
    // ---- scores and softmax: lane = token, warp = head (and head + 4) ----------
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int h = warp + 4 * j;
      if (h < heads) {
        float s = -INFINITY;
        if (lane < count && pid_s[lane] >= 0) {
          float dot = 0.f;
          for (int d = 0; d < D; ++d) dot = fmaf(q_s[h][d], tile_s[lane * row + d], dot);
          s = dot;
        }
        const float m_new = fmaxf(m_run[j], warp_max(s));
        // exp(-inf - -inf) is defined as 0: nothing seen yet contributes nothing
        const float alpha = m_run[j] == -INFINITY ? 0.f : __expf(m_run[j] - m_new);
        const float pr = (s == -INFINITY || m_new == -INFINITY) ? 0.f : __expf(s - m_new);
        l_run[j] = alpha * l_run[j] + warp_sum(pr);
        m_run[j] = m_new;
        p_s[h][lane] = pr;
        if (lane == 0) alpha_s[h] = alpha;
      }
    }
    __syncthreads();
    stage(p.v_pages, p.v_page_stride, p.v_head_stride);
    __syncthreads();
    // ---- values: thread = output coordinate -------------------------------------
#pragma unroll
    for (int slot = 0; slot < 2; ++slot) {
      const int d = tid + slot * kThreads;
      if (d < D) {
#pragma unroll
        for (int h = 0; h < kMaxHeads; ++h) {
          if (h < heads) {
            float a = alpha_s[h] * acc[h][slot];
            for (int t = 0; t < count; ++t) a = fmaf(p_s[h][t], tile_s[t * row + d], a);
            acc[h][slot] = a;
          }
        }
      }
    }
    __syncthreads();
  }
  // partial state of this split; an empty split writes (m = -inf, l = 0, acc = 0)
#pragma unroll
  for (int h = 0; h < kMaxHeads; ++h) {
    if (h < heads) {
      const int64_t prow = ((int64_t)b * p.Hq + qh0 + h) * p.num_splits + split;
      if (tid < D) p.part_acc[prow * D + tid] = acc[h][0];
      if (tid + kThreads < D) p.part_acc[prow * D + tid + kThreads] = acc[h][1];
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int h = warp + 4 * j;
    if (h < heads && lane == 0) {
      const int64_t prow = ((int64_t)b * p.Hq + qh0 + h) * p.num_splits + split;
      p.part_m[prow] = m_run[j];
      p.part_l[prow] = l_run[j];
    }
  }
}

// out[b, h, :] = sum_s w_s acc_s / sum_s w_s l_s, w_s = exp(m_s - max m); rows that
// saw no key are exact zeros.  One block per (sequence, head).
__global__ void __launch_bounds__(kThreads) merge_kernel(Params p) {
  __shared__ float w_s[1024];
  __shared__ float inv_s;
  const int rowi = blockIdx.x, b = rowi / p.Hq, h = rowi - b * p.Hq;
  const int tid = threadIdx.x;
  const int64_t base = (int64_t)rowi * p.num_splits;
  if (tid == 0) {
    float gmax = -INFINITY;
    for (int s = 0; s < p.num_splits; ++s) gmax = fmaxf(gmax, p.part_m[base + s]);
    float denom = 0.f;
    for (int s = 0; s < p.num_splits; ++s) {
      const float m = p.part_m[base + s];
      const float w = m == -INFINITY ? 0.f : __expf(m - gmax);
      w_s[s] = w;
      denom += w * p.part_l[base + s];
    }
    inv_s = denom > 0.f ? 1.f / fmaxf(denom, 1e-30f) : 0.f;
  }
  __syncthreads();
  for (int d = tid; d < p.D; d += kThreads) {
    float a = 0.f;
    for (int s = 0; s < p.num_splits; ++s) a = fmaf(w_s[s], p.part_acc[(base + s) * p.D + d], a);
    store_from_float(p.out, (int64_t)b * p.osb + (int64_t)h * p.osh + d, a * inv_s, p.q_dtype);
  }
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace dense
}  // namespace wtq

using namespace wtq;

extern "C" size_t wtq_dense_workspace_bytes(int B, int Hq, int D, int num_splits) {
  if (B < 1 || Hq < 1 || D < 1 || num_splits < 1) return 256;
  const size_t rows = (size_t)B * Hq * num_splits;
  return dense::round_up(rows * D * sizeof(float), 256) + 2 * dense::round_up(rows * sizeof(float), 256);
}

extern "C" int wtq_dense_decode(const void *q, int q_dtype, const int64_t q_strides[2], void *out,
                                const int64_t out_strides[2], const void *k_pages,
                                const void *v_pages, int page_dtype, const int64_t k_strides[2],
                                const int64_t v_strides[2], const int32_t *page_table,
                                int64_t table_stride, const int32_t *seq_lens, float scale, int B,
                                int Hq, int Hkv, int D, int S, int P, int max_pages,
                                int num_splits, void *workspace, size_t workspace_bytes,
                                int32_t *status, void *stream) {
  if (B < 0 || Hq < 1 || Hkv < 1 || S < 1 || P < 1 || max_pages < 1 || Hq % Hkv)
    return fail(WTQ_ERR_ARG, "wtq_dense_decode: bad sizes");
  if (D < 1 || D > dense::kMaxD) return fail(WTQ_ERR_ARG, "wtq_dense_decode: need 1 <= head_dim <= 256");
  if (q_dtype < WTQ_F32 || q_dtype > WTQ_BF16 || page_dtype < WTQ_F32 || page_dtype > WTQ_BF16)
    return fail(WTQ_ERR_ARG, "wtq_dense_decode: bad dtype");
  if (num_splits < 1 || num_splits > 1024)
    return fail(WTQ_ERR_ARG, "wtq_dense_decode: need 1 <= num_splits <= 1024");
  if (B == 0) return WTQ_OK;
  if (!q || !out || !k_pages || !v_pages || !page_table || !seq_lens || !workspace || !q_strides ||
      !out_strides || !k_strides || !v_strides)
    return fail(WTQ_ERR_ARG, "wtq_dense_decode: null argument");
  const size_t need = wtq_dense_workspace_bytes(B, Hq, D, num_splits);
  if (workspace_bytes < need)
    return fail(WTQ_ERR_WORKSPACE, "wtq_dense_decode: workspace %zu < %zu bytes", workspace_bytes, need);
  dense::Params p;
  p.q = q; p.k_pages = k_pages; p.v_pages = v_pages; p.out = out;
  p.q_dtype = q_dtype; p.page_dtype = page_dtype;
  p.qsb = q_strides[0]; p.qsh = q_strides[1]; p.osb = out_strides[0]; p.osh = out_strides[1];
  p.k_page_stride = k_strides[0]; p.k_head_stride = k_strides[1];
  p.v_page_stride = v_strides[0]; p.v_head_stride = v_strides[1];
  p.page_table = page_table; p.table_stride = table_stride; p.seq_lens = seq_lens; p.scale = scale;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.n_rep = Hq / Hkv; p.D = D; p.S = S; p.P = P;
  p.max_pages = max_pages; p.num_splits = num_splits; p.status = status;
  const size_t rows = (size_t)B * Hq * num_splits;
  char *ws = (char *)workspace;
  p.part_acc = (float *)ws;
  ws += dense::round_up(rows * D * sizeof(float), 256);
  p.part_m = (float *)ws;
  ws += dense::round_up(rows * sizeof(float), 256);
  p.part_l = (float *)ws;
  const int groups = (p.n_rep + dense::kMaxHeads - 1) / dense::kMaxHeads;
  const dim3 grid((unsigned)num_splits, (unsigned)(Hkv * groups), (unsigned)B);
  const size_t smem = (size_t)dense::kTile * (D + 1) * sizeof(float);
  dense::decode_kernel<<<grid, dense::kThreads, smem, (cudaStream_t)stream>>>(p);
  if (int rc = check_cuda(cudaGetLastError(), "wtq_dense_decode launch")) return rc;
  dense::merge_kernel<<<(unsigned)(B * Hq), dense::kThreads, 0, (cudaStream_t)stream>>>(p);
  note_launches(2);
  return check_cuda(cudaGetLastError(), "wtq_dense_decode merge launch");
}
