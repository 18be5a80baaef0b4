// Fused append: rotate -> norm -> Lloyd-Max quantize -> bit-pack -> page scatter.
//
// One thread block owns one vector at a time and one rotation matrix for its
// whole life (grid.y picks the K or V side), so Pi is staged in shared memory
// once per block and every vector after that costs D chained FMAs per thread.
//
// Arithmetic contract (bit-exactness with the reference's CPU PyTorch path,
// turboquant_kv/cache.py:108-115).  Every operation below is an explicit
// round-to-nearest intrinsic so no compiler flag can fuse or reorder it:
//   norm     : 8 interleaved partial sums (partial j takes d = j mod 8), each
//              step round(x*x) then round(acc + .), partials added left to
//              right, IEEE sqrt, clamp at 1e-10;
//   x / norm : IEEE division;
//   rotation : WTQ_ORDER_SEQUENTIAL    one FMA chain per output, d ascending;
//              WTQ_ORDER_INTERLEAVED16 16 chains (chain j takes d = j mod 16),
//              ((c[j]+c[j+4])+c[j+8])+c[j+12] for j = 0..3, then
//              (s0+s1)+(s2+s3);
//   bucket   : number of boundaries strictly below y (bucketize, right=False);
//   norm out : fp16 round-to-nearest-even for pages, fp32 for wtq_quantize.
#include "wtq_common.cuh"

namespace wtq {

struct QuantSideDev {
  const float *Pi;
  const float *bounds;
  int bw, nb, nbounds;
  bool vec4;      // Pi is 16-byte aligned and D a multiple of 4: rows can be read as float4
};

struct QuantScratch {
  float x[256];
  float lane[8];
  float norm;
  float bounds[255];
  uint8_t idx[256];
};

template <bool STAGE>
__device__ __forceinline__ float pi_at(const float *pi_s, const float *pi_g, int D, int c, int d) {
  return STAGE ? pi_s[c * (D + 1) + d] : pi_g[(int64_t)c * D + d];
}

// All threads of the block call this.  On return scratch.idx holds the D codes
// and scratch.norm the clamped fp32 norm; the caller synchronises before use.
template <bool STAGE>
__device__ void quantize_vector(QuantScratch &s, const float *pi_s, const QuantSideDev &q, int D,
                                int order) {
  const int c = threadIdx.x;
  if (c < 8) {
    float acc = 0.0f;
    for (int d = c; d < D; d += 8) acc = __fadd_rn(acc, __fmul_rn(s.x[d], s.x[d]));
    s.lane[c] = acc;
  }
  __syncthreads();
  if (c == 0) {
    float t = s.lane[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) t = __fadd_rn(t, s.lane[j]);
    s.norm = fmaxf(__fsqrt_rn(t), 1e-10f);
  }
  __syncthreads();
  if (c < D) s.x[c] = __fdiv_rn(s.x[c], s.norm);
  __syncthreads();
  if (c < D) {
    float y;
    if (!STAGE && q.vec4) {
      // Few vectors per block: staging all of Pi would cost more than it saves.
      // The thread walks its own row of Pi with 16-byte loads, eight in flight;
      // the summation order is the same as below.
      const float4 *row = reinterpret_cast<const float4 *>(q.Pi + (int64_t)c * D);
      if (order == WTQ_ORDER_INTERLEAVED16) {
        float ch[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) ch[j] = 0.0f;
        for (int d0 = 0; d0 < D; d0 += 16) {
          float4 w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) w[j] = d0 + 4 * j < D ? __ldg(row + d0 / 4 + j) : make_float4(0, 0, 0, 0);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (d0 + 4 * j < D) {
              ch[4 * j + 0] = __fmaf_rn(s.x[d0 + 4 * j + 0], w[j].x, ch[4 * j + 0]);
              ch[4 * j + 1] = __fmaf_rn(s.x[d0 + 4 * j + 1], w[j].y, ch[4 * j + 1]);
              ch[4 * j + 2] = __fmaf_rn(s.x[d0 + 4 * j + 2], w[j].z, ch[4 * j + 2]);
              ch[4 * j + 3] = __fmaf_rn(s.x[d0 + 4 * j + 3], w[j].w, ch[4 * j + 3]);
            }
          }
        }
        float part[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          part[j] = __fadd_rn(__fadd_rn(__fadd_rn(ch[j], ch[j + 4]), ch[j + 8]), ch[j + 12]);
        y = __fadd_rn(__fadd_rn(part[0], part[1]), __fadd_rn(part[2], part[3]));
      } else {
        float acc = 0.0f;
        for (int j0 = 0; j0 < D / 4; j0 += 8) {
          float4 w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) w[j] = j0 + j < D / 4 ? __ldg(row + j0 + j) : make_float4(0, 0, 0, 0);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (j0 + j < D / 4) {
              const int d = 4 * (j0 + j);
              acc = __fmaf_rn(s.x[d + 0], w[j].x, acc);
              acc = __fmaf_rn(s.x[d + 1], w[j].y, acc);
              acc = __fmaf_rn(s.x[d + 2], w[j].z, acc);
              acc = __fmaf_rn(s.x[d + 3], w[j].w, acc);
            }
          }
        }
        y = acc;
      }
    } else if (order == WTQ_ORDER_INTERLEAVED16) {
      float ch[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) ch[j] = 0.0f;
      for (int d0 = 0; d0 < D; d0 += 16) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (d0 + j < D)
            ch[j] = __fmaf_rn(s.x[d0 + j], pi_at<STAGE>(pi_s, q.Pi, D, c, d0 + j), ch[j]);
      }
      float part[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        part[j] = __fadd_rn(__fadd_rn(__fadd_rn(ch[j], ch[j + 4]), ch[j + 8]), ch[j + 12]);
      y = __fadd_rn(__fadd_rn(part[0], part[1]), __fadd_rn(part[2], part[3]));
    } else {
      float acc = 0.0f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) acc = __fmaf_rn(s.x[d], pi_at<STAGE>(pi_s, q.Pi, D, c, d), acc);
      y = acc;
    }
    int lo = 0, hi = q.nbounds;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (s.bounds[mid] < y) lo = mid + 1;
      else hi = mid;
    }
    s.idx[c] = (uint8_t)lo;
  }
}

__device__ __forceinline__ uint8_t packed_byte(const uint8_t *idx, int j, int bw) {
  if (bw == 8) return idx[j];
  if (bw == 4) return (uint8_t)(idx[2 * j] | (idx[2 * j + 1] << 4));
  unsigned out = 0;
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    const int bit = 8 * j + b;
    const int i = bit / bw;
    out |= ((idx[i] >> (bit - i * bw)) & 1u) << b;
  }
  return (uint8_t)out;
}

template <bool STAGE>
__device__ void stage_side(float *pi_s, QuantScratch &s, const QuantSideDev &q, int D) {
  if (STAGE) {
    for (int e = threadIdx.x; e < D * D; e += blockDim.x) {
      const int r = e / D, col = e - r * D;
      pi_s[r * (D + 1) + col] = q.Pi[e];
    }
  }
  for (int e = threadIdx.x; e < q.nbounds; e += blockDim.x) s.bounds[e] = q.bounds[e];
  __syncthreads();
}

struct QuantizeParams {
  const void *x;
  int dtype;
  int64_t rows, row_stride;
  int D, order;
  QuantSideDev side;
  uint8_t *idx, *packed;
  float *norms;
};

template <bool STAGE>
__global__ void quantize_kernel(QuantizeParams p) {
  extern __shared__ float pi_s[];
  __shared__ QuantScratch s;
  stage_side<STAGE>(pi_s, s, p.side, p.D);
  const int c = threadIdx.x;
  for (int64_t r = blockIdx.x; r < p.rows; r += gridDim.x) {
    if (c < p.D) s.x[c] = load_as_float(p.x, r * p.row_stride + c, p.dtype);
    __syncthreads();
    quantize_vector<STAGE>(s, pi_s, p.side, p.D, p.order);
    __syncthreads();
    if (p.idx && c < p.D) p.idx[r * p.D + c] = s.idx[c];
    if (p.packed && c < p.side.nb) p.packed[r * p.side.nb + c] = packed_byte(s.idx, c, p.side.bw);
    if (p.norms && c == 0) p.norms[r] = s.norm;
    __syncthreads();
  }
}

struct AppendSideDev {
  QuantSideDev q;
  const void *src;
  int64_t sb, sh, st;  // element strides: batch, head, token
  uint8_t *pages;
  __half *norms;
  int64_t page_stride, head_stride, norm_page_stride, norm_head_stride;
};

struct AppendParams {
  AppendSideDev side[2];
  const int32_t *page_table;
  int64_t table_stride;
  const int32_t *seq_lens;
  int dtype, B, Hkv, n, D, S, P, max_pages, order;
  int32_t *status;
};

template <bool STAGE>
__global__ void append_kernel(AppendParams p) {
  extern __shared__ float pi_s[];
  __shared__ QuantScratch s;
  __shared__ int64_t dest[2];
  const AppendSideDev &a = p.side[blockIdx.y];
  stage_side<STAGE>(pi_s, s, a.q, p.D);
  const int c = threadIdx.x;
  const int64_t vectors = (int64_t)p.B * p.Hkv * p.n;
  for (int64_t vec = blockIdx.x; vec < vectors; vec += gridDim.x) {
    const int i = (int)(vec % p.n);
    const int h = (int)((vec / p.n) % p.Hkv);
    const int b = (int)(vec / ((int64_t)p.n * p.Hkv));
    if (c == 0) {
      // Where the token goes; -1 marks a position or page the table does not
      // cover, which is reported through `status` and not written.
      const int pos = p.seq_lens[b] - p.n + i;
      int64_t code_off = -1, norm_off = -1;
      const int slot_page = pos >= 0 ? pos / p.S : -1;
      if (pos < 0 || slot_page >= p.max_pages) {
        if (p.status) atomicOr(p.status, WTQ_STATUS_BAD_POSITION);
      } else {
        const int pid = p.page_table[(int64_t)b * p.table_stride + slot_page];
        if (pid < 0 || pid >= p.P) {
          if (p.status) atomicOr(p.status, WTQ_STATUS_BAD_PAGE);
        } else {
          const int slot = pos - slot_page * p.S;
          code_off = (int64_t)pid * a.page_stride + (int64_t)h * a.head_stride +
                     (int64_t)slot * a.q.nb;
          norm_off = (int64_t)pid * a.norm_page_stride + (int64_t)h * a.norm_head_stride + slot;
        }
      }
      dest[0] = code_off;
      dest[1] = norm_off;
    }
    if (c < p.D)
      s.x[c] = load_as_float(a.src, (int64_t)b * a.sb + (int64_t)h * a.sh + (int64_t)i * a.st + c,
                             p.dtype);
    __syncthreads();
    quantize_vector<STAGE>(s, pi_s, a.q, p.D, p.order);
    __syncthreads();
    if (dest[0] >= 0) {
      if (c < a.q.nb) a.pages[dest[0] + c] = packed_byte(s.idx, c, a.q.bw);
      if (c == 0) a.norms[dest[1]] = __float2half_rn(s.norm);
    }
    __syncthreads();
  }
}

// A decode step's append at head_dim 128: NV vectors per block, so that the one
// pass a thread makes over its row of Pi (32 16-byte loads) serves NV FMA
// chains.  A block per vector makes the step L2-bound (64 KB of Pi per
// vector); sharing the pass divides that traffic by NV.  Same arithmetic, in
// the same order, as quantize_vector with WTQ_ORDER_SEQUENTIAL.
template <int NV>
__global__ void __launch_bounds__(128) append_multi_kernel(AppendParams p) {
  __shared__ float x_s[NV][128];
  __shared__ float lane_s[NV][8];
  __shared__ float norm_s[NV];
  __shared__ float bounds_s[255];
  __shared__ uint8_t idx_s[NV][128];
  __shared__ int64_t dest_s[NV][2];
  const AppendSideDev &a = p.side[blockIdx.y];
  const int c = threadIdx.x;
  for (int e = c; e < a.q.nbounds; e += 128) bounds_s[e] = a.q.bounds[e];
  const int64_t vectors = (int64_t)p.B * p.Hkv * p.n;
  const float4 *row = reinterpret_cast<const float4 *>(a.q.Pi + (int64_t)c * 128);
  for (int64_t v0 = (int64_t)blockIdx.x * NV; v0 < vectors; v0 += (int64_t)gridDim.x * NV) {
    // the first half of the thread's row of Pi is requested before anything
    // else: its trip to L2 overlaps the loads and barriers of the normalisation
    float4 wa[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) wa[k] = __ldg(row + k);
    if (c < NV) {
      // Where the token goes; -1 marks a position or page the table does not
      // cover (reported through `status`, not written) or a vector past the end.
      const int64_t vec = v0 + c;
      int64_t code_off = -1, norm_off = -1;
      if (vec < vectors) {
        const int i = (int)(vec % p.n);
        const int h = (int)((vec / p.n) % p.Hkv);
        const int b = (int)(vec / ((int64_t)p.n * p.Hkv));
        const int pos = p.seq_lens[b] - p.n + i;
        const int slot_page = pos >= 0 ? pos / p.S : -1;
        if (pos < 0 || slot_page >= p.max_pages) {
          if (p.status) atomicOr(p.status, WTQ_STATUS_BAD_POSITION);
        } else {
          const int pid = p.page_table[(int64_t)b * p.table_stride + slot_page];
          if (pid < 0 || pid >= p.P) {
            if (p.status) atomicOr(p.status, WTQ_STATUS_BAD_PAGE);
          } else {
            const int slot = pos - slot_page * p.S;
            code_off = (int64_t)pid * a.page_stride + (int64_t)h * a.head_stride +
                       (int64_t)slot * a.q.nb;
            norm_off = (int64_t)pid * a.norm_page_stride + (int64_t)h * a.norm_head_stride + slot;
          }
        }
      }
      dest_s[c][0] = code_off;
      dest_s[c][1] = norm_off;
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int64_t vec = v0 + j;
      float v = 0.0f;
      if (vec < vectors) {
        const int i = (int)(vec % p.n);
        const int h = (int)((vec / p.n) % p.Hkv);
        const int b = (int)(vec / ((int64_t)p.n * p.Hkv));
        v = load_as_float(a.src, (int64_t)b * a.sb + (int64_t)h * a.sh + (int64_t)i * a.st + c,
                          p.dtype);
      }
      x_s[j][c] = v;
    }
    __syncthreads();
    if (c < 8 * NV) {
      const int j = c >> 3, l = c & 7;
      float acc = 0.0f;
      for (int d = l; d < 128; d += 8) acc = __fadd_rn(acc, __fmul_rn(x_s[j][d], x_s[j][d]));
      lane_s[j][l] = acc;
    }
    __syncthreads();
    if (c < NV) {
      float t = lane_s[c][0];
#pragma unroll
      for (int l = 1; l < 8; ++l) t = __fadd_rn(t, lane_s[c][l]);
      norm_s[c] = fmaxf(__fsqrt_rn(t), 1e-10f);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NV; ++j) x_s[j][c] = __fdiv_rn(x_s[j][c], norm_s[j]);
    __syncthreads();
    float acc[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) acc[j] = 0.0f;
    float4 wb[16];                                         // second half, while the first is used
#pragma unroll
    for (int k = 0; k < 16; ++k) wb[k] = __ldg(row + 16 + k);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const float4 w = half ? wb[k] : wa[k];
        const int d = 64 * half + 4 * k;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          acc[j] = __fmaf_rn(x_s[j][d + 0], w.x, acc[j]);
          acc[j] = __fmaf_rn(x_s[j][d + 1], w.y, acc[j]);
          acc[j] = __fmaf_rn(x_s[j][d + 2], w.z, acc[j]);
          acc[j] = __fmaf_rn(x_s[j][d + 3], w.w, acc[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      int lo = 0, hi = a.q.nbounds;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (bounds_s[mid] < acc[j]) lo = mid + 1;
        else hi = mid;
      }
      idx_s[j][c] = (uint8_t)lo;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (dest_s[j][0] >= 0) {
        if (c < a.q.nb) a.pages[dest_s[j][0] + c] = packed_byte(idx_s[j], c, a.q.bw);
        if (c == 0) a.norms[dest_s[j][1]] = __float2half_rn(norm_s[j]);
      }
    }
    __syncthreads();
  }
}

static int block_threads(int D) { return ((D + 31) / 32) * 32; }

template <typename K, typename P>
static int launch_staged(K staged, K direct, P &params, int D, int64_t work, int sides,
                         cudaStream_t stream, const char *what) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // Staging Pi in shared memory (64 KB per block at head_dim 128) pays off when
  // a block quantizes many vectors (bulk fills); a decode step appends a few
  // hundred vectors in all, so there every vector gets its own block and the
  // threads read their rows of Pi directly.
  int64_t blocks = work < (int64_t)sms * 3 ? work : (int64_t)sms * 3;
  if (blocks < 1) blocks = 1;
  const bool stage = D <= 128 && work > 4 * blocks;
  const size_t smem = stage ? (size_t)D * (D + 1) * sizeof(float) : 0;
  if (stage && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(staged, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return check_cuda(e, what);
  }
  dim3 grid((unsigned)blocks, (unsigned)sides);
  if (stage) staged<<<grid, block_threads(D), smem, stream>>>(params);
  else direct<<<grid, block_threads(D), 0, stream>>>(params);
  note_launches(1);
  return check_cuda(cudaGetLastError(), what);
}

}  // namespace wtq

using namespace wtq;

extern "C" int wtq_quantize(const void *x, int dtype, int64_t rows, int64_t row_stride, int D,
                            const float *Pi, const float *bounds, int bw, int order,
                            uint8_t *idx, uint8_t *packed, float *norms, void *stream) {
  if (rows < 0 || D < 1 || D > 256) return fail(WTQ_ERR_ARG, "wtq_quantize: need 1 <= D <= 256");
  if (!width_supported(bw) || (D * bw) % 8)
    return fail(WTQ_ERR_ARG, "wtq_quantize: bit width %d unsupported for D=%d", bw, D);
  if (dtype < WTQ_F32 || dtype > WTQ_BF16) return fail(WTQ_ERR_ARG, "wtq_quantize: bad dtype");
  if (rows == 0) return WTQ_OK;
  if (!x || !Pi || !bounds) return fail(WTQ_ERR_ARG, "wtq_quantize: null input");
  QuantizeParams p;
  p.x = x; p.dtype = dtype; p.rows = rows; p.row_stride = row_stride; p.D = D;
  p.order = resolve_order(order, rows);
  p.side = {Pi, bounds, bw, D * bw / 8, (1 << bw) - 1, D % 4 == 0 && ((uintptr_t)Pi & 15) == 0};
  p.idx = idx; p.packed = packed; p.norms = norms;
  return launch_staged(quantize_kernel<true>, quantize_kernel<false>, p, D, rows, 1,
                       (cudaStream_t)stream, "wtq_quantize launch");
}

extern "C" int wtq_append(const void *k, const void *v, int dtype, const int64_t k_strides[3],
                          const int64_t v_strides[3], const wtq_side_t *k_side,
                          const wtq_side_t *v_side, const int32_t *page_table,
                          int64_t table_stride, const int32_t *seq_lens, int B, int Hkv, int n,
                          int D, int S, int P, int max_pages, int order, int32_t *status,
                          void *stream) {
  if (B < 0 || Hkv < 1 || n < 0 || S < 1 || P < 1 || max_pages < 1)
    return fail(WTQ_ERR_ARG, "wtq_append: bad sizes");
  if (D < 1 || D > 256) return fail(WTQ_ERR_ARG, "wtq_append: need 1 <= D <= 256");
  if (dtype < WTQ_F32 || dtype > WTQ_BF16) return fail(WTQ_ERR_ARG, "wtq_append: bad dtype");
  if (!k_side || !v_side || !k_strides || !v_strides)
    return fail(WTQ_ERR_ARG, "wtq_append: null descriptor");
  const wtq_side_t *sides[2] = {k_side, v_side};
  const void *src[2] = {k, v};
  const int64_t *strides[2] = {k_strides, v_strides};
  AppendParams p;
  for (int s = 0; s < 2; ++s) {
    const wtq_side_t &w = *sides[s];
    if (!width_supported(w.bw) || (D * w.bw) % 8)
      return fail(WTQ_ERR_ARG, "wtq_append: bit width %d unsupported for D=%d", w.bw, D);
    if (!w.pages || !w.norms || !w.Pi || !w.bounds)
      return fail(WTQ_ERR_ARG, "wtq_append: null pages, norms, Pi or bounds");
    AppendSideDev &a = p.side[s];
    a.q = {w.Pi, w.bounds, w.bw, D * w.bw / 8, (1 << w.bw) - 1,
           D % 4 == 0 && ((uintptr_t)w.Pi & 15) == 0};
    a.src = src[s];
    a.sb = strides[s][0]; a.sh = strides[s][1]; a.st = strides[s][2];
    a.pages = w.pages; a.norms = (__half *)w.norms;
    a.page_stride = w.page_stride; a.head_stride = w.head_stride;
    a.norm_page_stride = w.norm_page_stride; a.norm_head_stride = w.norm_head_stride;
  }
  const int64_t vectors = (int64_t)B * Hkv * n;
  if (vectors == 0) return WTQ_OK;
  if (!k || !v || !page_table || !seq_lens) return fail(WTQ_ERR_ARG, "wtq_append: null input");
  p.page_table = page_table; p.table_stride = table_stride; p.seq_lens = seq_lens;
  p.dtype = dtype; p.B = B; p.Hkv = Hkv; p.n = n; p.D = D; p.S = S; p.P = P;
  p.max_pages = max_pages; p.order = resolve_order(order, vectors); p.status = status;
  // decode-step sizes at head_dim 128: four vectors share a block's pass over Pi
  constexpr int kMultiVectors = 4;
  if (D == 128 && p.order == WTQ_ORDER_SEQUENTIAL && vectors >= 2 * kMultiVectors &&
      vectors <= 4 * 3 * 148 && p.side[0].q.vec4 && p.side[1].q.vec4) {
    dim3 grid((unsigned)((vectors + kMultiVectors - 1) / kMultiVectors), 2);
    append_multi_kernel<kMultiVectors><<<grid, 128, 0, (cudaStream_t)stream>>>(p);
    note_launches(1);
    return check_cuda(cudaGetLastError(), "wtq_append launch");
  }
  return launch_staged(append_kernel<true>, append_kernel<false>, p, D, vectors, 2,
                       (cudaStream_t)stream, "wtq_append launch");
}
