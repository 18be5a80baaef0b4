// Fused dequantisation of packed rows: unpack -> centroid gather -> rotation
// by Pi -> norm rescale -> one store in the output dtype.  Serves the prefill
// fallback and the contiguous legacy cache, which hand over a
// (planes, MAXLEN, NB) buffer viewed through its first L positions
// (turboquant_kv/kernel.py:47-53).
//
// A block takes kRows rows.  Their centroid values sit in shared memory; thread
// c owns output column c and walks Pi[:, c] once for all kRows rows, so every
// Pi element fetched (coalesced across the block) feeds kRows FMAs.
#include "wtq_common.cuh"

namespace wtq {

constexpr int kRows = 16;

struct DequantParams {
  const uint8_t *packed;
  const __half *norms;
  const float *centroids, *Pi;
  void *out;
  int out_dtype, bw, D, nb;
  int64_t N, L, MAXLEN;
};

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

}  // namespace wtq

using namespace wtq;

extern "C" int wtq_dequant(const uint8_t *packed, const void *norms_f16, const float *centroids,
                           const float *Pi, void *out, int out_dtype, int bw, int D, int64_t N,
                           int64_t L, int64_t MAXLEN, void *stream) {
  if (N < 0 || D < 1 || D > 256) return fail(WTQ_ERR_ARG, "wtq_dequant: need 1 <= D <= 256");
  if (!width_supported(bw) || (D * bw) % 8)
    return fail(WTQ_ERR_ARG, "wtq_dequant: bit width %d unsupported for D=%d", bw, D);
  if (out_dtype < WTQ_F32 || out_dtype > WTQ_BF16)
    return fail(WTQ_ERR_ARG, "wtq_dequant: bad output dtype");
  if (N == 0) return WTQ_OK;
  if (L < 1 || MAXLEN < L) return fail(WTQ_ERR_ARG, "wtq_dequant: need 1 <= L <= MAXLEN");
  if (!packed || !norms_f16 || !centroids || !Pi || !out)
    return fail(WTQ_ERR_ARG, "wtq_dequant: null buffer");
  DequantParams p;
  p.packed = packed; p.norms = (const __half *)norms_f16; p.centroids = centroids; p.Pi = Pi;
  p.out = out; p.out_dtype = out_dtype; p.bw = bw; p.D = D; p.nb = D * bw / 8;
  p.N = N; p.L = L; p.MAXLEN = MAXLEN;
  int64_t blocks = (N + kRows - 1) / kRows;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const int threads = D <= 32 ? 32 : D <= 64 ? 64 : 128;
  dequant_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(p);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_dequant launch");
}
