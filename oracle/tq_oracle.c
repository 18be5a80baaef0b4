/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement, in plain C, of the byte/integer
 * half of the TurboQuant packed-KV path of lgoyal6/winnow.  Nothing in the
 * product package may link, load or call this file; it exists so that the
 * tests, the smoke check and the benchmark's CPU-baseline leg can check the
 * CUDA kernels against an independent implementation.
 *
 * What is restated (reference file:line):
 *   tq_pack / tq_unpack     turboquant_kv/packing.py:38-89  (LSB-first bit
 *                           stream; index i occupies stream bits
 *                           [i*bw,(i+1)*bw), byte j bit b = stream bit 8j+b)
 *   tq_quantize             turboquant_kv/cache.py:108-115  (fp32 norm,
 *                           clamp 1e-10, fp32 division, rotation by Pi^T,
 *                           bucketize(right=False) -> uint8)
 *   tq_dequantize           turboquant_kv/cache.py:117-131 (centroid gather,
 *                           rotation by Pi, norm rescale), fp32 out
 *
 * Floating-point order.  The reference is PyTorch on CPU, so its bits depend
 * on the summation order of torch's norm kernel and of the BLAS it calls.
 * Measured against the reference in the build container (PyTorch 2.11 CPU,
 * MKL 2024.2, AVX-512), with zero mismatches over 1e5 vectors:
 *   norm      : 8 interleaved fp32 partial sums (lane j takes d = j mod 8),
 *               each step round(x*x) then round(acc + .) (no FMA); lanes are
 *               then added left to right; sqrtf.
 *   rotation  : rows >= 6 in the call  -> one fp32 FMA chain per output,
 *                                         d = 0..D-1 in order;
 *               2 <= rows <= 5         -> 16 interleaved FMA chains (chain j
 *                                         takes d = j mod 16); chains
 *                                         j, j+4, j+8, j+12 are added left to
 *                                         right for j = 0..3, then
 *                                         (s0+s1)+(s2+s3);
 *               rows == 1              -> the BLAS takes a matrix-vector path
 *                                         whose order was not identified;
 *                                         the sequential chain is used.
 * `order` selects the rotation order explicitly: 0 sequential, 1 interleaved.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off; every fused
 * multiply-add below is an explicit fmaf so the compiler may not invent or
 * remove one).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define TQ_ORDER_SEQUENTIAL 0
#define TQ_ORDER_INTERLEAVED16 1

int tq_rotation_order_for_rows(int64_t rows) {
  return (rows >= 2 && rows <= 5) ? TQ_ORDER_INTERLEAVED16 : TQ_ORDER_SEQUENTIAL;
}

static float tq_norm(const float *x, int D) {
  volatile float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int d = 0; d < D; ++d) {
    volatile float sq = x[d] * x[d];
    lane[d & 7] = lane[d & 7] + sq;
  }
  volatile float s = lane[0];
  for (int j = 1; j < 8; ++j) s = s + lane[j];
  return sqrtf(s);
}

static float tq_dot_sequential(const float *a, const float *p, int D) {
  float acc = 0.0f;
  for (int d = 0; d < D; ++d) acc = fmaf(a[d], p[d], acc);
  return acc;
}

static float tq_dot_interleaved16(const float *a, const float *p, int D) {
  float c[16];
  for (int j = 0; j < 16; ++j) c[j] = 0.0f;
  for (int d = 0; d < D; ++d) c[d & 15] = fmaf(a[d], p[d], c[d & 15]);
  volatile float s[4];
  for (int j = 0; j < 4; ++j) {
    volatile float t = c[j] + c[j + 4];
    t = t + c[j + 8];
    t = t + c[j + 12];
    s[j] = t;
  }
  volatile float lo = s[0] + s[1];
  volatile float hi = s[2] + s[3];
  return lo + hi;
}

/* x: rows x D fp32 contiguous.  idx: rows x D.  norms: rows (fp32, clamped). */
void tq_quantize(const float *x, int64_t rows, int D, const float *Pi,
                 const float *bounds, int nbounds, int order, uint8_t *idx,
                 float *norms) {
  float xn[1024];
  for (int64_t r = 0; r < rows; ++r) {
    const float *row = x + r * D;
    float n = tq_norm(row, D);
    if (n < 1e-10f) n = 1e-10f;
    norms[r] = n;
    for (int d = 0; d < D; ++d) xn[d] = row[d] / n;
    for (int c = 0; c < D; ++c) {
      const float *p = Pi + (int64_t)c * D;
      float y = order == TQ_ORDER_INTERLEAVED16 ? tq_dot_interleaved16(xn, p, D)
                                                : tq_dot_sequential(xn, p, D);
      int k = 0; /* bucketize(right=False): number of boundaries < y */
      while (k < nbounds && bounds[k] < y) ++k;
      idx[r * D + c] = (uint8_t)k;
    }
  }
}

void tq_pack(const uint8_t *idx, int64_t rows, int D, int bw, uint8_t *out) {
  const int nb = D * bw / 8;
  memset(out, 0, (size_t)rows * nb);
  for (int64_t r = 0; r < rows; ++r) {
    uint8_t *o = out + r * nb;
    for (int i = 0; i < D; ++i) {
      const unsigned v = idx[r * D + i];
      for (int b = 0; b < bw; ++b) {
        const int bit = i * bw + b;
        o[bit >> 3] |= (uint8_t)(((v >> b) & 1u) << (bit & 7));
      }
    }
  }
}

void tq_unpack(const uint8_t *packed, int64_t rows, int D, int bw, uint8_t *idx) {
  const int nb = D * bw / 8;
  for (int64_t r = 0; r < rows; ++r) {
    const uint8_t *p = packed + r * nb;
    for (int i = 0; i < D; ++i) {
      unsigned v = 0;
      for (int b = 0; b < bw; ++b) {
        const int bit = i * bw + b;
        v |= (unsigned)((p[bit >> 3] >> (bit & 7)) & 1u) << b;
      }
      idx[r * D + i] = (uint8_t)v;
    }
  }
}

/* out[r] = (centroids[idx[r]] @ Pi) * norm[r], fp32, sequential FMA chains. */
void tq_dequantize(const uint8_t *idx, const float *norms, int64_t rows, int D,
                   const float *Pi, const float *centroids, float *out) {
  float y[1024];
  for (int64_t r = 0; r < rows; ++r) {
    for (int d = 0; d < D; ++d) y[d] = centroids[idx[r * D + d]];
    for (int c = 0; c < D; ++c) {
      float acc = 0.0f;
      for (int d = 0; d < D; ++d) acc = fmaf(y[d], Pi[(int64_t)d * D + c], acc);
      out[r * D + c] = acc * norms[r];
    }
  }
}
