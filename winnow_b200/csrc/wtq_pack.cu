// Bit-packing of codebook indices (LSB-first stream) and its inverse, plus the
// library's error plumbing.
#include "wtq_common.cuh"

namespace wtq {

char *error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return WTQ_OK;
  return fail(WTQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// One thread per output byte: byte j of a row gathers stream bits 8j..8j+7.
__global__ void pack_kernel(const uint8_t *idx, uint8_t *out, int64_t rows, int D, int bw, int nb) {
  const int64_t total = rows * nb;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / nb;
    const int j = (int)(e - r * nb);
    const uint8_t *src = idx + r * D;
    unsigned v = 0;
    if (bw == 8) {
      v = src[j];
    } else {
      for (int b = 0; b < 8; ++b) {
        const int bit = 8 * j + b;
        const int i = bit / bw;
        v |= ((src[i] >> (bit - i * bw)) & 1u) << b;
      }
    }
    out[e] = (uint8_t)v;
  }
}

// One thread per code.
__global__ void unpack_kernel(const uint8_t *packed, uint8_t *idx, int64_t rows, int D, int bw,
                              int nb) {
  const int64_t total = rows * D;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / D;
    const int i = (int)(e - r * D);
    idx[e] = (uint8_t)extract_code(packed + r * nb, i, bw, nb);
  }
}

static int grid_for(int64_t total) {
  int64_t g = (total + 255) / 256;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

}  // namespace wtq

using namespace wtq;

extern "C" int wtq_version(void) { return 100; }
extern "C" const char *wtq_last_error(void) { return error_buffer(); }

static int check_pack_args(const char *who, const void *a, const void *b, int64_t rows, int D,
                           int bw) {
  if (rows < 0 || D < 1) return fail(WTQ_ERR_ARG, "%s: bad sizes", who);
  if (!width_supported(bw) || (D * bw) % 8)
    return fail(WTQ_ERR_ARG, "%s: head_dim*bit_width must be a multiple of 8 and the width one of "
                "2,3,4,5,6,8 (got %d*%d)", who, D, bw);
  if (rows > 0 && (!a || !b)) return fail(WTQ_ERR_ARG, "%s: null buffer", who);
  return WTQ_OK;
}

extern "C" int wtq_pack(const uint8_t *idx, uint8_t *out, int64_t rows, int D, int bw,
                        void *stream) {
  if (int rc = check_pack_args("wtq_pack", idx, out, rows, D, bw)) return rc;
  if (rows == 0) return WTQ_OK;
  const int nb = D * bw / 8;
  pack_kernel<<<grid_for(rows * nb), 256, 0, (cudaStream_t)stream>>>(idx, out, rows, D, bw, nb);
  return check_cuda(cudaGetLastError(), "wtq_pack launch");
}

extern "C" int wtq_unpack(const uint8_t *packed, uint8_t *idx, int64_t rows, int D, int bw,
                          void *stream) {
  if (int rc = check_pack_args("wtq_unpack", packed, idx, rows, D, bw)) return rc;
  if (rows == 0) return WTQ_OK;
  const int nb = D * bw / 8;
  unpack_kernel<<<grid_for(rows * D), 256, 0, (cudaStream_t)stream>>>(packed, idx, rows, D, bw, nb);
  return check_cuda(cudaGetLastError(), "wtq_unpack launch");
}
