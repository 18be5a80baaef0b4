// Shared device helpers and host-side error plumbing for libwinnow_tq.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/winnow_tq.h"

namespace wtq {

// ---- host: thread-local error text -----------------------------------------
char *error_buffer();
int fail(int code, const char *fmt, ...);
int check_cuda(cudaError_t e, const char *what);
void note_launches(int n);
int device_sms();          // multiprocessors of the current device
// Recorder of event pairs around the decode page-scan kernel (see
// wtq_profile_enable); both are no-ops while profiling is off.
void profile_mark_begin(cudaStream_t stream);
void profile_mark_end(cudaStream_t stream);
void profile_mark_call(cudaStream_t stream, bool begin);

inline bool width_supported(int bw) {
  return bw == 2 || bw == 3 || bw == 4 || bw == 5 || bw == 6 || bw == 8;
}

// The CPU BLAS behind the reference's `(x/|x|) @ Pi^T` switches summation
// order with the number of vectors in the call: 2..5 vectors take 16
// interleaved chains, everything else one chain per output.
inline int resolve_order(int order, int64_t rows) {
  if (order == WTQ_ORDER_AUTO)
    return (rows >= 2 && rows <= 5) ? WTQ_ORDER_INTERLEAVED16 : WTQ_ORDER_SEQUENTIAL;
  return order;
}

// ---- device: element loads / stores ----------------------------------------
template <int DT> struct Elem;
template <> struct Elem<WTQ_F32> {
  using type = float;
  __device__ static float load(const void *p, int64_t i) { return ((const float *)p)[i]; }
  __device__ static void store(void *p, int64_t i, float v) { ((float *)p)[i] = v; }
};
template <> struct Elem<WTQ_F16> {
  using type = __half;
  __device__ static float load(const void *p, int64_t i) {
    return __half2float(((const __half *)p)[i]);
  }
  __device__ static void store(void *p, int64_t i, float v) {
    ((__half *)p)[i] = __float2half_rn(v);
  }
};
template <> struct Elem<WTQ_BF16> {
  using type = __nv_bfloat16;
  __device__ static float load(const void *p, int64_t i) {
    return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
  }
  __device__ static void store(void *p, int64_t i, float v) {
    ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v);
  }
};

__device__ __forceinline__ float load_as_float(const void *p, int64_t i, int dtype) {
  if (dtype == WTQ_F16) return Elem<WTQ_F16>::load(p, i);
  if (dtype == WTQ_BF16) return Elem<WTQ_BF16>::load(p, i);
  return Elem<WTQ_F32>::load(p, i);
}
__device__ __forceinline__ void store_from_float(void *p, int64_t i, float v, int dtype) {
  if (dtype == WTQ_F16) Elem<WTQ_F16>::store(p, i, v);
  else if (dtype == WTQ_BF16) Elem<WTQ_BF16>::store(p, i, v);
  else Elem<WTQ_F32>::store(p, i, v);
}

// Code i of a row packed LSB-first at `bw` bits per code: stream bits
// [i*bw, (i+1)*bw).  The second byte is read only when the code crosses into
// it, so the last code of a row never touches the byte after the row.
__device__ __forceinline__ unsigned extract_code(const uint8_t *row, int i, int bw, int nb) {
  const int bit = i * bw;
  const int b0 = bit >> 3;
  const int sh = bit & 7;
  unsigned w = row[b0];
  if (sh + bw > 8 && b0 + 1 < nb) w |= (unsigned)row[b0 + 1] << 8;
  return (w >> sh) & ((1u << bw) - 1u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace wtq
