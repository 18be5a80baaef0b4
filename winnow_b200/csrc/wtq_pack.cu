// Bit-packing of codebook indices (LSB-first stream) and its inverse, plus the
// library's error plumbing.
#include <atomic>
#include <mutex>
#include <vector>

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

static std::atomic<uint64_t> g_launches{0};
void note_launches(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// Multiprocessor count of the current device (cached per device; the cache is
// only ever written with the value the driver reports, so concurrent first
// calls are harmless).
int device_sms() {
  static std::atomic<int> cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  std::atomic<int> &slot = cached[dev & 63];
  int sms = dev < 64 ? slot.load(std::memory_order_relaxed) : 0;
  if (sms == 0) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    if (dev < 64) slot.store(sms, std::memory_order_relaxed);
  }
  return sms;
}
uint64_t launches_so_far() { return g_launches.load(std::memory_order_relaxed); }

static std::mutex g_profile_lock;
static std::vector<cudaEvent_t> g_begin, g_end;
static int g_recorded = 0;
static bool g_open = false;

void profile_mark_begin(cudaStream_t stream) {
  std::lock_guard<std::mutex> hold(g_profile_lock);
  if (g_recorded < (int)g_begin.size() && !g_open) {
    cudaEventRecord(g_begin[g_recorded], stream);
    g_open = true;
  }
}
void profile_mark_end(cudaStream_t stream) {
  std::lock_guard<std::mutex> hold(g_profile_lock);
  if (g_open) {
    cudaEventRecord(g_end[g_recorded++], stream);
    g_open = false;
  }
}
// Call boundaries (before the first and after the last launch of a wtq_decode
// call), recorded alongside the scan's pair.
static std::vector<cudaEvent_t> g_call_begin, g_call_end;
void profile_mark_call(cudaStream_t stream, bool begin) {
  std::lock_guard<std::mutex> hold(g_profile_lock);
  if (begin) {
    if (g_recorded < (int)g_call_begin.size() && !g_open) cudaEventRecord(g_call_begin[g_recorded], stream);
  } else if (g_recorded > 0 && g_recorded <= (int)g_call_end.size()) {
    cudaEventRecord(g_call_end[g_recorded - 1], stream);
  }
}
static void profile_release() {
  for (cudaEvent_t e : g_call_begin) cudaEventDestroy(e);
  for (cudaEvent_t e : g_call_end) cudaEventDestroy(e);
  g_call_begin.clear();
  g_call_end.clear();
  for (cudaEvent_t e : g_begin) cudaEventDestroy(e);
  for (cudaEvent_t e : g_end) cudaEventDestroy(e);
  g_begin.clear();
  g_end.clear();
  g_recorded = 0;
  g_open = false;
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
extern "C" uint64_t wtq_launch_count(void) { return launches_so_far(); }

extern "C" int wtq_profile_enable(int capacity) {
  if (capacity < 1) return fail(WTQ_ERR_ARG, "wtq_profile_enable: capacity must be positive");
  std::lock_guard<std::mutex> hold(g_profile_lock);
  profile_release();
  for (int i = 0; i < capacity; ++i) {
    cudaEvent_t b, e;
    if (cudaEventCreate(&b) != cudaSuccess || cudaEventCreate(&e) != cudaSuccess) {
      profile_release();
      return check_cuda(cudaGetLastError(), "wtq_profile_enable");
    }
    g_begin.push_back(b);
    g_end.push_back(e);
    cudaEvent_t cb, ce;
    if (cudaEventCreate(&cb) != cudaSuccess || cudaEventCreate(&ce) != cudaSuccess) {
      profile_release();
      return check_cuda(cudaGetLastError(), "wtq_profile_enable");
    }
    g_call_begin.push_back(cb);
    g_call_end.push_back(ce);
  }
  return WTQ_OK;
}

extern "C" int wtq_profile_collect(double *total_ms, int *launches) {
  if (!total_ms || !launches) return fail(WTQ_ERR_ARG, "wtq_profile_collect: null output");
  std::lock_guard<std::mutex> hold(g_profile_lock);
  double sum = 0.0;
  for (int i = 0; i < g_recorded; ++i) {
    float ms = 0.0f;
    cudaError_t e = cudaEventSynchronize(g_end[i]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, g_begin[i], g_end[i]);
    if (e != cudaSuccess) return check_cuda(e, "wtq_profile_collect");
    sum += ms;
  }
  *total_ms = sum;
  *launches = g_recorded;
  g_recorded = 0;
  return WTQ_OK;
}

extern "C" int wtq_profile_phases(double *before_scan_ms, double *scan_ms, double *after_scan_ms,
                                  int *calls) {
  if (!before_scan_ms || !scan_ms || !after_scan_ms || !calls)
    return fail(WTQ_ERR_ARG, "wtq_profile_phases: null output");
  std::lock_guard<std::mutex> hold(g_profile_lock);
  double a = 0.0, b = 0.0, c = 0.0;
  for (int i = 0; i < g_recorded; ++i) {
    float t0 = 0.f, t1 = 0.f, t2 = 0.f;
    cudaError_t e = cudaEventSynchronize(g_call_end[i]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t0, g_call_begin[i], g_begin[i]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t1, g_begin[i], g_end[i]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t2, g_end[i], g_call_end[i]);
    if (e != cudaSuccess) return check_cuda(e, "wtq_profile_phases");
    a += t0; b += t1; c += t2;
  }
  *before_scan_ms = a; *scan_ms = b; *after_scan_ms = c; *calls = g_recorded;
  g_recorded = 0;
  return WTQ_OK;
}

extern "C" int wtq_profile_disable(void) {
  std::lock_guard<std::mutex> hold(g_profile_lock);
  profile_release();
  return WTQ_OK;
}

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
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_pack launch");
}

extern "C" int wtq_unpack(const uint8_t *packed, uint8_t *idx, int64_t rows, int D, int bw,
                          void *stream) {
  if (int rc = check_pack_args("wtq_unpack", packed, idx, rows, D, bw)) return rc;
  if (rows == 0) return WTQ_OK;
  const int nb = D * bw / 8;
  unpack_kernel<<<grid_for(rows * D), 256, 0, (cudaStream_t)stream>>>(packed, idx, rows, D, bw, nb);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_unpack launch");
}
