// wtq_decode_static: decode attention for callers that must not allocate.
//
// Some hosts of this library cannot hand it a workspace: a plugin loaded into
// an inference server whose arena owns every byte of device memory and forbids
// further cudaMalloc calls, a real-time loop that may not take the device-wide
// synchronisation an allocation implies, or a process whose memory budget was
// fixed at start-up.  For them the split-K workspace of wtq_decode lives in a
// fixed array inside the library image.  Every GPU that loads the library
// holds kStaticScratchBytes of it until the process exits, whether or not this
// entry point is ever called.
#include <mutex>

#include "wtq_decode.cuh"

namespace {

constexpr size_t kStaticScratchBytes = 16u << 20;       // 16 MiB, the stated maximum
static __device__ __align__(256) unsigned char g_scratch[kStaticScratchBytes];

// In host code `g_scratch` is only a handle for the runtime, not an address a
// kernel can use; the device address is asked for once per device, with that
// device current, and kept.
constexpr int kMaxDevices = 64;
void *g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_lock;

int scratch_for_current_device(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return wtq::check_cuda(e, "wtq_decode_static: cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices)
    return wtq::fail(WTQ_ERR_UNSUPPORTED, "wtq_decode_static: device index %d not supported", dev);
  std::lock_guard<std::mutex> hold(g_setup_lock);
  if (g_scratch_ptr[dev] == nullptr) {
    void *ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return wtq::check_cuda(e != cudaSuccess ? e : cudaErrorInvalidSymbol,
                             "wtq_decode_static: cudaGetSymbolAddress");
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return WTQ_OK;
}

}  // namespace

extern "C" size_t wtq_decode_static_capacity(void) { return kStaticScratchBytes; }

extern "C" int wtq_decode_static(const void *q, int dtype, const int64_t q_strides[2], void *out,
                                 const int64_t out_strides[2], const wtq_side_t *k_side,
                                 const wtq_side_t *v_side, const int32_t *page_table,
                                 int64_t table_stride, const int32_t *seq_lens, float scale, int B,
                                 int Hq, int Hkv, int D, int S, int P, int max_pages,
                                 int num_splits, int32_t *status, void *stream) {
  // every argument is checked before anything is queued on the stream
  if (int rc = wtq::decode_validate(q, dtype, q_strides, out, out_strides, false, k_side, v_side,
                                    page_table, seq_lens, B, Hq, Hkv, D, S, P, max_pages))
    return rc;
  if (!out) return wtq::fail(WTQ_ERR_ARG, "wtq_decode_static: null output");
  // num_splits goes through unchanged (<= 0: the library's own choice), so this
  // entry point runs the same schedule as wtq_decode; the size asked for is the
  // one wtq_decode_workspace_bytes reports for that argument.
  const size_t need = wtq_decode_workspace_bytes(B, Hq, Hkv, D, max_pages, S, num_splits);
  if (need > kStaticScratchBytes)
    return wtq::fail(WTQ_ERR_WORKSPACE,
                     "wtq_decode_static: this call needs %zu bytes of scratch, the built-in array "
                     "holds %zu; lower num_splits or use wtq_decode with your own workspace",
                     need, kStaticScratchBytes);
  if (B == 0) return WTQ_OK;
  void *scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  // The array keeps whatever the previous call left.  Only the leading counter
  // block has to start at zero; everything else is written before it is read.
  cudaError_t e = cudaMemsetAsync(scratch, 0, wtq_decode_counter_bytes(B, Hkv), (cudaStream_t)stream);
  if (e != cudaSuccess) return wtq::check_cuda(e, "wtq_decode_static: clearing counters");
  return wtq_decode(q, dtype, q_strides, out, out_strides, k_side, v_side, page_table, table_stride,
                    seq_lens, scale, B, Hq, Hkv, D, S, P, max_pages, num_splits, scratch,
                    kStaticScratchBytes, status, stream);
}
