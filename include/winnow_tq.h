/*
 * winnow_tq.h - C ABI of libwinnow_tq.so: the sm_100a CUDA backend for the
 * TurboQuant packed-KV decode path of lgoyal6/winnow (turboquant_kv/).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its comment says "host";
 *   - buffers are borrowed for the duration of the call's work on `stream`;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream); calls only enqueue work, they never synchronise;
 *   - return value: WTQ_OK or a negative WTQ_ERR_* code, with a text in
 *     wtq_last_error() (thread-local).  Nothing throws or aborts.  Argument
 *     errors are reported before anything is launched;
 *   - `status` (optional, may be NULL) is a device int32 the kernels OR bits
 *     into when they meet data they refuse to follow (a page id outside the
 *     pool, a position outside the page table); such accesses are skipped,
 *     never performed.  The caller zeroes it and reads it when it likes;
 *   - dtype codes: WTQ_F32 / WTQ_F16 / WTQ_BF16.
 *
 * Layouts (reference: turboquant_kv/packed_attention.py:20-29,
 * turboquant_kv/page_pool.py:63-86)
 *   pages      (P, Hkv, S, NB) uint8, NB = D*bw/8, rows of NB bytes contiguous,
 *              S rows contiguous; page and head strides given in BYTES
 *   norms      (P, Hkv, S) fp16, S contiguous; strides given in ELEMENTS
 *   page_table (B, max_pages) int32, unused slots -1; row stride in elements
 *   seq_lens   (B,) int32, tokens stored per sequence (including this step's)
 *   codes      LSB-first bit stream per row (turboquant_kv/packing.py:14-18)
 */
#ifndef WINNOW_TQ_H_
#define WINNOW_TQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WTQ_OK 0
#define WTQ_ERR_ARG (-1)         /* malformed argument (shape, stride, null) */
#define WTQ_ERR_UNSUPPORTED (-2) /* legal request this build has no kernel for */
#define WTQ_ERR_CUDA (-3)        /* a CUDA runtime call failed */
#define WTQ_ERR_WORKSPACE (-4)   /* workspace too small */

#define WTQ_F32 0
#define WTQ_F16 1
#define WTQ_BF16 2

/* status bits written by kernels */
#define WTQ_STATUS_BAD_PAGE 1     /* page id outside [0, P) was skipped */
#define WTQ_STATUS_BAD_POSITION 2 /* token position outside the page table */
/* (4 is WTQ_STATUS_EXCHANGE_TIMEOUT, below) */
#define WTQ_STATUS_LAYOUT 8        /* the scan kernel found its shared-memory plan unusable and did nothing */
#define WTQ_STATUS_SCAN_TIMEOUT 16 /* a page copy of the scan kernel did not complete within its bounded wait */

/* order of the fp32 summation in the rotation of wtq_quantize / wtq_append.
 * The reference computes (x/|x|) @ Pi^T with a CPU BLAS whose order depends
 * on the number of vectors in the call (turboquant_kv/cache.py:108-115);
 * WTQ_ORDER_AUTO picks the order that BLAS uses for `rows` vectors. */
#define WTQ_ORDER_AUTO (-1)
#define WTQ_ORDER_SEQUENTIAL 0
#define WTQ_ORDER_INTERLEAVED16 1

/* Library version (major*10000 + minor*100 + patch) and last error text. */
int wtq_version(void);
const char *wtq_last_error(void);

/* Replaces packing.pack (turboquant_kv/packing.py:38-64).
 * idx (rows, D) uint8 contiguous -> out (rows, D*bw/8) uint8 contiguous. */
int wtq_pack(const uint8_t *idx, uint8_t *out, int64_t rows, int D, int bw, void *stream);

/* Replaces packing.unpack (turboquant_kv/packing.py:68-89). */
int wtq_unpack(const uint8_t *packed, uint8_t *idx, int64_t rows, int D, int bw, void *stream);

/* Replaces TurboQuantMSE.quantize (turboquant_kv/cache.py:108-115), optionally
 * fused with packing.pack.  x: `rows` vectors of D elements of `dtype`,
 * vector r at x + r*row_stride (elements), contiguous inside a vector.
 * Pi (D, D) fp32 row-major; bounds (2^bw - 1) fp32 ascending.
 * Outputs, each optional (NULL to skip): idx (rows, D) uint8; packed
 * (rows, D*bw/8) uint8; norms (rows) fp32 (clamped at 1e-10, as returned by
 * the reference). */
int wtq_quantize(const void *x, int dtype, int64_t rows, int64_t row_stride, int D,
                 const float *Pi, const float *bounds, int bw, int order, uint8_t *idx,
                 uint8_t *packed, float *norms, void *stream);

/* Replaces the packed branch of PagedPackedCache.update
 * (turboquant_kv/packed_backend.py:135-170): rotate, take the norm, quantize,
 * bit-pack and scatter n new tokens per sequence into one layer's pages, for K
 * and V, in one launch.  k, v: (B, Hkv, n, D) of `dtype` with element strides
 * {batch, head, token} (the last dimension is contiguous).  Token i of
 * sequence b lands at position seq_lens[b] - n + i, i.e. in page
 * page_table[b][pos / S], slot pos % S.  Norms are stored as fp16 (round to
 * nearest even).  `order` as in wtq_quantize, with rows = B*Hkv*n. */
typedef struct {
  uint8_t *pages;        /* one layer: (P, Hkv, S, NB) */
  void *norms;           /* fp16 (P, Hkv, S) */
  int64_t page_stride;   /* bytes between pages */
  int64_t head_stride;   /* bytes between kv heads */
  int64_t norm_page_stride; /* elements */
  int64_t norm_head_stride; /* elements */
  const float *Pi;       /* (D, D) */
  const float *bounds;   /* 2^bw - 1 (append) */
  const float *centroids;/* 2^bw     (decode) */
  int bw;
} wtq_side_t;

int wtq_append(const void *k, const void *v, int dtype, const int64_t k_strides[3],
               const int64_t v_strides[3], const wtq_side_t *k_side, const wtq_side_t *v_side,
               const int32_t *page_table, int64_t table_stride, const int32_t *seq_lens, int B,
               int Hkv, int n, int D, int S, int P, int max_pages, int order, int32_t *status,
               void *stream);

/* Replaces packed_decode_attention (turboquant_kv/packed_attention_triton.py:
 * 180-187, 204-262): one query token per sequence attends to its packed
 * history.  q: (B, Hq, D) of `dtype`, element strides {batch, head}; out:
 * same shape, own strides, same dtype (it may be a slice of a larger gathered
 * buffer).  Query head h reads kv head h / (Hq/Hkv).  num_splits <= 0 lets the
 * library choose.  The rotated query, the split-K partial states and the merge
 * live in `workspace` (wtq_decode_workspace_bytes); nothing else is allocated.
 * The first wtq_decode_counter_bytes() of the workspace must be zero on entry
 * and are zero again when the call's work completes.  Sequences of length 0
 * produce exact zeros. */
size_t wtq_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int max_pages, int S,
                                  int num_splits);
size_t wtq_decode_counter_bytes(int B, int Hkv);
int wtq_decode_auto_splits(int B, int Hq, int Hkv, int D, int max_pages, int S, int bw_k,
                           int bw_v);
int wtq_decode(const void *q, int dtype, const int64_t q_strides[2], void *out,
               const int64_t out_strides[2], const wtq_side_t *k_side, const wtq_side_t *v_side,
               const int32_t *page_table, int64_t table_stride, const int32_t *seq_lens,
               float scale, int B, int Hq, int Hkv, int D, int S, int P, int max_pages,
               int num_splits, void *workspace, size_t workspace_bytes, int32_t *status,
               void *stream);

/* wtq_decode fused with the output exchange of KV-head tensor parallelism (no
 * counterpart in the reference, which has no multi-GPU form of this path).
 * Every rank holds `Hq` of the `world * Hq` query heads.  Instead of writing a
 * local (B, Hq, D) result, the merge kernel stores this rank's rows straight
 * into EVERY rank's full (B, world*Hq, D) buffer at head offset
 * `head_offset`, through peer-mapped pointers (plain stores over NVLink; no
 * multicast); when the last merge block has fenced its stores, one arrival is
 * added to slot `rank` of every rank's flag array, so a rank's rows of call
 * number s are complete in a buffer once that slot has reached s x (arrivals
 * per call).  wtq_exchange_wait, enqueued after it, returns once all `world` slots
 * of the local flag array have got there, i.e. the local full buffer is
 * complete.  Waits are bounded: after `spin_limit` polls of a slot the kernel
 * gives up, sets WTQ_STATUS_EXCHANGE_TIMEOUT in `status` and returns; the buffer
 * then still holds the late rank's previous rows, so the result is valid only
 * while that bit is clear.  The bookkeeping lives in device memory
 * (`step_counter`: FOUR uint32 words, zero at start: calls completed, waits
 * completed, arrivals per call, spare), so the arguments never change and
 * the pair of calls can be replayed from a CUDA graph; call number s (1, 2, ...)
 * uses buffer set s & 1: the full buffers alternate between two sets because a
 * peer may already be writing step s+1 while this rank still reads step s.
 * Every rank must make the same sequence of calls with the same shapes (they
 * then launch the same number of merge blocks).
 * Only the tensor-core path (head_dim 128, widths 4/4, 4/6, 6/6, 8/8) has this
 * epilogue; other shapes get WTQ_ERR_UNSUPPORTED and should gather with NCCL
 * (wtq_decode_exchange_supported answers ahead of time). */
#define WTQ_STATUS_EXCHANGE_TIMEOUT 4
typedef struct {
  void *const *peer_out[2];       /* DEVICE arrays [world]: every rank's full buffer, sets 0 and 1 */
  uint32_t *const *peer_flags;    /* DEVICE array [world]: every rank's flag array (world uint32) */
  int64_t out_strides[2];         /* element strides {batch, head} of the full buffers */
  int rank, world;
  int head_offset;                /* first head of the full buffer this rank writes */
  uint32_t *step_counter;         /* local device uint32[4]: see above */
  uint32_t *done_counter;         /* local device uint32, zero between calls */
} wtq_exchange_t;
int wtq_decode_exchange(const void *q, int dtype, const int64_t q_strides[2],
                        const wtq_exchange_t *exchange, const wtq_side_t *k_side,
                        const wtq_side_t *v_side, const int32_t *page_table, int64_t table_stride,
                        const int32_t *seq_lens, float scale, int B, int Hq, int Hkv, int D, int S,
                        int P, int max_pages, int num_splits, void *workspace,
                        size_t workspace_bytes, int32_t *status, void *stream);
/* 1 when wtq_decode_exchange has its fused epilogue for these descriptors (the
 * test the call applies: shape, widths, alignment of pointers and strides, the
 * WTQ_FORCE_GENERIC switch), 0 when the caller should gather with NCCL.
 * `workspace`: the buffer the call will be given.  Launches nothing. */
int wtq_decode_exchange_supported(const wtq_side_t *k_side, const wtq_side_t *v_side, int Hq,
                                  int Hkv, int D, int S, const void *workspace);
int wtq_exchange_wait(const uint32_t *local_flags, int world, uint32_t *step_counter,
                      int64_t spin_limit, int32_t *status, void *stream);

/* wtq_decode without a caller-supplied workspace.  It has no counterpart in the
 * reference.  It exists for hosts that cannot allocate device memory for this
 * library (a server whose arena owns all of it, a loop that may not take the
 * device-wide synchronisation an allocation implies): the workspace is a
 * 16 MiB array built into the library image, which every GPU that loads the
 * library holds until the process exits.  Same arguments and results as
 * wtq_decode minus the workspace pair.  Calls whose workspace
 * (wtq_decode_workspace_bytes for the chosen num_splits) exceeds
 * wtq_decode_static_capacity() are refused with WTQ_ERR_WORKSPACE.  The first
 * call on each device looks the array's device address up (with that device
 * current); that is also when the CUDA runtime, which loads modules lazily,
 * places the array in that device's memory.  Make that first call at start-up,
 * before any stream capture begins; later calls leave the device's free memory
 * unchanged.  All calls
 * on a device share the one array: calls that can overlap on the GPU (two
 * streams, two threads) race and must be serialised by the caller.  Nothing
 * here calls cudaMalloc, cudaFree or any allocating routine. */
size_t wtq_decode_static_capacity(void);
int wtq_decode_static(const void *q, int dtype, const int64_t q_strides[2], void *out,
                      const int64_t out_strides[2], const wtq_side_t *k_side,
                      const wtq_side_t *v_side, const int32_t *page_table, int64_t table_stride,
                      const int32_t *seq_lens, float scale, int B, int Hq, int Hkv, int D, int S,
                      int P, int max_pages, int num_splits, int32_t *status, void *stream);

/* Replaces dense_decode_attention (turboquant_kv/packed_attention_triton.py:190-201),
 * the matched unquantised arm of the decode operator: the same split-K schedule
 * over the same page table, on pages (P, Hkv, S, D) of `page_dtype` (fp16, bf16
 * or fp32; the last two dimensions contiguous; k_strides / v_strides = element
 * strides {page, head}).  q, out as in wtq_decode.  num_splits >= 1 (the
 * caller's choice; 1 = one block per (kv head, sequence)).  Workspace:
 * wtq_dense_workspace_bytes. */
size_t wtq_dense_workspace_bytes(int B, int Hq, int D, int num_splits);
int wtq_dense_decode(const void *q, int q_dtype, const int64_t q_strides[2], void *out,
                     const int64_t out_strides[2], const void *k_pages, const void *v_pages,
                     int page_dtype, const int64_t k_strides[2], const int64_t v_strides[2],
                     const int32_t *page_table, int64_t table_stride, const int32_t *seq_lens,
                     float scale, int B, int Hq, int Hkv, int D, int S, int P, int max_pages,
                     int num_splits, void *workspace, size_t workspace_bytes, int32_t *status,
                     void *stream);

/* Chunked prefill over packed pages: causal attention of the last Q tokens of
 * every sequence (their K/V already appended, so seq_lens includes them) over
 * the sequence's packed history, the pages read and decoded once for all query
 * rows.  Replaces the reference's prefill fallback, dequantize_history +
 * _reconstruct_sdpa (turboquant_kv/packed_backend.py:192-226), and computes
 * what tiled_compressed_attention (turboquant_kv/packed_attention.py:260-311)
 * computes for Q > 1.
 *
 *   q    row (b * Q + i) holds query token i of sequence b: element (row, head, d)
 *        at q + row * q_strides[0] + head * q_strides[1] + d (elements);
 *   out  the same indexing with out_strides, i.e. a (B, Q, Hq, D) tensor.
 * Token i sees keys [0, seq_lens[b] - Q + i]; a token that sees none gets zeros.
 * Requires what the tensor-core decode path requires (head_dim 128, widths
 * 4/4, 4/6, 6/6, 8/8, power-of-two page size >= 16, Hq / Hkv <= 8, 16-byte
 * aligned pages); otherwise WTQ_ERR_UNSUPPORTED, and the caller may run the
 * B * Q rows through wtq_decode instead.  num_splits > 0 cuts every history
 * into that many equal chunks.  num_splits <= 0 leaves the schedule to the
 * library: with enough groups and rows the 64-token tiles of all histories are
 * dealt evenly to the thread blocks (at most three chunk states per row),
 * otherwise equal chunks from a cost model; wtq_prefill_auto_splits returns the
 * number of chunk states per row that choice needs, and the workspace must hold
 * wtq_prefill_workspace_bytes(..., num_splits) for that number (or for the
 * explicit num_splits).  Status bits as for wtq_decode.  Three launches and up
 * to two small memsets, no allocation, no synchronisation. */
int wtq_prefill_auto_splits(int B, int Hq, int Hkv, int Q, int max_pages, int S);
/* Schedule of this thread's last wtq_prefill call that got as far as launching:
 * 0 equal chunks, 1 tiles dealt evenly to the blocks; -1 before any call. */
int wtq_prefill_last_schedule(void);
size_t wtq_prefill_workspace_bytes(int B, int Hq, int Hkv, int Q, int D, int num_splits);
int wtq_prefill(const void *q, int dtype, const int64_t q_strides[2], void *out,
                const int64_t out_strides[2], const wtq_side_t *k_side, const wtq_side_t *v_side,
                const int32_t *page_table, int64_t table_stride, const int32_t *seq_lens,
                float scale, int B, int Hq, int Hkv, int Q, int D, int S, int P, int max_pages,
                int num_splits, void *workspace, size_t workspace_bytes, int32_t *status,
                void *stream);

/* Replaces tq_dequant / tq_dequant_cuda (turboquant_kv/kernel.py:78-115,
 * turboquant_kv/csrc/tq_dequant.cu:186-211): N packed rows -> (N, D) of
 * `out_dtype`.  Logical row r is read from source row (r / L) * MAXLEN + r % L
 * (a (planes, MAXLEN, NB) buffer viewed through its first L positions);
 * out[r] = (centroids[codes] @ Pi) * norm.
 *
 * wtq_dequant_mode chooses the arithmetic:
 *   WTQ_DEQUANT_EXACT    fp32 contraction on the CUDA cores (any D <= 256, any width);
 *   WTQ_DEQUANT_TC       tensor cores, centroids and Pi each split into fp16 high
 *                        and low parts, three products accumulated in fp32;
 *   WTQ_DEQUANT_TC_FAST  tensor cores, single fp16 operands: the accuracy class of
 *                        the reference's allow_tf32=True (turboquant_kv/kernel.py:69);
 *   WTQ_DEQUANT_AUTO     TC for fp16/bf16 outputs where the tensor-core kernel
 *                        applies, EXACT otherwise (what wtq_dequant does).
 * The tensor-core kernel needs D = 128, a width of 4, 6 or 8, `packed` 16-byte
 * aligned (8 for 6-bit), `out` 16-byte aligned and MAXLEN < 2^31; an explicit
 * TC mode outside that returns WTQ_ERR_UNSUPPORTED.  The first tensor-core call
 * of each (width, mode, dtype) on a device synchronises the stream once to set
 * the kernel up, so it cannot be made while the stream is capturing (AUTO then
 * runs EXACT for that call). */
#define WTQ_DEQUANT_AUTO (-1)
#define WTQ_DEQUANT_EXACT 0
#define WTQ_DEQUANT_TC 1
#define WTQ_DEQUANT_TC_FAST 2
/* the same two with the mma.sync kernels named explicitly (TC and TC_FAST run the
 * tcgen05 kernel, accumulator in tensor memory, and fall back to these) */
#define WTQ_DEQUANT_TC_MMA 3
#define WTQ_DEQUANT_TC_FAST_MMA 4
int wtq_dequant(const uint8_t *packed, const void *norms_f16, const float *centroids,
                const float *Pi, void *out, int out_dtype, int bw, int D, int64_t N, int64_t L,
                int64_t MAXLEN, void *stream);
int wtq_dequant_mode(const uint8_t *packed, const void *norms_f16, const float *centroids,
                     const float *Pi, void *out, int out_dtype, int bw, int D, int64_t N, int64_t L,
                     int64_t MAXLEN, int mode, void *stream);

/* Instrumentation; no counterpart in the reference.
 * wtq_launch_count: kernels this library has launched in this process.
 * wtq_profile_enable: from now on every wtq_decode call records a pair of CUDA
 * events on its stream around its page-scan kernel (up to `capacity` calls).
 * wtq_profile_collect waits for the recorded pairs, returns their summed
 * duration in milliseconds and their number, and rearms the recorder.
 * wtq_profile_disable releases the events.  Not meant for production use: the
 * events serialise nothing, but enable/disable create and destroy them. */
uint64_t wtq_launch_count(void);
int wtq_profile_enable(int capacity);
int wtq_profile_collect(double *total_ms, int *launches);
/* Like wtq_profile_collect, split per call into: first launch to scan start
 * (query rotation), the scan, scan end to last launch's end (merge). */
int wtq_profile_phases(double *before_scan_ms, double *scan_ms, double *after_scan_ms, int *calls);
int wtq_profile_disable(void);

/* Plain streaming read of `bytes` bytes of device memory (16-byte loads, every
 * byte once), for calibrating the read-only HBM ceiling beside the scan's
 * numbers; `sink` (optional device word) only keeps the loads alive.  Same role
 * as the reference study's streaming control (experiments/c27/controls.cu:15-36). */
int wtq_probe_read(const void *src, size_t bytes, uint32_t *sink, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* WINNOW_TQ_H_ */
