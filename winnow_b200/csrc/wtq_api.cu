// Host entry points of wtq_decode: argument checks, workspace carving, launch
// order.  Nothing here allocates or synchronises.
#include <cstdlib>

#include "wtq_decode.cuh"

using namespace wtq;

namespace {

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// lookup tables of the tensor-core scan: at most 256 entries x 2 sides x 32 lanes
constexpr size_t kLutBytesMax = 256 * 256;

int clamp_splits(int splits, int max_pages, int S) {
  const int64_t tokens = (int64_t)max_pages * S;
  int64_t tiles = (tokens + 127) / 128;
  if (tiles < 1) tiles = 1;
  if (splits > tiles) splits = (int)tiles;
  if (splits > kMaxSplits) splits = kMaxSplits;
  if (splits < 1) splits = 1;
  return splits;
}

// WTQ_FORCE_GENERIC=1 in the environment routes every call through the generic
// CUDA-core kernels (used by the tests to cover both paths on the same inputs).
bool force_generic() {
  const char *v = getenv("WTQ_FORCE_GENERIC");
  return v && v[0] == '1';
}

bool fill_side(DecodeSideDev &d, const wtq_side_t &w, int D) {
  d.pages = w.pages;
  d.norms = (const __half *)w.norms;
  d.page_stride = w.page_stride;
  d.head_stride = w.head_stride;
  d.norm_page_stride = w.norm_page_stride;
  d.norm_head_stride = w.norm_head_stride;
  d.Pi = w.Pi;
  d.centroids = w.centroids;
  d.bw = w.bw;
  d.nb = D * w.bw / 8;
  return w.pages && w.norms && w.Pi && w.centroids;
}

}  // namespace

extern "C" size_t wtq_decode_counter_bytes(int B, int Hkv) {
  (void)Hkv;
  // [0] work queue of the tensor-core scan; from byte 128 (its own cache line, so
  // that queue traffic does not delay readers): chunk prefix, B + 1 ints
  return round_up(128 + ((size_t)(B > 0 ? B : 0) + 1) * sizeof(int32_t), 256);
}

extern "C" int wtq_decode_auto_splits(int B, int Hq, int Hkv, int D, int max_pages, int S,
                                      int bw_k, int bw_v) {
  if (B < 1 || Hkv < 1 || Hq < 1) return 1;
  const int64_t groups = (int64_t)B * Hkv;
  const int64_t max_tokens = (int64_t)max_pages * S;
  const int warps = mma_warps_per_sm(bw_k, bw_v);
  if (D == 128 && warps > 0 && S >= 16 && (S & (S - 1)) == 0 && Hq / Hkv <= 8) {
    // tensor-core path.  Every warp of the persistent grid is a worker and
    // takes whole chunks; a step costs about rounds * (chunk + 34) token
    // times, where 34 tokens stand for the fixed cost of a chunk (its partial
    // state written and merged) and `rounds` lies half way between
    // items / workers and that ratio rounded up: warps of one SM share its
    // throughput, so a part-filled last round costs less than a full one but
    // is not free.  Measured on B200, the best chunk is the one that fills
    // the last round (items just under a multiple of the workers); the search
    // below finds it.  Lengths are taken at the table's full width.  Chunks are
    // capped at 1024 tokens: beyond that one warp runs long after the others.
    const int64_t workers = (int64_t)device_sms() * warps;
    int64_t lo = ((max_tokens + kMaxSplits - 1) / kMaxSplits + 31) / 32 * 32;
    if (lo < 64) lo = 64;
    int64_t hi = lo > 1024 ? lo : 1024;
    int64_t best = hi;
    double best_cost = 0;
    for (int64_t chunk = hi; chunk >= lo; chunk -= 32) {
      const int64_t items = groups * ((max_tokens + chunk - 1) / chunk);
      const double frac = (double)items / (double)workers;
      const double rounds = 0.5 * (frac + (double)((items + workers - 1) / workers));
      const double cost = rounds * (double)(chunk + 34);
      if (chunk == hi || cost < best_cost) { best = chunk; best_cost = cost; }
    }
    int64_t splits = (max_tokens + best - 1) / best;
    if (splits > kMaxSplits) splits = kMaxSplits;
    return splits < 1 ? 1 : (int)splits;
  }
  // generic path: about eight 128-thread blocks per SM
  const int64_t want = (int64_t)device_sms() * 8;
  return clamp_splits((int)((want + groups - 1) / groups), max_pages, S);
}

static size_t workspace_for(int B, int Hq, int Hkv, int D, int splits) {
  const size_t rows = (size_t)B * Hq;
  size_t bytes = wtq_decode_counter_bytes(B, Hkv);
  bytes += round_up(rows * D * sizeof(float), 256);                   // rotated query
  bytes += round_up(rows * splits * D * sizeof(float), 256);          // partial acc
  bytes += 2 * round_up(rows * splits * sizeof(float), 256);          // partial m, l
  bytes += kLutBytesMax;                                              // lookup tables of the scan
  return bytes;
}

extern "C" size_t wtq_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int max_pages, int S,
                                             int num_splits) {
  if (B < 1 || Hq < 1 || Hkv < 1 || D < 1) return 256;
  int splits;
  if (num_splits > 0) {
    splits = clamp_splits(num_splits, max_pages, S);
  } else {                       // whichever kernel the call will pick, it fits
    splits = 1;
    for (int bw : {4, 6, 8}) {
      const int a = wtq_decode_auto_splits(B, Hq, Hkv, D, max_pages, S, bw, bw);
      if (a > splits) splits = a;
    }
    const int a = wtq_decode_auto_splits(B, Hq, Hkv, D, max_pages, S, 4, 6);
    if (a > splits) splits = a;
    const int g = wtq_decode_auto_splits(B, Hq, Hkv, D, max_pages, S, 3, 3);
    if (g > splits) splits = g;
  }
  return workspace_for(B, Hq, Hkv, D, splits);
}

// Argument checks shared by every decode entry point; nothing is launched or
// queued before they pass.
int wtq::decode_validate(const void *q, int dtype, const int64_t q_strides[2], const void *out,
                         const int64_t out_strides[2], bool has_exchange, const wtq_side_t *k_side,
                         const wtq_side_t *v_side, const int32_t *page_table,
                         const int32_t *seq_lens, int B, int Hq, int Hkv, int D, int S, int P,
                         int max_pages) {
  if (B < 0 || Hq < 1 || Hkv < 1 || S < 1 || P < 1 || max_pages < 1)
    return fail(WTQ_ERR_ARG, "wtq_decode: bad sizes");
  if (Hq % Hkv) return fail(WTQ_ERR_ARG, "wtq_decode: Hq=%d is not a multiple of Hkv=%d", Hq, Hkv);
  if (D < 1 || D > 256) return fail(WTQ_ERR_ARG, "wtq_decode: need 1 <= head_dim <= 256");
  if (dtype < WTQ_F32 || dtype > WTQ_BF16) return fail(WTQ_ERR_ARG, "wtq_decode: bad dtype");
  if (!k_side || !v_side || !q_strides || !out_strides)
    return fail(WTQ_ERR_ARG, "wtq_decode: null descriptor");
  for (const wtq_side_t *w : {k_side, v_side}) {
    if (!width_supported(w->bw) || (D * w->bw) % 8)
      return fail(WTQ_ERR_ARG, "wtq_decode: bit width %d unsupported for head_dim %d", w->bw, D);
    if (!w->pages || !w->norms || !w->Pi || !w->centroids)
      return fail(WTQ_ERR_ARG, "wtq_decode: null pages, norms, Pi or centroids");
  }
  if (B > 0 && (!q || (!out && !has_exchange) || !page_table || !seq_lens))
    return fail(WTQ_ERR_ARG, "wtq_decode: null input");
  return WTQ_OK;
}

static int decode_common(const void *q, int dtype, const int64_t q_strides[2], void *out,
                         const int64_t out_strides[2], const wtq_exchange_t *exchange,
                         const wtq_side_t *k_side, const wtq_side_t *v_side,
                         const int32_t *page_table, int64_t table_stride, const int32_t *seq_lens,
                         float scale, int B, int Hq, int Hkv, int D, int S, int P, int max_pages,
                         int num_splits, void *workspace, size_t workspace_bytes, int32_t *status,
                         void *stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (int rc = decode_validate(q, dtype, q_strides, out, out_strides, exchange != nullptr, k_side,
                               v_side, page_table, seq_lens, B, Hq, Hkv, D, S, P, max_pages))
    return rc;
  if (B == 0) return WTQ_OK;
  DecodeParams p;
  fill_side(p.k, *k_side, D);
  fill_side(p.v, *v_side, D);
  if (!workspace) return fail(WTQ_ERR_ARG, "wtq_decode: null workspace");
  const int splits = num_splits > 0 ? clamp_splits(num_splits, max_pages, S)
                                    : wtq_decode_auto_splits(B, Hq, Hkv, D, max_pages, S,
                                                             k_side->bw, v_side->bw);
  const size_t need = workspace_for(B, Hq, Hkv, D, splits);
  if (workspace_bytes < need)
    return fail(WTQ_ERR_WORKSPACE, "wtq_decode: workspace %zu < %zu bytes", workspace_bytes, need);

  const size_t rows = (size_t)B * Hq;
  p.work_counter = (int32_t *)workspace;
  int32_t *chunk_prefix = (int32_t *)((char *)workspace + 128);
  p.chunk_prefix = chunk_prefix;
  char *ws = (char *)workspace + wtq_decode_counter_bytes(B, Hkv);
  float *q_rot = (float *)ws;
  ws += round_up(rows * D * sizeof(float), 256);
  p.part_acc = (float *)ws;
  ws += round_up(rows * splits * D * sizeof(float), 256);
  p.part_m = (float *)ws;
  ws += round_up(rows * splits * sizeof(float), 256);
  p.part_l = (float *)ws;
  ws += round_up(rows * splits * sizeof(float), 256);
  p.lut = (const uint32_t *)ws;

  p.q_rot = q_rot;
  p.page_table = page_table;
  p.table_stride = table_stride;
  p.seq_lens = seq_lens;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.n_rep = Hq / Hkv; p.D = D; p.S = S; p.P = P;
  p.max_pages = max_pages; p.num_splits = splits; p.status = status;

  MergeParams m;
  m.part_acc = p.part_acc; m.part_m = p.part_m; m.part_l = p.part_l;
  m.Pi_v = v_side->Pi; m.out = out; m.osb = out_strides[0]; m.osh = out_strides[1];
  m.dtype = dtype; m.Hq = Hq; m.D = D; m.num_splits = splits;
  m.peer_out[0] = m.peer_out[1] = nullptr; m.peer_flags = nullptr;
  m.done_counter = m.step_counter = nullptr;
  m.rank = m.world = m.head_offset = 0;
  if (exchange) {
    if (exchange->world < 1 || exchange->rank < 0 || exchange->rank >= exchange->world ||
        !exchange->peer_out[0] || !exchange->peer_out[1] || !exchange->peer_flags ||
        !exchange->done_counter || !exchange->step_counter)
      return fail(WTQ_ERR_ARG, "wtq_decode_exchange: malformed exchange descriptor");
    m.peer_out[0] = exchange->peer_out[0]; m.peer_out[1] = exchange->peer_out[1];
    m.peer_flags = exchange->peer_flags; m.done_counter = exchange->done_counter;
    m.step_counter = exchange->step_counter; m.rank = exchange->rank; m.world = exchange->world;
    m.head_offset = exchange->head_offset;
  }
  const bool fast = mma_eligible(p) && !force_generic();
  if (exchange && !fast)
    return fail(WTQ_ERR_UNSUPPORTED, "wtq_decode_exchange: this shape runs on the generic kernels, "
                "which have no exchange epilogue; gather with NCCL instead");
  // the tensor-core path works in the exp2 domain: fold log2(e) into the query
  const float q_scale = fast ? scale * 1.4426950408889634f : scale;
  const int max_tokens = max_pages * S;
  m.work_counter = fast ? p.work_counter : nullptr;
  profile_mark_call(stream, true);
  ScanSetup setup = {nullptr, nullptr, nullptr, nullptr, 0, 0, 0};
  if (fast) {
    setup.chunk_prefix = chunk_prefix;
    setup.lut = (uint32_t *)p.lut;
    setup.cent_k = k_side->centroids; setup.cent_v = v_side->centroids;
    setup.bw_k = k_side->bw; setup.bw_v = v_side->bw;
    setup.lut_words = mma_lut_words(k_side->bw, v_side->bw);
  }
  if (int rc = launch_rotate_q(q, dtype, q_strides, k_side->Pi, q_scale, B, Hq, D, q_rot, seq_lens,
                               fast ? mma_chunk_tokens(max_tokens, splits) : 1, max_tokens, setup,
                               stream))
    return rc;
  int rc = 0;
  if (fast) {
    rc = launch_decode_mma(p, m, stream);
  } else {
    rc = launch_decode_generic(p, stream);
    if (rc == 0) rc = launch_merge(m, B, stream);
  }
  profile_mark_call(stream, false);
  return rc;
}

extern "C" int wtq_decode(const void *q, int dtype, const int64_t q_strides[2], void *out,
                          const int64_t out_strides[2], const wtq_side_t *k_side,
                          const wtq_side_t *v_side, const int32_t *page_table,
                          int64_t table_stride, const int32_t *seq_lens, float scale, int B,
                          int Hq, int Hkv, int D, int S, int P, int max_pages, int num_splits,
                          void *workspace, size_t workspace_bytes, int32_t *status,
                          void *stream) {
  if (!out || !out_strides) return fail(WTQ_ERR_ARG, "wtq_decode: null output");
  return decode_common(q, dtype, q_strides, out, out_strides, nullptr, k_side, v_side, page_table,
                       table_stride, seq_lens, scale, B, Hq, Hkv, D, S, P, max_pages, num_splits,
                       workspace, workspace_bytes, status, stream);
}

extern "C" int wtq_decode_exchange(const void *q, int dtype, const int64_t q_strides[2],
                                   const wtq_exchange_t *exchange, const wtq_side_t *k_side,
                                   const wtq_side_t *v_side, const int32_t *page_table,
                                   int64_t table_stride, const int32_t *seq_lens, float scale,
                                   int B, int Hq, int Hkv, int D, int S, int P, int max_pages,
                                   int num_splits, void *workspace, size_t workspace_bytes,
                                   int32_t *status, void *stream) {
  if (!exchange) return fail(WTQ_ERR_ARG, "wtq_decode_exchange: null exchange descriptor");
  return decode_common(q, dtype, q_strides, nullptr, exchange->out_strides, exchange, k_side,
                       v_side, page_table, table_stride, seq_lens, scale, B, Hq, Hkv, D, S, P,
                       max_pages, num_splits, workspace, workspace_bytes, status, stream);
}

extern "C" int wtq_exchange_wait(const uint32_t *local_flags, int world, uint32_t *step_counter,
                                 int64_t spin_limit, int32_t *status, void *stream) {
  if (!local_flags || !step_counter || world < 1 || world > 32 || spin_limit < 1)
    return fail(WTQ_ERR_ARG, "wtq_exchange_wait: need flags, 1 <= world <= 32, spin_limit >= 1");
  return launch_exchange_wait(local_flags, world, step_counter, spin_limit, status,
                              (cudaStream_t)stream);
}

// ---- measurement aids ---------------------------------------------------------
// Plain streaming read of `bytes` bytes (16-byte loads, grid-stride, every byte
// once): the read-only HBM ceiling that the page scan is compared with beside
// the copy bandwidth.  Same role as the streaming control of the reference's
// kernel study (experiments/c27/controls.cu:15-36).
namespace {
__global__ void __launch_bounds__(256) stream_read_kernel(const uint4 *src, size_t n16,
                                                          uint32_t *sink) {
  uint32_t x = 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {          // four loads in flight per thread
    const uint4 a = __ldcs(src + i), b = __ldcs(src + i + stride);
    const uint4 c = __ldcs(src + i + 2 * stride), d = __ldcs(src + i + 3 * stride);
    x ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
  }
  for (; i < n16; i += stride) {
    const uint4 a = __ldcs(src + i);
    x ^= a.x ^ a.y ^ a.z ^ a.w;
  }
  if (x == 0x9e3779b9u && sink != nullptr) atomicXor(sink, x);   // keeps the loads alive
}
}  // namespace

extern "C" int wtq_probe_read(const void *src, size_t bytes, uint32_t *sink, void *stream) {
  if (!src || ((uintptr_t)src & 15) || bytes < 16)
    return fail(WTQ_ERR_ARG, "wtq_probe_read: need a 16-byte aligned buffer of at least 16 bytes");
  const int sms = device_sms();
  stream_read_kernel<<<sms * 8, 256, 0, (cudaStream_t)stream>>>((const uint4 *)src, bytes / 16, sink);
  note_launches(1);
  return check_cuda(cudaGetLastError(), "wtq_probe_read launch");
}

// Whether wtq_decode_exchange has its fused epilogue for these descriptors: the
// same test the call itself applies (shape, widths, alignment of every pointer
// and stride, and the environment switch that forces the generic kernels),
// without launching anything.  1 = yes, 0 = no (gather with NCCL instead).
extern "C" int wtq_decode_exchange_supported(const wtq_side_t *k_side, const wtq_side_t *v_side,
                                             int Hq, int Hkv, int D, int S,
                                             const void *workspace) {
  if (!k_side || !v_side || Hkv < 1 || Hq < 1 || Hq % Hkv || !workspace) return 0;
  DecodeParams p = {};
  fill_side(p.k, *k_side, D);
  fill_side(p.v, *v_side, D);
  p.D = D; p.S = S; p.n_rep = Hq / Hkv;
  p.q_rot = (const float *)workspace; p.part_acc = (float *)workspace;
  p.lut = (const uint32_t *)workspace;
  return mma_eligible(p) && !force_generic() ? 1 : 0;
}
