// Parameter blocks shared by the decode kernels and their host launcher.
#pragma once

#include "wtq_common.cuh"

namespace wtq {

constexpr int kMaxSplits = 1024;

struct DecodeSideDev {
  const uint8_t *pages;
  const __half *norms;
  int64_t page_stride, head_stride;            // bytes
  int64_t norm_page_stride, norm_head_stride;  // elements
  const float *Pi;
  const float *centroids;
  int bw, nb;
};

struct DecodeParams {
  DecodeSideDev k, v;
  const float *q_rot;  // (B, Hq, D) fp32, already scaled
  const int32_t *page_table;
  int64_t table_stride;
  const int32_t *seq_lens;
  int B, Hq, Hkv, n_rep, D, S, P, max_pages, num_splits;
  float *part_acc;  // (B, Hq, splits, D)
  float *part_m;    // (B, Hq, splits)
  float *part_l;
  int32_t *status;
  // tensor-core path: work queue (one int, zero between calls) and the exclusive
  // prefix of chunks per sequence (B + 1 ints), both inside the workspace's
  // counter block
  int32_t *work_counter;
  const int32_t *chunk_prefix;
  // tensor-core path: the lookup tables in the layout the scan kernel keeps in
  // shared memory, [index][key | value][lane] words, built by the rotation kernel
  const uint32_t *lut;
};

// Table words the tensor-core scan wants for widths (bw_k, bw_v); 0 when the
// pair has no tensor-core kernel.
int mma_lut_words(int bw_k, int bw_v);

// What the query-rotation launch also prepares for the tensor-core scan (all
// optional): the exclusive prefix of ceil(seq_len / chunk_tokens) over the B
// sequences (B + 1 ints), and the lookup tables.
struct ScanSetup {
  int32_t *chunk_prefix;
  uint32_t *lut;
  const float *cent_k, *cent_v;
  int bw_k, bw_v, lut_words;
};

struct MergeParams {
  const float *part_acc, *part_m, *part_l;
  const float *Pi_v;
  void *out;
  int64_t osb, osh;
  int dtype, Hq, D, num_splits;
  int32_t *work_counter;   // reset to zero by the merge (null on the generic path)
  // output exchange of KV-head tensor parallelism (world == 0: plain local store)
  void *const *peer_out[2];
  uint32_t *const *peer_flags;
  uint32_t *done_counter, *step_counter;
  int rank, world, head_offset;
};

// Argument checks of the decode entry points (wtq_api.cu); WTQ_OK or an error
// code with the text set.
int decode_validate(const void *q, int dtype, const int64_t q_strides[2], const void *out,
                    const int64_t out_strides[2], bool has_exchange, const wtq_side_t *k_side,
                    const wtq_side_t *v_side, const int32_t *page_table, const int32_t *seq_lens,
                    int B, int Hq, int Hkv, int D, int S, int P, int max_pages);

int launch_rotate_q(const void *q, int dtype, const int64_t *q_strides, const float *Pi,
                    float scale, int B, int Hq, int D, float *q_rot, const int32_t *seq_lens,
                    int chunk_tokens, int max_tokens, const ScanSetup &setup, cudaStream_t stream);
int launch_decode_generic(const DecodeParams &p, cudaStream_t stream);
int launch_merge(const MergeParams &p, int B, cudaStream_t stream);

// head_dim 128 tensor-core path (wtq_decode_mma.cu).  In that path `num_splits`
// counts chunks of mma_chunk_tokens() tokens per sequence, the partial m values
// are in the log2 domain and q_rot carries scale * log2(e).
int mma_warps_per_sm(int bw_k, int bw_v);
bool mma_eligible(const DecodeParams &p);
int mma_chunk_tokens(int max_tokens, int splits);
int launch_decode_mma(const DecodeParams &p, const MergeParams &m, cudaStream_t stream);
int launch_mma_merge(const MergeParams &m, const int32_t *seq_lens, int B, int Hkv, int n_rep,
                     int chunk_tokens, int max_tokens, cudaStream_t stream);
// Tensor-core forms of the query rotation and of the chunk merge for calls with
// thousands of rows (wtq_rows_mma.cu); the *_eligible functions say whether a
// call qualifies (contiguous rows of 128, at least 4096 of them, 16-byte aligned
// buffers; the merge also: at most 8 chunks per row, no exchange).
bool rows_mma_rotate_eligible(const void *q, int64_t row_stride, int64_t head_stride, int Hq, int D,
                              int64_t rows, const float *Pi, const float *q_rot);
int launch_rotate_rows_mma(const void *q, int dtype, const float *Pi, float mult, int64_t rows,
                           float *q_rot, const ScanSetup &setup, int32_t *status, cudaStream_t stream);
bool rows_mma_merge_eligible(const MergeParams &m, int64_t rows);
int launch_merge_rows_mma(const MergeParams &m, const int32_t *row_lens, int64_t rows, int chunk_tokens,
                          int max_tokens, int32_t *status, cudaStream_t stream);
int launch_exchange_wait(const uint32_t *flags, int world, uint32_t *state, long long spin_limit,
                         int32_t *status, cudaStream_t stream);

}  // namespace wtq
