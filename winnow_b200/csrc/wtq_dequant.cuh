// Parameter block and launchers shared by the dequantisation kernels.
#pragma once

#include "wtq_common.cuh"

namespace wtq {

struct DequantParams {
  const uint8_t *packed;
  const __half *norms;
  const float *centroids, *Pi;
  void *out;
  int out_dtype, bw, D, nb;
  int64_t N, L, MAXLEN;
};

// tcgen05 kernel (wtq_dequant_umma.cu); `terms` = 1 or 3.  *usable = false and
// nothing launched when the kernel cannot serve this call here.
int launch_dequant_umma(const DequantParams &p, int terms, cudaStream_t stream, bool *usable);
int dequant_umma_gave_up();

}  // namespace wtq
