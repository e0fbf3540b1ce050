// Host-side launch interface of the persistent (streaming) matmul kernels; one translation unit per bit width
// (qmm_stream_inst.cu compiled with -DTF_BITS=b).
#pragma once

#include <cuda_runtime.h>

#include "qmm_stream.cuh"

namespace tf {

#define TF_DECLARE_STREAM_BITS(B)                                                                                          \
  cudaError_t qmm_stream_launch_b##B(const CUtensorMap& tmx, const StreamParams& p, int gs, int mt, int kw, int grid,      \
                                     cudaStream_t stream, bool pdl);                                                       \
  int qmm_stream_resident_b##B(int gs, int mt, int kw); /* blocks of that shape an SM holds (0: the query failed) */       \
  cudaError_t qmm_stream_configure_b##B();
TF_DECLARE_STREAM_BITS(2)
TF_DECLARE_STREAM_BITS(3)
TF_DECLARE_STREAM_BITS(4)
TF_DECLARE_STREAM_BITS(5)
TF_DECLARE_STREAM_BITS(6)
TF_DECLARE_STREAM_BITS(8)
#undef TF_DECLARE_STREAM_BITS

// The grouped (mixture-of-experts) form, 4-bit tables: mt = 1 (items of up to 8 rows) or 2 (16 rows).
cudaError_t qmm_stream_grouped_launch(const StreamParams& p, int gs, int mt, int grid, cudaStream_t stream, bool pdl);
int qmm_stream_grouped_resident(int gs, int mt);

}  // namespace tf
