// Host-side launch interface of the tiled matmul kernels; one translation unit per bit width (qmm_inst.cu compiled
// with -DTF_BITS=b) keeps the build parallel.
#pragma once

#include <cuda_runtime.h>

#include "qmm_tiled.cuh"

namespace tf {

// Row-tile shape for a row count: 8, 16, 32 or 64 rows per block (1, 2, 4 or 8 m8 tiles).
inline int mt_for_rows(int m) { return m <= 8 ? 1 : m <= 16 ? 2 : m <= 32 ? 4 : 8; }
// Slice lanes a block may hold for a row tile: up to 4 for 8 or 16 rows, 2 for 32 rows, 1 for 64 rows.
inline int max_lanes(int mt) { return mt <= 2 ? 4 : mt == 4 ? 2 : 1; }

#define TF_DECLARE_BITS(B)                                                                        \
  cudaError_t qmm_launch_b##B(const CUtensorMap& tmx, const QmmParams& p, int gs, int mt, int kw, cudaStream_t stream, bool pdl); \
  cudaError_t qmm_configure_b##B();
TF_DECLARE_BITS(2)
TF_DECLARE_BITS(3)
TF_DECLARE_BITS(4)
TF_DECLARE_BITS(5)
TF_DECLARE_BITS(6)
TF_DECLARE_BITS(8)
#undef TF_DECLARE_BITS

}  // namespace tf
