// Instantiates qmm_tiled_kernel for one bit width (TF_BITS) over every group size and row tile.
#include "qmm_launch.h"

#ifndef TF_BITS
#error "compile with -DTF_BITS=<2|3|4|5|6|8>"
#endif

namespace tf {

namespace {

template <int GS, int MT>
cudaError_t launch(const QmmParams& p, cudaStream_t stream, bool pdl) {
  using Geo = QmmGeo<TF_BITS, GS, MT>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + SB_COLS - 1) / SB_COLS, (p.M + Geo::ROWS - 1) / Geo::ROWS, p.sk);
  cfg.blockDim = dim3(QMM_THREADS);
  cfg.dynamicSmemBytes = Geo::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (p.cluster && p.sk > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 1;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = p.sk;
    ++na;
  }
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, qmm_tiled_kernel<TF_BITS, GS, MT>, p);
}

template <int GS, int MT>
cudaError_t configure() {
  return cudaFuncSetAttribute(qmm_tiled_kernel<TF_BITS, GS, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              QmmGeo<TF_BITS, GS, MT>::SMEM);
}

template <int GS>
cudaError_t launch_gs(const QmmParams& p, int mt, cudaStream_t stream, bool pdl) {
  switch (mt) {
    case 1: return launch<GS, 1>(p, stream, pdl);
    case 2: return launch<GS, 2>(p, stream, pdl);
    case 4: return launch<GS, 4>(p, stream, pdl);
    case 8: return launch<GS, 8>(p, stream, pdl);
    default: return cudaErrorInvalidValue;
  }
}

template <int GS>
cudaError_t configure_gs() {
  cudaError_t e = configure<GS, 1>();
  if (e == cudaSuccess) e = configure<GS, 2>();
  if (e == cudaSuccess) e = configure<GS, 4>();
  if (e == cudaSuccess) e = configure<GS, 8>();
  return e;
}

}  // namespace

#define TF_CAT2(a, b) a##b
#define TF_CAT(a, b) TF_CAT2(a, b)

cudaError_t TF_CAT(qmm_launch_b, TF_BITS)(const QmmParams& p, int gs, int mt, cudaStream_t stream, bool pdl) {
  switch (gs) {
    case 32: return launch_gs<32>(p, mt, stream, pdl);
    case 64: return launch_gs<64>(p, mt, stream, pdl);
    case 128: return launch_gs<128>(p, mt, stream, pdl);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t TF_CAT(qmm_configure_b, TF_BITS)() {
  cudaError_t e = configure_gs<32>();
  if (e == cudaSuccess) e = configure_gs<64>();
  if (e == cudaSuccess) e = configure_gs<128>();
  return e;
}

}  // namespace tf
