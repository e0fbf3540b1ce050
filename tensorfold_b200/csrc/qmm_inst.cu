// Instantiates qmm_tiled_kernel for one bit width (TF_BITS) over every group size, row tile and lane count.
#include "qmm_launch.h"

#ifndef TF_BITS
#error "compile with -DTF_BITS=<2|3|4|5|6|8>"
#endif

namespace tf {

namespace {

template <int GS, int MT, int KW>
cudaError_t launch(const CUtensorMap& tmx, const QmmParams& p, cudaStream_t stream, bool pdl) {
  using Geo = QmmGeo<TF_BITS, GS, MT, KW>;
  const int nblocks = p.sk;
  const int nsb = (p.N + SB_COLS - 1) / SB_COLS;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((nsb + KW - 1) / KW, p.items != nullptr ? p.M : (p.M + Geo::ROWS - 1) / Geo::ROWS, nblocks);   // grouped: M = plan capacity in items
  cfg.blockDim = dim3(Geo::THREADS);
  cfg.dynamicSmemBytes = Geo::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (p.cluster && nblocks > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 1;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = nblocks;
    ++na;
  }
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, qmm_tiled_kernel<TF_BITS, GS, MT, KW>, tmx, p);
}

template <int GS, int MT, int KW>
cudaError_t configure() {
  return cudaFuncSetAttribute(qmm_tiled_kernel<TF_BITS, GS, MT, KW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              QmmGeo<TF_BITS, GS, MT, KW>::SMEM);
}

template <int GS>
cudaError_t launch_gs(const CUtensorMap& tmx, const QmmParams& p, int mt, int kw, cudaStream_t stream, bool pdl) {
  switch (mt * 10 + kw) {
    case 11: return launch<GS, 1, 1>(tmx, p, stream, pdl);
    case 12: return launch<GS, 1, 2>(tmx, p, stream, pdl);
    case 14: return launch<GS, 1, 4>(tmx, p, stream, pdl);
    case 21: return launch<GS, 2, 1>(tmx, p, stream, pdl);
    case 22: return launch<GS, 2, 2>(tmx, p, stream, pdl);
    case 24: return launch<GS, 2, 4>(tmx, p, stream, pdl);
    case 41: return launch<GS, 4, 1>(tmx, p, stream, pdl);
    case 42: return launch<GS, 4, 2>(tmx, p, stream, pdl);
    case 81: return launch<GS, 8, 1>(tmx, p, stream, pdl);
    default: return cudaErrorInvalidValue;
  }
}

template <int GS>
cudaError_t configure_gs() {
  cudaError_t e = configure<GS, 1, 1>();
  if (e == cudaSuccess) e = configure<GS, 1, 2>();
  if (e == cudaSuccess) e = configure<GS, 1, 4>();
  if (e == cudaSuccess) e = configure<GS, 2, 1>();
  if (e == cudaSuccess) e = configure<GS, 2, 2>();
  if (e == cudaSuccess) e = configure<GS, 2, 4>();
  if (e == cudaSuccess) e = configure<GS, 4, 1>();
  if (e == cudaSuccess) e = configure<GS, 4, 2>();
  if (e == cudaSuccess) e = configure<GS, 8, 1>();
  return e;
}

}  // namespace

#define TF_CAT2(a, b) a##b
#define TF_CAT(a, b) TF_CAT2(a, b)

cudaError_t TF_CAT(qmm_launch_b, TF_BITS)(const CUtensorMap& tmx, const QmmParams& p, int gs, int mt, int kw, cudaStream_t stream, bool pdl) {
  switch (gs) {
    case 32: return launch_gs<32>(tmx, p, mt, kw, stream, pdl);
    case 64: return launch_gs<64>(tmx, p, mt, kw, stream, pdl);
    case 128: return launch_gs<128>(tmx, p, mt, kw, stream, pdl);
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
