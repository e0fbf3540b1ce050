// Instantiates qmm_stream_kernel for one bit width (TF_BITS) over every group size, row tile (8 or 16 rows) and lane
// count (1, 2 or 4 super-blocks a block).
#include "qmm_stream_launch.h"

#ifndef TF_BITS
#error "compile with -DTF_BITS=<2|3|4|5|6|8>"
#endif

namespace tf {

namespace {

template <int GS, int MT, int KW>
cudaError_t launch(const CUtensorMap& tmx, const StreamParams& p, int grid, cudaStream_t stream, bool pdl) {
  using Geo = StreamGeo<TF_BITS, GS, MT, KW>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(Geo::THREADS);
  cfg.dynamicSmemBytes = Geo::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, qmm_stream_kernel<TF_BITS, GS, MT, KW>, tmx, p);
}

template <int GS, int MT, int KW>
cudaError_t configure() {
  return cudaFuncSetAttribute(qmm_stream_kernel<TF_BITS, GS, MT, KW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              StreamGeo<TF_BITS, GS, MT, KW>::SMEM);
}

template <int GS, int MT, int KW>
int resident() {
  using Geo = StreamGeo<TF_BITS, GS, MT, KW>;
  int blocks = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, qmm_stream_kernel<TF_BITS, GS, MT, KW>, Geo::THREADS, Geo::SMEM) !=
      cudaSuccess)
    return 0;
  return blocks;
}

#define TF_STREAM_CASES(CALL)          \
  switch (mt * 10 + kw) {              \
    case 11: return CALL(GS, 1, 1);    \
    case 12: return CALL(GS, 1, 2);    \
    case 14: return CALL(GS, 1, 4);    \
    case 21: return CALL(GS, 2, 1);    \
    case 22: return CALL(GS, 2, 2);    \
    case 24: return CALL(GS, 2, 4);    \
    default: break;                    \
  }

template <int GS>
cudaError_t launch_gs(const CUtensorMap& tmx, const StreamParams& p, int mt, int kw, int grid, cudaStream_t stream, bool pdl) {
#define TF_CALL(G_, M_, K_) launch<G_, M_, K_>(tmx, p, grid, stream, pdl)
  TF_STREAM_CASES(TF_CALL)
#undef TF_CALL
  return cudaErrorInvalidValue;
}

template <int GS>
int resident_gs(int mt, int kw) {
#define TF_CALL(G_, M_, K_) resident<G_, M_, K_>()
  TF_STREAM_CASES(TF_CALL)
#undef TF_CALL
  return 0;
}

template <int GS>
cudaError_t configure_gs() {
  cudaError_t e = configure<GS, 1, 1>();
  if (e == cudaSuccess) e = configure<GS, 1, 2>();
  if (e == cudaSuccess) e = configure<GS, 1, 4>();
  if (e == cudaSuccess) e = configure<GS, 2, 1>();
  if (e == cudaSuccess) e = configure<GS, 2, 2>();
  if (e == cudaSuccess) e = configure<GS, 2, 4>();
  return e;
}

#if TF_BITS == 4
// The grouped (mixture-of-experts) form: expert tables are 4-bit; one lane a block, 8 or 16 rows an item.
template <int GS, int MT>
cudaError_t launch_grouped(const StreamParams& p, int grid, cudaStream_t stream, bool pdl) {
  using Geo = StreamGeo<4, GS, MT, 1>;
  static const CUtensorMap none = {};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(Geo::THREADS);
  cfg.dynamicSmemBytes = Geo::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, qmm_stream_kernel<4, GS, MT, 1, true>, none, p);
}

template <int GS, int MT>
int resident_grouped() {
  using Geo = StreamGeo<4, GS, MT, 1>;
  int blocks = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, qmm_stream_kernel<4, GS, MT, 1, true>, Geo::THREADS, Geo::SMEM) != cudaSuccess)
    return 0;
  return blocks;
}

template <int GS, int MT>
cudaError_t configure_grouped() {
  return cudaFuncSetAttribute(qmm_stream_kernel<4, GS, MT, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              StreamGeo<4, GS, MT, 1>::SMEM);
}
#endif

}  // namespace

#define TF_CAT2(a, b) a##b
#define TF_CAT(a, b) TF_CAT2(a, b)

cudaError_t TF_CAT(qmm_stream_launch_b, TF_BITS)(const CUtensorMap& tmx, const StreamParams& p, int gs, int mt, int kw, int grid,
                                                 cudaStream_t stream, bool pdl) {
  switch (gs) {
    case 32: return launch_gs<32>(tmx, p, mt, kw, grid, stream, pdl);
    case 64: return launch_gs<64>(tmx, p, mt, kw, grid, stream, pdl);
    case 128: return launch_gs<128>(tmx, p, mt, kw, grid, stream, pdl);
    default: return cudaErrorInvalidValue;
  }
}

int TF_CAT(qmm_stream_resident_b, TF_BITS)(int gs, int mt, int kw) {
  switch (gs) {
    case 32: return resident_gs<32>(mt, kw);
    case 64: return resident_gs<64>(mt, kw);
    case 128: return resident_gs<128>(mt, kw);
    default: return 0;
  }
}

cudaError_t TF_CAT(qmm_stream_configure_b, TF_BITS)() {
  cudaError_t e = configure_gs<32>();
  if (e == cudaSuccess) e = configure_gs<64>();
  if (e == cudaSuccess) e = configure_gs<128>();
#if TF_BITS == 4
  if (e == cudaSuccess) e = configure_grouped<32, 1>();
  if (e == cudaSuccess) e = configure_grouped<32, 2>();
  if (e == cudaSuccess) e = configure_grouped<64, 1>();
  if (e == cudaSuccess) e = configure_grouped<64, 2>();
  if (e == cudaSuccess) e = configure_grouped<128, 1>();
  if (e == cudaSuccess) e = configure_grouped<128, 2>();
#endif
  return e;
}

#if TF_BITS == 4
cudaError_t qmm_stream_grouped_launch(const StreamParams& p, int gs, int mt, int grid, cudaStream_t stream, bool pdl) {
  switch (gs * 10 + mt) {
    case 321: return launch_grouped<32, 1>(p, grid, stream, pdl);
    case 322: return launch_grouped<32, 2>(p, grid, stream, pdl);
    case 641: return launch_grouped<64, 1>(p, grid, stream, pdl);
    case 642: return launch_grouped<64, 2>(p, grid, stream, pdl);
    case 1281: return launch_grouped<128, 1>(p, grid, stream, pdl);
    case 1282: return launch_grouped<128, 2>(p, grid, stream, pdl);
    default: return cudaErrorInvalidValue;
  }
}

int qmm_stream_grouped_resident(int gs, int mt) {
  switch (gs * 10 + mt) {
    case 321: return resident_grouped<32, 1>();
    case 322: return resident_grouped<32, 2>();
    case 641: return resident_grouped<64, 1>();
    case 642: return resident_grouped<64, 2>();
    case 1281: return resident_grouped<128, 1>();
    case 1282: return resident_grouped<128, 2>();
    default: return 0;
  }
}
#endif

}  // namespace tf
