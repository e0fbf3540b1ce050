// Instantiates qmm_stream_kernel for one bit width (TF_BITS) over every group size and lane count (1, 2 or 4
// super-blocks a block) that fits an SM's shared and tensor memory.
#include "qmm_stream_launch.h"

#ifndef TF_BITS
#error "compile with -DTF_BITS=<2|3|4|5|6>"
#endif

namespace tf {

namespace {

template <int GS, int KW>
cudaError_t launch(const CUtensorMap& tmx, const StreamParams& p, int grid, cudaStream_t stream, bool pdl) {
  using Geo = StreamGeo<TF_BITS, GS, KW>;
  if constexpr (!Geo::FITS) {
    return cudaErrorInvalidConfiguration;
  } else {
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
    return cudaLaunchKernelEx(&cfg, qmm_stream_kernel<TF_BITS, GS, KW>, tmx, p);
  }
}

template <int GS, int KW>
cudaError_t configure() {
  using Geo = StreamGeo<TF_BITS, GS, KW>;
  if constexpr (!Geo::FITS) {
    return cudaSuccess;
  } else {
    return cudaFuncSetAttribute(qmm_stream_kernel<TF_BITS, GS, KW>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo::SMEM);
  }
}

// Blocks of that shape an SM holds: the design figure.  The launch bounds guarantee the registers and the static
// assertion the shared memory for that many; the runtime's occupancy query answers 1 for any kernel that allocates
// tensor memory, whatever it allocates, so it only serves to tell whether the kernel can be launched at all.
template <int GS, int KW>
int resident() {
  using Geo = StreamGeo<TF_BITS, GS, KW>;
  if constexpr (!Geo::FITS) {
    return 0;
  } else {
    static_assert(Geo::BLOCKS * (Geo::SMEM + 1024) <= 228 * 1024, "the resident blocks fit the shared memory of an SM");
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, qmm_stream_kernel<TF_BITS, GS, KW>, Geo::THREADS, Geo::SMEM) != cudaSuccess)
      return 0;
    return blocks < 1 ? 0 : Geo::BLOCKS;
  }
}

template <int GS>
cudaError_t launch_gs(const CUtensorMap& tmx, const StreamParams& p, int kw, int grid, cudaStream_t stream, bool pdl) {
  switch (kw) {
    case 1: return launch<GS, 1>(tmx, p, grid, stream, pdl);
    case 2: return launch<GS, 2>(tmx, p, grid, stream, pdl);
    case 4: return launch<GS, 4>(tmx, p, grid, stream, pdl);
    default: return cudaErrorInvalidValue;
  }
}

template <int GS>
int resident_gs(int kw) {
  switch (kw) {
    case 1: return resident<GS, 1>();
    case 2: return resident<GS, 2>();
    case 4: return resident<GS, 4>();
    default: return 0;
  }
}

template <int GS>
cudaError_t configure_gs() {
  cudaError_t e = configure<GS, 1>();
  if (e == cudaSuccess) e = configure<GS, 2>();
  if (e == cudaSuccess) e = configure<GS, 4>();
  return e;
}

}  // namespace

#define TF_CAT2(a, b) a##b
#define TF_CAT(a, b) TF_CAT2(a, b)

cudaError_t TF_CAT(qmm_stream_launch_b, TF_BITS)(const CUtensorMap& tmx, const StreamParams& p, int gs, int kw, int grid,
                                                 cudaStream_t stream, bool pdl) {
  switch (gs) {
    case 32: return launch_gs<32>(tmx, p, kw, grid, stream, pdl);
    case 64: return launch_gs<64>(tmx, p, kw, grid, stream, pdl);
    case 128: return launch_gs<128>(tmx, p, kw, grid, stream, pdl);
    default: return cudaErrorInvalidValue;
  }
}

int TF_CAT(qmm_stream_resident_b, TF_BITS)(int gs, int kw) {
  switch (gs) {
    case 32: return resident_gs<32>(kw);
    case 64: return resident_gs<64>(kw);
    case 128: return resident_gs<128>(kw);
    default: return 0;
  }
}

cudaError_t TF_CAT(qmm_stream_configure_b, TF_BITS)() {
  cudaError_t e = configure_gs<32>();
  if (e == cudaSuccess) e = configure_gs<64>();
  if (e == cudaSuccess) e = configure_gs<128>();
  return e;
}

}  // namespace tf
