// Row-wise glue that feeds the quantised matmuls: residual add + RMSNorm, and SwiGLU, each also writing the fp32 sums of
// its bf16 output over the quantisation groups (the matmul's `xs` input), so the rows make one trip through memory.
// A row is handled by one block in a fixed order of operations: its bits never depend on how many rows share the call.
// Replaces the Triton `_add_rmsnorm` and `_swiglu` of families/qwen3_5/cuda/glue.py:10-40,130-151.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tensorfold_b200.h"

namespace tf {

int fail_moe(int code, const char* msg);
int cuda_fail_moe(cudaError_t e, const char* what);

namespace {

constexpr int GLUE_THREADS = 256;

__device__ __forceinline__ void unpack8(const uint4& q, float (&v)[8]) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(u[i] << 16);
    v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
  }
}

// Rounds eight floats to bf16, returns them packed and leaves the rounded values in v.
__device__ __forceinline__ uint4 pack8(float (&v)[8]) {
  uint32_t u[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    u[i] = *reinterpret_cast<const uint32_t*>(&t);
    v[2 * i] = __uint_as_float(u[i] << 16);
    v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
  }
  return make_uint4(u[0], u[1], u[2], u[3]);
}

// Sum of the eight values of a thread, then over the `lanes` consecutive lanes that hold one quantisation group
// (a butterfly: every lane of the group ends with the same sum).  All 32 lanes of the warp call it.
__device__ __forceinline__ float group_sum(const float (&v)[8], int lanes) {
  float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
  for (int m = 1; m < lanes; m <<= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, m);
  return s;
}

// One block per row.  Pass 1: h = bf16(x + r) (stored when r is given), sum of h^2 per thread over its 8-element pieces
// in order, then a shuffle tree inside each warp and the warps' sums added in warp order.  Pass 2: y = bf16(h * inv * w)
// and the group sums of y.
__global__ void __launch_bounds__(GLUE_THREADS) add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ r,
                                                                   const __nv_bfloat16* __restrict__ w, int d, float eps,
                                                                   __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ y,
                                                                   float* __restrict__ xs, int gs) {
  __shared__ float warp_ss[GLUE_THREADS / 32];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pieces = d / 8, rounds = (pieces + GLUE_THREADS - 1) / GLUE_THREADS;
  const uint4* x8 = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * d);
  const uint4* r8 = r ? reinterpret_cast<const uint4*>(r + static_cast<int64_t>(row) * d) : nullptr;
  uint4* h8 = h ? reinterpret_cast<uint4*>(h + static_cast<int64_t>(row) * d) : nullptr;
  float ss = 0.f;
  for (int it = 0; it < rounds; ++it) {
    const int c = it * GLUE_THREADS + tid;
    if (c < pieces) {
      float v[8];
      unpack8(x8[c], v);
      if (r8) {
        float rv[8];
        unpack8(r8[c], rv);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += rv[i];
        h8[c] = pack8(v);                                    // v now holds the rounded sums
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
    }
  }
  for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, m);
  if (lane == 0) warp_ss[warp] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < GLUE_THREADS / 32; ++i) total += warp_ss[i];
  const float inv = 1.0f / sqrtf(total / static_cast<float>(d) + eps);

  const uint4* src = r8 ? reinterpret_cast<const uint4*>(h8) : x8;   // this thread wrote the pieces of h it reads back
  const uint4* w8 = reinterpret_cast<const uint4*>(w);
  uint4* y8 = reinterpret_cast<uint4*>(y + static_cast<int64_t>(row) * d);
  const int lanes = gs / 8;
  for (int it = 0; it < rounds; ++it) {
    const int c = it * GLUE_THREADS + tid;
    float v[8] = {};
    if (c < pieces) {
      float wv[8];
      unpack8(src[c], v);
      unpack8(w8[c], wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * wv[i];
      y8[c] = pack8(v);
    }
    const float s = group_sum(v, lanes);
    if (xs && c < pieces && (lane & (lanes - 1)) == 0) xs[static_cast<int64_t>(row) * (d / gs) + c / lanes] = s;
  }
}

// out = bf16(g * sigmoid(g) * u) in fp32 from bf16 inputs, one rounding; group sums of out.  Block (x, row).
__global__ void __launch_bounds__(GLUE_THREADS) swiglu_kernel(const __nv_bfloat16* __restrict__ gate,
                                                              const __nv_bfloat16* __restrict__ up, int n,
                                                              __nv_bfloat16* __restrict__ out, float* __restrict__ xs, int gs) {
  const int row = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
  const int pieces = n / 8, lanes = gs / 8;
  const int c = blockIdx.x * GLUE_THREADS + tid;
  float v[8] = {};
  if (c < pieces) {
    float g[8], u[8];
    unpack8(reinterpret_cast<const uint4*>(gate + static_cast<int64_t>(row) * n)[c], g);
    unpack8(reinterpret_cast<const uint4*>(up + static_cast<int64_t>(row) * n)[c], u);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = g[i] * (1.0f / (1.0f + expf(-g[i]))) * u[i];
    reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * n)[c] = pack8(v);
  }
  const float s = group_sum(v, lanes);
  if (xs && c < pieces && (lane & (lanes - 1)) == 0) xs[static_cast<int64_t>(row) * (n / gs) + c / lanes] = s;
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

}  // namespace tf

using namespace tf;

extern "C" {

int tf_add_rmsnorm(const void* x, const void* r, const void* w, int rows, int d, float eps, void* h, void* y, float* xs,
                   int gs, void* stream) {
  if (rows < 1 || d < 8 || !x || !w || !y || (r && !h)) return fail_moe(TF_ERR_ARG, "tf_add_rmsnorm: bad arguments");
  if (gs != 32 && gs != 64 && gs != 128) return fail_moe(TF_ERR_ARG, "tf_add_rmsnorm: groups of 32, 64 or 128");
  if (d % gs) return fail_moe(TF_ERR_ARG, "tf_add_rmsnorm: the row length must be a multiple of the group");
  if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (r && (!aligned16(r) || !aligned16(h))))
    return fail_moe(TF_ERR_ALIGN, "tf_add_rmsnorm: tensors must be 16-byte aligned");
  add_rmsnorm_kernel<<<rows, GLUE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(r), static_cast<const __nv_bfloat16*>(w), d, eps,
      static_cast<__nv_bfloat16*>(r ? h : nullptr), static_cast<__nv_bfloat16*>(y), xs, gs);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_add_rmsnorm");
}

int tf_swiglu(const void* gate, const void* up, int rows, int n, void* out, float* xs, int gs, void* stream) {
  if (rows < 1 || rows > 65535 || n < 8 || !gate || !up || !out) return fail_moe(TF_ERR_ARG, "tf_swiglu: bad arguments");
  if (gs != 32 && gs != 64 && gs != 128) return fail_moe(TF_ERR_ARG, "tf_swiglu: groups of 32, 64 or 128");
  if (n % gs) return fail_moe(TF_ERR_ARG, "tf_swiglu: the row length must be a multiple of the group");
  if (!aligned16(gate) || !aligned16(up) || !aligned16(out)) return fail_moe(TF_ERR_ALIGN, "tf_swiglu: tensors must be 16-byte aligned");
  dim3 grid((n / 8 + GLUE_THREADS - 1) / GLUE_THREADS, rows);
  swiglu_kernel<<<grid, GLUE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up), n, static_cast<__nv_bfloat16*>(out), xs, gs);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_swiglu");
}

}  // extern "C"
