// extern "C" entry points (include/tensorfold_b200.h), argument checks, and the small kernels around the matmul:
// load-time repack and its inverse, group sums, slice reduction.
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <string>

#include "../../include/tensorfold_b200.h"
#include "qmm_launch.h"
#include "qmm_stream_launch.h"

namespace tf {

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_error, sizeof g_error, "%s: %s", what, cudaGetErrorString(e));
  return static_cast<int>(e);
}

bool format_ok(int bits, int gs) {
  return (bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8) && (gs == 32 || gs == 64 || gs == 128);
}

constexpr int MAX_DEVICES = 64;
struct DeviceState {
  bool ready = false;
  int* err = nullptr;
  int sms = 0;
  signed char resident[6][3][2][3] = {};   // blocks of a streaming kernel an SM holds: [bits][group][row tile][lanes]
  signed char resident_grouped[3][2] = {}; // the same for the grouped form: [group][row tile]
};
DeviceState g_devices[MAX_DEVICES];
int g_lanes_pref = 0;                 // tuning knob (tf_tune): preferred slice lanes per block, 0 = default
int g_stream_lanes = 0;               // tuning knob: super-blocks a streaming block holds side by side, 0 = default
int g_stream_blocks = 0;              // tuning knob: streaming blocks an SM may hold, 0 = as many as fit
int g_grouped_tiled = 0;              // tuning knob: 1 sends the experts' decode form through the tiled kernel (one block an item)

constexpr int BIT_WIDTHS[6] = {2, 3, 4, 5, 6, 8};
int bits_index(int bits) { return bits == 8 ? 5 : bits - 2; }
int gs_index(int gs) { return gs == 32 ? 0 : gs == 64 ? 1 : 2; }
int kw_index(int kw) { return kw == 1 ? 0 : kw == 2 ? 1 : 2; }
std::mutex g_init_mutex;

}  // namespace

cudaError_t prefill_configure();      // qmm_prefill.cu
void peer_reduce_plain(int on);       // peer_reduce.cu
cudaError_t moe_static_init(int device);   // moe.cu: the built-in plan scratch's address on that device
int encode_rows(CUtensorMap* map, const void* x, int64_t ldx, int rows, int k, int box_rows);

int* device_error_word() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES || !g_devices[dev].ready) return nullptr;
  return g_devices[dev].err;
}

int fail_moe(int code, const char* msg) { return fail(code, "%s", msg); }
int cuda_fail_moe(cudaError_t e, const char* what) { return cuda_fail(e, what); }

__device__ int g_error_word;          // set by a kernel whose bounded wait gave up; read by tf_device_error

// ---------------------------------------------------------------------------------------------------------------------
// repack: one thread per output word of the tiled tensor
// ---------------------------------------------------------------------------------------------------------------------

// With a second source (words2 != null) the packed rows interleave 16 rows of the first with 16 rows of the second
// (gate and up projections of an expert): packed row r comes from source (r / 16) % 2, row (r / 32) * 16 + r % 16.
__global__ void pack_kernel(const uint32_t* __restrict__ words, const uint16_t* __restrict__ scales,
                            const uint16_t* __restrict__ biases, const uint32_t* __restrict__ words2,
                            const uint16_t* __restrict__ scales2, const uint16_t* __restrict__ biases2, int n, int k,
                            int bits, int gs, uint32_t* __restrict__ tiled, int64_t total) {
  const int wpl = words_per_lane(bits, gs), unitw = unit_words(bits, gs), kg = k / gs;
  const int64_t wpr = static_cast<int64_t>(k) * bits / 32;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int wi_unit = static_cast<int>(i % unitw);
    const int64_t unit = i / unitw;
    const int g = static_cast<int>(unit % kg);
    const int64_t sb = unit / kg;
    const int code_words = TILE_PAIRS * 32 * wpl;
    uint32_t value;
    if (wi_unit < code_words) {
      const int tp = wi_unit / (32 * wpl), lane = (wi_unit / wpl) % 32, wi = wi_unit % wpl;
      auto code = [&](int col, int kk) -> uint32_t {
        int64_t row = sb * SB_COLS + col;
        if (row >= n) return 0u;
        const uint32_t* src = words;
        if (words2 != nullptr) {
          if ((row >> 4) & 1) src = words2;
          row = (row >> 5) * 16 + (row & 15);
        }
        return stored_code(src + row * wpr, static_cast<int64_t>(g) * gs + kk, bits, wpr);
      };
      value = lane_word(bits, gs, tp, lane, wi, code);
    } else {
      const int ai = wi_unit - code_words;
      const int tp = ai >> 5, gg = (ai >> 2) & 7, h = (ai >> 1) & 1, r8 = ai & 1;
      int64_t row = sb * SB_COLS + 32 * tp + 16 * h + 8 * r8 + gg;
      value = 0u;
      if (row < n) {
        const uint16_t *sc = scales, *bi = biases;
        if (words2 != nullptr) {
          if ((row >> 4) & 1) sc = scales2, bi = biases2;
          row = (row >> 5) * 16 + (row & 15);
        }
        value = static_cast<uint32_t>(sc[row * kg + g]) | (static_cast<uint32_t>(bi[row * kg + g]) << 16);
      }
    }
    tiled[i] = value;
  }
}

// inverse: one thread per (row, block of 32 codes) writes `bits` words; one thread per (row, group) writes the affine pair
__global__ void unpack_kernel(const uint32_t* __restrict__ tiled, int n, int k, int bits, int gs,
                              uint32_t* __restrict__ words, uint16_t* __restrict__ scales, uint16_t* __restrict__ biases) {
  const int wpl = words_per_lane(bits, gs), unitw = unit_words(bits, gs), kg = k / gs, blocks = k / 32;
  const int64_t total = static_cast<int64_t>(n) * blocks;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / blocks;
    const int blk = static_cast<int>(i % blocks);
    const int64_t sb = row / SB_COLS;
    const int c = static_cast<int>(row % SB_COLS);
    uint32_t outw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < 32; ++j) {
      const int kk_all = blk * 32 + j, g = kk_all / gs, kk = kk_all % gs;
      const CodeLoc loc = code_loc(c, kk, gs);
      const uint32_t* lw = tiled + (sb * kg + g) * unitw + (loc.tp * 32 + loc.lane) * wpl;
      const uint64_t code = lane_code(bits, gs, lw, loc.p, loc.half);
      const int bit = j * bits;
      const uint64_t shifted = code << (bit & 31);
      outw[bit >> 5] |= static_cast<uint32_t>(shifted);
      if ((bit & 31) + bits > 32) outw[(bit >> 5) + 1] |= static_cast<uint32_t>(shifted >> 32);
    }
    for (int w = 0; w < bits; ++w) words[row * (static_cast<int64_t>(k) * bits / 32) + blk * bits + w] = outw[w];
    if (blk < kg) {                                   // kg <= blocks: reuse the first kg threads of a row
      const int g = blk;
      const uint32_t v = tiled[(sb * kg + g) * unitw + TILE_PAIRS * 32 * wpl + affine_index(c)];
      scales[row * kg + g] = static_cast<uint16_t>(v & 0xFFFFu);
      biases[row * kg + g] = static_cast<uint16_t>(v >> 16);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// group sums with the matmul kernel's own arithmetic: x against a tile of ones, one warp per (8 rows, group)
// ---------------------------------------------------------------------------------------------------------------------

__global__ void group_sums_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int m, int kg, int gs,
                                  float* __restrict__ xs) {
  const int lane = threadIdx.x & 31, g8 = lane >> 2, t = lane & 3;
  const int group = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (group >= kg) return;
  const int m0 = blockIdx.y * 8, row = m0 + g8;
  const uint32_t ones[4] = {0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u};
  float d[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t* src = reinterpret_cast<const uint32_t*>(x + static_cast<int64_t>(row < m ? row : 0) * ldx + static_cast<int64_t>(group) * gs);
  for (int s = 0; s < gs / 16; ++s) {
    uint32_t b0 = 0, b1 = 0;
    if (row < m) {
      b0 = src[s * 8 + t];           // inputs 16 s + 2 t, + 1
      b1 = src[s * 8 + 4 + t];       // inputs 16 s + 8 + 2 t, + 1
    }
    mma_bf16(d, ones, b0, b1);
  }
  if (lane < 4) {
    const int r = m0 + 2 * lane;
    if (r < m) xs[static_cast<int64_t>(r) * kg + group] = d[0];
    if (r + 1 < m) xs[static_cast<int64_t>(r + 1) * kg + group] = d[1];
  }
}

// out[r, c] = round(part[0][r, c] + part[1][r, c] + ...): slices [sk, total] fp32 with rows of n values, added in slice
// order; out rows ldo elements apart.
__global__ void reduce_slices_kernel(const float* __restrict__ part, int sk, int64_t total, int n, int64_t ldo, void* out,
                                     int out_f32) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc = part[i];
    for (int s = 1; s < sk; ++s) acc = acc + part[static_cast<int64_t>(s) * total + i];
    const int64_t o = ldo == n ? i : (i / n) * ldo + i % n;
    if (out_f32) reinterpret_cast<float*>(out)[o] = acc;
    else reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(acc);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// stored-layout helpers: dequantised rows (embedding gather, diagnostics) and the rank-ordered sum of partials
// ---------------------------------------------------------------------------------------------------------------------

__device__ __forceinline__ float meta_value(const void* p, int64_t i, int dtype) {      // 0 bf16, 1 fp16, 2 fp32
  if (dtype == 0) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  if (dtype == 1) return __half2float(static_cast<const __half*>(p)[i]);
  return static_cast<const float*>(p)[i];
}

// out[r, k] = q[row(r), k] * scale + bias in fp32 (one rounding when out is bf16); row(r) = ids[r], or r without ids.
__global__ void affine_rows_kernel(const void* __restrict__ ids, int ids64, int rows, const uint32_t* __restrict__ words,
                                   const void* __restrict__ scales, const void* __restrict__ biases, int meta, int n, int k,
                                   int bits, int gs, void* __restrict__ out, int out_f32) {
  const int r = blockIdx.y;
  const int kk = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows || kk >= k) return;
  int64_t row = r;
  if (ids != nullptr) row = ids64 ? static_cast<const int64_t*>(ids)[r] : static_cast<const int*>(ids)[r];
  float v = 0.f;
  if (row >= 0 && row < n) {                                   // ids outside the table give zeros, never a fault
    const int64_t wpr = static_cast<int64_t>(k) * bits / 32, kg = k / gs;
    const float q = static_cast<float>(stored_code(words + row * wpr, kk, bits, wpr));
    v = q * meta_value(scales, row * kg + kk / gs, meta) + meta_value(biases, row * kg + kk / gs, meta);
  }
  if (out_f32) static_cast<float*>(out)[static_cast<int64_t>(r) * k + kk] = v;
  else static_cast<__nv_bfloat16*>(out)[static_cast<int64_t>(r) * k + kk] = __float2bfloat16_rn(v);
}

// out[i] = round(((p[0][i] + p[1][i]) + p[2][i]) + ...) in fp32, rank order; partials fp32 or bf16.
__global__ void sum_ranks_kernel(const void* __restrict__ parts, int world, int64_t total, int parts_bf16, void* out,
                                 int out_f32) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) {
      const float v = parts_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(parts)[r * total + i])
                                 : static_cast<const float*>(parts)[r * total + i];
      acc = r == 0 ? v : acc + v;
    }
    if (out_f32) static_cast<float*>(out)[i] = acc;
    else static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(acc);
  }
}

// A wait nothing will ever satisfy, with a short limit: what a lost copy or a lost peer looks like to the host.  One
// warp polls a barrier no one arrives on `polls` times, gives up, and reports through the device error word.
__global__ void lost_wait_kernel(int polls, int* err) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  bool done = false;
  for (int i = 0; i < polls && !done; ++i) done = mbar_try_wait_sleep(&bar, 0, 1000u);
  if (!__all_sync(0xFFFFFFFFu, done) && threadIdx.x == 0) atomicCAS(err, 0, ERR_WAIT_FULL);
}

namespace {

// The dense form fetches the rows of x with tensor-map copies ([64 inputs x row tile] boxes, 128-byte swizzle); the map
// is built per call on the host and travels as a kernel parameter.  The grouped form gathers rows itself (map unused).
cudaError_t launch_bits(const QmmParams& p, int bits, int gs, int mt, int kw, cudaStream_t s, bool pdl) {
  CUtensorMap tmx = {};
  // (a single row has no stride to speak of: give the map a legal one)
  if (p.items == nullptr && encode_rows(&tmx, p.x, p.M == 1 ? p.K : p.ldx, p.M, p.K, 8 * mt) != TF_OK) return cudaErrorInvalidValue;
  switch (bits) {
    case 2: return qmm_launch_b2(tmx, p, gs, mt, kw, s, pdl);
    case 3: return qmm_launch_b3(tmx, p, gs, mt, kw, s, pdl);
    case 4: return qmm_launch_b4(tmx, p, gs, mt, kw, s, pdl);
    case 5: return qmm_launch_b5(tmx, p, gs, mt, kw, s, pdl);
    case 6: return qmm_launch_b6(tmx, p, gs, mt, kw, s, pdl);
    default: return qmm_launch_b8(tmx, p, gs, mt, kw, s, pdl);
  }
}

cudaError_t stream_launch_bits(const CUtensorMap& tmx, const StreamParams& p, int bits, int gs, int mt, int kw, int grid,
                               cudaStream_t s, bool pdl) {
  switch (bits) {
    case 2: return qmm_stream_launch_b2(tmx, p, gs, mt, kw, grid, s, pdl);
    case 3: return qmm_stream_launch_b3(tmx, p, gs, mt, kw, grid, s, pdl);
    case 4: return qmm_stream_launch_b4(tmx, p, gs, mt, kw, grid, s, pdl);
    case 5: return qmm_stream_launch_b5(tmx, p, gs, mt, kw, grid, s, pdl);
    case 6: return qmm_stream_launch_b6(tmx, p, gs, mt, kw, grid, s, pdl);
    default: return qmm_stream_launch_b8(tmx, p, gs, mt, kw, grid, s, pdl);
  }
}

int stream_resident_bits(int bits, int gs, int mt, int kw) {
  switch (bits) {
    case 2: return qmm_stream_resident_b2(gs, mt, kw);
    case 3: return qmm_stream_resident_b3(gs, mt, kw);
    case 4: return qmm_stream_resident_b4(gs, mt, kw);
    case 5: return qmm_stream_resident_b5(gs, mt, kw);
    case 6: return qmm_stream_resident_b6(gs, mt, kw);
    default: return qmm_stream_resident_b8(gs, mt, kw);
  }
}

// Scratch of a set: a counter area of fixed size first (4 ints per super-block; fixed, so that no call's slices ever
// land where another call's counters live: the counters must stay zero between calls), then the slices of every
// projection with more than one K slice.
constexpr int64_t SET_COUNTER_BYTES = 64 * 1024;            // 4096 super-blocks a set: 524,288 output columns

int64_t set_counter_bytes(int nproj, const int* n) {
  int64_t ints = 0;
  for (int i = 0; i < nproj; ++i) ints += static_cast<int64_t>((n[i] + SB_COLS - 1) / SB_COLS) * 4;
  return ints * 4 <= SET_COUNTER_BYTES ? SET_COUNTER_BYTES : -1;
}

int64_t set_part_bytes(int n, int sk) {
  return sk > 1 ? static_cast<int64_t>((n + SB_COLS - 1) / SB_COLS) * sk * STREAM_PART_FLOATS * 4 : 0;
}

int grid_for(int64_t total, int threads) {
  const int64_t blocks = (total + threads - 1) / threads;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 32 ? 148 * 32 : blocks));
}

int current_state(DeviceState** st) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= MAX_DEVICES || !g_devices[dev].ready)
    return fail(TF_ERR_STATE, "tf_init(%d) has not been called for the current device", dev);
  *st = &g_devices[dev];
  return TF_OK;
}

}  // namespace

}  // namespace tf

using namespace tf;

extern "C" {

int tf_version(void) { return 100; }
const char* tf_arch(void) { return "sm_100a"; }
const char* tf_last_error(void) { return g_error; }

int tf_init(int device) {
  if (device < 0 || device >= MAX_DEVICES) return fail(TF_ERR_ARG, "device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_init_mutex);
  if (g_devices[device].ready) return TF_OK;
  int prev = -1;
  cudaError_t e = cudaGetDevice(&prev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  e = cudaSetDevice(device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e == cudaSuccess && prop.major != 10) {
    cudaSetDevice(prev);
    return fail(TF_ERR_UNSUPPORTED, "built for sm_100a; device %d is sm_%d%d", device, prop.major, prop.minor);
  }
  if (e == cudaSuccess) e = qmm_configure_b2();
  if (e == cudaSuccess) e = qmm_configure_b3();
  if (e == cudaSuccess) e = qmm_configure_b4();
  if (e == cudaSuccess) e = qmm_configure_b5();
  if (e == cudaSuccess) e = qmm_configure_b6();
  if (e == cudaSuccess) e = qmm_configure_b8();
  if (e == cudaSuccess) e = prefill_configure();
  if (e == cudaSuccess) e = qmm_stream_configure_b2();
  if (e == cudaSuccess) e = qmm_stream_configure_b3();
  if (e == cudaSuccess) e = qmm_stream_configure_b4();
  if (e == cudaSuccess) e = qmm_stream_configure_b5();
  if (e == cudaSuccess) e = qmm_stream_configure_b6();
  if (e == cudaSuccess) e = qmm_stream_configure_b8();
  int sms = 0;
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (e == cudaSuccess) {
    for (int b = 0; b < 6; ++b)
      for (int g = 0; g < 3; ++g)
        for (int m = 0; m < 2; ++m)
          for (int k = 0; k < 3; ++k)
            g_devices[device].resident[b][g][m][k] =
                static_cast<signed char>(stream_resident_bits(BIT_WIDTHS[b], 32 << g, m + 1, 1 << k));
  }
  if (e == cudaSuccess) {
    for (int g = 0; g < 3; ++g)
      for (int m = 0; m < 2; ++m)
        g_devices[device].resident_grouped[g][m] = static_cast<signed char>(qmm_stream_grouped_resident(32 << g, m + 1));
  }
  if (e == cudaSuccess) e = moe_static_init(device);
  int* err = nullptr;
  if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&err), g_error_word);
  if (e == cudaSuccess) e = cudaMemset(err, 0, sizeof(int));
  cudaSetDevice(prev);
  if (e != cudaSuccess) return cuda_fail(e, "tf_init");
  g_devices[device].err = err;
  g_devices[device].sms = sms;
  g_devices[device].ready = true;
  return TF_OK;
}

int tf_device_error(int device, void* stream, int* code) {
  if (device < 0 || device >= MAX_DEVICES || !g_devices[device].ready || code == nullptr)
    return fail(TF_ERR_STATE, "tf_init(%d) has not been called", device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(code, g_devices[device].err, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && *code != 0) e = cudaMemsetAsync(g_devices[device].err, 0, sizeof(int), s);
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_device_error");
}

int tf_selftest_lost_wait(int polls, void* stream) {
  if (polls < 1 || polls > 4096) return fail(TF_ERR_ARG, "tf_selftest_lost_wait: 1 to 4096 polls");
  DeviceState* st = nullptr;
  if (int rc = current_state(&st)) return rc;
  lost_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(polls, st->err);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_selftest_lost_wait");
}

int tf_tune(const char* key, int value) {
  if (key != nullptr && std::string(key) == "qmm_lanes" && (value == 0 || value == 1 || value == 2 || value == 4)) {
    g_lanes_pref = value;
    return TF_OK;
  }
  if (key != nullptr && std::string(key) == "stream_lanes" && (value == 0 || value == 1 || value == 2 || value == 4)) {
    g_stream_lanes = value;
    return TF_OK;
  }
  if (key != nullptr && std::string(key) == "stream_blocks" && value >= 0 && value <= 8) {
    g_stream_blocks = value;
    return TF_OK;
  }
  if (key != nullptr && std::string(key) == "peer_plain" && (value == 0 || value == 1)) {
    peer_reduce_plain(value);
    return TF_OK;
  }
  if (key != nullptr && std::string(key) == "grouped_tiled" && (value == 0 || value == 1)) {
    g_grouped_tiled = value;
    return TF_OK;
  }
  return fail(TF_ERR_ARG, "tf_tune: unknown key or value");
}

int tf_split_k(int n, int k, int gs, int target) {
  if (n < 1 || k < 1 || gs < 1) return TF_ERR_ARG;
  const int tiles = (n + 63) / 64, groups = k / gs;
  int sk = 1;
  while (sk < 8 && tiles * sk < target && groups % (sk * 2) == 0 && groups / (sk * 2) >= 8) sk *= 2;
  return sk;
}

int tf_bucket(int m) { return m < 1 ? TF_ERR_ARG : m <= 16 ? 16 : m <= 32 ? 32 : 64; }

int tf_unit_words(int bits, int gs) { return format_ok(bits, gs) ? unit_words(bits, gs) : TF_ERR_ARG; }

int64_t tf_tiled_words(int n, int k, int bits, int gs) {
  if (!format_ok(bits, gs) || n < 1 || k < gs || k % gs) return TF_ERR_ARG;
  return static_cast<int64_t>((n + SB_COLS - 1) / SB_COLS) * (k / gs) * unit_words(bits, gs);
}

int tf_pack(const void* words, const void* scales, const void* biases, int n, int k, int bits, int gs, void* tiled,
            void* stream) {
  if (!format_ok(bits, gs)) return fail(TF_ERR_ARG, "tf_pack: %d bits / groups of %d is not an affine format", bits, gs);
  if (n < 1 || k < gs || k % gs || (static_cast<int64_t>(k) * bits) % 32)
    return fail(TF_ERR_ARG, "tf_pack: (%d, %d) does not split into whole groups and words", n, k);
  if (!words || !scales || !biases || !tiled) return fail(TF_ERR_ARG, "tf_pack: null pointer");
  const int64_t total = tf_tiled_words(n, k, bits, gs);
  pack_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(words), static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases), nullptr,
      nullptr, nullptr, n, k, bits, gs, static_cast<uint32_t*>(tiled), total);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_pack");
}

int tf_pack_pair(const void* words_a, const void* scales_a, const void* biases_a, const void* words_b, const void* scales_b,
                 const void* biases_b, int n_each, int k, int bits, int gs, void* tiled, void* stream) {
  if (!format_ok(bits, gs)) return fail(TF_ERR_ARG, "tf_pack_pair: %d bits / groups of %d is not an affine format", bits, gs);
  if (n_each < 16 || n_each % 16 || k < gs || k % gs || (static_cast<int64_t>(k) * bits) % 32)
    return fail(TF_ERR_ARG, "tf_pack_pair: (%d, %d) needs rows in whole 16-row tiles and whole groups and words", n_each, k);
  if (!words_a || !scales_a || !biases_a || !words_b || !scales_b || !biases_b || !tiled)
    return fail(TF_ERR_ARG, "tf_pack_pair: null pointer");
  const int64_t total = tf_tiled_words(2 * n_each, k, bits, gs);
  pack_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(words_a), static_cast<const uint16_t*>(scales_a), static_cast<const uint16_t*>(biases_a),
      static_cast<const uint32_t*>(words_b), static_cast<const uint16_t*>(scales_b), static_cast<const uint16_t*>(biases_b),
      2 * n_each, k, bits, gs, static_cast<uint32_t*>(tiled), total);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_pack_pair");
}

int tf_unpack(const void* tiled, int n, int k, int bits, int gs, void* words, void* scales, void* biases, void* stream) {
  if (!format_ok(bits, gs)) return fail(TF_ERR_ARG, "tf_unpack: %d bits / groups of %d is not an affine format", bits, gs);
  if (n < 1 || k < gs || k % gs || (static_cast<int64_t>(k) * bits) % 32)
    return fail(TF_ERR_ARG, "tf_unpack: (%d, %d) does not split into whole groups and words", n, k);
  if (!words || !scales || !biases || !tiled) return fail(TF_ERR_ARG, "tf_unpack: null pointer");
  unpack_kernel<<<grid_for(static_cast<int64_t>(n) * (k / 32), 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(tiled), n, k, bits, gs, static_cast<uint32_t*>(words), static_cast<uint16_t*>(scales),
      static_cast<uint16_t*>(biases));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_unpack");
}

int tf_group_sums(const void* x, int64_t ldx, int m, int k, int gs, float* xs, void* stream) {
  if (gs != 32 && gs != 64 && gs != 128) return fail(TF_ERR_ARG, "tf_group_sums: groups of 32, 64 or 128, not %d", gs);
  if (m < 1 || k < gs || k % gs || !x || !xs) return fail(TF_ERR_ARG, "tf_group_sums: bad shape (%d, %d)", m, k);
  if (reinterpret_cast<uintptr_t>(x) % 4 || (m > 1 && ldx % 2)) return fail(TF_ERR_ALIGN, "tf_group_sums: rows must be 4-byte aligned");
  const int kg = k / gs;
  dim3 grid((kg + 3) / 4, (m + 7) / 8);
  group_sums_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x), ldx, m, kg, gs, xs);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_group_sums");
}

int tf_qmm(const void* x, int64_t ldx, int m, const float* xs, const void* tiled, int64_t sb_stride, int n, int k, int bits,
           int gs, int sk, void* out, int64_t ldo, int out_f32, float* part, int reduce, int pdl, void* stream) {
  if (!format_ok(bits, gs)) return fail(TF_ERR_ARG, "tf_qmm: %d bits / groups of %d is not an affine format", bits, gs);
  if (m < 1 || n < 1 || k < gs || k % gs) return fail(TF_ERR_ARG, "tf_qmm: bad shape m=%d n=%d k=%d", m, n, k);
  const int kg = k / gs;
  if (sk < 1 || sk > kg) return fail(TF_ERR_ARG, "tf_qmm: 1 to %d K slices (one group at least a slice), not %d", kg, sk);
  if (!x || !tiled) return fail(TF_ERR_ARG, "tf_qmm: null pointer");
  if (reinterpret_cast<uintptr_t>(x) % 16 || (m > 1 && ldx % 8) || ldx < k)
    return fail(TF_ERR_ALIGN, "tf_qmm: x rows must start on 16-byte boundaries (ldx %% 8 == 0, ldx >= k)");
  if (reinterpret_cast<uintptr_t>(tiled) % 16) return fail(TF_ERR_ALIGN, "tf_qmm: tiled weights must be 16-byte aligned");
  // A block streams kw super-blocks of 128 columns side by side (they share the rows of x); the sk blocks of the same
  // columns form a cluster (at most 8).  The geometry never changes a bit of the result; it is picked for occupancy.
  const int mt = mt_for_rows(m);
  const int nsb = (n + SB_COLS - 1) / SB_COLS;
  int kw = g_lanes_pref > 0 ? g_lanes_pref : (((nsb + 1) / 2) * sk >= 256 ? 2 : 1);    // measured on B200
  if (kw > max_lanes(mt)) kw = max_lanes(mt);
  const bool slices_out = sk > 1 && (!reduce || sk > 8);
  if (slices_out && !part) return fail(TF_ERR_ARG, "tf_qmm: part is required when the slices leave the kernel (reduce = 0, or more than 8 slices)");
  const bool out_used = !slices_out || reduce;
  if (out_used && (!out || ldo < n)) return fail(TF_ERR_ARG, "tf_qmm: out is null or its rows are shorter than n (ldo >= n)");
  if (sb_stride < 0) return fail(TF_ERR_ARG, "tf_qmm: negative super-block stride");
  if (m > 65535 * 8) return fail(TF_ERR_ARG, "tf_qmm: too many rows");
  DeviceState* st = nullptr;
  if (int rc = current_state(&st)) return rc;

  const int unitw = unit_words(bits, gs);
  QmmParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.ldx = ldx;
  p.M = m;
  p.xs = xs;
  p.w = static_cast<const uint32_t*>(tiled);
  p.sb_stride = sb_stride > 0 ? sb_stride : static_cast<int64_t>(kg) * unitw;
  p.N = n, p.K = k, p.KG = kg, p.sk = sk;
  p.out = out;
  p.ldo = ldo;
  p.out_f32 = out_f32;
  const int esize = out_f32 ? 4 : 2;
  p.out_vec = out && reinterpret_cast<uintptr_t>(out) % 16 == 0 && (ldo * esize) % 16 == 0;
  p.part = part;
  p.cluster = !slices_out;
  p.err = st->err;
  const cudaError_t e = launch_bits(p, bits, gs, mt, kw, static_cast<cudaStream_t>(stream), pdl != 0);
  if (e != cudaSuccess) return cuda_fail(e, "tf_qmm launch");
  if (slices_out && reduce) {                               // more slices than a cluster holds: summed by a second kernel
    const int64_t total = static_cast<int64_t>(m) * n;
    reduce_slices_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(part, sk, total, n, ldo, out, out_f32);
    const cudaError_t e2 = cudaGetLastError();
    return e2 == cudaSuccess ? TF_OK : cuda_fail(e2, "tf_qmm slice sum");
  }
  return TF_OK;
}

int64_t tf_qmm_set_scratch_bytes(int nproj, const int* n, const int* sk) {
  if (nproj < 1 || nproj > STREAM_MAX_PROJ || !n || !sk) return TF_ERR_ARG;
  int64_t total = set_counter_bytes(nproj, n);
  if (total < 0) return TF_ERR_ARG;
  for (int i = 0; i < nproj; ++i) {
    if (n[i] < 1 || sk[i] < 1) return TF_ERR_ARG;
    total += set_part_bytes(n[i], sk[i]);
  }
  return total;
}

int tf_qmm_set_geometry(int m, int bits, int gs, int nproj, const int* n, const int* sk, int* lanes, int* blocks_per_sm,
                        int* grid) {
  if (!format_ok(bits, gs) || m < 1 || m > 16 || nproj < 1 || nproj > STREAM_MAX_PROJ || !n || !sk)
    return fail(TF_ERR_ARG, "tf_qmm_set_geometry: bad arguments");
  DeviceState* st = nullptr;
  if (int rc = current_state(&st)) return rc;
  const int mt = mt_for_rows(m);
  int64_t units = 0;
  for (int i = 0; i < nproj; ++i) units += static_cast<int64_t>((n[i] + SB_COLS - 1) / SB_COLS) * sk[i];
  const int kw = g_stream_lanes > 0 ? g_stream_lanes : (units > 3 * st->sms ? 2 : 1);
  int resident = st->resident[bits_index(bits)][gs_index(gs)][mt - 1][kw_index(kw)];
  if (resident < 1) return fail(TF_ERR_STATE, "tf_qmm_set_geometry: the streaming kernel does not fit an SM of this device");
  if (g_stream_blocks > 0 && g_stream_blocks < resident) resident = g_stream_blocks;
  int64_t items = 0;
  for (int i = 0; i < nproj; ++i) items += static_cast<int64_t>(((n[i] + SB_COLS - 1) / SB_COLS + kw - 1) / kw) * sk[i];
  if (lanes) *lanes = kw;
  if (blocks_per_sm) *blocks_per_sm = resident;
  if (grid) *grid = static_cast<int>(std::min<int64_t>(items, static_cast<int64_t>(st->sms) * resident));
  return TF_OK;
}

int tf_qmm_set(const void* x, int64_t ldx, int m, const float* xs, int k, int bits, int gs, int nproj,
               const void* const* tiled, const int64_t* sb_stride, const int* n, const int* sk, void* const* out,
               const int64_t* ldo, int out_f32, void* scratch, int64_t scratch_bytes, int pdl, void* stream) {
  if (!format_ok(bits, gs)) return fail(TF_ERR_ARG, "tf_qmm_set: %d bits / groups of %d is not an affine format", bits, gs);
  if (nproj < 1 || nproj > STREAM_MAX_PROJ) return fail(TF_ERR_ARG, "tf_qmm_set: 1 to %d projections a set, not %d", STREAM_MAX_PROJ, nproj);
  if (m < 1 || m > 16) return fail(TF_ERR_ARG, "tf_qmm_set: 1 to 16 rows, not %d (larger windows go through tf_qmm)", m);
  if (k < gs || k % gs) return fail(TF_ERR_ARG, "tf_qmm_set: K = %d must be a positive multiple of the group", k);
  if (!x || !tiled || !n || !sk || !out || !ldo) return fail(TF_ERR_ARG, "tf_qmm_set: null pointer");
  if (reinterpret_cast<uintptr_t>(x) % 16 || (m > 1 && ldx % 8) || ldx < k)
    return fail(TF_ERR_ALIGN, "tf_qmm_set: x rows must start on 16-byte boundaries (ldx %% 8 == 0, ldx >= k)");
  const int kg = k / gs;
  int64_t need = set_counter_bytes(nproj, n);
  if (need < 0) return fail(TF_ERR_ARG, "tf_qmm_set: a set holds at most 4096 super-blocks of 128 columns");
  for (int i = 0; i < nproj; ++i) {
    if (n[i] < 1 || sk[i] < 1 || sk[i] > kg)
      return fail(TF_ERR_ARG, "tf_qmm_set: projection %d: n = %d, %d slices over %d groups", i, n[i], sk[i], kg);
    if (!tiled[i] || !out[i] || ldo[i] < n[i]) return fail(TF_ERR_ARG, "tf_qmm_set: projection %d: null pointer or short out rows", i);
    if (reinterpret_cast<uintptr_t>(tiled[i]) % 16) return fail(TF_ERR_ALIGN, "tf_qmm_set: tiled weights must be 16-byte aligned");
    need += set_part_bytes(n[i], sk[i]);
  }
  if (!scratch || reinterpret_cast<uintptr_t>(scratch) % 256 || scratch_bytes < need)
    return fail(TF_ERR_ARG, "tf_qmm_set: scratch must be 256-byte aligned and hold tf_qmm_set_scratch_bytes = %lld bytes",
                static_cast<long long>(need));
  DeviceState* st = nullptr;
  if (int rc = current_state(&st)) return rc;

  const int mt = mt_for_rows(m), unitw = unit_words(bits, gs);
  // super-blocks a block streams side by side: one while single-lane blocks (three an SM) hold the set in one wave, else two
  int64_t units = 0;
  for (int i = 0; i < nproj; ++i) units += static_cast<int64_t>((n[i] + SB_COLS - 1) / SB_COLS) * sk[i];
  int kw = g_stream_lanes > 0 ? g_stream_lanes : (units > 3 * st->sms ? 2 : 1);
  int resident = st->resident[bits_index(bits)][gs_index(gs)][mt - 1][kw_index(kw)];
  if (resident < 1) return fail(TF_ERR_STATE, "tf_qmm_set: the streaming kernel does not fit an SM of this device");
  if (g_stream_blocks > 0 && g_stream_blocks < resident) resident = g_stream_blocks;

  // longer slices first, so the blocks that get one item more get a short one
  int order[STREAM_MAX_PROJ];
  for (int i = 0; i < nproj; ++i) order[i] = i;
  for (int i = 1; i < nproj; ++i)
    for (int j = i; j > 0 && sk[order[j]] < sk[order[j - 1]]; --j) std::swap(order[j], order[j - 1]);

  StreamParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.xs = xs;
  p.M = m, p.K = k, p.KG = kg;
  p.nproj = nproj;
  p.err = st->err;
  int* counters = static_cast<int*>(scratch);
  uint8_t* parts = static_cast<uint8_t*>(scratch) + set_counter_bytes(nproj, n);
  int items = 0;
  for (int q = 0; q < nproj; ++q) {
    const int i = order[q];
    StreamProj& pr = p.proj[q];
    pr.w = static_cast<const uint32_t*>(tiled[i]);
    pr.sb_stride = sb_stride && sb_stride[i] > 0 ? sb_stride[i] : static_cast<int64_t>(kg) * unitw;
    pr.out = out[i];
    pr.ldo = ldo[i];
    pr.N = n[i], pr.sk = sk[i];
    pr.nsb = (n[i] + SB_COLS - 1) / SB_COLS;
    pr.out_f32 = out_f32;
    pr.count = counters;
    counters += pr.nsb * 4;
    pr.part = reinterpret_cast<float*>(parts);
    parts += set_part_bytes(n[i], sk[i]);
    pr.item0 = items;
    items += (pr.nsb + kw - 1) / kw * pr.sk;
  }
  p.items = items;
  CUtensorMap tmx = {};
  if (int rc = encode_rows(&tmx, x, m == 1 ? k : ldx, m, k, 8 * mt)) return rc;
  const int grid = std::min(items, st->sms * resident);
  const cudaError_t e = stream_launch_bits(tmx, p, bits, gs, mt, kw, grid, static_cast<cudaStream_t>(stream), pdl != 0);
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_qmm_set launch");
}

int tf_qmm_act(const void* x, int64_t ldx, int m, const void* tiled, int64_t sb_stride, int n, int k, int bits, int gs,
               void* out, int64_t ldo, int epi, float limit, int pdl, void* stream) {
  if (!format_ok(bits, gs)) return fail(TF_ERR_ARG, "tf_qmm_act: %d bits / groups of %d is not an affine format", bits, gs);
  if (m < 1 || n < 1 || k < gs || k % gs) return fail(TF_ERR_ARG, "tf_qmm_act: bad shape m=%d n=%d k=%d", m, n, k);
  if (epi != 1 && epi != 2) return fail(TF_ERR_ARG, "tf_qmm_act: epilogue 1 (relu^2) or 2 (SwiGLU)");
  if (epi == 2 && n % 32) return fail(TF_ERR_ARG, "tf_qmm_act: SwiGLU rows interleave gate and up in tiles of 16");
  const int ncols = epi == 2 ? n / 2 : n;
  if (!x || !tiled || !out || ldo < ncols) return fail(TF_ERR_ARG, "tf_qmm_act: null pointer or short out rows");
  if (reinterpret_cast<uintptr_t>(x) % 16 || (m > 1 && ldx % 8) || ldx < k)
    return fail(TF_ERR_ALIGN, "tf_qmm_act: x rows must start on 16-byte boundaries");
  DeviceState* st = nullptr;
  if (int rc = current_state(&st)) return rc;
  QmmParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.ldx = ldx, p.M = m;
  p.w = static_cast<const uint32_t*>(tiled);
  p.sb_stride = sb_stride > 0 ? sb_stride : static_cast<int64_t>(k / gs) * unit_words(bits, gs);
  p.N = n, p.K = k, p.KG = k / gs, p.sk = 1;
  p.out = out, p.ldo = ldo, p.out_f32 = 0;
  p.out_vec = reinterpret_cast<uintptr_t>(out) % 16 == 0 && (ldo * 2) % 16 == 0;
  p.cluster = 1;
  p.err = st->err;
  p.epi = epi, p.limit = limit;
  const cudaError_t e = launch_bits(p, bits, gs, mt_for_rows(m), 1, static_cast<cudaStream_t>(stream), pdl != 0);
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_qmm_act launch");
}

int tf_moe_experts(const void* x, int64_t ldx, int slots, const void* tiled, int64_t expert_stride, int experts, int n, int k,
                   int gs, const int* items, const int* counts, const int* members, int max_items, int tile, void* out,
                   int64_t ldo, int out_f32, int epi, float limit, void* stream) {
  if (experts < 1) return fail(TF_ERR_ARG, "tf_moe_experts: the table holds at least one expert");
  if (!format_ok(4, gs)) return fail(TF_ERR_ARG, "tf_moe_experts: groups of 32, 64 or 128, not %d", gs);
  if (n < 1 || k < gs || k % gs || max_items < 1) return fail(TF_ERR_ARG, "tf_moe_experts: bad shape n=%d k=%d items=%d", n, k, max_items);
  if (tile != 8 && tile != 16 && tile != 32 && tile != 64) return fail(TF_ERR_ARG, "tf_moe_experts: items of 8, 16, 32 or 64 pairs");
  if (epi < 0 || epi > 2 || (epi == 2 && n % 32)) return fail(TF_ERR_ARG, "tf_moe_experts: bad epilogue for %d columns", n);
  if (epi != 0 && out_f32) return fail(TF_ERR_ARG, "tf_moe_experts: activations are written as bf16");
  const int ncols = epi == 2 ? n / 2 : n;
  if (!x || !tiled || !items || !counts || !members || !out || ldo < ncols || slots < 0)
    return fail(TF_ERR_ARG, "tf_moe_experts: null pointer or short out rows");
  if (reinterpret_cast<uintptr_t>(x) % 16 || ldx % 8 || ldx < k) return fail(TF_ERR_ALIGN, "tf_moe_experts: x rows must start on 16-byte boundaries");
  if (max_items > 65535) return fail(TF_ERR_ARG, "tf_moe_experts: too many items");
  DeviceState* st = nullptr;
  if (int rc = current_state(&st)) return rc;
  const cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const int nsb = (n + SB_COLS - 1) / SB_COLS;
  const int resident = tile <= 16 ? st->resident_grouped[gs_index(gs)][tile / 8 - 1] : 0;
  cudaError_t e;
  if (resident > 0 && !g_grouped_tiled) {
    // items of up to 16 pairs: the persistent kernel in its grouped form, (plan item, super-block) units dealt to the
    // resident blocks (the item count is read on the device, so the grid covers the most the plan can hold)
    StreamParams sp = {};
    sp.x = static_cast<const __nv_bfloat16*>(x);
    sp.ldx = ldx, sp.M = tile, sp.K = k, sp.KG = k / gs, sp.nproj = 1, sp.items = 0, sp.err = st->err;
    sp.proj[0].w = static_cast<const uint32_t*>(tiled);
    sp.proj[0].sb_stride = static_cast<int64_t>(k / gs) * unit_words(4, gs);
    sp.proj[0].out = out, sp.proj[0].ldo = ldo, sp.proj[0].N = n, sp.proj[0].sk = 1, sp.proj[0].nsb = nsb;
    sp.proj[0].out_f32 = out_f32;
    sp.plan_items = items, sp.counts = counts, sp.members = members, sp.slots = slots;
    sp.expert_stride = expert_stride, sp.experts = experts, sp.epi = epi, sp.limit = limit;
    const int64_t units = static_cast<int64_t>(max_items) * nsb;
    int64_t grid = static_cast<int64_t>(g_stream_blocks > 0 ? std::min(g_stream_blocks, resident) : resident) * st->sms;
    if (grid > units) grid = units;
    e = qmm_stream_grouped_launch(sp, gs, tile / 8, static_cast<int>(grid), cs, true);
  } else {
    QmmParams p = {};
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.ldx = ldx, p.M = max_items;
    p.w = static_cast<const uint32_t*>(tiled);
    p.sb_stride = static_cast<int64_t>(k / gs) * unit_words(4, gs);
    p.N = n, p.K = k, p.KG = k / gs, p.sk = 1;
    p.out = out, p.ldo = ldo, p.out_f32 = out_f32;
    p.out_vec = reinterpret_cast<uintptr_t>(out) % 16 == 0 && (ldo * (out_f32 ? 4 : 2)) % 16 == 0;
    p.cluster = 1;
    p.err = st->err;
    p.items = items, p.counts = counts, p.members = members, p.slots = slots;
    p.expert_stride = expert_stride;
    p.experts = experts;
    p.epi = epi, p.limit = limit;
    e = launch_bits(p, 4, gs, tile / 8, 1, cs, false);
  }
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_moe_experts launch");
}

int tf_affine_rows(const void* ids, int ids64, int rows, const void* words, const void* scales, const void* biases, int meta,
                   int n, int k, int bits, int gs, void* out, int out_f32, void* stream) {
  if (!format_ok(bits, gs)) return fail(TF_ERR_ARG, "tf_affine_rows: %d bits / groups of %d is not an affine format", bits, gs);
  if (rows < 1 || rows > 65535 * 32 || n < 1 || k < gs || k % gs || (static_cast<int64_t>(k) * bits) % 32 || meta < 0 || meta > 2)
    return fail(TF_ERR_ARG, "tf_affine_rows: bad shape rows=%d n=%d k=%d", rows, n, k);
  if (!words || !scales || !biases || !out) return fail(TF_ERR_ARG, "tf_affine_rows: null pointer");
  if (rows > 65535) return fail(TF_ERR_ARG, "tf_affine_rows: at most 65535 rows a call");
  dim3 grid((k + 255) / 256, rows);
  affine_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(ids, ids64, rows, static_cast<const uint32_t*>(words),
                                                                         scales, biases, meta, n, k, bits, gs, out, out_f32);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_affine_rows");
}

int tf_sum_ranks(const void* parts, int world, int64_t total, int parts_bf16, void* out, int out_f32, void* stream) {
  if (!parts || !out || world < 1 || total < 1) return fail(TF_ERR_ARG, "tf_sum_ranks: bad arguments");
  sum_ranks_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(parts, world, total, parts_bf16, out, out_f32);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_sum_ranks");
}

int tf_reduce_slices(const float* part, int sk, int64_t total, void* out, int out_f32, void* stream) {
  if (!part || !out || sk < 1 || total < 1) return fail(TF_ERR_ARG, "tf_reduce_slices: bad arguments");
  reduce_slices_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(part, sk, total, 1, 1, out, out_f32);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail(e, "tf_reduce_slices");
}

}  // extern "C"
