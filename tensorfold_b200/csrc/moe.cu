// Routed mixture-of-experts plumbing around the grouped matmul: router logits, top-k selection with renormalised
// weights, the plan (a stable counting sort of the (row, slot) pairs by expert) and the slot-ordered combine.
// Every kernel computes a row from that row alone, so a row's bits never depend on how many rows share the call.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>

#include "../../include/tensorfold_b200.h"

namespace tf {

int fail_moe(int code, const char* msg);          // defined in tf_api.cu (sets the thread's error text)
int cuda_fail_moe(cudaError_t e, const char* what);

namespace {

constexpr int PLAN_BLOCK = 1024;                  // pairs a plan block ranks
constexpr int PLAN_MAX_EXPERTS = 4096;

// ---------------------------------------------------------------------------------------------------------------------
// plan
// ---------------------------------------------------------------------------------------------------------------------

// Phase A: block b ranks pairs [1024 b, 1024 b + 1024): rank[i] = number of earlier pairs of the block with the same
// expert; hist[b][e] = pairs of expert e in the block.  Warps take turns so ranks follow pair order (a stable sort).
__device__ void plan_rank_block(const int* __restrict__ picks, int pairs, int experts, int* __restrict__ rank,
                                int* __restrict__ hist, int blk, int* cnt /* shared [experts] */) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int e = tid; e < experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  const int i = blk * PLAN_BLOCK + tid;
  int e = i < pairs ? picks[i] : -1;
  const bool valid = e >= 0 && e < experts;
  for (int turn = 0; turn < PLAN_BLOCK / 32; ++turn) {
    if (warp == turn) {
      const unsigned act = __ballot_sync(0xFFFFFFFFu, valid);
      if (valid) {
        const unsigned same = __match_any_sync(act, e);
        const int base = cnt[e];
        __syncwarp(act);
        rank[i] = base + __popc(same & ((1u << lane) - 1u));
        if (lane == __ffs(same) - 1) cnt[e] = base + __popc(same);
      }
    }
    __syncthreads();
  }
  for (int x = tid; x < experts; x += blockDim.x) hist[blk * experts + x] = cnt[x];
}

// Phase B (one block): turn hist[b][e] into the offset in `members` of block b's first pair of expert e, and write the
// items (expert, first, count <= tile) in expert order plus counts = (items, distinct experts).
__device__ void plan_offsets_block(int* __restrict__ hist, int nblk, int experts, int tile, int* __restrict__ items,
                                   int* __restrict__ counts, int max_items, int* scan /* shared [2 * 1024 + 64] */) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ept = (experts + blockDim.x - 1) / blockDim.x;       // experts a thread owns (consecutive)
  int tot[4], nit[4];
  int sum_t = 0, sum_i = 0, distinct = 0;
  for (int j = 0; j < ept; ++j) {
    const int e = tid * ept + j;
    int t = 0;
    if (e < experts)
      for (int b = 0; b < nblk; ++b) {
        const int c = hist[b * experts + e];
        hist[b * experts + e] = t;                               // exclusive over blocks
        t += c;
      }
    tot[j] = t, nit[j] = (t + tile - 1) / tile;
    sum_t += t, sum_i += nit[j], distinct += t > 0;
  }
  // block-wide exclusive scans of (sum_t, sum_i) and the total of `distinct`
  int inc_t = sum_t, inc_i = sum_i, dis = distinct;
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xFFFFFFFFu, inc_t, o), b = __shfl_up_sync(0xFFFFFFFFu, inc_i, o);
    if (lane >= o) inc_t += a, inc_i += b;
  }
  for (int o = 16; o > 0; o >>= 1) dis += __shfl_xor_sync(0xFFFFFFFFu, dis, o);
  int* wt = scan;
  int* wi = scan + 32;
  int* wd = scan + 64;
  if (lane == 31) wt[warp] = inc_t, wi[warp] = inc_i;
  if (lane == 0) wd[warp] = dis;
  __syncthreads();
  int base_t = 0, base_i = 0;
  for (int w = 0; w < warp; ++w) base_t += wt[w], base_i += wi[w];
  int start = base_t + inc_t - sum_t, ibase = base_i + inc_i - sum_i;
  for (int j = 0; j < ept; ++j) {
    const int e = tid * ept + j;
    if (e < experts) {
      for (int b = 0; b < nblk; ++b) hist[b * experts + e] += start;
      for (int q = 0; q < nit[j]; ++q)
        if (ibase + q < max_items) {
          items[3 * (ibase + q)] = e;
          items[3 * (ibase + q) + 1] = start + q * tile;
          items[3 * (ibase + q) + 2] = min(tile, tot[j] - q * tile);
        }
    }
    start += tot[j], ibase += nit[j];
  }
  if (tid == blockDim.x - 1) {
    int d = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) d += wd[w];
    counts[0] = min(ibase, max_items);
    counts[1] = d;
  }
}

__device__ void plan_scatter_block(const int* __restrict__ picks, int pairs, int experts, const int* __restrict__ rank,
                                   const int* __restrict__ hist, int* __restrict__ members, int blk) {
  const int i = blk * PLAN_BLOCK + threadIdx.x;
  if (i >= pairs) return;
  const int e = picks[i];
  if (e < 0 || e >= experts) return;
  members[hist[blk * experts + e] + rank[i]] = i;
}

// phase 0: rank (grid = blocks), 1: offsets (one block), 2: scatter (grid = blocks), -1: all three in one block
__global__ void __launch_bounds__(PLAN_BLOCK) plan_kernel(const int* __restrict__ picks, int pairs, int experts, int tile,
                                                         int* members, int* items, int* counts, int* rank, int* hist,
                                                         int max_items, int nblk, int phase) {
  __shared__ int shared[PLAN_MAX_EXPERTS + 128];
  if (phase == 0) {
    plan_rank_block(picks, pairs, experts, rank, hist, blockIdx.x, shared);
  } else if (phase == 1) {
    plan_offsets_block(hist, nblk, experts, tile, items, counts, max_items, shared);
  } else if (phase == 2) {
    plan_scatter_block(picks, pairs, experts, rank, hist, members, blockIdx.x);
  } else {
    plan_rank_block(picks, pairs, experts, rank, hist, 0, shared);
    __syncthreads();
    plan_offsets_block(hist, 1, experts, tile, items, counts, max_items, shared);
    __syncthreads();
    plan_scatter_block(picks, pairs, experts, rank, hist, members, 0);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// router: logits[r, e] = fp32 dot of bf16 rows x[r] and w[e]; one warp per (row, expert), fixed order
// ---------------------------------------------------------------------------------------------------------------------

__global__ void router_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int rows, int d,
                              const __nv_bfloat16* __restrict__ w, int ne, float* __restrict__ out, int64_t ldo) {
  const int lane = threadIdx.x & 31, e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), r = blockIdx.y;
  if (e >= ne || r >= rows) return;
  const __nv_bfloat16* xr = x + r * ldx;
  const __nv_bfloat16* wr = w + static_cast<int64_t>(e) * d;
  float acc = 0.f;
  const int vec = (d % 8 == 0 && (reinterpret_cast<uintptr_t>(xr) % 16 == 0) && (reinterpret_cast<uintptr_t>(wr) % 16 == 0)) ? d / 8 : 0;
  for (int v = lane; v < vec; v += 32) {
    const uint4 a = reinterpret_cast<const uint4*>(xr)[v], b = reinterpret_cast<const uint4*>(wr)[v];
    const uint32_t aa[4] = {a.x, a.y, a.z, a.w}, bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc = fmaf(__uint_as_float(aa[i] << 16), __uint_as_float(bb[i] << 16), acc);
      acc = fmaf(__uint_as_float(aa[i] & 0xFFFF0000u), __uint_as_float(bb[i] & 0xFFFF0000u), acc);
    }
  }
  for (int k = vec * 8 + lane; k < d; k += 32) acc = fmaf(__bfloat162float(xr[k]), __bfloat162float(wr[k]), acc);
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if (lane == 0) out[r * ldo + e] = acc;
}

__device__ __forceinline__ void router_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same logits in the prefill arithmetic: one warp per (16 rows, 16 experts) tile walks K in 16-input steps in order
// (m16n8k16, fp32 accumulate), operands straight from global memory (the block's four warps share the 16 rows through
// L1).  A row's logits depend on that row alone, whatever the row count; they are this kernel's bits, not the one-warp
// kernel's, so a caller picks one form per model and keeps it.
__global__ void __launch_bounds__(128) router_tiles_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int rows, int d,
                                                           const __nv_bfloat16* __restrict__ w, int ne,
                                                           float* __restrict__ out, int64_t ldo) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int e0 = (blockIdx.x * 4 + warp) * 16, r0 = blockIdx.y * 16;
  if (e0 >= ne) return;
  const int ra = min(r0 + g, rows - 1), rb = min(r0 + g + 8, rows - 1);
  const uint32_t* xa = reinterpret_cast<const uint32_t*>(x + ra * ldx);
  const uint32_t* xb = reinterpret_cast<const uint32_t*>(x + rb * ldx);
  const uint32_t* w0 = reinterpret_cast<const uint32_t*>(w + static_cast<int64_t>(min(e0 + g, ne - 1)) * d);
  const uint32_t* w1 = reinterpret_cast<const uint32_t*>(w + static_cast<int64_t>(min(e0 + 8 + g, ne - 1)) * d);
  float acc[2][4] = {};
#pragma unroll 4
  for (int k = 0; k < d / 16; ++k) {
    const int o = k * 8 + t;
    const uint32_t a0 = xa[o], a1 = xb[o], a2 = xa[o + 4], a3 = xb[o + 4];
    router_mma(acc[0], a0, a1, a2, a3, w0[o], w0[o + 4]);
    router_mma(acc[1], a0, a1, a2, a3, w1[o], w1[o + 4]);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int c = e0 + 8 * j + 2 * t;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = r0 + g + 8 * h;
      if (r < rows && c < ne) out[r * ldo + c] = acc[j][2 * h];
      if (r < rows && c + 1 < ne) out[r * ldo + c + 1] = acc[j][2 * h + 1];
    }
  }
}

// The same arithmetic from shared memory: a block of four warps takes 64 rows x 32 experts, 64 inputs a step, staged by
// 16-byte cp.async copies into 128-byte rows with the chunk index xor-ed by the row (conflict-free ldmatrix), four
// buffers (one chunk in flight made every step wait a full trip to memory: 44 us for 2048 rows x 160 experts x 6144).
// Each (row, expert) accumulator sees the same m16n8k16 operands in the same order as in router_tiles_kernel, so both
// give the same bits; this one reads x once per 32 experts instead of once per 16 and
// fetches fragments with ldmatrix instead of 4-byte global loads.
__device__ __forceinline__ void router_ldm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

constexpr int ROUTER_BUFS = 4;                               // stages in flight: three chunks are on their way while one is used
constexpr int ROUTER_STAGE = (64 + 32) * 128;                // 64 rows of x and 32 experts, 64 inputs (128 bytes) each

__global__ void __launch_bounds__(128) router_tiles_staged_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int rows,
                                                                  int d, const __nv_bfloat16* __restrict__ w, int ne,
                                                                  float* __restrict__ out, int64_t ldo) {
  extern __shared__ __align__(128) uint8_t router_smem[];    // [ROUTER_BUFS][x tile | expert tile]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int e0 = blockIdx.x * 32, r0 = blockIdx.y * 64;
  const int chunks = d / 64;
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(router_smem));
  // where this thread's six 16-byte pieces of a chunk come from and go to: worked out once (with one warp a scheduler,
  // the address arithmetic of every chunk was most of the instructions the loop issued)
  const __nv_bfloat16* xsrc[4];
  const __nv_bfloat16* wsrc[2];
  uint32_t xdst[4], wdst[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {                                // 64 rows x 8 pieces of 16 bytes
    const int p = tid + 128 * i, row = p >> 3, ch = p & 7;
    xsrc[i] = x + static_cast<int64_t>(min(r0 + row, rows - 1)) * ldx + ch * 8;
    xdst[i] = row * 128 + ((ch ^ (row & 7)) << 4);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {                                // 32 experts x 8 pieces
    const int p = tid + 128 * i, row = p >> 3, ch = p & 7;
    wsrc[i] = w + static_cast<int64_t>(min(e0 + row, ne - 1)) * d + ch * 8;
    wdst[i] = 64 * 128 + row * 128 + ((ch ^ (row & 7)) << 4);
  }
  auto stage = [&](int c, int buf) {
    const uint32_t sb = base + buf * ROUTER_STAGE;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sb + xdst[i]), "l"(xsrc[i] + c * 64) : "memory");
#pragma unroll
    for (int i = 0; i < 2; ++i)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sb + wdst[i]), "l"(wsrc[i] + c * 64) : "memory");
  };
  const uint32_t a_row = (16 * warp + (lane & 15)) * 128, a_half = lane >> 4, a_x = (lane & 15) & 7;
  const uint32_t b_row = ((lane & 7) + 8 * (lane >> 4)) * 128, b_half = (lane >> 3) & 1, b_x = lane & 7;
  float acc[4][4] = {};
  // every iteration commits exactly one group (an empty one past the end), so "all but the last ROUTER_BUFS - 1 groups
  // have landed" always means chunk c has
#pragma unroll
  for (int c = 0; c < ROUTER_BUFS - 1; ++c) {
    if (c < chunks) stage(c, c);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int c = 0; c < chunks; ++c) {
    const int buf = c % ROUTER_BUFS;
    asm volatile("cp.async.wait_group %0;" ::"n"(ROUTER_BUFS - 2) : "memory");
    __syncthreads();                                          // chunk c is visible; the buffer of chunk c - 1 is free
    if (c + ROUTER_BUFS - 1 < chunks) stage(c + ROUTER_BUFS - 1, (c + ROUTER_BUFS - 1) % ROUTER_BUFS);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const uint32_t xs = base + buf * ROUTER_STAGE, ws = xs + 64 * 128;
#pragma unroll
    for (int k16 = 0; k16 < 4; ++k16) {
      uint32_t a[4], b0[4], b1[4];
      // rows 0-7 / 8-15 x inputs 0-7 / 8-15 of the step; experts 0-15 then 16-31 ((row + 16) & 7 == row & 7)
      router_ldm4(a, xs + a_row + (((2 * k16 + a_half) ^ a_x) << 4));
      router_ldm4(b0, ws + b_row + (((2 * k16 + b_half) ^ b_x) << 4));
      router_ldm4(b1, ws + b_row + 16 * 128 + (((2 * k16 + b_half) ^ b_x) << 4));
      router_mma(acc[0], a[0], a[1], a[2], a[3], b0[0], b0[1]);
      router_mma(acc[1], a[0], a[1], a[2], a[3], b0[2], b0[3]);
      router_mma(acc[2], a[0], a[1], a[2], a[3], b1[0], b1[1]);
      router_mma(acc[3], a[0], a[1], a[2], a[3], b1[2], b1[3]);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = e0 + 8 * j + 2 * t;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = r0 + 16 * warp + g + 8 * h;
      if (r < rows && c < ne) out[r * ldo + c] = acc[j][2 * h];
      if (r < rows && c + 1 < ne) out[r * ldo + c + 1] = acc[j][2 * h + 1];
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// top-k: one warp per row
// ---------------------------------------------------------------------------------------------------------------------

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// With count > 0 the ids are rewritten for a rank that owns experts [first, first + count): local ids for those, -1 and a
// zero weight for every other slot (the shared slot among them), so the planner and the combine leave them out.
__global__ void topk_kernel(const float* __restrict__ logits, int64_t ldl, int rows, int experts, int topk, int shared,
                            int first, int count, int* __restrict__ pick, float* __restrict__ wts) {
  const int lane = threadIdx.x & 31, r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const float* l = logits + r * ldl;
  const int slots = topk + (shared ? 1 : 0);
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = (lane + 32 * j) < experts ? l[lane + 32 * j] : -INFINITY;
  float top = 0.f, total = 0.f, mine_ex = 0.f;
  int mine_id = 0;
  for (int k = 0; k < topk; ++k) {
    float best = -INFINITY;
    int id = 0x7FFFFFFF;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (v[j] > best) best = v[j], id = lane + 32 * j;           // ascending ids: the first maximum is the lowest id
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, id, o);
      if (ob > best || (ob == best && oi < id)) best = ob, id = oi;
    }
    if (k == 0) top = best;
    const float ex = expf(best - top);
    total += ex;
    if (lane == k % 32) mine_ex = ex, mine_id = id;              // lane k keeps slot k (topk <= 32)
    if ((id & 31) == lane) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j == (id >> 5)) v[j] = -INFINITY;
    }
  }
  if (lane < topk) {
    float w = bf16r(mine_ex / total);
    if (count > 0) {
      mine_id -= first;
      if (mine_id < 0 || mine_id >= count) mine_id = -1, w = 0.f;
    }
    pick[r * slots + lane] = mine_id;
    wts[r * slots + lane] = w;
  }
  if (shared && lane == 0) {
    if (count > 0) {
      pick[r * slots + topk] = -1;
      wts[r * slots + topk] = 0.f;
    } else {
      const float sg = bf16r(l[experts]);
      pick[r * slots + topk] = experts;
      wts[r * slots + topk] = bf16r(1.f / (1.f + expf(-sg)));
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// combine: out[r, d] = bf16(sum over slots in slot order of w[r, k] * y[r, k, d]) in fp32
// ---------------------------------------------------------------------------------------------------------------------

template <bool YBF16>
__global__ void combine_kernel(const void* __restrict__ y, const float* __restrict__ wts, int rows, int slots, int d,
                               __nv_bfloat16* __restrict__ out) {
  const int r = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (r >= rows || c >= d) return;
  float a0 = 0.f, a1 = 0.f;
  for (int k = 0; k < slots; ++k) {
    const float w = wts[r * slots + k];
    if (w == 0.f) continue;                                      // a slot another rank owns: its y is never read
    const int64_t off = (static_cast<int64_t>(r) * slots + k) * d + c;
    float y0, y1 = 0.f;
    if (YBF16) {
      const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(y) + off;
      y0 = __bfloat162float(p[0]);
      if (c + 1 < d) y1 = __bfloat162float(p[1]);
    } else {
      const float* p = reinterpret_cast<const float*>(y) + off;
      y0 = p[0];
      if (c + 1 < d) y1 = p[1];
    }
    a0 = fmaf(w, y0, a0);
    a1 = fmaf(w, y1, a1);
  }
  out[static_cast<int64_t>(r) * d + c] = __float2bfloat16_rn(a0);
  if (c + 1 < d) out[static_cast<int64_t>(r) * d + c + 1] = __float2bfloat16_rn(a1);
}

// The same sums, eight columns a thread with 16-byte loads (d a multiple of 8, y and out 16-byte aligned): every
// element still takes its slots in slot order with one fma each, so the bits are those of combine_kernel.
template <bool YBF16>
__global__ void __launch_bounds__(128) combine_wide_kernel(const void* __restrict__ y, const float* __restrict__ wts, int rows,
                                                           int slots, int d, __nv_bfloat16* __restrict__ out) {
  const int r = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (r >= rows || c >= d) return;
  float a[8] = {};
#pragma unroll 3
  for (int k = 0; k < slots; ++k) {
    const float w = wts[r * slots + k];
    if (w == 0.f) continue;                                      // a slot another rank owns: its y is never read
    const int64_t off = (static_cast<int64_t>(r) * slots + k) * d + c;
    float v[8];
    if (YBF16) {
      const uint4 q = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(y) + off);
      const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(u[i] << 16);
        v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
      }
    } else {
      const float4 lo = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(y) + off);
      const float4 hi = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(y) + off + 4);
      v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = fmaf(w, v[i], a[i]);
  }
  uint4 o;
  __nv_bfloat162 t0 = __floats2bfloat162_rn(a[0], a[1]), t1 = __floats2bfloat162_rn(a[2], a[3]);
  __nv_bfloat162 t2 = __floats2bfloat162_rn(a[4], a[5]), t3 = __floats2bfloat162_rn(a[6], a[7]);
  o.x = *reinterpret_cast<uint32_t*>(&t0), o.y = *reinterpret_cast<uint32_t*>(&t1);
  o.z = *reinterpret_cast<uint32_t*>(&t2), o.w = *reinterpret_cast<uint32_t*>(&t3);
  *reinterpret_cast<uint4*>(out + static_cast<int64_t>(r) * d + c) = o;
}

}  // namespace

}  // namespace tf

using namespace tf;

extern "C" {

int tf_moe_plan_blocks(int pairs) { return pairs < 1 ? TF_ERR_ARG : (pairs + PLAN_BLOCK - 1) / PLAN_BLOCK; }

int tf_moe_plan(const int* picks, int pairs, int experts, int tile, int* members, int* items, int* counts, int* rank,
                int* hist, int max_items, void* stream) {
  if (pairs < 1 || experts < 1 || experts > PLAN_MAX_EXPERTS || tile < 1 || max_items < 1)
    return fail_moe(TF_ERR_ARG, "tf_moe_plan: bad sizes (at most 4096 experts)");
  if (!picks || !members || !items || !counts || !rank || !hist) return fail_moe(TF_ERR_ARG, "tf_moe_plan: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int nblk = (pairs + PLAN_BLOCK - 1) / PLAN_BLOCK;
  if (nblk == 1) {
    plan_kernel<<<1, PLAN_BLOCK, 0, s>>>(picks, pairs, experts, tile, members, items, counts, rank, hist, max_items, 1, -1);
  } else {
    plan_kernel<<<nblk, PLAN_BLOCK, 0, s>>>(picks, pairs, experts, tile, members, items, counts, rank, hist, max_items, nblk, 0);
    plan_kernel<<<1, PLAN_BLOCK, 0, s>>>(picks, pairs, experts, tile, members, items, counts, rank, hist, max_items, nblk, 1);
    plan_kernel<<<nblk, PLAN_BLOCK, 0, s>>>(picks, pairs, experts, tile, members, items, counts, rank, hist, max_items, nblk, 2);
  }
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_moe_plan");
}

// ---------------------------------------------------------------------------------------------------------------------
// plan without caller scratch
// ---------------------------------------------------------------------------------------------------------------------

}  // extern "C"

namespace tf {
namespace {

constexpr int STATIC_PLAN_PAIRS = 16384;              // pairs a tf_moe_plan_static call may sort
constexpr int STATIC_PLAN_HIST = 65536;               // blocks * experts it may count (16 blocks of up to 4096 experts)

// The plan's working memory for callers that own none: ranks of the pairs, then the per-block expert counts.  Every
// GPU that loads the library holds these 320 KB until the process exits.
static __device__ __align__(256) int g_plan_scratch[STATIC_PLAN_PAIRS + STATIC_PLAN_HIST];

int* g_plan_scratch_ptr[64] = {};                     // device address of the array, per device (set once, under tf_init's lock)

}  // namespace

// Called by tf_init with `device` current: looks the array's address up once, so that tf_moe_plan_static itself is a
// pure look-up afterwards (no symbol query, no module load: safe under stream capture).  The array's name is only a
// host-side handle; the kernels need its address on that device.
cudaError_t moe_static_init(int device) {
  if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
  if (g_plan_scratch_ptr[device] != nullptr) return cudaSuccess;
  int* ptr = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_plan_scratch);
  if (e != cudaSuccess) return e;
  if (ptr == nullptr) return cudaErrorInvalidSymbol;
  g_plan_scratch_ptr[device] = ptr;
  return cudaSuccess;
}

}  // namespace tf

extern "C" {

int tf_moe_plan_static(const int* picks, int pairs, int experts, int tile, int* members, int* items, int* counts,
                       int max_items, void* stream) {
  if (pairs < 1 || experts < 1) return fail_moe(TF_ERR_ARG, "tf_moe_plan_static: bad sizes");
  const int nblk = (pairs + PLAN_BLOCK - 1) / PLAN_BLOCK;
  if (pairs > STATIC_PLAN_PAIRS || static_cast<int64_t>(nblk) * experts > STATIC_PLAN_HIST) {
    char msg[200];
    snprintf(msg, sizeof msg,
             "tf_moe_plan_static: %d pairs x %d experts exceed the built-in scratch (at most %d pairs and %d block-expert "
             "counters); use tf_moe_plan with caller scratch", pairs, experts, STATIC_PLAN_PAIRS, STATIC_PLAN_HIST);
    return fail_moe(TF_ERR_ARG, msg);
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail_moe(e, "tf_moe_plan_static: cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail_moe(TF_ERR_ARG, "tf_moe_plan_static: device index out of range");
  if (g_plan_scratch_ptr[dev] == nullptr)
    return fail_moe(TF_ERR_STATE, "tf_moe_plan_static: tf_init has not been called for the current device");
  int* rank = g_plan_scratch_ptr[dev];
  return tf_moe_plan(picks, pairs, experts, tile, members, items, counts, rank, rank + STATIC_PLAN_PAIRS, max_items, stream);
}

int tf_moe_router(const void* x, int64_t ldx, int rows, int d, const void* w, int ne, float* out, int64_t ldo, void* stream) {
  if (rows < 1 || d < 1 || ne < 1 || !x || !w || !out || ldx < d || ldo < ne) return fail_moe(TF_ERR_ARG, "tf_moe_router: bad arguments");
  if (rows > 65535) return fail_moe(TF_ERR_ARG, "tf_moe_router: too many rows");
  dim3 grid((ne + 7) / 8, rows);
  router_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x), ldx, rows, d,
                                                                     static_cast<const __nv_bfloat16*>(w), ne, out, ldo);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_moe_router");
}

int tf_moe_router_tiles(const void* x, int64_t ldx, int rows, int d, const void* w, int ne, float* out, int64_t ldo,
                        void* stream) {
  if (rows < 1 || d < 16 || ne < 1 || !x || !w || !out || ldx < d || ldo < ne)
    return fail_moe(TF_ERR_ARG, "tf_moe_router_tiles: bad arguments");
  if (d % 16 || ldx % 2 || reinterpret_cast<uintptr_t>(x) % 4 || reinterpret_cast<uintptr_t>(w) % 4)
    return fail_moe(TF_ERR_ARG, "tf_moe_router_tiles: d must be a multiple of 16, rows of x and w 4-byte aligned");
  if (rows > 65535 * 16) return fail_moe(TF_ERR_ARG, "tf_moe_router_tiles: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  if (d % 64 == 0 && ldx % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0) {
    dim3 grid((ne + 31) / 32, (rows + 63) / 64);             // staged through shared memory: the same bits, faster
    router_tiles_staged_kernel<<<grid, 128, ROUTER_BUFS * ROUTER_STAGE, st>>>(xp, ldx, rows, d, wp, ne, out, ldo);
  } else {
    dim3 grid((ne + 63) / 64, (rows + 15) / 16);
    router_tiles_kernel<<<grid, 128, 0, st>>>(xp, ldx, rows, d, wp, ne, out, ldo);
  }
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_moe_router_tiles");
}

int tf_moe_topk(const float* logits, int64_t ldl, int rows, int experts, int topk, int shared, int* pick, float* wts,
                void* stream) {
  if (rows < 1 || experts < 1 || experts > 1024 || topk < 1 || topk > 32 || topk > experts || !logits || !pick || !wts ||
      ldl < experts + (shared ? 1 : 0))
    return fail_moe(TF_ERR_ARG, "tf_moe_topk: bad arguments (at most 1024 experts, top 32)");
  topk_kernel<<<(rows + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(logits, ldl, rows, experts, topk, shared, 0, 0, pick,
                                                                             wts);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_moe_topk");
}

int tf_moe_topk_local(const float* logits, int64_t ldl, int rows, int experts, int topk, int shared, int first, int count,
                      int* pick, float* wts, void* stream) {
  if (rows < 1 || experts < 1 || experts > 1024 || topk < 1 || topk > 32 || topk > experts || !logits || !pick || !wts ||
      ldl < experts || first < 0 || count < 1 || first + count > experts)
    return fail_moe(TF_ERR_ARG, "tf_moe_topk_local: bad arguments (at most 1024 experts, top 32, a range inside them)");
  topk_kernel<<<(rows + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(logits, ldl, rows, experts, topk, shared, first,
                                                                             count, pick, wts);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_moe_topk_local");
}

int tf_moe_combine(const void* y, int y_bf16, const float* wts, int rows, int slots, int d, void* out, void* stream) {
  if (rows < 1 || slots < 1 || d < 1 || !y || !wts || !out || rows > 65535) return fail_moe(TF_ERR_ARG, "tf_moe_combine: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (d % 8 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    dim3 wide((d / 8 + 127) / 128, rows);
    if (y_bf16) combine_wide_kernel<true><<<wide, 128, 0, s>>>(y, wts, rows, slots, d, static_cast<__nv_bfloat16*>(out));
    else combine_wide_kernel<false><<<wide, 128, 0, s>>>(y, wts, rows, slots, d, static_cast<__nv_bfloat16*>(out));
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_moe_combine");
  }
  dim3 grid((d / 2 + 127) / 128 + 1, rows);
  if (y_bf16) combine_kernel<true><<<grid, 128, 0, s>>>(y, wts, rows, slots, d, static_cast<__nv_bfloat16*>(out));
  else combine_kernel<false><<<grid, 128, 0, s>>>(y, wts, rows, slots, d, static_cast<__nv_bfloat16*>(out));
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_moe_combine");
}

}  // extern "C"
