// Row-exact affine quantised matmul over the tiled layout (tf_layout.h): out[m, n] = sum_k x[m, k] * (s q[n, k] + b).
//
// Arithmetic contract (identical for every row count, tile shape and launch geometry):
//   for each K slice (a function of the weight shape only), acc = 0, and for each quantisation group in order
//       P'  = sum over the group of x * (q + C)      m16n8k16 bf16 MMAs chained from zero, fp32 accumulate
//       acc = fma(xs, b - C s, fma(P', s, acc))      xs = the group's sum of x, also from MMAs (x against ones)
//   slices are added in slice order and the sum is rounded once to bf16 (or returned as fp32).
// C = 128 is the constant the magic-number dequantisation leaves on every code (128 * 17 for 8-bit codes, whose two
// nibbles are multiplied separately); folding it into the bias term saves a subtraction per weight pair.
// The weights are the MMA's A operand (16 output columns x 16 inputs) and the rows of x are the B operand's columns,
// so one to eight rows cost a single MMA per 256 weights.  An MMA output element depends only on its own A row and B
// column, hence a row's bits never depend on the rows beside it.
//
// Block = 4 consumer warps (32 output columns each, all rows of the row tile) + 1 producer warp that issues the bulk
// copies (one per stage for the packed weights, one per row of x) and computes the group sums of x for the consumers.
// K slices of one column block run as one thread-block cluster and are summed in slice order through distributed
// shared memory; with more than 8 slices, or when the caller wants the slices, they go to `part` in global memory.
#pragma once

#include <cooperative_groups.h>

#include "tf_layout.h"
#include "tf_ptx.cuh"

namespace tf {

namespace cg = cooperative_groups;

struct QmmParams {
  const __nv_bfloat16* x;     // [M, K] bf16, row stride ldx elements, rows 16-byte aligned
  int64_t ldx;
  int M;
  const float* xs;            // optional [M, K / GS] fp32 group sums (row stride KG); null: computed here
  const uint32_t* w;          // tiled units
  int64_t sb_stride;          // words from one 128-column super-block to the next
  int N, K, KG;
  int sk;                     // K slices
  void* out;                  // [M, N] bf16 or fp32, row stride ldo elements
  int64_t ldo;
  int out_f32;
  int out_vec;                // rows of out allow 16-byte vector stores
  float* part;                // [sk, M, N] fp32 when the slices leave the kernel
  int cluster;                // 1: slices form a cluster and are summed here
  int* err;                   // device error word (0 = none)
};

constexpr int QMM_THREADS = 160;
constexpr int QMM_CONSUMERS = 128;
constexpr int XROW_BYTES = 272;            // 128 inputs of bf16 + 16 bytes so ldmatrix rows fall in distinct banks
constexpr int RED_STRIDE = 132;            // floats per row of the output staging tile (conflict-free fragment stores)

template <int BITS, int GS, int MT>
struct QmmGeo {
  static constexpr int S = GS / 16;                         // MMA k-steps per group
  static constexpr int G = 128 / GS;                        // groups per stage (a stage covers 128 inputs)
  static constexpr int ROWS = 8 * MT;
  static constexpr int WPL = words_per_lane(BITS, GS);
  static constexpr int UNITW = unit_words(BITS, GS);
  static constexpr int W_BYTES = G * UNITW * 4;
  static constexpr int X_BYTES = ROWS * XROW_BYTES;
  static constexpr int XS_BYTES = ROWS * G * 4;
  static constexpr int STAGE = W_BYTES + X_BYTES + XS_BYTES;
  static constexpr int RED_BYTES = ROWS * RED_STRIDE * 4;
  static constexpr int NST_RAW = 98304 / STAGE;
  static constexpr int NST = NST_RAW < 2 ? 2 : (NST_RAW > 12 ? 12 : NST_RAW);
  static constexpr int BAR_BYTES = 3 * NST * 8 + 16;
  static constexpr int SMEM = NST * STAGE + BAR_BYTES;
  static_assert(STAGE % 16 == 0 && W_BYTES % 16 == 0 && X_BYTES % 16 == 0, "stage parts stay 16-byte aligned");
  static_assert(NST * STAGE >= RED_BYTES, "the output staging tile reuses the stage memory");
  static_assert(SMEM <= 227 * 1024, "fits the shared memory of an SM");
};

// Group sums of one m8 tile by MMA against a tile of ones: d[0], d[1] = sums of rows 2t and 2t + 1 of the tile.
template <int GS>
__device__ __forceinline__ void ones_mma_group(float (&d)[4], uint32_t xaddr_lane) {
  const uint32_t ones[4] = {0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u};
  d[0] = d[1] = d[2] = d[3] = 0.f;
#pragma unroll
  for (int s = 0; s < GS / 16; s += 2) {
    uint32_t b[4];
    ldmatrix_x4(b, xaddr_lane + s * 32);
    mma_bf16(d, ones, b[0], b[1]);
    mma_bf16(d, ones, b[2], b[3]);
  }
}

template <int BITS, int GS, int MT>
__global__ void __launch_bounds__(QMM_THREADS) qmm_tiled_kernel(const QmmParams p) {
  using Geo = QmmGeo<BITS, GS, MT>;
  constexpr int S = Geo::S, G = Geo::G, ROWS = Geo::ROWS, WPL = Geo::WPL, UNITW = Geo::UNITW, NST = Geo::NST;
  constexpr bool SPLIT = Fmt<BITS>::SPLIT;

  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + NST * Geo::STAGE);
  uint64_t* empty = full + NST;
  uint64_t* sums = empty + NST;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sums + NST);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sb = blockIdx.x, m0 = blockIdx.y * ROWS, slice = blockIdx.z;
  const int per = p.KG / p.sk;                              // groups of this slice
  const int g_first = slice * per;
  const int nstages = (per + G - 1) / G;
  const int rows_here = min(ROWS, p.M - m0);

  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      mbar_init(full + i, 1);
      mbar_init(empty + i, 4);
      mbar_init(sums + i, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  const uint32_t* wbase = p.w + static_cast<int64_t>(sb) * p.sb_stride + static_cast<int64_t>(g_first) * UNITW;

  auto stage_ptr = [&](int slot) { return smem + slot * Geo::STAGE; };
  auto groups_of = [&](int st) { return min(G, per - st * G); };

  float acc[2][MT][4];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[h][mt][e] = 0.f;

  if (warp == 4) {
    // ------------------------------------------------------------------ producer: copies and group sums
    auto issue_w = [&](int st, int slot) {
      if (lane == 0) {
        const int ng = groups_of(st);
        const uint32_t bytes = ng * UNITW * 4 + rows_here * ng * GS * 2;
        mbar_expect_tx(full + slot, bytes);
        bulk_load(stage_ptr(slot), wbase + static_cast<int64_t>(st) * G * UNITW, ng * UNITW * 4, full + slot);
      }
    };
    auto issue_x = [&](int st, int slot) {
      const int ng = groups_of(st);
      const int64_t k0 = static_cast<int64_t>(g_first + st * G) * GS;
      for (int r = lane; r < rows_here; r += 32)
        bulk_load(stage_ptr(slot) + Geo::W_BYTES + r * XROW_BYTES, p.x + (m0 + r) * p.ldx + k0, ng * GS * 2, full + slot);
    };
    const int pro = min(NST, nstages);
    for (int st = 0; st < pro; ++st) issue_w(st, st);      // weights never depend on the previous kernel
    __syncwarp();
    pdl_wait();                                            // x (and out) may be the previous kernel's
    for (int st = 0; st < pro; ++st) issue_x(st, st);

    bool ok = true;
    for (int st = 0; st < nstages && ok; ++st) {
      const int slot = st % NST;
      ok = mbar_wait(full + slot, (st / NST) & 1, abort_flag);
      if (!ok) {
        if (lane == 0) {
          *abort_flag = ERR_WAIT_FULL;
          atomicCAS(p.err, 0, ERR_WAIT_FULL);
        }
        break;
      }
      const int ng = groups_of(st);
      float* xs_s = reinterpret_cast<float*>(stage_ptr(slot) + Geo::W_BYTES + Geo::X_BYTES);
      if (p.xs != nullptr) {
        for (int i = lane; i < ng * ROWS; i += 32) {
          const int u = i / ROWS, r = i % ROWS;
          xs_s[u * ROWS + r] = r < rows_here ? p.xs[static_cast<int64_t>(m0 + r) * p.KG + g_first + st * G + u] : 0.f;
        }
      } else {
        const uint32_t xs0 = smem_addr(stage_ptr(slot) + Geo::W_BYTES) + (lane & 7) * XROW_BYTES + (lane >> 3) * 16;
        for (int u = 0; u < ng; ++u)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            float d[4];
            ones_mma_group<GS>(d, xs0 + mt * 8 * XROW_BYTES + u * GS * 2);
            if (lane < 4) *reinterpret_cast<float2*>(xs_s + u * ROWS + mt * 8 + 2 * lane) = make_float2(d[0], d[1]);
          }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(sums + slot);
      // refill the slot the consumers are about to finish: stage st - 1 + NST goes where stage st - 1 was
      const int nst = st - 1 + NST;
      if (st >= 1 && nst < nstages) {
        const int slot2 = (st - 1) % NST;
        ok = mbar_wait(empty + slot2, ((st - 1) / NST) & 1, abort_flag);
        if (!ok) {
          if (lane == 0) {
            *abort_flag = ERR_WAIT_EMPTY;
            atomicCAS(p.err, 0, ERR_WAIT_EMPTY);
          }
          break;
        }
        issue_w(nst, slot2);
        __syncwarp();
        issue_x(nst, slot2);
      }
    }
    if (!ok) {
      // give copies still in flight time to land before this block's shared memory is released
      for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
  } else {
    // ------------------------------------------------------------------ consumers: dequantise, MMA, affine epilogue
    pdl_wait();
    const int g = lane >> 2, t = lane & 3;
    constexpr float OFFSET = code_offset(BITS);
    bool ok = true;
    for (int st = 0; st < nstages && ok; ++st) {
      const int slot = st % NST;
      const uint32_t parity = (st / NST) & 1;
      ok = mbar_wait(full + slot, parity, abort_flag);
      if (!ok) {
        if (lane == 0) {
          *abort_flag = ERR_WAIT_FULL;
          atomicCAS(p.err, 0, ERR_WAIT_FULL);
        }
        break;
      }
      const int ng = groups_of(st);
      const uint8_t* sp = stage_ptr(slot);
      const uint32_t* wst = reinterpret_cast<const uint32_t*>(sp);
      const uint32_t xaddr = smem_addr(sp + Geo::W_BYTES) + (lane & 7) * XROW_BYTES + (lane >> 3) * 16;
      const float* xs_s = reinterpret_cast<const float*>(sp + Geo::W_BYTES + Geo::X_BYTES);
      bool sums_ready = false;
#pragma unroll 1
      for (int u = 0; u < ng; ++u) {
        uint32_t wd[WPL];
        {
          const uint32_t* src = wst + u * UNITW + (warp * 32 + lane) * WPL;
          if constexpr (WPL % 4 == 0) {
#pragma unroll
            for (int i = 0; i < WPL; i += 4) {
              const uint4 v = *reinterpret_cast<const uint4*>(src + i);
              wd[i] = v.x, wd[i + 1] = v.y, wd[i + 2] = v.z, wd[i + 3] = v.w;
            }
          } else if constexpr (WPL % 2 == 0) {
#pragma unroll
            for (int i = 0; i < WPL; i += 2) {
              const uint2 v = *reinterpret_cast<const uint2*>(src + i);
              wd[i] = v.x, wd[i + 1] = v.y;
            }
          } else {
#pragma unroll
            for (int i = 0; i < WPL; ++i) wd[i] = src[i];
          }
        }
        const uint4 sbw = *reinterpret_cast<const uint4*>(wst + u * UNITW + TILE_PAIRS * 32 * WPL + warp * 32 + g * 4);

        float P[2][MT][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) P[h][mt][e] = 0.f;

        uint32_t bf[MT][4];
#pragma unroll
        for (int s = 0; s < S; ++s) {
          if ((s & 1) == 0) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(bf[mt], xaddr + mt * 8 * XROW_BYTES + u * GS * 2 + s * 32);
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t a[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) a[j] = pair_reg<BITS, GS, false>(wd, (h * S + s) * 4 + j);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) mma_bf16(P[h][mt], a, bf[mt][2 * (s & 1)], bf[mt][2 * (s & 1) + 1]);
            if constexpr (SPLIT) {
              uint32_t ah[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) ah[j] = pair_reg<BITS, GS, true>(wd, (h * S + s) * 4 + j);
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                const __nv_bfloat162 k16 = __floats2bfloat162_rn(16.f, 16.f);
                __nv_bfloat162 b0 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&bf[mt][2 * (s & 1)]), k16);
                __nv_bfloat162 b1 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&bf[mt][2 * (s & 1) + 1]), k16);
                mma_bf16(P[h][mt], ah, *reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1));
              }
            }
          }
        }

        if (!sums_ready) {
          ok = mbar_wait(sums + slot, parity, abort_flag);
          if (!ok) {
            if (lane == 0) {
              *abort_flag = ERR_WAIT_SUMS;
              atomicCAS(p.err, 0, ERR_WAIT_SUMS);
            }
            break;
          }
          sums_ready = true;
        }
        const uint32_t sbv[4] = {sbw.x, sbw.y, sbw.z, sbw.w};       // (tile 0, col g), (0, g + 8), (1, g), (1, g + 8)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float s0 = bf16_lo(sbv[2 * h]), s1 = bf16_lo(sbv[2 * h + 1]);
          const float c0 = fmaf(-OFFSET, s0, bf16_hi(sbv[2 * h])), c1 = fmaf(-OFFSET, s1, bf16_hi(sbv[2 * h + 1]));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const float2 xv = *reinterpret_cast<const float2*>(xs_s + u * ROWS + mt * 8 + 2 * t);
            fma2(acc[h][mt][0], acc[h][mt][1], P[h][mt][0], P[h][mt][1], s0);
            fma2(acc[h][mt][0], acc[h][mt][1], xv.x, xv.y, c0);
            fma2(acc[h][mt][2], acc[h][mt][3], P[h][mt][2], P[h][mt][3], s1);
            fma2(acc[h][mt][2], acc[h][mt][3], xv.x, xv.y, c1);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + slot);
    }
  }

  // -------------------------------------------------------------------- output: stage, sum the slices in order, store
  __syncthreads();                                          // every stage consumed: its memory becomes the staging tile
  float* red = reinterpret_cast<float*>(smem);
  if (warp < 4) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int n = warp * 32 + h * 16 + g, m = mt * 8 + 2 * t;
        red[m * RED_STRIDE + n] = acc[h][mt][0];
        red[(m + 1) * RED_STRIDE + n] = acc[h][mt][1];
        red[m * RED_STRIDE + n + 8] = acc[h][mt][2];
        red[(m + 1) * RED_STRIDE + n + 8] = acc[h][mt][3];
      }
  }
  const bool clustered = p.cluster && p.sk > 1;
  cg::cluster_group cluster = cg::this_cluster();
  if (clustered) cluster.sync(); else __syncthreads();

  const bool failed = *abort_flag != 0;
  const int n0 = sb * SB_COLS;
  const int share = clustered ? p.sk : 1, mine = clustered ? slice : 0;
  if (!failed) {
    for (int idx = tid; idx < ROWS * 16; idx += QMM_THREADS) {
      if (idx % share != mine) continue;
      const int ml = idx >> 4, c8 = (idx & 15) * 8, m = m0 + ml, n = n0 + c8;
      if (ml >= rows_here || n >= p.N) continue;
      float v[8];
      {
        const float4 a = *reinterpret_cast<const float4*>(red + ml * RED_STRIDE + c8);
        const float4 b = *reinterpret_cast<const float4*>(red + ml * RED_STRIDE + c8 + 4);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
      }
      if (clustered) {
        // slice order: ((s0 + s1) + s2) + ...; this block holds slice `slice`, the others are read remotely
        float tot[8];
#pragma unroll 1
        for (int r = 0; r < p.sk; ++r) {
          const float* src = r == slice ? red : cluster.map_shared_rank(red, r);
          const float4 a = *reinterpret_cast<const float4*>(src + ml * RED_STRIDE + c8);
          const float4 b = *reinterpret_cast<const float4*>(src + ml * RED_STRIDE + c8 + 4);
          const float w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) tot[e] = r == 0 ? w[e] : tot[e] + w[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = tot[e];
      }
      const int valid = min(8, p.N - n);
      if (!clustered && p.sk > 1) {
        float* dst = p.part + (static_cast<int64_t>(slice) * p.M + m) * p.N + n;
        for (int e = 0; e < valid; ++e) dst[e] = v[e];
      } else if (p.out_f32) {
        float* dst = reinterpret_cast<float*>(p.out) + m * p.ldo + n;
        if (p.out_vec && valid == 8) {
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
          for (int e = 0; e < valid; ++e) dst[e] = v[e];
        }
      } else {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + m * p.ldo + n;
        if (p.out_vec && valid == 8) {
          uint4 o;
          __nv_bfloat162 t0 = __floats2bfloat162_rn(v[0], v[1]), t1 = __floats2bfloat162_rn(v[2], v[3]);
          __nv_bfloat162 t2 = __floats2bfloat162_rn(v[4], v[5]), t3 = __floats2bfloat162_rn(v[6], v[7]);
          o.x = *reinterpret_cast<uint32_t*>(&t0), o.y = *reinterpret_cast<uint32_t*>(&t1);
          o.z = *reinterpret_cast<uint32_t*>(&t2), o.w = *reinterpret_cast<uint32_t*>(&t3);
          *reinterpret_cast<uint4*>(dst) = o;
        } else {
          for (int e = 0; e < valid; ++e) dst[e] = __float2bfloat16_rn(v[e]);
        }
      }
    }
  }
  if (clustered) cluster.sync();                            // peers may still be reading this block's tile
}

}  // namespace tf
