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
// Block = KW slice lanes x 4 consumer warps (a lane streams one K slice of the block's 128 output columns; each of its
// warps owns 32 columns and all rows of the row tile) + a copy warp that issues the bulk copies (one per lane and stage
// for the packed weights, one per row of x) + a sums warp that computes the group sums of x for the consumers.
// The sk / KW blocks that hold the slices of one column block form a thread-block cluster; the slices are summed in
// slice order through (distributed) shared memory.  When the caller wants the slices, or there are more than the
// cluster can hold, they go to `part` in global memory.  How slices map to lanes and blocks never changes a bit.
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
  int cluster;                // 1: the blocks of a column block form a cluster and the slices are summed here
  int* err;                   // device error word (0 = none)
};

constexpr int XROW_BYTES = 272;            // 128 inputs of bf16 + 16 bytes so ldmatrix rows fall in distinct banks
constexpr int RED_STRIDE = 132;            // floats per row of the output staging tile (conflict-free fragment stores)

template <int BITS, int GS, int MT, int KW>
struct QmmGeo {
  static constexpr int CONSUMERS = 4 * KW;                  // consumer warps
  static constexpr int THREADS = 32 * (CONSUMERS + 2);
  static constexpr int S = GS / 16;                         // MMA k-steps per group
  static constexpr int G = 128 / GS;                        // groups per stage (a stage covers 128 inputs)
  static constexpr int ROWS = 8 * MT;
  static constexpr int WPL = words_per_lane(BITS, GS);
  static constexpr int UNITW = unit_words(BITS, GS);
  static constexpr int W_BYTES = G * UNITW * 4;
  static constexpr int X_BYTES = ROWS * XROW_BYTES;
  static constexpr int XS_BYTES = ROWS * G * 4;
  static constexpr int LANE_STAGE = W_BYTES + X_BYTES + XS_BYTES;
  static constexpr int STAGE = KW * LANE_STAGE;
  static constexpr int RED_BYTES = KW * ROWS * RED_STRIDE * 4;
  static constexpr int BUDGET = KW == 1 ? (MT <= 2 ? 73 * 1024 : 110 * 1024) : KW == 2 ? 110 * 1024 : 222 * 1024;
  static constexpr int NST_RAW = BUDGET / STAGE;
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

template <int BITS, int GS, int MT, int KW>
__global__ void __launch_bounds__(QmmGeo<BITS, GS, MT, KW>::THREADS) qmm_tiled_kernel(const QmmParams p) {
  using Geo = QmmGeo<BITS, GS, MT, KW>;
  constexpr int S = Geo::S, G = Geo::G, ROWS = Geo::ROWS, WPL = Geo::WPL, UNITW = Geo::UNITW, NST = Geo::NST;
  constexpr int CONSUMERS = Geo::CONSUMERS, THREADS = Geo::THREADS;
  constexpr bool SPLIT = Fmt<BITS>::SPLIT;

  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + NST * Geo::STAGE);
  uint64_t* empty = full + NST;
  uint64_t* sums = empty + NST;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sums + NST);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sb = blockIdx.x, m0 = blockIdx.y * ROWS;
  const int per = p.KG / p.sk;                              // groups of a slice
  const int nstages = (per + G - 1) / G;
  const int rows_here = min(ROWS, p.M - m0);

  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      mbar_init(full + i, 1);
      mbar_init(empty + i, CONSUMERS);
      mbar_init(sums + i, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  // lane kw of this block streams slice blockIdx.z * KW + kw
  auto slice_of = [&](int kw) { return static_cast<int>(blockIdx.z) * KW + kw; };
  auto lane_ptr = [&](int slot, int kw) { return smem + slot * Geo::STAGE + kw * Geo::LANE_STAGE; };
  auto groups_of = [&](int st) { return min(G, per - st * G); };
  auto give_up = [&](int code) {
    if (lane == 0) {
      *abort_flag = code;
      atomicCAS(p.err, 0, code);
    }
  };

  float acc[2][MT][4];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[h][mt][e] = 0.f;

  if (warp == CONSUMERS) {
    // ------------------------------------------------------------------ copy warp: weights and rows of x
    const uint32_t* wsb = p.w + static_cast<int64_t>(sb) * p.sb_stride;
    auto issue_w = [&](int st, int slot) {
      if (lane == 0) {
        const int ng = groups_of(st);
        mbar_expect_tx(full + slot, KW * (ng * UNITW * 4 + rows_here * ng * GS * 2));
#pragma unroll
        for (int kw = 0; kw < KW; ++kw)
          bulk_load(lane_ptr(slot, kw), wsb + (static_cast<int64_t>(slice_of(kw)) * per + st * G) * UNITW, ng * UNITW * 4,
                    full + slot);
      }
    };
    auto issue_x = [&](int st, int slot) {
      const int ng = groups_of(st);
      for (int i = lane; i < KW * rows_here; i += 32) {
        const int kw = i / rows_here, r = i % rows_here;
        const int64_t k0 = (static_cast<int64_t>(slice_of(kw)) * per + st * G) * GS;
        bulk_load(lane_ptr(slot, kw) + Geo::W_BYTES + r * XROW_BYTES, p.x + (m0 + r) * p.ldx + k0, ng * GS * 2,
                  full + slot);
      }
    };
    const int pro = min(NST, nstages);
    for (int st = 0; st < pro; ++st) issue_w(st, st);      // weights never depend on the previous kernel
    __syncwarp();
    pdl_wait();                                            // x may be the previous kernel's output
    for (int st = 0; st < pro; ++st) issue_x(st, st);
    bool ok = true;
    for (int st = NST; st < nstages; ++st) {               // stage st goes where stage st - NST was
      const int slot = st % NST;
      ok = mbar_wait(empty + slot, ((st - NST) / NST) & 1, abort_flag);
      if (!ok) {
        give_up(ERR_WAIT_EMPTY);
        break;
      }
      issue_w(st, slot);
      __syncwarp();
      issue_x(st, slot);
    }
    if (!ok) {
      // give copies still in flight time to land before this block's shared memory is released
      for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
  } else if (warp == CONSUMERS + 1) {
    // ------------------------------------------------------------------ sums warp: group sums of x for every lane
    pdl_wait();
    for (int st = 0; st < nstages; ++st) {
      const int slot = st % NST;
      if (!mbar_wait(full + slot, (st / NST) & 1, abort_flag)) {
        give_up(ERR_WAIT_FULL);
        break;
      }
      const int ng = groups_of(st);
#pragma unroll 1
      for (int kw = 0; kw < KW; ++kw) {
        float* xs_s = reinterpret_cast<float*>(lane_ptr(slot, kw) + Geo::W_BYTES + Geo::X_BYTES);
        if (p.xs != nullptr) {
          const int g0 = slice_of(kw) * per + st * G;
          for (int i = lane; i < ng * ROWS; i += 32) {
            const int u = i / ROWS, r = i % ROWS;
            xs_s[u * ROWS + r] = r < rows_here ? p.xs[static_cast<int64_t>(m0 + r) * p.KG + g0 + u] : 0.f;
          }
        } else {
          const uint32_t xs0 = smem_addr(lane_ptr(slot, kw) + Geo::W_BYTES) + (lane & 7) * XROW_BYTES + (lane >> 3) * 16;
          for (int u = 0; u < ng; ++u)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              float d[4];
              ones_mma_group<GS>(d, xs0 + mt * 8 * XROW_BYTES + u * GS * 2);
              if (lane < 4) *reinterpret_cast<float2*>(xs_s + u * ROWS + mt * 8 + 2 * lane) = make_float2(d[0], d[1]);
            }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(sums + slot);
    }
  } else {
    // ------------------------------------------------------------------ consumers: dequantise, MMA, affine epilogue
    const int kw = warp >> 2, tp = warp & 3;
    const int g = lane >> 2, t = lane & 3;
    constexpr float OFFSET = code_offset(BITS);
    bool ok = true;
    for (int st = 0; st < nstages && ok; ++st) {
      const int slot = st % NST;
      const uint32_t parity = (st / NST) & 1;
      ok = mbar_wait(full + slot, parity, abort_flag);
      if (!ok) {
        give_up(ERR_WAIT_FULL);
        break;
      }
      const int ng = groups_of(st);
      const uint8_t* sp = lane_ptr(slot, kw);
      const uint32_t* wst = reinterpret_cast<const uint32_t*>(sp);
      const uint32_t xaddr = smem_addr(sp + Geo::W_BYTES) + (lane & 7) * XROW_BYTES + (lane >> 3) * 16;
      const float* xs_s = reinterpret_cast<const float*>(sp + Geo::W_BYTES + Geo::X_BYTES);
      bool sums_ready = false;
#pragma unroll 1
      for (int u = 0; u < ng; ++u) {
        uint32_t wd[WPL];
        {
          const uint32_t* src = wst + u * UNITW + (tp * 32 + lane) * WPL;
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
        const uint4 sbw = *reinterpret_cast<const uint4*>(wst + u * UNITW + TILE_PAIRS * 32 * WPL + tp * 32 + g * 4);

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
            give_up(ERR_WAIT_SUMS);
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
  __syncthreads();                                          // every stage consumed: its memory becomes the staging tiles
  pdl_wait();                                               // nothing is written before the previous kernel is done
  float* red = reinterpret_cast<float*>(smem);              // [KW][ROWS][RED_STRIDE]
  constexpr int RED_TILE = ROWS * RED_STRIDE;
  if (warp < CONSUMERS) {
    const int kw = warp >> 2, tp = warp & 3, g = lane >> 2, t = lane & 3;
    float* mine = red + kw * RED_TILE;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int n = tp * 32 + h * 16 + g, m = mt * 8 + 2 * t;
        mine[m * RED_STRIDE + n] = acc[h][mt][0];
        mine[(m + 1) * RED_STRIDE + n] = acc[h][mt][1];
        mine[m * RED_STRIDE + n + 8] = acc[h][mt][2];
        mine[(m + 1) * RED_STRIDE + n + 8] = acc[h][mt][3];
      }
  }
  const int nblocks = p.sk / KW;                            // blocks holding the slices of this column block
  const bool clustered = p.cluster && nblocks > 1;
  cg::cluster_group cluster = cg::this_cluster();
  if (clustered) cluster.sync(); else __syncthreads();

  const bool failed = *abort_flag != 0;
  const int n0 = sb * SB_COLS;
  const bool summed = p.cluster != 0;                       // slices are summed here (else they go to part)
  const int share = clustered ? nblocks : 1, mine_rank = clustered ? static_cast<int>(blockIdx.z) : 0;
  if (!failed) {
    const int items = summed ? ROWS * 16 : KW * ROWS * 16;
    for (int idx = tid; idx < items; idx += THREADS) {
      if (idx % share != mine_rank) continue;
      const int kw_item = idx / (ROWS * 16), rem = idx % (ROWS * 16);
      const int ml = rem >> 4, c8 = (rem & 15) * 8, m = m0 + ml, n = n0 + c8;
      if (ml >= rows_here || n >= p.N) continue;
      const int off = ml * RED_STRIDE + c8;
      float v[8];
      if (summed) {
        // slice order ((s0 + s1) + s2) + ...: slice s is lane s % KW of block s / KW of the cluster
#pragma unroll 1
        for (int s = 0; s < p.sk; ++s) {
          const int b = s / KW;
          const float* tile = (b == mine_rank || !clustered) ? red : cluster.map_shared_rank(red, b);
          const float* src = tile + (s % KW) * RED_TILE + off;
          const float4 lo = *reinterpret_cast<const float4*>(src);
          const float4 hi = *reinterpret_cast<const float4*>(src + 4);
          const float w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = s == 0 ? w[e] : v[e] + w[e];
        }
      } else {
        const float* src = red + kw_item * RED_TILE + off;
        const float4 lo = *reinterpret_cast<const float4*>(src);
        const float4 hi = *reinterpret_cast<const float4*>(src + 4);
        v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
      }
      const int valid = min(8, p.N - n);
      if (!summed) {
        float* dst = p.part + (static_cast<int64_t>(slice_of(kw_item)) * p.M + m) * p.N + n;
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
  if (clustered) cluster.sync();                            // peers may still be reading this block's tiles
}

}  // namespace tf
