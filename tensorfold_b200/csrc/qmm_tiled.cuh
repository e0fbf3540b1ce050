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
// Block = KW column lanes x 4 consumer warps (a lane streams one 128-column super-block over the block's K slice; each
// of its warps owns 32 columns and all rows of the row tile) + a copy warp (one bulk copy per lane and stage for the
// packed weights; tensor-map copies into 128-byte-swizzled half tiles for the rows of x, which all lanes share, 16-byte
// asynchronous copies in the grouped form that gathers rows) + a sums warp that computes the group sums of x once for
// the whole block.  The blocks that hold the K slices of the same columns form a thread-block cluster: after one
// cluster barrier every block pushes its slice of each 8-column piece into the shared memory of the block that owns
// the piece, and the owner adds the slices in slice order.  When the caller wants the slices, or there are more than a
// cluster can hold, they go to `part` in global memory.  Geometry never changes a bit.
#pragma once

#include <cooperative_groups.h>
#include <cuda.h>

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
  int cluster;                // 1: the sk blocks of a column block form a cluster and the slices are summed here
  int* err;                   // device error word (0 = none)
  // grouped (mixture-of-experts) mode, items != null: block (x, y) runs plan item y = (expert, first, count <= ROWS):
  // its rows are pairs members[first .. first + count), read from row pair / slots of x (slots > 0) or row pair of x
  // (slots == 0), against expert `expert`'s weights, written to row `pair` of out.  sk must be 1.
  const int* items;           // [max items][3]
  const int* counts;          // [0] = items in use; blocks past it leave at once
  const int* members;         // pair ids grouped by expert
  int slots;
  int64_t expert_stride;      // words from one expert's units to the next
  int experts;                // experts the table holds: an item that names another one is skipped and reported
  // epilogue: 0 store as is; 1 bf16(relu(bf16 v)^2); 2 SwiGLU over column pairs: the weight rows interleave 16 gate
  // columns with 16 up columns, so a tile pair holds both halves and out has N / 2 columns.
  int epi;
  float limit;                // SwiGLU clip (0: none)
};

// SwiGLU as the families define it: bf16(bf16(silu(bf16 g)) * bf16 u), clipped first when limit > 0.
__device__ __forceinline__ float bf16_round_f(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float swiglu_f(float g, float u, float limit) {
  float gv = bf16_round_f(g), uv = bf16_round_f(u);
  if (limit > 0.f) {
    gv = fminf(gv, limit);
    uv = fminf(fmaxf(uv, -limit), limit);
  }
  return bf16_round_f(gv / (1.f + expf(-gv))) * uv;
}
__device__ __forceinline__ float relu2_f(float v) {
  const float u = fmaxf(bf16_round_f(v), 0.f);
  return u * u;
}

// A stage's rows of x: two half tiles of 64 inputs (128 bytes a row) in the 128-byte swizzle pattern (16-byte chunk c of
// row r sits at chunk c ^ (r & 7)): what a tensor-map copy writes, and conflict-free for ldmatrix.
constexpr int XHALF_ROW = 128;
constexpr int RED_STRIDE = 132;            // floats per row of the output staging tile (conflict-free fragment stores)

#ifndef TF_BUDGET1_KB
#define TF_BUDGET1_KB 73
#endif
#ifndef TF_BUDGET2_KB
#define TF_BUDGET2_KB 110
#endif
#ifndef TF_BUDGET4_KB
#define TF_BUDGET4_KB 222
#endif

template <int BITS, int GS, int MT, int KW>
struct QmmGeo {
  static constexpr int CONSUMERS = 4 * KW;                  // consumer warps
  static constexpr int THREADS = 32 * (CONSUMERS + 2);
  static constexpr int S = GS / 16;                         // MMA k-steps per group
  static constexpr int G = 128 / GS;                        // groups per stage (a stage covers 128 inputs)
  static constexpr int ROWS = 8 * MT;
  static constexpr int WPL = words_per_lane(BITS, GS);
  static constexpr int UNITW = unit_words(BITS, GS);
  static constexpr int W_BYTES = G * UNITW * 4;             // one lane's weights of a stage
  static constexpr int XHALF = ROWS * XHALF_ROW;           // bytes of a half tile (64 inputs of every row)
  static constexpr int X_BYTES = 2 * XHALF;
  static constexpr int XS_BYTES = ROWS * G * 4;
  static constexpr int X_OFF = 0;                          // first: a stage starts 1024-byte aligned, as the swizzle needs
  static constexpr int W_OFF = X_BYTES;
  static constexpr int XS_OFF = W_OFF + KW * W_BYTES;
  static constexpr int STAGE = (XS_OFF + XS_BYTES + 1023) / 1024 * 1024;
  static constexpr int RED_BYTES = KW * ROWS * RED_STRIDE * 4;
  // slices pushed by the cluster's blocks: 16 pieces of 32 bytes a row and lane (+ one piece a slice of rounding)
  static constexpr int RECV_BYTES = KW * ROWS * 512 + 8 * 32;
  static constexpr int BUDGET = (MT > 2 ? 110 : KW == 1 ? TF_BUDGET1_KB : KW == 2 ? TF_BUDGET2_KB : TF_BUDGET4_KB) * 1024;
  static constexpr int NST_A = BUDGET / STAGE, NST_B = (RED_BYTES + RECV_BYTES + STAGE - 1) / STAGE;
  static constexpr int NST_C = NST_A < 2 ? 2 : (NST_A > 12 ? 12 : NST_A);
  static constexpr int NST = NST_C < NST_B ? NST_B : NST_C;
  static constexpr int BAR_BYTES = 3 * NST * 8 + 8 + 16;   // full, empty, sums per stage; the receive barrier; abort flag
  static constexpr int SMEM = NST * STAGE + BAR_BYTES + 1024;     // + slack to align the first stage
  // blocks per SM the register file should allow (64 registers a thread is the floor the kernel needs)
  static constexpr int BY_SMEM = (227 * 1024) / (SMEM + 1024), BY_REGS = 65536 / (THREADS * (MT == 2 ? 80 : 64));
  static constexpr int MINB = MT > 2 ? 1 : (BY_SMEM < BY_REGS ? BY_SMEM : BY_REGS) < 1 ? 1 : (BY_SMEM < BY_REGS ? BY_SMEM : BY_REGS);
  static_assert(STAGE % 1024 == 0 && W_BYTES % 16 == 0 && XS_OFF % 16 == 0, "stage parts stay aligned");
  static_assert(NST * STAGE >= RED_BYTES + RECV_BYTES, "the output staging tile and the receive area reuse the stage memory");
  static_assert(SMEM <= 227 * 1024, "fits the shared memory of an SM");
};

// Shared-memory address of the ldmatrix.x4 that fetches inputs [k0, k0 + 32) (k0 a multiple of 32, relative to the stage)
// of the m8 tile `mt`: lane l addresses row l & 7 of matrix l >> 3 (8 inputs each).  xrow = byte offset of the lane's row
// in a half tile, sw0 / sw1 = the lane's swizzled chunk offsets for chunk bases 0 and 4.
template <int XHALF>
__device__ __forceinline__ uint32_t x_ldm_addr(uint32_t xbase, uint32_t xrow, uint32_t sw0, uint32_t sw1, int mt, int k0) {
  const int chunk = k0 >> 3;                                // 16-byte chunk of the row where the 32 inputs start: 0, 4, 8 or 12
  return xbase + (chunk >> 3) * XHALF + mt * 8 * XHALF_ROW + xrow + ((chunk & 4) ? sw1 : sw0);
}

// Group sums of one m8 tile by MMA against a tile of ones: d[0], d[1] = sums of rows 2t and 2t + 1 of the tile.
template <int GS, int XHALF>
__device__ __forceinline__ void ones_mma_group(float (&d)[4], uint32_t xbase, uint32_t xrow, uint32_t sw0, uint32_t sw1, int mt,
                                               int k0) {
  const uint32_t ones[4] = {0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u};
  d[0] = d[1] = d[2] = d[3] = 0.f;
#pragma unroll
  for (int s = 0; s < GS / 16; s += 2) {
    uint32_t b[4];
    ldmatrix_x4(b, x_ldm_addr<XHALF>(xbase, xrow, sw0, sw1, mt, k0 + 16 * s));
    mma_bf16(d, ones, b[0], b[1]);
    mma_bf16(d, ones, b[2], b[3]);
  }
}

template <int BITS, int GS, int MT, int KW>
__global__ void __launch_bounds__(QmmGeo<BITS, GS, MT, KW>::THREADS, QmmGeo<BITS, GS, MT, KW>::MINB)
qmm_tiled_kernel(const __grid_constant__ CUtensorMap tmx, const QmmParams p) {
  using Geo = QmmGeo<BITS, GS, MT, KW>;
  constexpr int S = Geo::S, G = Geo::G, ROWS = Geo::ROWS, WPL = Geo::WPL, UNITW = Geo::UNITW, NST = Geo::NST;
  constexpr int CONSUMERS = Geo::CONSUMERS, THREADS = Geo::THREADS;
  constexpr bool SPLIT = Fmt<BITS>::SPLIT;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + NST * Geo::STAGE);   // weights and x of a stage have landed
  uint64_t* empty = full + NST;                                           // every consumer warp is done with a stage
  uint64_t* sums = empty + NST;                                           // the stage's group sums are written
  uint64_t* recv_bar = sums + NST;                                        // every block of the cluster has pushed its slice
  volatile int* abort_flag = reinterpret_cast<volatile int*>(recv_bar + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nsb = (p.N + SB_COLS - 1) / SB_COLS;
  const int sb0 = blockIdx.x * KW;                          // lane kw streams super-block sb0 + kw (if it exists)
  const int lanes_here = min(KW, nsb - sb0);
  const int slice = blockIdx.z;
  // slice s covers groups [s KG / sk, (s + 1) KG / sk): a function of the shape only; sizes differ by at most one group
  const int g_first = static_cast<int>(static_cast<int64_t>(slice) * p.KG / p.sk);
  const int per = static_cast<int>(static_cast<int64_t>(slice + 1) * p.KG / p.sk) - g_first;
  const int nstages = (per + G - 1) / G;
  const bool grouped = p.items != nullptr;
  int m0 = blockIdx.y * ROWS, rows_here, first = 0;
  const uint32_t* wroot = p.w;
  if (grouped) {
    pdl_wait();                                             // the plan may be the previous kernel's output
    if (static_cast<int>(blockIdx.y) >= p.counts[0]) return;
    const int* item = p.items + 3 * blockIdx.y;
    if (item[0] < 0 || item[0] >= p.experts) {              // never read past the table: skip the item, tell the host
      if (tid == 0) atomicCAS(p.err, 0, ERR_BAD_ITEM);
      return;
    }
    wroot += static_cast<int64_t>(item[0]) * p.expert_stride;
    first = item[1];
    rows_here = min(ROWS, item[2]);
    m0 = 0;
  } else {
    rows_here = min(ROWS, p.M - m0);
  }
  auto row_of = [&](int r) -> int64_t {                      // the row of x that row r of this block reads
    if (!grouped) return m0 + r;
    const int pair = p.members[first + r];
    return p.slots > 0 ? pair / p.slots : pair;
  };

  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      mbar_init(full + i, 1 + 32);                          // the expect_tx arrive + each copy-warp lane's cp.async arrive
      mbar_init(empty + i, CONSUMERS);
      mbar_init(sums + i, 1);
    }
    mbar_init(recv_bar, p.sk);
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  auto stage_ptr = [&](int slot) { return smem + slot * Geo::STAGE; };
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
    // ------------------------------------------------------------------ copy warp: weights (bulk) and rows of x (16 B)
    const uint32_t* wbase = wroot + static_cast<int64_t>(sb0) * p.sb_stride + static_cast<int64_t>(g_first) * UNITW;
    auto issue_w = [&](int st, int slot) {
      if (lane == 0) {
        const int ng = groups_of(st);
        mbar_expect_tx(full + slot, lanes_here * ng * UNITW * 4);
        for (int kw = 0; kw < lanes_here; ++kw)
          bulk_load(stage_ptr(slot) + Geo::W_OFF + kw * Geo::W_BYTES, wbase + kw * p.sb_stride + static_cast<int64_t>(st) * G * UNITW,
                    ng * UNITW * 4, full + slot);
      }
    };
    auto issue_x = [&](int st, int slot) {
      const int kext = groups_of(st) * GS;                  // inputs of this stage (at most 128)
      uint8_t* dst = stage_ptr(slot) + Geo::X_OFF;
      if (!grouped) {
        // one tensor-map copy per 64 inputs: a [64 x ROWS] box lands in the swizzled half tile; rows past M read zero
        if (lane == 0) {
          const int boxes = (kext + 63) / 64;
          mbar_expect_tx_only(full + slot, boxes * Geo::XHALF);
          const int k0 = (g_first + st * G) * GS;
          for (int b = 0; b < boxes; ++b) tma_load_2d(dst + b * Geo::XHALF, &tmx, k0 + 64 * b, m0, full + slot);
        }
      } else {
        // gathered rows: 16-byte copies placed in the same swizzle pattern
        const int cpr = kext / 8;                           // 16-byte chunks a row
        const __nv_bfloat16* src = p.x + static_cast<int64_t>(g_first + st * G) * GS;
        for (int c = lane; c < rows_here * cpr; c += 32) {
          const int r = c / cpr, q = c - r * cpr;
          cp_async16(dst + (q >> 3) * Geo::XHALF + r * XHALF_ROW + (((q & 7) ^ (r & 7)) << 4), src + row_of(r) * p.ldx + q * 8);
        }
      }
      cp_async_arrive(full + slot);
    };
    const int pro = min(NST, nstages);
    for (int st = 0; st < pro; ++st) issue_w(st, st);      // weights never depend on the previous kernel
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
      issue_x(st, slot);
    }
    if (!ok) {
      // give copies still in flight time to land before this block's shared memory is released
      for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
  } else if (warp == CONSUMERS + 1) {
    // ------------------------------------------------------------------ sums warp: group sums of x, once per block
    pdl_wait();
    for (int st = 0; st < nstages; ++st) {
      const int slot = st % NST;
      if (!mbar_wait(full + slot, (st / NST) & 1, abort_flag)) {
        give_up(ERR_WAIT_FULL);
        break;
      }
      const int ng = groups_of(st);
      float* xs_s = reinterpret_cast<float*>(stage_ptr(slot) + Geo::XS_OFF);
      if (p.xs != nullptr) {
        const int g0 = g_first + st * G;
        for (int i = lane; i < ng * ROWS; i += 32) {
          const int u = i / ROWS, r = i % ROWS;
          xs_s[u * ROWS + r] = r < rows_here ? p.xs[row_of(r) * p.KG + g0 + u] : 0.f;
        }
      } else {
        const uint32_t xbase = smem_addr(stage_ptr(slot) + Geo::X_OFF), xrow = (lane & 7) * XHALF_ROW;
        const uint32_t sw0 = (((lane >> 3) ^ (lane & 7)) << 4), sw1 = (((4 | (lane >> 3)) ^ (lane & 7)) << 4);
#pragma unroll
        for (int u = 0; u < G; ++u) {
          if (u >= ng) break;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            float d[4];
            ones_mma_group<GS, Geo::XHALF>(d, xbase, xrow, sw0, sw1, mt, u * GS);
            if (lane < 4) *reinterpret_cast<float2*>(xs_s + u * ROWS + mt * 8 + 2 * lane) = make_float2(d[0], d[1]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(sums + slot);               // also tells the consumers that the stage has landed
    }
  } else {
    // ------------------------------------------------------------------ consumers: dequantise, MMA, affine epilogue
    const int kw = warp >> 2, tp = warp & 3;
    const int g = lane >> 2, t = lane & 3;
    const bool active = kw < lanes_here;
    constexpr float OFFSET = code_offset(BITS);
    bool ok = true;
    bool ready = mbar_try_wait(sums + 0, 0);                // probe early: the answer is needed only after the loop head
    for (int st = 0; st < nstages && ok; ++st) {
      const int slot = st % NST;
      const uint32_t parity = (st / NST) & 1;
      ok = mbar_wait_probed(ready, sums + slot, parity, abort_flag);
      if (!ok) {
        give_up(ERR_WAIT_SUMS);
        break;
      }
      const int ng = groups_of(st);
      const uint8_t* sp = stage_ptr(slot);
      const uint32_t* wst = reinterpret_cast<const uint32_t*>(sp + Geo::W_OFF + kw * Geo::W_BYTES);
      const uint32_t xbase = smem_addr(sp + Geo::X_OFF), xrow = (lane & 7) * XHALF_ROW;
      const uint32_t sw0 = (((lane >> 3) ^ (lane & 7)) << 4), sw1 = (((4 | (lane >> 3)) ^ (lane & 7)) << 4);
      const float* xs_s = reinterpret_cast<const float*>(sp + Geo::XS_OFF);
#pragma unroll
      for (int u = 0; u < G; ++u) {
        if (u >= ng) break;
        if (u == ng - 1 && st + 1 < nstages)               // probe the next stage while this group computes
          ready = mbar_try_wait(sums + (st + 1) % NST, ((st + 1) / NST) & 1);
        if (!active) continue;
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
        uint32_t bf[MT][4];
#pragma unroll
        for (int s = 0; s < S; ++s) {
          if ((s & 1) == 0) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
              ldmatrix_x4(bf[mt], x_ldm_addr<Geo::XHALF>(xbase, xrow, sw0, sw1, mt, u * GS + 16 * s));
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t a[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) a[j] = pair_reg<BITS, GS, false>(wd, (h * S + s) * 4 + j);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              if (s == 0) mma_bf16_zero(P[h][mt], a, bf[mt][0], bf[mt][1]);
              else mma_bf16(P[h][mt], a, bf[mt][2 * (s & 1)], bf[mt][2 * (s & 1) + 1]);
            }
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

        const uint32_t sbv[4] = {sbw.x, sbw.y, sbw.z, sbw.w};       // (tile 0, col g), (0, g + 8), (1, g), (1, g + 8)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float s0 = bf16_lo(sbv[2 * h]), s1 = bf16_lo(sbv[2 * h + 1]);
          const float c0 = fmaf(-OFFSET, s0, bf16_hi(sbv[2 * h])), c1 = fmaf(-OFFSET, s1, bf16_hi(sbv[2 * h + 1]));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const float2 xv = *reinterpret_cast<const float2*>(xs_s + u * ROWS + mt * 8 + 2 * t);
            acc[h][mt][0] = fmaf(xv.x, c0, fmaf(P[h][mt][0], s0, acc[h][mt][0]));
            acc[h][mt][1] = fmaf(xv.y, c0, fmaf(P[h][mt][1], s0, acc[h][mt][1]));
            acc[h][mt][2] = fmaf(xv.x, c1, fmaf(P[h][mt][2], s1, acc[h][mt][2]));
            acc[h][mt][3] = fmaf(xv.y, c1, fmaf(P[h][mt][3], s1, acc[h][mt][3]));
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
  const bool clustered = p.cluster && p.sk > 1;
  cg::cluster_group cluster = cg::this_cluster();
  if (clustered) cluster.sync(); else __syncthreads();

  const bool failed = *abort_flag != 0;
  if (!failed && p.epi == 2) {
    // SwiGLU: a tile pair holds 16 gate columns then the 16 up columns of the same outputs; out has N / 2 columns (bf16)
    const int nout = p.N / 2;
    for (int idx = tid; idx < lanes_here * ROWS * 8; idx += THREADS) {
      const int kw = idx / (ROWS * 8), rem = idx % (ROWS * 8);
      const int ml = rem >> 3, j8 = rem & 7, n = (sb0 + kw) * (SB_COLS / 2) + j8 * 8;
      if (ml >= rows_here || n >= nout) continue;
      const float* src = red + kw * RED_TILE + ml * RED_STRIDE + 32 * (j8 >> 1) + 8 * (j8 & 1);
      const int64_t m = grouped ? p.members[first + ml] : m0 + ml;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + m * p.ldo + n;
      const int valid = min(8, nout - n);
      for (int e = 0; e < valid; ++e) dst[e] = __float2bfloat16_rn(swiglu_f(src[e], src[16 + e], p.limit));
    }
  } else if (!failed) {
    // One 8-column piece (row ml of lane kw, columns c8 .. c8 + 7) goes out: epilogue, then slices / fp32 / bf16.
    auto emit = [&](float (&v)[8], int kw, int ml, int c8) {
      const int n = (sb0 + kw) * SB_COLS + c8;
      if (n >= p.N) return;
      const int64_t m = grouped ? p.members[first + ml] : m0 + ml;
      const int valid = min(8, p.N - n);
      if (p.epi == 1) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = relu2_f(v[e]);
      }
      if (!p.cluster && p.sk > 1) {
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
    };
    const int pieces = lanes_here * ROWS * 16;              // 8-column pieces of the block's tiles
    if (clustered) {
      // Piece idx is summed by block idx % sk of the cluster.  Every block PUSHES its pieces into their owners' receive
      // areas (slot [slice][idx / sk], 32 bytes; the area sits behind the staging tile in every block's stage memory,
      // free since the cluster barrier above), then arrives on each owner's receive barrier.  An owner that has seen
      // all sk arrivals holds every slice of its pieces locally, sums them in slice order and may leave: nothing is
      // read remotely and no second cluster barrier is needed (a block is written to only before its own last wait).
      const int per_owner = (pieces + p.sk - 1) / p.sk;
      float* recv = red + (Geo::RED_BYTES + 15) / 16 * 4;     // [sk][per_owner][8], the same place in every block
      for (int idx = tid; idx < pieces; idx += THREADS) {
        const int kw = idx / (ROWS * 16), rem = idx % (ROWS * 16), ml = rem >> 4, c8 = (rem & 15) * 8;
        if (ml >= rows_here) continue;
        const float* src = red + kw * RED_TILE + ml * RED_STRIDE + c8;
        float* dst = cluster.map_shared_rank(recv, idx % p.sk) + (static_cast<int64_t>(slice) * per_owner + idx / p.sk) * 8;
        *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
        *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
      }
      __syncthreads();                                        // every thread's pushes come before the arrivals
      if (tid < p.sk) mbar_arrive_cluster(recv_bar, tid);
      if (!mbar_wait_cluster(recv_bar, 0, abort_flag)) {
        give_up(ERR_WAIT_FULL);
      } else {
        for (int j = tid; j * p.sk + slice < pieces; j += THREADS) {
          const int idx = j * p.sk + slice;
          const int kw = idx / (ROWS * 16), rem = idx % (ROWS * 16), ml = rem >> 4, c8 = (rem & 15) * 8;
          if (ml >= rows_here) continue;
          float v[8];
          {
            const float4 lo = *reinterpret_cast<const float4*>(recv + j * 8);
            const float4 hi = *reinterpret_cast<const float4*>(recv + j * 8 + 4);
            v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
          }
          for (int sl = 1; sl < p.sk; ++sl) {                 // slice order ((s0 + s1) + s2) + ...
            const float* src = recv + (static_cast<int64_t>(sl) * per_owner + j) * 8;
            const float4 lo = *reinterpret_cast<const float4*>(src);
            const float4 hi = *reinterpret_cast<const float4*>(src + 4);
            v[0] += lo.x, v[1] += lo.y, v[2] += lo.z, v[3] += lo.w, v[4] += hi.x, v[5] += hi.y, v[6] += hi.z, v[7] += hi.w;
          }
          emit(v, kw, ml, c8);
        }
      }
    } else {
      for (int idx = tid; idx < pieces; idx += THREADS) {
        const int kw = idx / (ROWS * 16), rem = idx % (ROWS * 16), ml = rem >> 4, c8 = (rem & 15) * 8;
        if (ml >= rows_here) continue;
        const float* src = red + kw * RED_TILE + ml * RED_STRIDE + c8;
        const float4 lo = *reinterpret_cast<const float4*>(src);
        const float4 hi = *reinterpret_cast<const float4*>(src + 4);
        float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        emit(v, kw, ml, c8);
      }
    }
  }
  if (failed && clustered) {
    // a block that gave up pushes nothing, but it still tells its peers and stays until they have pushed (or their
    // own waits run out): they write into this block's shared memory
    __syncthreads();
    if (tid < p.sk) mbar_arrive_cluster(recv_bar, tid);
    volatile int never = 0;
    mbar_wait_cluster(recv_bar, 0, &never);
  }
}

}  // namespace tf
