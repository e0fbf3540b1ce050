// Row-exact affine matmul for decode and verify windows (at most 16 rows a launch) on the 5th-generation tensor cores:
// one persistent launch runs a SET of projections that read the same rows of x (q/k/v, gate/up, or one projection).
//
// Arithmetic contract (identical for every row count and launch geometry; wider windows run as 16-row launches):
//   for each K slice (a function of the weight's shape only), acc = 0, and for each quantisation group in order
//       P'  = sum over the group of x * (q + C)      tcgen05.mma (M = 128 columns, N = 16 rows, K = 16) chained from
//                                                     zero over the group's 16-input steps, fp32 in tensor memory
//       acc = fma(xs, b - C s, fma(P', s, acc))      xs = the group's sum of x (m16n8k16 MMAs of x against ones, the
//                                                     bits tf_group_sums gives), C = 128 (the magic-number offset)
//   slices are added in slice order and the sum is rounded once to bf16 (or returned as fp32).
// An output element depends only on its own weight column and its own row of x, so a row's bits never depend on the
// rows beside it.
//
// Data flow.  The weights stay in the tiled layout (tf_layout.h): a lane of a consumer warp holds exactly the codes of
// its m16n8k16 A fragments, and the register pattern of such a fragment is also the pattern tcgen05.st.16x128b writes:
// a consumer warp dequantises a group of its 32 columns in registers ((word >> shift) & mask | magic, one shift and
// one logic instruction per two weights) and stores the 16 registers of each 16-column tile straight into tensor
// memory as the MMA's A operand (lane = column, 32-bit column = two inputs).  The last of a lane's four warps to finish
// its stores (a counter in shared memory tells) issues the group's MMAs from one thread, against the rows of x in
// shared memory (the B operand: a [64 inputs x 16 rows] tensor-map box in the 128-byte swizzle), and commits them to
// a barrier; the consumer warps read P' back with tcgen05.ld (one column a thread, 16 rows) and apply the affine step.  Two A and two P' buffers per 128-column lane alternate, so a warp
// dequantises group n + 1 while the tensor core works on group n and before it folds in group n.
//
// Schedule.  The grid is persistent; work items (projection, KW adjacent 128-column super-blocks, K slice) are dealt
// round-robin and a block's copy warp keeps its ring of stages (128 inputs: packed units by bulk copies, rows of x by
// tensor-map copies) full ACROSS items.  Blocks never wait for one another: a warp that finishes a slice writes it to
// scratch in global memory (L2-resident) and counts itself in; the warp that counts in last adds the slices in slice
// order and stores.  Who comes last changes nothing: the order of the additions is the slice order.
//
// Scratch: `count` must be zero when a launch starts and every launch leaves it zero; `part` needs no initial value.
// Two launches that share scratch must not overlap on the GPU (with programmatic dependent launch a block touches
// global memory only after the previous kernel in the stream has finished).  Every wait is bounded and reports through
// the device error word; tensor memory is released on every path.
#pragma once

#include "qmm_tiled.cuh"
#ifdef TF_WAIT_STATS
#include <cstdio>
#endif

namespace tf {

constexpr int STREAM_MAX_PROJ = 4;
constexpr int STREAM_ROWS = 16;            // rows of x a launch takes (the MMA's N)
constexpr int STREAM_PART_FLOATS = 2048;   // one (super-block, slice) partial: 128 columns x 16 rows

struct StreamProj {
  const uint32_t* w;          // tiled units of this projection
  int64_t sb_stride;          // words from one 128-column super-block to the next
  void* out;                  // [M, N] bf16 or fp32, row stride ldo elements; or [sk, M, N] fp32 slices (slices_out)
  int64_t ldo;
  float* part;                // [nsb][sk][STREAM_PART_FLOATS] slices, one column a thread; unused when sk == 1
  int* count;                 // [nsb][4] warps that have written their slice of (super-block, 32-column tile pair)
  int N, sk, nsb;
  int item0;                  // first work item of this projection
  int out_f32;
};

struct StreamParams {
  const __nv_bfloat16* x;     // [M, K] bf16, shared by the projections of the set
  const float* xs;            // optional [M, KG] group sums
  int M, K, KG;               // M: rows of this launch (1 to 16)
  int nproj, items;
  int slices_out;             // 1: every slice goes to out as fp32 [sk, rows_total, N] and nothing is summed
  int row0, rows_total;       // a wider window runs as 16-row launches: this launch's first row, and the window's rows
  int* err;
  StreamProj proj[STREAM_MAX_PROJ];
};

template <int BITS, int GS, int KW>
struct StreamGeo {
  static constexpr int CONSUMERS = 4 * KW;
  static constexpr int THREADS = 32 * (CONSUMERS + 2);      // + copy warp, sums / MMA warp
  static constexpr int S = GS / 16;                         // MMAs (16-input steps) per group
  static constexpr int G = 128 / GS;                        // groups per stage (a stage covers 128 inputs)
  static constexpr int ROWS = STREAM_ROWS;
  static constexpr int WPL = words_per_lane(BITS, GS);
  static constexpr int UNITW = unit_words(BITS, GS);
  static constexpr int W_BYTES = G * UNITW * 4;             // one lane's packed units of a stage
  static constexpr int XHALF = ROWS * XHALF_ROW;            // 64 inputs of every row: one swizzled B tile
  static constexpr int X_BYTES = 2 * XHALF;
  static constexpr int XS_BYTES = ROWS * G * 4;
  static constexpr int X_OFF = 0;                           // first: a stage starts 1024-byte aligned, as the swizzle needs
  static constexpr int W_OFF = X_BYTES;
  static constexpr int XS_OFF = W_OFF + KW * W_BYTES;
  static constexpr int STAGE = (XS_OFF + XS_BYTES + 1023) / 1024 * 1024;
  // tensor memory of a lane: two A buffers (a group's inputs, two to a 32-bit column) and two P' buffers (16 rows)
  static constexpr int A_COLS = GS / 2, D_COLS = ROWS;
  static constexpr int LANE_COLS = 2 * A_COLS + 2 * D_COLS;
  static constexpr int TMEM_NEED = KW * LANE_COLS;
  static constexpr int TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  // blocks an SM should hold: as many as tensor memory (512 columns) and the lane count suggest; shared memory is sized
  // so that no more than that ever become resident (a block that cannot get its tensor memory would sit and wait)
  static constexpr int BY_TMEM = 512 / TMEM_COLS < 1 ? 1 : 512 / TMEM_COLS;
  static constexpr int WANT = KW == 1 ? 3 : KW == 2 ? 2 : 1;
  static constexpr int BLOCKS = WANT < BY_TMEM ? WANT : BY_TMEM;
  static constexpr int BUDGET = (BLOCKS == 3 ? 72 : BLOCKS == 2 ? 110 : 220) * 1024;
  static constexpr int NST_A = BUDGET / STAGE;
  static constexpr int NST = NST_A < 3 ? 3 : (NST_A > 12 ? 12 : NST_A);
  static constexpr int NBAR = 3 * NST + 2 * KW;             // full, empty, sums per stage; d_full per lane buffer
  static constexpr int BAR_BYTES = NBAR * 8 + 2 * KW * 4 + 16;   // + store counters per lane buffer, abort word, tensor-memory base
  static constexpr int SMEM_USED = NST * STAGE + BAR_BYTES + 1024;
  static constexpr int SMEM_FLOOR = BLOCKS == 1 ? 116 * 1024 : BLOCKS == 2 ? 76 * 1024 : 0;   // keeps a further block out
  static constexpr int SMEM = SMEM_USED > SMEM_FLOOR ? SMEM_USED : SMEM_FLOOR;
  static constexpr bool FITS = TMEM_NEED <= 512 && SMEM <= 227 * 1024 && THREADS <= 1024 && !Fmt<BITS>::SPLIT;
  static_assert(STAGE % 1024 == 0 && W_BYTES % 16 == 0 && XS_OFF % 16 == 0, "stage parts stay aligned");
};

// One work item, decoded from its flat index (the same on every warp of the block).  Kernel parameters are read
// with constant indices only.
struct StreamItem {
  int p;                      // projection
  int sb0;                    // first super-block
  int lanes;                  // super-blocks in use (the last item of a projection may hold fewer than KW)
  int slice;
  int sk;
  int g_first;                // first group of the slice
  int per;                    // groups of the slice
  int nst;                    // stages of the slice
};

#define TF_PROJ_FIELD(p, pi, field)                                                                   \
  ((pi) == 0 ? (p).proj[0].field : (pi) == 1 ? (p).proj[1].field : (pi) == 2 ? (p).proj[2].field : (p).proj[3].field)

template <int KW, int G>
__device__ __forceinline__ StreamItem stream_item(const StreamParams& p, int i) {
  StreamItem it;
  int pi = 0;
#pragma unroll
  for (int q = 1; q < STREAM_MAX_PROJ; ++q)
    if (q < p.nproj && i >= p.proj[q].item0) pi = q;
  const int sk = TF_PROJ_FIELD(p, pi, sk), nsb = TF_PROJ_FIELD(p, pi, nsb);
  const int j = i - TF_PROJ_FIELD(p, pi, item0);
  it.p = pi;
  it.sk = sk;
  it.slice = j % sk;
  it.sb0 = (j / sk) * KW;
  it.lanes = min(KW, nsb - it.sb0);
  it.per = p.KG / sk;
  it.g_first = it.slice * it.per;
  it.nst = (it.per + G - 1) / G;
  return it;
}

// tcgen05.st.16x128b.x2: registers 0..3 of thread T go to lanes T / 4, T / 4 + 8 (registers 0, 1) and the same lanes four
// columns on (registers 2, 3), column T % 4: the register pattern of one m16n8k16 A fragment (16 columns x 16 inputs).
// Four registers a store keep the operands where the dequantisation left them (wider stores made the compiler copy).
__device__ __forceinline__ void tmem_store_frag(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}

// P' of one column: 16 fp32 values (one per row of x) from the thread's own tensor-memory lane.
__device__ __forceinline__ void tmem_load_rows(uint32_t taddr, float (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]), "=f"(v[9]),
        "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int BITS, int GS, int KW>
__global__ void __launch_bounds__(StreamGeo<BITS, GS, KW>::THREADS, StreamGeo<BITS, GS, KW>::BLOCKS)
qmm_stream_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ StreamParams p) {
  using Geo = StreamGeo<BITS, GS, KW>;
  constexpr int S = Geo::S, G = Geo::G, ROWS = Geo::ROWS, WPL = Geo::WPL, UNITW = Geo::UNITW, NST = Geo::NST;
  constexpr int CONSUMERS = Geo::CONSUMERS;
  constexpr int COPY_WARP = CONSUMERS, AUX_WARP = CONSUMERS + 1;

  extern __shared__ uint8_t smem_raw[];
  // everything in shared memory is addressed by 32-bit shared addresses: stage s at smem32 + s * STAGE, then the barriers
  const uint32_t smem32 = (smem_addr(smem_raw) + 1023u) & ~1023u;
  const uint32_t full32 = smem32 + NST * Geo::STAGE;        // weights and x of a stage have landed
  const uint32_t empty32 = full32 + NST * 8;                // every consumer warp is done with a stage
  const uint32_t sums32 = empty32 + NST * 8;                // the stage's group sums are written
  const uint32_t dfull32 = sums32 + NST * 8;                // [kw][2]: the group's MMAs have completed
  const uint32_t stored32 = dfull32 + KW * 16;              // [kw][2] counters: warps of the lane that have stored a group's A operand
  const uint32_t abort32 = stored32 + KW * 8;               // non-zero once a warp of the block has given up a wait
  const uint32_t tslot32 = abort32 + 4;                     // tensor-memory base address, written by tcgen05.alloc

  // the warp index through a shuffle: the compiler then knows it is the same in every lane, keeps what derives from it
  // (roles, tensor-memory and barrier addresses) in uniform registers and branches on it without divergence handling
  const int tid = threadIdx.x, warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0), lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full32 + 8 * i), "r"(2) : "memory");    // weights' bytes + bytes of x
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty32 + 8 * i), "r"(CONSUMERS) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sums32 + 8 * i), "r"(1) : "memory");
    }
    for (int i = 0; i < 2 * KW; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dfull32 + 8 * i), "r"(1) : "memory");
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(stored32 + 4 * i), "r"(0) : "memory");
    }
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort32), "r"(0) : "memory");
    mbar_fence_init();
  }
  if (warp == AUX_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tslot32), "r"(Geo::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = __shfl_sync(0xFFFFFFFFu, lds32(tslot32), 0);
  pdl_launch_dependents();

  auto give_up = [&](int code) {
    if (lane == 0) {
      asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort32), "r"(code) : "memory");
      atomicCAS(p.err, 0, code);
    }
  };
  const int first_item = blockIdx.x, step = gridDim.x;

  if (warp == COPY_WARP) {
    // ------------------------------------------------------------------ copy warp: one bulk copy per lane and stage
    auto issue_w = [&](const StreamItem& it, int st, int slot) {
      if (lane == 0) {
        const uint32_t* w = TF_PROJ_FIELD(p, it.p, w);
        const int64_t sb_stride = TF_PROJ_FIELD(p, it.p, sb_stride);
        const int ng = min(G, it.per - st * G);
        const uint32_t* src = w + static_cast<int64_t>(it.sb0) * sb_stride +
                              (static_cast<int64_t>(it.g_first) + static_cast<int64_t>(st) * G) * UNITW;
        const uint32_t bar = full32 + 8 * slot, dst = smem32 + slot * Geo::STAGE + Geo::W_OFF;
        mbar32_expect_tx(bar, it.lanes * ng * UNITW * 4);
        for (int kw = 0; kw < it.lanes; ++kw) bulk_load32(dst + kw * Geo::W_BYTES, src + kw * sb_stride, ng * UNITW * 4, bar);
      }
    };
    auto issue_x = [&](const StreamItem& it, int st, int slot) {
      if (lane == 0) {
        const int ng = min(G, it.per - st * G);
        const int boxes = (ng * GS + 63) / 64;              // a [64 inputs x 16 rows] box lands in a swizzled B tile
        const uint32_t bar = full32 + 8 * slot, dst = smem32 + slot * Geo::STAGE + Geo::X_OFF;
        mbar32_expect_tx(bar, boxes * Geo::XHALF);
        const int k0 = (it.g_first + st * G) * GS;
        for (int b = 0; b < boxes; ++b) tma_load_2d32(dst + b * Geo::XHALF, &tmx, k0 + 64 * b, 0, bar);
      }
    };
    // the weights of the first NST stages never depend on the previous kernel: they go out before the dependency wait
    {
      int gst = 0;
      for (int i = first_item; i < p.items && gst < NST; i += step) {
        const StreamItem it = stream_item<KW, G>(p, i);
        for (int st = 0; st < it.nst && gst < NST; ++st, ++gst) issue_w(it, st, gst);
      }
    }
    pdl_wait();                                             // x may be the previous kernel's output
    bool ok = true;
    uint32_t polls_empty = 0;
    int gst = 0, slot = 0;
    uint32_t phase = 1;                                     // parity of the `empty` phase that frees the slot (first round: none)
    for (int i = first_item; i < p.items && ok; i += step) {
      const StreamItem it = stream_item<KW, G>(p, i);
      for (int st = 0; st < it.nst; ++st, ++gst) {
        if (gst >= NST) {                                   // the stage goes where stage gst - NST was
          ok = mbar32_wait(empty32 + 8 * slot, phase, abort32, 256, &polls_empty);
          if (!ok) {
            give_up(ERR_WAIT_EMPTY);
            break;
          }
          issue_w(it, st, slot);
        }
        issue_x(it, st, slot);
        if (++slot == NST) slot = 0, phase ^= 1;
      }
    }
    if (!ok) {
      for (int i = 0; i < 64; ++i) __nanosleep(20000);      // copies in flight land before the shared memory is released
    }
#ifdef TF_WAIT_STATS
    if (lane == 0 && blockIdx.x < 2) printf("block %d copy warp: polls empty %u stages %d\n", blockIdx.x, polls_empty, gst);
#endif
  } else if (warp == AUX_WARP) {
    // ------------------------------------------------------------------ sums warp: group sums of x, once per block
    // (x against a tile of ones on the legacy tensor path: the bits tf_group_sums gives; the arrival also tells the
    // consumers that the stage has landed)
    pdl_wait();                                              // xs may be the previous kernel's output
    bool ok = true;
    uint32_t polls_full = 0;
    int slot = 0;
    uint32_t phase = 0;
    const uint32_t xrow = (lane & 7) * XHALF_ROW;
    const uint32_t sw0 = (((lane >> 3) ^ (lane & 7)) << 4), sw1 = (((4 | (lane >> 3)) ^ (lane & 7)) << 4);
    for (int i = first_item; i < p.items && ok; i += step) {
      const StreamItem it = stream_item<KW, G>(p, i);
      for (int st = 0; st < it.nst; ++st) {
        ok = mbar32_wait(full32 + 8 * slot, phase, abort32, 128, &polls_full);
        if (!ok) {
          give_up(ERR_WAIT_FULL);
          break;
        }
        const int ng = min(G, it.per - st * G);
        const uint32_t sp32 = smem32 + slot * Geo::STAGE, xs32 = sp32 + Geo::XS_OFF;
        if (p.xs != nullptr) {
          const int g0 = it.g_first + st * G;
          for (int e = lane; e < ng * ROWS; e += 32) {
            const int u = e / ROWS, r = e % ROWS;
            const float v = r < p.M ? p.xs[static_cast<int64_t>(r) * p.KG + g0 + u] : 0.f;
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(xs32 + (u * ROWS + r) * 4), "f"(v) : "memory");
          }
        } else {
#pragma unroll
          for (int u = 0; u < G; ++u) {
            if (u >= ng) break;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
              float d[4];
              ones_mma_group<GS, Geo::XHALF>(d, sp32 + Geo::X_OFF, xrow, sw0, sw1, mt, u * GS);
              if (lane < 4)
                asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xs32 + (u * ROWS + mt * 8 + 2 * lane) * 4), "f"(d[0]), "f"(d[1])
                             : "memory");
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar32_arrive(sums32 + 8 * slot);
        if (++slot == NST) slot = 0, phase ^= 1;
      }
    }
#ifdef TF_WAIT_STATS
    if (lane == 0 && blockIdx.x < 2) printf("block %d sums warp: polls full %u\n", blockIdx.x, polls_full);
#endif
  } else {
    // ------------------------------------------------------------------ consumers: dequantise -> tensor memory, then P' -> acc
    const int kw = warp >> 2, tp = warp & 3;
    constexpr float OFFSET = code_offset(BITS);
    // byte offsets inside a stage that depend on the thread only
    const uint32_t w_off = Geo::W_OFF + kw * Geo::W_BYTES + (tp * 32 + lane) * WPL * 4;
    // the thread's column is 32 tp + lane = 32 tp + 16 h + 8 r8 + g: its (scale, bias) word sits at tp * 32 + g * 4 + h * 2 + r8
    const uint32_t sb_off =
        Geo::W_OFF + kw * Geo::W_BYTES + (TILE_PAIRS * 32 * WPL + tp * 32 + (lane & 7) * 4 + (lane >> 4) * 2 + ((lane >> 3) & 1)) * 4;
    const uint32_t a_lane = tmem + (static_cast<uint32_t>(32 * tp) << 16) + kw * Geo::LANE_COLS;     // this warp's 32 tensor-memory lanes

    // D (128 columns x 16 rows, fp32) = A (tensor memory: lane = column, 32-bit column = two inputs) x B (the rows of x in
    // shared memory, K-major, 128-byte swizzle); bf16 inputs, M = 128, N = 16
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
    float acc[ROWS];                                        // the thread's column, one value a row of x
    uint32_t polls_sums = 0, polls_dfull = 0;               // (counted in instrumented builds only)

    // dequantise group u of the stage into the A buffer `buf` of this lane (the stores are left in flight)
    auto push_issue = [&](uint32_t sp32, int u, uint32_t buf) {
      uint32_t wd[WPL];
      const uint32_t src = sp32 + w_off + u * (UNITW * 4);
      if constexpr (WPL % 4 == 0) {
#pragma unroll
        for (int i = 0; i < WPL; i += 4) {
          const uint4 v = lds128(src + i * 4);
          wd[i] = v.x, wd[i + 1] = v.y, wd[i + 2] = v.z, wd[i + 3] = v.w;
        }
      } else if constexpr (WPL % 2 == 0) {
#pragma unroll
        for (int i = 0; i < WPL; i += 2) {
          const uint2 v = lds64(src + i * 4);
          wd[i] = v.x, wd[i + 1] = v.y;
        }
      } else {
#pragma unroll
        for (int i = 0; i < WPL; ++i) wd[i] = lds32(src + i * 4);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t tile = a_lane + (static_cast<uint32_t>(16 * h) << 16) + buf * Geo::A_COLS;
#pragma unroll
        for (int st = 0; st < S; ++st) {                      // one A fragment (16 columns x 16 inputs) a store
          uint32_t a[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) a[j] = pair_reg<BITS, GS, false>(wd, (h * S + st) * 4 + j);
          tmem_store_frag(tile + 8 * st, a);
        }
      }
    };
    // the stores have landed: count this warp in; the lane's last warp issues the group's MMAs (one thread) and
    // commits them to the buffer's barrier.  The counter only ever grows: every group adds four.
    auto push_commit = [&](uint32_t sp32, int u, uint32_t buf) {
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      uint32_t seen = 0;
      if (lane == 0)
        asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], 1;" : "=r"(seen) : "r"(stored32 + 4 * (2 * kw + buf)) : "memory");
      seen = __shfl_sync(0xFFFFFFFFu, seen, 0);
      if ((seen & 3u) == 3u) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (lane == 0) {
          const uint32_t a_t = tmem + kw * Geo::LANE_COLS + buf * Geo::A_COLS;
          const uint32_t d_t = tmem + kw * Geo::LANE_COLS + 2 * Geo::A_COLS + buf * Geo::D_COLS;
          const uint32_t xb = sp32 + Geo::X_OFF;
#pragma unroll
          for (int st = 0; st < S; ++st) {
            // 64 inputs a swizzled tile, 32 bytes a 16-input step inside its 128-byte rows
            const uint32_t kin = u * GS + 16 * st;
            const uint32_t baddr = xb + (kin >> 6) * Geo::XHALF + (kin & 63) * 2;
            const uint32_t lo = ((baddr >> 4) & 0x3FFFu) | (1u << 16);
            const uint32_t hi = 64u | (1u << 14) | (2u << 29);
            const uint64_t bdesc = (static_cast<uint64_t>(hi) << 32) | lo;
            asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(d_t),
                         "r"(a_t + 8 * st), "l"(bdesc), "r"(IDESC), "r"(st > 0 ? 1 : 0)
                         : "memory");
          }
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(dfull32 + 8 * (2 * kw + buf))
                       : "memory");
        }
        __syncwarp();
      }
    };

    // fold a finished group into acc: acc[r] = fma(xs[r], b - C s, fma(P'[r], s, acc[r]))
    // group m's MMAs have completed: its A buffer may be written again and its P' read
    auto wait_group = [&](uint32_t m) -> bool {
      if (!mbar32_wait(dfull32 + 8 * (2 * kw + (m & 1)), (m >> 1) & 1, abort32, 0, &polls_dfull)) return false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      return true;
    };
    auto fold_group = [&](uint32_t sp32, int u, uint32_t buf) {
      float P[ROWS];
      tmem_load_rows(a_lane + 2 * Geo::A_COLS + buf * Geo::D_COLS, P);
      const uint32_t sbw = lds32(sp32 + sb_off + u * (UNITW * 4));
      const float s = bf16_lo(sbw), c = fmaf(-OFFSET, s, bf16_hi(sbw));
      const uint32_t xs32 = sp32 + Geo::XS_OFF + u * ROWS * 4;
#pragma unroll
      for (int r4 = 0; r4 < ROWS; r4 += 4) {
        const uint4 xq = lds128(xs32 + r4 * 4);
        acc[r4] = fmaf(__uint_as_float(xq.x), c, fmaf(P[r4], s, acc[r4]));
        acc[r4 + 1] = fmaf(__uint_as_float(xq.y), c, fmaf(P[r4 + 1], s, acc[r4 + 1]));
        acc[r4 + 2] = fmaf(__uint_as_float(xq.z), c, fmaf(P[r4 + 2], s, acc[r4 + 2]));
        acc[r4 + 3] = fmaf(__uint_as_float(xq.w), c, fmaf(P[r4 + 3], s, acc[r4 + 3]));
      }
    };

    struct OutProj {
      void* out;
      int64_t ldo;
      int N, out_f32;
    };
    // the thread's column n of rows 0 .. M - 1 (row0: first row of the destination)
    auto store_out = [&](const OutProj& pr, int n, const float (&v)[ROWS], int64_t row0) {
      if (n >= pr.N) return;
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        if (r < p.M) {
          if (pr.out_f32) reinterpret_cast<float*>(pr.out)[(row0 + r) * pr.ldo + n] = v[r];
          else reinterpret_cast<__nv_bfloat16*>(pr.out)[(row0 + r) * pr.ldo + n] = __float2bfloat16_rn(v[r]);
        }
      }
    };

    // the output of a finished item: the slice itself, or (last warp in) the sum of the slices in slice order
    auto finish_item = [&](const StreamItem& it) {
      pdl_wait();                                           // nothing is written before the previous kernel is done
      const float (&a)[ROWS] = acc;
      OutProj pr;
      pr.out = TF_PROJ_FIELD(p, it.p, out), pr.ldo = TF_PROJ_FIELD(p, it.p, ldo);
      pr.N = TF_PROJ_FIELD(p, it.p, N), pr.out_f32 = TF_PROJ_FIELD(p, it.p, out_f32);
      const int sb = it.sb0 + kw, n = sb * SB_COLS + tp * 32 + lane;
      if (p.slices_out) {                                   // fp32 [sk, rows_total, N]
        pr.out_f32 = 1, pr.ldo = pr.N;
        store_out(pr, n, a, static_cast<int64_t>(it.slice) * p.rows_total + p.row0);
      } else if (it.sk == 1) {
        store_out(pr, n, a, p.row0);
      } else {
        // rows 4 f .. 4 f + 3 of slice s: float4 index (((sb * sk + s) * 4 + tp) * 4 + f) * 32 + lane
        float* part = TF_PROJ_FIELD(p, it.p, part);
        float4* mine = reinterpret_cast<float4*>(part) + ((static_cast<int64_t>(sb) * it.sk + it.slice) * 4 + tp) * 128 + lane;
#pragma unroll
        for (int f = 0; f < 4; ++f) __stcg(mine + f * 32, make_float4(a[4 * f], a[4 * f + 1], a[4 * f + 2], a[4 * f + 3]));
        __threadfence();                                    // the slice is visible before this warp counts itself in
        __syncwarp();
        int* counter = TF_PROJ_FIELD(p, it.p, count) + sb * 4 + tp;
        int seen = 0;
        if (lane == 0) seen = atomicAdd(counter, 1);
        seen = __shfl_sync(0xFFFFFFFFu, seen, 0);
        if (seen == it.sk - 1) {
          __threadfence();                                  // the other warps' slices are visible before they are read
          const float4* base = reinterpret_cast<const float4*>(part) + (static_cast<int64_t>(sb) * it.sk * 4 + tp) * 128 + lane;
          float v[ROWS];
#pragma unroll
          for (int f = 0; f < 4; ++f) {
            const float4 q = __ldcg(base + f * 32);
            v[4 * f] = q.x, v[4 * f + 1] = q.y, v[4 * f + 2] = q.z, v[4 * f + 3] = q.w;
          }
#pragma unroll 4
          for (int s = 1; s < it.sk; ++s) {                 // slice order ((s0 + s1) + s2) + ...
            const float4* src = base + static_cast<int64_t>(s) * 512;
#pragma unroll
            for (int f = 0; f < 4; ++f) {
              const float4 q = __ldcg(src + f * 32);
              v[4 * f] += q.x, v[4 * f + 1] += q.y, v[4 * f + 2] += q.z, v[4 * f + 3] += q.w;
            }
          }
          if (lane == 0) *counter = 0;                      // the next launch finds the counter at zero again
          store_out(pr, n, v, p.row0);
        }
      }
    };

    // Main loop.  Step n of a lane: wait for group n - 2's MMAs (its tensor-memory buffers are the ones group n takes),
    // issue group n's dequantised stores, fold group n - 2 into acc while they fly, then hand group n to the tensor
    // core.  Group n - 1's MMAs run through the whole step, so their round trip (last warp in, issue, execute, commit)
    // hides behind a full dequantisation.  A stage's slot is released when its last group has been folded in; at the
    // end of an item both groups in flight are folded, the item's output goes out and acc starts from zero.
    bool ok = true;
    int slot = 0;
    uint32_t phase = 0;                                     // parity of the `sums` phase the current slot waits for
    uint32_t n = 0;                                         // groups this lane has pushed so far
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;

    struct Flight {                                         // a group whose MMAs may still be running
      uint32_t sp32;                                        // its stage
      int u;                                                // its index in the stage (-1: none)
      int release;                                          // >= 0: the stage's slot, to release once the group is folded in
    };
    auto retire = [&](const Flight& f, uint32_t m) {        // fold group m (already waited for) and release what ends with it
      fold_group(f.sp32, f.u, m & 1);
      if (f.release >= 0) {
        __syncwarp();
        if (lane == 0) mbar32_arrive(empty32 + 8 * f.release);
      }
    };

    for (int i = first_item; i < p.items && ok; i += step) {
      const StreamItem it = stream_item<KW, G>(p, i);
      if (kw >= it.lanes) {
        // an idle lane of a narrow item: it only keeps the ring turning
        for (int st = 0; st < it.nst && ok; ++st) {
          ok = mbar32_wait(sums32 + 8 * slot, phase, abort32, 128);
          if (!ok) {
            give_up(ERR_WAIT_SUMS);
            break;
          }
          if (lane == 0) mbar32_arrive(empty32 + 8 * slot);
          if (++slot == NST) slot = 0, phase ^= 1;
        }
        continue;
      }
      Flight f1 = {0, -1, -1}, f2 = {0, -1, -1};            // groups n - 1 and n - 2
      for (int st = 0; st < it.nst && ok; ++st) {
        const uint32_t sp32 = smem32 + slot * Geo::STAGE;
        ok = mbar32_wait(sums32 + 8 * slot, phase, abort32, 0, &polls_sums);
        if (!ok) {
          give_up(ERR_WAIT_SUMS);
          break;
        }
        const int ng = min(G, it.per - st * G);
#pragma unroll
        for (int u = 0; u < G; ++u) {
          if (u >= ng) break;
          if (f2.u >= 0) {
            ok = wait_group(n - 2);
            if (!ok) break;
          }
          push_issue(sp32, u, n & 1);
          if (f2.u >= 0) retire(f2, n - 2);
          push_commit(sp32, u, n & 1);
          f2 = f1;
          f1.sp32 = sp32, f1.u = u, f1.release = u == ng - 1 ? slot : -1;
          ++n;
        }
        if (!ok) {
          give_up(ERR_WAIT_FULL);
          break;
        }
        if (++slot == NST) slot = 0, phase ^= 1;
      }
      if (!ok) break;
      // drain: the item's last two groups
      if (f2.u >= 0) {
        ok = wait_group(n - 2);
        if (ok) retire(f2, n - 2);
      }
      if (ok) ok = wait_group(n - 1);
      if (!ok) {
        give_up(ERR_WAIT_FULL);
        break;
      }
      retire(f1, n - 1);
      finish_item(it);
#pragma unroll
      for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
    }
#ifdef TF_WAIT_STATS
    if (lane == 0 && blockIdx.x < 2) printf("block %d warp %d: polls sums %u dfull %u groups %u\n", blockIdx.x, warp, polls_sums, polls_dfull, n);
#endif
  }

  // ---------------------------------------------------------------------- tensor memory goes back on every path
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == AUX_WARP) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Geo::TMEM_COLS) : "memory");
  }
}

#undef TF_PROJ_FIELD

}  // namespace tf
