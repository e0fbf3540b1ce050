// Persistent form of the row-exact affine matmul for decode and verify windows (at most 16 rows): one launch runs a SET
// of projections that read the same rows of x (q/k/v, gate/up, or a single projection) and never stops streaming.
//
// The arithmetic is qmm_tiled.cuh's, bit for bit: per K slice (a function of the weight's shape only) and per group in
// order, P' = sum of x * (q + C) from chained m16n8k16 MMAs, acc = fma(xs, b - C s, fma(P', s, acc)); slices added in
// slice order; one rounding.  Only the schedule differs:
//
//   * the grid is persistent (blocks resident on every SM); work items (projection, KW adjacent 128-column
//     super-blocks, K slice) are dealt to the blocks round-robin, and a block's copy warp keeps its ring of stages
//     full ACROSS items, so a block pays the first-byte latency once per launch, not once per item;
//   * blocks never wait for one another: a warp that finishes a slice of its 32 columns writes the slice (its
//     accumulator fragment, as it sits in registers) to a scratch area in global memory, which stays in L2, and counts
//     itself in; the warp that counts in last reads every slice back in slice order, adds and stores the result.  Who
//     comes last changes nothing: the order of the additions is the slice order;
//   * for windows of up to 8 rows a consumer warp keeps the next group's packed words in registers while the tensor
//     cores work on the current group (the ring hides HBM latency, the registers hide shared-memory latency).
//
// Scratch: `count` must be zero when a launch starts and every launch leaves it zero; `part` needs no initial value.
// Two launches that share scratch must not overlap on the GPU (with programmatic dependent launch a block touches
// global memory only after the previous kernel in the stream has finished).
#pragma once

#include "qmm_tiled.cuh"

namespace tf {

constexpr int STREAM_MAX_PROJ = 4;
constexpr int STREAM_PART_FLOATS = 2048;   // one (super-block, slice) partial: 4 tile pairs x 4 fragments x 32 lanes x 4 floats

struct StreamProj {
  const uint32_t* w;          // tiled units of this projection
  int64_t sb_stride;          // words from one 128-column super-block to the next
  void* out;                  // [M, N] bf16 or fp32, row stride ldo elements
  int64_t ldo;
  float* part;                // [nsb][sk][STREAM_PART_FLOATS] slices in fragment order; unused when sk == 1
  int* count;                 // [nsb][4] warps that have written their slice of (super-block, tile pair)
  int N, sk, nsb;
  int item0;                  // first work item of this projection
  int out_f32;
};

struct StreamParams {
  const __nv_bfloat16* x;     // [M, K] bf16, shared by the projections of the set
  const float* xs;            // optional [M, KG] group sums
  int M, K, KG;
  int nproj, items;
  int* err;
  StreamProj proj[STREAM_MAX_PROJ];
  // grouped (mixture-of-experts) form, GROUPED kernels only: one projection (proj[0], one K slice) whose weights are a
  // table of experts; plan item y = (expert, first, count <= ROWS) runs rows members[first .. first + count), read from
  // row pair / slots of x (slots > 0) or row pair (slots == 0), and writes row `pair` of out.  Work item i is plan item
  // i / groups_of_sb for the super-blocks (i % groups_of_sb) * KW ...; the item count comes from counts[0] on the device.
  int64_t ldx;                // row stride of x in elements
  const int* plan_items;      // [max items][3]
  const int* counts;          // [0] = plan items in use
  const int* members;         // pair ids grouped by expert
  int slots;
  int64_t expert_stride;      // words from one expert's units to the next
  int experts;                // experts the table holds: an item that names another one is skipped and reported
  int epi;                    // 0 store as is; 1 bf16(relu(bf16 v)^2); 2 SwiGLU over the gate / up halves of a tile pair
  float limit;                // SwiGLU clip (0: none)
};

template <int BITS, int GS, int MT, int KW>
struct StreamGeo {
  static constexpr int CONSUMERS = 4 * KW;
  static constexpr int THREADS = 32 * (CONSUMERS + 2);
  static constexpr int S = GS / 16;
  static constexpr int G = 128 / GS;                        // groups per stage (a stage covers 128 inputs)
  static constexpr int ROWS = 8 * MT;
  static constexpr int WPL = words_per_lane(BITS, GS);
  static constexpr int UNITW = unit_words(BITS, GS);
  static constexpr int W_BYTES = G * UNITW * 4;
  static constexpr int XHALF = ROWS * XHALF_ROW;
  static constexpr int X_BYTES = 2 * XHALF;
  static constexpr int XS_BYTES = ROWS * G * 4;
  static constexpr int X_OFF = 0;
  static constexpr int W_OFF = X_BYTES;
  static constexpr int XS_OFF = W_OFF + KW * W_BYTES;
  static constexpr int STAGE = (XS_OFF + XS_BYTES + 1023) / 1024 * 1024;
  // shared memory a block may take: three blocks an SM with one lane, two with two lanes, one with four
  static constexpr int BUDGET = (KW == 1 ? 72 : KW == 2 ? 110 : 220) * 1024;
  static constexpr int NST_A = BUDGET / STAGE;
  static constexpr int NST = NST_A < 2 ? 2 : (NST_A > 12 ? 12 : NST_A);
  static constexpr int BAR_BYTES = 3 * NST * 8 + 16;
  static constexpr int SMEM = NST * STAGE + BAR_BYTES + 1024;
  static constexpr int BY_SMEM = (227 * 1024) / (SMEM + 1024) < 1 ? 1 : (227 * 1024) / (SMEM + 1024);
  static constexpr int MINB = BY_SMEM > 3 ? 3 : BY_SMEM;
  // The next group's words wait in registers while the current group computes: worth its registers for windows of up to
  // 8 rows (measured on B200: a layer of the dense 27B model in 68 us instead of 74); at 16 rows the accumulators
  // need the registers more (83 us without, 89 with).
#ifdef TF_STREAM_NO_PREFETCH
  static constexpr bool PREFETCH = false;
#else
  static constexpr bool PREFETCH = MT == 1 && WPL <= 8 && G % 2 == 0;
#endif
  static_assert(STAGE % 1024 == 0 && W_BYTES % 16 == 0 && XS_OFF % 16 == 0, "stage parts stay aligned");
  static_assert(SMEM <= 227 * 1024, "fits the shared memory of an SM");
};

// One work item, decoded from its flat index (the same on every warp of the block).  Kernel parameters are read
// with constant indices only (a run-time index would make the compiler keep a copy of the parameters in local memory).
struct StreamItem {
  int p;                      // projection
  int sb0;                    // first super-block
  int lanes;                  // super-blocks in use (the last item of a projection may hold fewer than KW)
  int slice;
  int sk;
  int g_first;                // first group of the slice
  int per;                    // groups of the slice
  int nst;                    // stages of the slice
  int expert, first, rows;    // grouped form: the plan item (rows == 0: nothing to do)
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
  // slice s covers groups [s KG / sk, (s + 1) KG / sk): a function of the shape only; sizes differ by at most one group
  it.g_first = static_cast<int>(static_cast<int64_t>(it.slice) * p.KG / sk);
  it.per = static_cast<int>(static_cast<int64_t>(it.slice + 1) * p.KG / sk) - it.g_first;
  it.nst = (it.per + G - 1) / G;
  return it;
}

// Grouped form: work item i = (plan item i / sbg, super-blocks (i % sbg) * KW ...), sbg = ceil(nsb / KW).
template <int KW, int G, int ROWS>
__device__ __forceinline__ StreamItem grouped_item(const StreamParams& p, int i, int sbg) {
  StreamItem it;
  const int y = i / sbg;
  const int* item = p.plan_items + 3 * y;
  it.p = 0, it.sk = 1, it.slice = 0, it.g_first = 0;
  it.sb0 = (i - y * sbg) * KW;
  it.lanes = min(KW, p.proj[0].nsb - it.sb0);
  it.per = p.KG;
  it.nst = (p.KG + G - 1) / G;
  it.expert = __ldg(item), it.first = __ldg(item + 1), it.rows = min(ROWS, __ldg(item + 2));
  if (it.expert < 0 || it.expert >= p.experts) {             // never read past the table: skip the item, tell the host
    atomicCAS(p.err, 0, ERR_BAD_ITEM);
    it.rows = 0, it.nst = 0;
  }
  return it;
}

template <int BITS, int GS, int MT, int KW, bool GROUPED = false>
__global__ void __launch_bounds__(StreamGeo<BITS, GS, MT, KW>::THREADS, StreamGeo<BITS, GS, MT, KW>::MINB)
qmm_stream_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ StreamParams p) {
  using Geo = StreamGeo<BITS, GS, MT, KW>;
  constexpr int S = Geo::S, G = Geo::G, ROWS = Geo::ROWS, WPL = Geo::WPL, UNITW = Geo::UNITW, NST = Geo::NST;
  constexpr int CONSUMERS = Geo::CONSUMERS;
  constexpr bool SPLIT = Fmt<BITS>::SPLIT;

  extern __shared__ uint8_t smem_raw[];
  // everything in shared memory is addressed by 32-bit shared addresses: stage s at smem32 + s * STAGE, then the barriers
  const uint32_t smem32 = (smem_addr(smem_raw) + 1023u) & ~1023u;
  const uint32_t full32 = smem32 + NST * Geo::STAGE;        // weights and x of a stage have landed
  const uint32_t empty32 = full32 + NST * 8;                // every consumer warp is done with a stage
  const uint32_t sums32 = empty32 + NST * 8;                // the stage's group sums are written
  const uint32_t abort32 = sums32 + NST * 8;                // non-zero once a warp of the block has given up a wait

  // the warp index through a shuffle: the compiler then knows it is the same in every lane, keeps what derives from it
  // (roles, stage and barrier addresses) in uniform registers and branches on it without divergence handling
  const int tid = threadIdx.x, warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0), lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      // dense: the weights' bytes and the bytes of x each come with an arrival; grouped: the weights' arrival and one
      // from every lane of the copy warp when its 16-byte copies of x have landed
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full32 + 8 * i), "r"(GROUPED ? 33 : 2) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty32 + 8 * i), "r"(CONSUMERS) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sums32 + 8 * i), "r"(1) : "memory");
    }
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort32), "r"(0) : "memory");
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  auto give_up = [&](int code) {
    if (lane == 0) {
      asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort32), "r"(code) : "memory");
      atomicCAS(p.err, 0, code);
    }
  };
  const int first_item = blockIdx.x, step = gridDim.x;
  int n_items = p.items, sbg = 1;
  if constexpr (GROUPED) {
    pdl_wait();                                             // the plan may be the previous kernel's output
    sbg = (p.proj[0].nsb + KW - 1) / KW;
    n_items = __ldg(p.counts) * sbg;
  }
  auto item_at = [&](int i) -> StreamItem {
    if constexpr (GROUPED) return grouped_item<KW, G, ROWS>(p, i, sbg);
    else return stream_item<KW, G>(p, i);
  };

  if (warp == CONSUMERS) {
    // ------------------------------------------------------------------ copy warp: one bulk copy per lane and stage
    auto issue_w = [&](const StreamItem& it, int st, int slot) {
      if (lane == 0) {
        const uint32_t* w = TF_PROJ_FIELD(p, it.p, w);
        if constexpr (GROUPED) w += static_cast<int64_t>(it.expert) * p.expert_stride;
        const int64_t sb_stride = TF_PROJ_FIELD(p, it.p, sb_stride);
        const int ng = min(G, it.per - st * G);
        const uint32_t* src = w + static_cast<int64_t>(it.sb0) * sb_stride +
                              (static_cast<int64_t>(it.g_first) + static_cast<int64_t>(st) * G) * UNITW;
        const uint32_t bar = full32 + 8 * slot, dst = smem32 + slot * Geo::STAGE + Geo::W_OFF;
        mbar32_expect_tx(bar, it.lanes * ng * UNITW * 4);
        for (int kw = 0; kw < it.lanes; ++kw) bulk_load32(dst + kw * Geo::W_BYTES, src + kw * sb_stride, ng * UNITW * 4, bar);
      }
    };
    auto issue_x = [&](const StreamItem& it, int st, int slot, int64_t my_row) {
      if constexpr (GROUPED) {
        // gathered rows: 16-byte copies placed in the swizzle pattern of the tensor-map boxes; lane r < rows holds the
        // row of x that row r reads (my_row)
        const int ng = min(G, it.per - st * G);
        const int cpr = ng * GS / 8;                        // 16-byte chunks a row
        const uint32_t bar = full32 + 8 * slot, dst = smem32 + slot * Geo::STAGE + Geo::X_OFF;
        const __nv_bfloat16* src = p.x + static_cast<int64_t>(it.g_first + st * G) * GS;
        const int chunks = it.rows * cpr;
        for (int c0 = 0; c0 < chunks; c0 += 32) {
          const int c = c0 + lane;
          const bool valid = c < chunks;
          const int r = valid ? c / cpr : 0, q = c - r * cpr;
          const int64_t row = __shfl_sync(0xFFFFFFFFu, my_row, r);
          if (valid)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (q >> 3) * Geo::XHALF + r * XHALF_ROW +
                                                                          (((q & 7) ^ (r & 7)) << 4)),
                         "l"(src + row * p.ldx + q * 8)
                         : "memory");
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
      } else if (lane == 0) {
        const int ng = min(G, it.per - st * G);
        const int boxes = (ng * GS + 63) / 64;              // a [64 inputs x ROWS] box lands in a swizzled half tile
        const uint32_t bar = full32 + 8 * slot, dst = smem32 + slot * Geo::STAGE + Geo::X_OFF;
        mbar32_expect_tx(bar, boxes * Geo::XHALF);
        const int k0 = (it.g_first + st * G) * GS;
        for (int b = 0; b < boxes; ++b) tma_load_2d32(dst + b * Geo::XHALF, &tmx, k0 + 64 * b, 0, bar);
      }
    };
    // the weights of the first NST stages never depend on the previous kernel: they go out before the dependency wait
    {
      int gst = 0;
      for (int i = first_item; i < n_items && gst < NST; i += step) {
        const StreamItem it = item_at(i);
        for (int st = 0; st < it.nst && gst < NST; ++st, ++gst) issue_w(it, st, gst);
      }
    }
    pdl_wait();                                             // x may be the previous kernel's output
    bool ok = true;
    int gst = 0, slot = 0;
    uint32_t phase = 1;                                     // parity of the `empty` phase that frees the slot (first round: none)
    for (int i = first_item; i < n_items && ok; i += step) {
      const StreamItem it = item_at(i);
      int64_t my_row = 0;
      if constexpr (GROUPED) {
        if (lane < it.rows) {
          const int pair = __ldg(p.members + it.first + lane);
          my_row = p.slots > 0 ? pair / p.slots : pair;
        }
      }
      for (int st = 0; st < it.nst; ++st, ++gst) {
        if (gst >= NST) {                                   // the stage goes where stage gst - NST was
          ok = mbar32_wait(empty32 + 8 * slot, phase, abort32, 256);     // (naps between polls: the ring has slack)
          if (!ok) {
            give_up(ERR_WAIT_EMPTY);
            break;
          }
          issue_w(it, st, slot);
        }
        issue_x(it, st, slot, my_row);
        if (++slot == NST) slot = 0, phase ^= 1;
      }
    }
    if (!ok) {
      for (int i = 0; i < 64; ++i) __nanosleep(20000);      // copies in flight land before the shared memory is released
    }
  } else if (warp == CONSUMERS + 1) {
    // ------------------------------------------------------------------ sums warp: group sums of x, once per block
    pdl_wait();
    bool ok = true;
    int slot = 0;
    uint32_t phase = 0;
    const uint32_t xrow = (lane & 7) * XHALF_ROW;
    const uint32_t sw0 = (((lane >> 3) ^ (lane & 7)) << 4), sw1 = (((4 | (lane >> 3)) ^ (lane & 7)) << 4);
    for (int i = first_item; i < n_items && ok; i += step) {
      const StreamItem it = item_at(i);
      for (int st = 0; st < it.nst; ++st) {
        ok = mbar32_wait(full32 + 8 * slot, phase, abort32, 64);
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
            for (int mt = 0; mt < MT; ++mt) {
              float d[4];
              ones_mma_group<GS, Geo::XHALF>(d, sp32 + Geo::X_OFF, xrow, sw0, sw1, mt, u * GS);
              if (lane < 4)
                asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xs32 + (u * ROWS + mt * 8 + 2 * lane) * 4), "f"(d[0]), "f"(d[1])
                             : "memory");
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar32_arrive(sums32 + 8 * slot);     // also tells the consumers that the stage has landed
        if (++slot == NST) slot = 0, phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers: dequantise, MMA, affine epilogue
    const int kw = warp >> 2, tp = warp & 3;
    const int g = lane >> 2, t = lane & 3;
    constexpr float OFFSET = code_offset(BITS);
    // byte offsets inside a stage that depend on the thread only (shared memory is addressed with 32-bit addresses)
    const uint32_t w_off = Geo::W_OFF + kw * Geo::W_BYTES + (tp * 32 + lane) * WPL * 4;
    const uint32_t sb_off = Geo::W_OFF + kw * Geo::W_BYTES + (TILE_PAIRS * 32 * WPL + tp * 32 + g * 4) * 4;
    const uint32_t xrow = (lane & 7) * XHALF_ROW;
    const uint32_t xa0 = Geo::X_OFF + xrow + (((lane >> 3) ^ (lane & 7)) << 4);          // ldmatrix rows, chunks 0..3
    const uint32_t xa1 = Geo::X_OFF + xrow + (((4 | (lane >> 3)) ^ (lane & 7)) << 4);    // chunks 4..7
    const uint32_t xs_off = Geo::XS_OFF + 2 * t * 4;

    struct GroupRegs {
      uint32_t wd[WPL];
      uint4 sbw;
    };
    auto load_group = [&](GroupRegs& r, uint32_t sp32, int u) {
      const uint32_t src = sp32 + w_off + u * (UNITW * 4);
      if constexpr (WPL % 4 == 0) {
#pragma unroll
        for (int i = 0; i < WPL; i += 4) {
          const uint4 v = lds128(src + i * 4);
          r.wd[i] = v.x, r.wd[i + 1] = v.y, r.wd[i + 2] = v.z, r.wd[i + 3] = v.w;
        }
      } else if constexpr (WPL % 2 == 0) {
#pragma unroll
        for (int i = 0; i < WPL; i += 2) {
          const uint2 v = lds64(src + i * 4);
          r.wd[i] = v.x, r.wd[i + 1] = v.y;
        }
      } else {
#pragma unroll
        for (int i = 0; i < WPL; ++i) r.wd[i] = lds32(src + i * 4);
      }
      r.sbw = lds128(sp32 + sb_off + u * (UNITW * 4));
    };

    float acc[2][MT][4];
    // one group: the chained MMAs of P', then the affine step into acc
    auto compute_group = [&](const GroupRegs& r, uint32_t sp32, int u) {
      float2 xv[MT];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) xv[mt] = lds64f(sp32 + xs_off + (u * ROWS + mt * 8) * 4);
      const uint32_t xu0 = sp32 + xa0 + ((u * GS) >> 6) * Geo::XHALF, xu1 = sp32 + xa1 + ((u * GS) >> 6) * Geo::XHALF;
      const uint32_t kin = (u * GS) & 63;                   // the group's first input inside its half tile (groups of 32)
      float P[2][MT][4];
      uint32_t bf[MT][4];
#pragma unroll
      for (int s = 0; s < S; ++s) {
        if ((s & 1) == 0) {
          // inputs [16 s, 16 s + 32) of the group: chunk (kin + 16 s) / 8 of a half tile (a group of 128 spans two)
          const int k0 = 16 * s;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint32_t half = (GS == 128 && k0 >= 64) ? Geo::XHALF : 0;
            const uint32_t c4 = GS == 32 ? (kin >> 5) : ((k0 >> 5) & 1);       // which four chunks of the half tile
            ldmatrix_x4(bf[mt], (c4 ? xu1 : xu0) + half + mt * 8 * XHALF_ROW);
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t a[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) a[j] = pair_reg<BITS, GS, false>(r.wd, (h * S + s) * 4 + j);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            if (s == 0) mma_bf16_zero(P[h][mt], a, bf[mt][0], bf[mt][1]);
            else mma_bf16(P[h][mt], a, bf[mt][2 * (s & 1)], bf[mt][2 * (s & 1) + 1]);
          }
          if constexpr (SPLIT) {
            uint32_t ah[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) ah[j] = pair_reg<BITS, GS, true>(r.wd, (h * S + s) * 4 + j);
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
      const uint32_t sbv[4] = {r.sbw.x, r.sbw.y, r.sbw.z, r.sbw.w};   // (tile 0, col g), (0, g + 8), (1, g), (1, g + 8)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float s0 = bf16_lo(sbv[2 * h]), s1 = bf16_lo(sbv[2 * h + 1]);
        const float c0 = fmaf(-OFFSET, s0, bf16_hi(sbv[2 * h])), c1 = fmaf(-OFFSET, s1, bf16_hi(sbv[2 * h + 1]));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#ifdef TF_NO_FMA2
          acc[h][mt][0] = fmaf(xv[mt].x, c0, fmaf(P[h][mt][0], s0, acc[h][mt][0]));
          acc[h][mt][1] = fmaf(xv[mt].y, c0, fmaf(P[h][mt][1], s0, acc[h][mt][1]));
          acc[h][mt][2] = fmaf(xv[mt].x, c1, fmaf(P[h][mt][2], s1, acc[h][mt][2]));
          acc[h][mt][3] = fmaf(xv[mt].y, c1, fmaf(P[h][mt][3], s1, acc[h][mt][3]));
#else
          fma2(acc[h][mt][0], acc[h][mt][1], P[h][mt][0], P[h][mt][1], s0, s0);
          fma2(acc[h][mt][0], acc[h][mt][1], xv[mt].x, xv[mt].y, c0, c0);
          fma2(acc[h][mt][2], acc[h][mt][3], P[h][mt][2], P[h][mt][3], s1, s1);
          fma2(acc[h][mt][2], acc[h][mt][3], xv[mt].x, xv[mt].y, c1, c1);
#endif
        }
      }
    };

    // rows mt * 8 + 2 t (+ 1), columns 32 tp + 16 h + g (+ 8) of super-block sb: the m16n8 accumulator fragment
    struct OutProj {
      void* out;
      int64_t ldo;
      int N, out_f32;
    };
    auto store_out = [&](const OutProj& pr, int sb, const float (&v)[2][MT][4]) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int m = mt * 8 + 2 * t + (e & 1), n = sb * SB_COLS + tp * 32 + h * 16 + g + 8 * (e >> 1);
            if (m < p.M && n < pr.N) {
              if (pr.out_f32) reinterpret_cast<float*>(pr.out)[m * pr.ldo + n] = v[h][mt][e];
              else reinterpret_cast<__nv_bfloat16*>(pr.out)[m * pr.ldo + n] = __float2bfloat16_rn(v[h][mt][e]);
            }
          }
    };

    bool ok = true;
    bool have_a = false;                                    // group 0 of the coming stage already sits in ra
    GroupRegs ra, rb;
    int slot = 0;
    uint32_t phase = 0;                                     // parity of the `sums` phase the current slot waits for
    for (int i = first_item; i < n_items && ok; i += step) {
      const StreamItem it = item_at(i);
      const bool active = kw < it.lanes;
      const bool more_items = i + step < n_items;
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[h][mt][e] = 0.f;

      for (int st = 0; st < it.nst; ++st) {
        const uint32_t sp32 = smem32 + slot * Geo::STAGE;
        if (!have_a) {
          ok = mbar32_wait(sums32 + 8 * slot, phase, abort32);
          if (!ok) {
            give_up(ERR_WAIT_SUMS);
            break;
          }
          if (active) load_group(ra, sp32, 0);
        }
        have_a = false;
        const int ng = min(G, it.per - st * G);
        const int nslot = slot + 1 == NST ? 0 : slot + 1;
        const uint32_t nphase = slot + 1 == NST ? phase ^ 1 : phase;
        if (active) {
          if (Geo::PREFETCH && ng == G) {
            // a whole stage: groups alternate between the two register sets, and the set for the group after next is
            // loaded before the current group computes (the next stage's first group only if that stage has landed)
            const bool more = st + 1 < it.nst || more_items;
#pragma unroll
            for (int u = 0; u < G; u += 2) {
              load_group(rb, sp32, u + 1);
              compute_group(ra, sp32, u);
              if (u + 2 < G) {
                load_group(ra, sp32, u + 2);
              } else if (more && __all_sync(0xFFFFFFFFu, mbar32_try_wait(sums32 + 8 * nslot, nphase))) {
                load_group(ra, smem32 + nslot * Geo::STAGE, 0);   // (an idle lane of the next item loads unused words)
                have_a = true;
              }
              compute_group(rb, sp32, u + 1);
            }
          } else {
            for (int u = 0; u < ng; ++u) {
              if (u > 0) load_group(ra, sp32, u);
              compute_group(ra, sp32, u);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar32_arrive(empty32 + 8 * slot);
        slot = nslot, phase = nphase;
      }
      if (!ok) break;

      // ---------------------------------------------------------------- the item's output
      if constexpr (GROUPED) {
        if (active && it.rows > 0) {
          // rows mt * 8 + 2 t (+ 1) of the item are pairs members[first + row]; each writes its own row of out
          const int sb = it.sb0 + kw;
          int64_t orow[MT][2];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int ml = mt * 8 + 2 * t + e;
              orow[mt][e] = ml < it.rows ? static_cast<int64_t>(__ldg(p.members + it.first + ml)) * p.proj[0].ldo : -1;
            }
          if (p.epi == 2) {
            // SwiGLU: half 0 of a tile pair holds 16 gate columns, half 1 the up columns of the same 16 outputs
            const int nout = p.proj[0].N / 2;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.proj[0].out);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int n = sb * (SB_COLS / 2) + tp * 16 + g + 8 * (e >> 1);
                if (orow[mt][e & 1] >= 0 && n < nout)
                  out[orow[mt][e & 1] + n] = __float2bfloat16_rn(swiglu_f(acc[0][mt][e], acc[1][mt][e], p.limit));
              }
          } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int n = sb * SB_COLS + tp * 32 + h * 16 + g + 8 * (e >> 1);
                  if (orow[mt][e & 1] < 0 || n >= p.proj[0].N) continue;
                  const float v = p.epi == 1 ? relu2_f(acc[h][mt][e]) : acc[h][mt][e];
                  if (p.proj[0].out_f32) reinterpret_cast<float*>(p.proj[0].out)[orow[mt][e & 1] + n] = v;
                  else reinterpret_cast<__nv_bfloat16*>(p.proj[0].out)[orow[mt][e & 1] + n] = __float2bfloat16_rn(v);
                }
          }
        }
      } else if (active) {
        pdl_wait();                                         // nothing is written before the previous kernel is done
        OutProj pr;
        pr.out = TF_PROJ_FIELD(p, it.p, out), pr.ldo = TF_PROJ_FIELD(p, it.p, ldo);
        pr.N = TF_PROJ_FIELD(p, it.p, N), pr.out_f32 = TF_PROJ_FIELD(p, it.p, out_f32);
        const int sb = it.sb0 + kw;
        if (it.sk == 1) {
          store_out(pr, sb, acc);
        } else {
          // fragment f = h * MT + mt of slice s: float4 index (((sb * sk + s) * 4 + tp) * 4 + f) * 32 + lane
          float* part = TF_PROJ_FIELD(p, it.p, part);
          float4* mine = reinterpret_cast<float4*>(part) + ((static_cast<int64_t>(sb) * it.sk + it.slice) * 4 + tp) * 128 + lane;
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
              __stcg(mine + (h * MT + mt) * 32, make_float4(acc[h][mt][0], acc[h][mt][1], acc[h][mt][2], acc[h][mt][3]));
          __threadfence();                                  // the slice is visible before this warp counts itself in
          __syncwarp();
          int* counter = TF_PROJ_FIELD(p, it.p, count) + sb * 4 + tp;
          int seen = 0;
          if (lane == 0) seen = atomicAdd(counter, 1);
          seen = __shfl_sync(0xFFFFFFFFu, seen, 0);
          if (seen == it.sk - 1) {
            __threadfence();                                // the other warps' slices are visible before they are read
            const float4* base = reinterpret_cast<const float4*>(part) + (static_cast<int64_t>(sb) * it.sk * 4 + tp) * 128 + lane;
            float v[2][MT][4];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                const float4 q = __ldcg(base + (h * MT + mt) * 32);
                v[h][mt][0] = q.x, v[h][mt][1] = q.y, v[h][mt][2] = q.z, v[h][mt][3] = q.w;
              }
#pragma unroll 4
            for (int s = 1; s < it.sk; ++s) {               // slice order ((s0 + s1) + s2) + ...
              const float4* src = base + static_cast<int64_t>(s) * 512;
#pragma unroll
              for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                  const float4 q = __ldcg(src + (h * MT + mt) * 32);
                  v[h][mt][0] += q.x, v[h][mt][1] += q.y, v[h][mt][2] += q.z, v[h][mt][3] += q.w;
                }
            }
            if (lane == 0) *counter = 0;                    // the next launch finds the counter at zero again
            store_out(pr, sb, v);
          }
        }
      }
    }
  }
}

#undef TF_PROJ_FIELD

}  // namespace tf
