// Prefill matmul on the 5th-generation tensor cores: out[m, n] = sum_k x[m, k] * bf16(q[n, k] * s + b).
//
// Arithmetic contract (the reference's prefill form, cuda/kernels/qmm_prefill.cu:1,115-118): every weight is rounded once
// to bf16, w = bf16(fma(q, s, b)) with q exact, then ONE fp32 accumulation chain runs over all of K in 16-input steps
// (tcgen05.mma, accumulator in tensor memory).  Any chunking of the rows gives the same bits; they are not the decode
// kernel's bits (that one keeps the affine terms in fp32).
//
// Block tile = 128 output columns x 256 rows of x, "swap-AB": the dequantised weights are the MMA's A operand (M = 128),
// the rows of x its B operand (N = 256), so every dequantised weight feeds 256 rows.  The kernel is persistent: a grid
// no larger than the number of SMs, tiles dealt round-robin, and every producer simply runs on into the block's next
// tile, so a tile's prologue (first bytes are about 2000 cycles away) and its drain overlap the neighbouring tiles'
// MMAs.  Two rings decouple the latencies: packed units arrive from HBM by bulk copies into a ring of small slots; a
// stage of the main ring holds the dequantised A tile and the x tile (a 2-D tensor-map copy with the 128-byte
// swizzle) of 64 inputs behind ONE full barrier and ONE empty barrier.  Two accumulators in tensor memory alternate
// between tiles.  Roles: warp 0 loads x, warp 1 owns tensor memory and issues the MMAs, warp 2 loads packed units,
// warps 4-19 are two groups of eight conversion warps that take alternate stages (a stage's conversion is a long
// dependent chain, so two stages are always in conversion), warps 20-23 drain the finished accumulator to global memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/tensorfold_b200.h"
#include "tf_layout.h"
#include "tf_ptx.cuh"

namespace tf {

int fail_moe(int code, const char* msg);
int cuda_fail_moe(cudaError_t e, const char* what);
int* device_error_word();          // tf_api.cu: the current device's error word (null before tf_init)

namespace {

constexpr int PF_COLS = 128;       // output columns of a block tile (MMA M)
constexpr int PF_STAGE_K = 64;     // inputs a stage
constexpr int PF_A_BYTES = PF_COLS * 128;
constexpr int PF_W_BYTES = 5120;   // packed units of a stage: one g64 unit (4608 B) or two g32 units (5120 B)
constexpr int PF_NW = 6;           // packed-unit slots in flight
constexpr int PF_THREADS = 768;    // 24 warps: x loads, MMA, unit loads, (idle), 2 x 8 conversion, 4 drain
constexpr int PF_CONV0 = 4;        // first conversion warp
constexpr int PF_DRAIN0 = 20;      // first drain warp (a multiple of 4: tensor-memory lane groups go by warp % 4)
constexpr int PF_BAR_BYTES = 512;

// ROWS = rows of x of a block tile (MMA N): 256 for dense prompts, 128 for the grouped expert form
template <int ROWS>
struct PfGeo {
  static constexpr int B_BYTES = ROWS * 128;
  static constexpr int STAGE = PF_A_BYTES + B_BYTES;
  static constexpr int NS = ROWS == 256 ? 4 : 6;           // stages in flight (even: the conversion groups alternate)
  static constexpr int W_OFF = NS * STAGE, BAR_OFF = W_OFF + PF_NW * PF_W_BYTES;
  static constexpr int SMEM = BAR_OFF + PF_BAR_BYTES + 1024 /* alignment slack */;
  static_assert(STAGE % 1024 == 0, "tiles stay 1024-byte aligned for the 128-byte swizzle");
  static_assert((2 * NS + 2 * PF_NW + 4) * 8 + 16 <= PF_BAR_BYTES, "barriers fit");
  static_assert(NS % 2 == 0, "conversion groups alternate stages");
  static_assert(SMEM <= 232448, "fits the opt-in shared memory of a block");
};

struct PrefillParams {
  const uint32_t* w;
  int64_t sb_stride;
  int N, K, M;
  void* out;
  int64_t ldo;
  int out_f32;
  int* err;
  // grouped form (items != null): block (x, y) = plan item y = (expert, first, count <= ROWS); the tensor map covers the
  // rows in member order, row first + r of it feeds pair members[first + r], which is the row of out that is written
  const int* items;
  const int* counts;
  const int* members;
  int64_t expert_stride;
  int experts;                // experts the table holds (grouped form)
  int epi;                    // 0 store, 1 relu^2, 2 SwiGLU over gate/up rows interleaved in tiles of 16 (out: N / 2 columns)
  float limit;
};

__device__ __forceinline__ float pf_bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float pf_swiglu(float g, float u, float limit) {
  float gv = pf_bf16r(g), uv = pf_bf16r(u);
  if (limit > 0.f) {
    gv = fminf(gv, limit);
    uv = fminf(fmaxf(uv, -limit), limit);
  }
  return pf_bf16r(gv / (1.f + expf(-gv))) * uv;
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr) {
  // K-major, 128-byte swizzle: rows 128 B apart inside an 8-row atom, atoms 1024 B apart (SBO), LBO unused (1),
  // descriptor version 1, layout type 2 (SWIZZLE_128B)
  const uint32_t lo = ((smem_byte_addr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = 64u | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

// The whole warp runs these with warp-uniform operands (so the descriptors can live in uniform registers); the
// instruction itself is predicated on `leader`, true in exactly one lane.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                          uint32_t leader) {
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar, uint32_t leader) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %1, 0;\n"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}" ::"r"(smem_addr(bar)),
      "r"(leader)
      : "memory");
}

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
      "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int GS, int ROWS>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_kernel(const __grid_constant__ CUtensorMap tmx, const PrefillParams p) {
  using Geo = PfGeo<ROWS>;
  constexpr int PF_ROWS = ROWS, PF_B_BYTES = Geo::B_BYTES, NS = Geo::NS;
  constexpr uint32_t PF_TMEM_COLS = 2 * ROWS;                // two accumulators: one fills while the other drains
  constexpr int S = GS / 16;                                 // k16 steps a group
  constexpr int UNITS = PF_STAGE_K / GS;                     // units a stage (1 for g64, 2 for g32)
  constexpr int WPL = words_per_lane(4, GS);
  constexpr int UNITW = unit_words(4, GS);
  static_assert(UNITS * UNITW * 4 <= PF_W_BYTES, "slot holds a stage's packed units");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Geo::BAR_OFF);
  uint64_t* full = bars;                            // stage ready: 8 conversion warps arrived and the x tile landed
  uint64_t* empty = full + NS;                      // the MMAs that read the stage are done
  uint64_t* w_full = empty + NS;                    // packed units landed (bulk copy)
  uint64_t* w_empty = w_full + PF_NW;               // the 8 conversion warps of the stage's group have read the slot
  uint64_t* acc_full = w_empty + PF_NW;             // [2] every MMA of a tile is done
  uint64_t* acc_empty = acc_full + 2;               // [2] the 4 drain warps have read the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nstages = (p.K + PF_STAGE_K - 1) / PF_STAGE_K;
  const int total_units = p.K / GS;
  const int nsb = (p.N + PF_COLS - 1) / PF_COLS;
  const bool grouped = p.items != nullptr;
  // Tiles = column blocks x row tiles (plan items in the grouped form), column block fastest, dealt round-robin to the
  // blocks of a grid no larger than the number of SMs.  Every role walks the same (tile, stage) sequence, so a running
  // stage count g names the ring slot (g % NS) and its phase without any exchange between the roles.
  const int row_tiles = grouped ? p.counts[0] : (p.M + PF_ROWS - 1) / PF_ROWS;
  const int tiles = nsb * row_tiles;
  const int first_tile = blockIdx.x;
  if (first_tile >= tiles) return;                           // before any barrier or tensor-memory use
  const int my_tiles = (tiles - first_tile + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int total = my_tiles * nstages;                      // stages this block runs

  struct Tile {
    int sb, m0, rows_here, first;
    const uint32_t* wroot;
  };
  auto tile_at = [&](int it) {
    const int t = first_tile + it * static_cast<int>(gridDim.x);
    Tile ti;
    ti.sb = t % nsb;
    const int y = t / nsb;
    ti.wroot = p.w;
    if (grouped) {
      const int* item = p.items + 3 * y;
      // an item that names an expert outside the table runs against expert 0 with no rows (nothing is stored) and
      // is reported: every role still walks the same tile sequence, and nothing is read past the table
      const bool known = item[0] >= 0 && item[0] < p.experts;
      if (!known && threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_ITEM);
      ti.wroot += static_cast<int64_t>(known ? item[0] : 0) * p.expert_stride;
      ti.first = item[1];
      ti.rows_here = known ? min(PF_ROWS, item[2]) : 0;
      ti.m0 = item[1];                                       // row of the member-ordered input
    } else {
      ti.first = 0;
      ti.m0 = y * PF_ROWS;
      ti.rows_here = min(PF_ROWS, p.M - ti.m0);
    }
    return ti;
  };

  auto a_tile = [&](int s) { return smem + s * Geo::STAGE; };
  auto b_tile = [&](int s) { return smem + s * Geo::STAGE + PF_A_BYTES; };
  auto w_slot = [&](int s) { return smem + Geo::W_OFF + s * PF_W_BYTES; };
  auto give_up = [&](int code) {
    if (lane == 0) {
      *abort_flag = code;
      atomicCAS(p.err, 0, code);
    }
  };

  if (tid == 0) {
    for (int i = 0; i < NS; ++i) mbar_init(full + i, 9), mbar_init(empty + i, 1);
    for (int i = 0; i < PF_NW; ++i) mbar_init(w_full + i, 1), mbar_init(w_empty + i, 8);
    for (int i = 0; i < 2; ++i) mbar_init(acc_full + i, 1), mbar_init(acc_empty + i, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(PF_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ x tiles (L2 -> shared, tensor-map copies)
    bool ok = true;
    int g = 0;
    for (int it = 0; it < my_tiles && ok; ++it) {
      const Tile ti = tile_at(it);
      for (int ls = 0; ls < nstages && ok; ++ls, ++g) {
        const int s = g % NS;
        if (g >= NS) {
          ok = mbar_wait(empty + s, (g / NS - 1) & 1, abort_flag);
          if (!ok) {
            give_up(ERR_WAIT_EMPTY);
            break;
          }
        }
        if (lane == 0) {
          mbar_expect_tx(full + s, PF_B_BYTES);
          tma_load_2d(b_tile(s), &tmx, ls * PF_STAGE_K, ti.m0, full + s);
        }
        __syncwarp();
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ packed units (HBM -> shared, bulk copies)
    bool ok = true;
    int g = 0;
    for (int it = 0; it < my_tiles && ok; ++it) {
      const Tile ti = tile_at(it);
      const uint32_t* wsb = ti.wroot + static_cast<int64_t>(ti.sb) * p.sb_stride;
      for (int ls = 0; ls < nstages && ok; ++ls, ++g) {
        const int s = g % PF_NW;
        if (g >= PF_NW) {
          ok = mbar_wait(w_empty + s, (g / PF_NW - 1) & 1, abort_flag);
          if (!ok) {
            give_up(ERR_WAIT_EMPTY);
            break;
          }
        }
        if (lane == 0) {
          const int units_here = min(UNITS, total_units - ls * UNITS);
          mbar_expect_tx(w_full + s, units_here * UNITW * 4);
          bulk_load(w_slot(s), wsb + static_cast<int64_t>(ls) * UNITS * UNITW, units_here * UNITW * 4, w_full + s);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue (one thread)
    // The tensor pipe's queue is short and every instruction of this warp between two MMA issues is dead time for
    // it, so the loop is unrolled over the ring (descriptors by constant offsets, no index arithmetic) and the next
    // stage's full barrier is tested between this stage's MMAs, while earlier ones are still executing.
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((PF_ROWS >> 3) << 17) | ((PF_COLS >> 4) << 24);
    constexpr uint64_t SLOT_STEP = Geo::STAGE >> 4;            // a ring slot further, in descriptor address units
    const uint32_t leader = lane == 0 ? 1u : 0u;
    const uint64_t ad0 = umma_desc(smem_addr(a_tile(0))), bd0 = umma_desc(smem_addr(b_tile(0)));
    bool ok = mbar_wait(full, 0, abort_flag);
    if (!ok) give_up(ERR_WAIT_FULL);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t phase = 0;                                          // parity of the full barriers of this pass over the ring
    int ls = 0, it = 0;                                          // stage inside the tile, tile count of this block
    for (int base = 0; base < total && ok; base += NS, phase ^= 1u) {
#pragma unroll
      for (int st = 0; st < NS; ++st) {
        const int g = base + st;
        if (g >= total || !ok) break;
        if (ls == 0 && it >= 2) {                                // the accumulator's last tile must have been drained
          ok = mbar_wait(acc_empty + (it & 1), ((it >> 1) - 1) & 1, abort_flag);
          if (!ok) {
            give_up(ERR_WAIT_EMPTY);
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t acc = tmem_base + static_cast<uint32_t>(it & 1) * PF_ROWS;
        const uint64_t ad = ad0 + st * SLOT_STEP, bd = bd0 + st * SLOT_STEP;
        const int nx = (st + 1) % NS;
        const uint32_t nx_phase = st + 1 == NS ? phase ^ 1u : phase;
        const bool more = g + 1 < total;
        bool next_ready = false;
        umma_bf16(acc, ad, bd, IDESC, ls > 0 ? 1u : 0u, leader);
        umma_bf16(acc, ad + 2, bd + 2, IDESC, 1u, leader);       // + 32 bytes a k16 step inside the swizzle atom
        umma_bf16(acc, ad + 4, bd + 4, IDESC, 1u, leader);
        if (more) {
          next_ready = mbar_test(full + nx, nx_phase);
          if (next_ready) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        umma_bf16(acc, ad + 6, bd + 6, IDESC, 1u, leader);
        umma_commit(empty + st, leader);
        if (ls == nstages - 1) {
          umma_commit(acc_full + (it & 1), leader);
          ls = 0, ++it;
        } else {
          ++ls;
        }
        if (more && !next_ready) {
          ok = mbar_wait(full + nx, nx_phase, abort_flag);
          if (!ok) give_up(ERR_WAIT_FULL);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
      }
    }
  } else if (warp >= PF_CONV0 && warp < PF_DRAIN0) {
    // ------------------------------------------------------------------ conversion: packed codes -> swizzled bf16 A tile
    // A warp owns 16 output columns (tile pair tp, half h) of every stage its group takes.  Per 16-input step a thread
    // holds the four m8n8 fragments (two column octets x two input octets) of its lane's codes, so one stmatrix.x4
    // writes four 8 x 16-byte row segments of the swizzled tile; lane l supplies the address of row l % 8 of fragment l / 8.
    const int cw = warp - PF_CONV0, group = cw >> 3, dw = cw & 7, tp = dw & 3, h = dw >> 2, g8 = lane >> 2;
    const __nv_bfloat162 k128 = __floats2bfloat162_rn(128.f, 128.f);
    uint32_t row_off[4];                                        // this lane's row segment of each 16-input step of a stage
#pragma unroll
    for (int q = 0; q < 4; ++q)
      row_off[q] = (32 * tp + 16 * h + 8 * ((lane >> 3) & 1) + (lane & 7)) * 128 + (((2 * q + (lane >> 4)) ^ (lane & 7)) << 4);
    bool ok = true;
    for (int i = group; i < total && ok; i += 2) {             // i = the block's running stage count
      const int sw = i % PF_NW, st = i % NS, ls = i % nstages;
      ok = mbar_wait(w_full + sw, (i / PF_NW) & 1, abort_flag);
      if (ok && i >= NS) ok = mbar_wait(empty + st, (i / NS - 1) & 1, abort_flag);
      if (!ok) {
        give_up(ERR_WAIT_FULL);
        break;
      }
      const uint32_t* wst = reinterpret_cast<const uint32_t*>(w_slot(sw));
      const uint32_t at = smem_addr(a_tile(st));
      const int units_here = min(UNITS, total_units - ls * UNITS);
#pragma unroll
      for (int u = 0; u < UNITS; ++u) {
        uint32_t wd[S] = {};
        __nv_bfloat162 sc[2], bi[2];
        sc[0] = sc[1] = bi[0] = bi[1] = __floats2bfloat162_rn(0.f, 0.f);
        // past the end of K (it ends inside this stage) x is zero (the tensor map fills it) and the weights must be
        // finite: codes, scales and biases of zero give zero weights
        if (u < units_here) {
          const uint32_t* unit = wst + u * UNITW;
          if constexpr (S == 4) {
            const uint4 v = *reinterpret_cast<const uint4*>(unit + (tp * 32 + lane) * WPL + h * S);
            wd[0] = v.x, wd[1] = v.y, wd[2] = v.z, wd[3] = v.w;
          } else {
            const uint2 v = *reinterpret_cast<const uint2*>(unit + (tp * 32 + lane) * WPL + h * S);
            wd[0] = v.x, wd[1] = v.y;
          }
          const uint2 sbw = *reinterpret_cast<const uint2*>(unit + TILE_PAIRS * 32 * WPL + tp * 32 + g8 * 4 + h * 2);
          const uint32_t sbv[2] = {sbw.x, sbw.y};                  // columns c0 and c0 + 8
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint32_t s2 = __byte_perm(sbv[r], 0u, 0x1010), b2 = __byte_perm(sbv[r], 0u, 0x3232);
            sc[r] = *reinterpret_cast<const __nv_bfloat162*>(&s2);
            bi[r] = *reinterpret_cast<const __nv_bfloat162*>(&b2);
          }
        }
#pragma unroll
        for (int sidx = 0; sidx < S; ++sidx) {
          uint32_t frag[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t v = ((wd[sidx] >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
            const __nv_bfloat162 q2 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), k128);       // exact code
            const __nv_bfloat162 w2 = __hfma2(q2, sc[j & 1], bi[j & 1]);                            // one rounding
            frag[j] = *reinterpret_cast<const uint32_t*>(&w2);
          }
          asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(at + row_off[u * S + sidx]),
                       "r"(frag[0]), "r"(frag[1]), "r"(frag[2]), "r"(frag[3])
                       : "memory");
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(full + st);
        mbar_arrive(w_empty + sw);                               // the slot's words are in registers or already used
      }
    }
  } else if (warp >= PF_DRAIN0) {
    // ------------------------------------------------------------------ drain: tensor memory -> global, a tile behind
    const int lg = warp & 3;                                   // this warp may touch TMEM lanes [32 lg, 32 lg + 32)
    for (int it = 0; it < my_tiles; ++it) {
      const Tile ti = tile_at(it);
      const int ab = it & 1, rows_here = ti.rows_here, first = ti.first, m0 = ti.m0, sb = ti.sb;
      const bool done = mbar_wait(acc_full + ab, (it >> 1) & 1, abort_flag);
      if (!done) {
        give_up(ERR_WAIT_FULL);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (*abort_flag != 0) break;
      // A lane holds one output column for 32 rows of x.  Each group of eight lanes transposes its 8 x 8 blocks in
      // registers (three butterfly steps), so a lane then holds eight neighbouring columns of one row and writes them
      // as 16 bytes: a store instruction costs about the same whatever its width, and narrow ones made the drain the
      // slowest part of a tile.
      const bool swiglu = p.epi == 2;
      const int col = swiglu ? sb * (PF_COLS / 2) + lg * 16 + lane : sb * PF_COLS + lg * 32 + lane;
      const int ncols = swiglu ? p.N / 2 : p.N;
      const bool live = col < ncols && (!swiglu || lane < 16);
      const bool wide = !p.out_f32 && (ncols & 7) == 0 && (p.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
      const int l8 = lane & 7;
#pragma unroll 1
      for (int col0 = 0; col0 < rows_here; col0 += 32) {         // 32 rows of x a pass
        uint32_t r[32];
        tmem_load32(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + static_cast<uint32_t>(ab * PF_ROWS + col0), r);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          v[j] = __uint_as_float(r[j]);
          if (swiglu) {                                          // lanes 0-15 hold gate columns, 16-31 the up columns
            const float up = __shfl_down_sync(0xFFFFFFFFu, v[j], 16);
            v[j] = pf_swiglu(v[j], up, p.limit);
          } else if (p.epi == 1) {
            v[j] = fmaxf(pf_bf16r(v[j]), 0.f);
            v[j] = v[j] * v[j];
          }
        }
        if (wide) {
#pragma unroll
          for (int blk = 0; blk < 4; ++blk) {                    // rows 8 blk .. 8 blk + 7 of the pass
            float* a = v + 8 * blk;
#pragma unroll
            for (int mask = 4; mask >= 1; mask >>= 1) {
              const bool upper = (l8 & mask) != 0;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (i & mask) continue;
                const float got = __shfl_xor_sync(0xFFFFFFFFu, upper ? a[i] : a[i | mask], mask);
                if (upper) a[i] = got;
                else a[i | mask] = got;
              }
            }
            const int rr = col0 + 8 * blk + l8;                  // a[c] = column (col - l8 + c) of row rr
            if (live && rr < rows_here) {
              const int64_t m = grouped ? p.members[first + rr] : m0 + rr;
              uint4 o;
              __nv_bfloat162 t0 = __floats2bfloat162_rn(a[0], a[1]), t1 = __floats2bfloat162_rn(a[2], a[3]);
              __nv_bfloat162 t2 = __floats2bfloat162_rn(a[4], a[5]), t3 = __floats2bfloat162_rn(a[6], a[7]);
              o.x = *reinterpret_cast<uint32_t*>(&t0), o.y = *reinterpret_cast<uint32_t*>(&t1);
              o.z = *reinterpret_cast<uint32_t*>(&t2), o.w = *reinterpret_cast<uint32_t*>(&t3);
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + m * p.ldo + (col - l8)) = o;
            }
          }
        } else if (live) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int rr = col0 + j;
            if (rr < rows_here) {
              const int64_t m = grouped ? p.members[first + rr] : m0 + rr;
              if (p.out_f32) reinterpret_cast<float*>(p.out)[m * p.ldo + col] = v[j];
              else reinterpret_cast<__nv_bfloat16*>(p.out)[m * p.ldo + col] = __float2bfloat16_rn(v[j]);
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + ab);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(PF_TMEM_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(sym);
  });
  return fn;
}

}  // namespace

// dst[pos, :] = src[row(members[pos]), :]: the rows of a grouped call in member order, so an item's rows are contiguous
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, int64_t ld, const int* __restrict__ members,
                                   const int* __restrict__ counts_total, int slots, int pairs, int k,
                                   __nv_bfloat16* __restrict__ dst) {
  const int lane = threadIdx.x & 31;
  const int pos = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pos >= pairs) return;
  const int pair = members[pos];
  if (pair < 0 || pair >= pairs) return;                     // members past the planned pairs hold no pair
  const int64_t row = slots > 0 ? pair / slots : pair;
  const uint4* s4 = reinterpret_cast<const uint4*>(src + row * ld);
  uint4* d4 = reinterpret_cast<uint4*>(dst + static_cast<int64_t>(pos) * k);
  for (int i = lane; i < k / 8; i += 32) d4[i] = s4[i];
}


// SMs of the current device (cached per device)
int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

cudaError_t prefill_configure() {
  cudaError_t e = cudaFuncSetAttribute(prefill_kernel<64, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfGeo<256>::SMEM);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(prefill_kernel<32, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfGeo<256>::SMEM);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(prefill_kernel<64, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfGeo<128>::SMEM);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(prefill_kernel<32, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, PfGeo<128>::SMEM);
  return e;
}

int encode_rows(CUtensorMap* map, const void* x, int64_t ldx, int rows, int k, int box_rows) {
  EncodeTiled encode = encode_fn();
  if (encode == nullptr) return fail_moe(TF_ERR_UNSUPPORTED, "prefill: the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldx) * 2};
  const cuuint32_t box[2] = {PF_STAGE_K, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TF_OK : fail_moe(TF_ERR_ARG, "prefill: cuTensorMapEncodeTiled refused the input tensor");
}

}  // namespace tf

using namespace tf;

extern "C" int tf_qmm_prefill_act(const void* x, int64_t ldx, int m, const void* tiled, int64_t sb_stride, int n, int k, int gs,
                                  void* out, int64_t ldo, int out_f32, int epi, float limit, void* stream);

extern "C" int tf_qmm_prefill(const void* x, int64_t ldx, int m, const void* tiled, int64_t sb_stride, int n, int k, int gs,
                              void* out, int64_t ldo, int out_f32, void* stream) {
  return tf_qmm_prefill_act(x, ldx, m, tiled, sb_stride, n, k, gs, out, ldo, out_f32, 0, 0.f, stream);
}

extern "C" int tf_qmm_prefill_act(const void* x, int64_t ldx, int m, const void* tiled, int64_t sb_stride, int n, int k, int gs,
                                  void* out, int64_t ldo, int out_f32, int epi, float limit, void* stream) {
  if (gs != 32 && gs != 64) return fail_moe(TF_ERR_UNSUPPORTED, "tf_qmm_prefill: 4-bit weights with groups of 32 or 64");
  if (m < 1 || n < 1 || k < gs || k % gs) return fail_moe(TF_ERR_ARG, "tf_qmm_prefill: K must be a positive multiple of the group");
  if (epi < 0 || epi > 2 || (epi == 2 && n % 32) || (epi != 0 && out_f32)) return fail_moe(TF_ERR_ARG, "tf_qmm_prefill: bad epilogue");
  if (!x || !tiled || !out || ldo < (epi == 2 ? n / 2 : n) || ldx < k) return fail_moe(TF_ERR_ARG, "tf_qmm_prefill: null pointer or short rows");
  if (reinterpret_cast<uintptr_t>(x) % 16 || ldx % 8) return fail_moe(TF_ERR_ALIGN, "tf_qmm_prefill: x rows must start on 16-byte boundaries");
  if (reinterpret_cast<uintptr_t>(tiled) % 16) return fail_moe(TF_ERR_ALIGN, "tf_qmm_prefill: tiled weights must be 16-byte aligned");
  int* err = device_error_word();
  if (err == nullptr) return fail_moe(TF_ERR_STATE, "tf_qmm_prefill: tf_init has not been called for the current device");
  CUtensorMap map;
  if (int rc = encode_rows(&map, x, ldx, m, k, 256)) return rc;
  PrefillParams p = {};
  p.w = static_cast<const uint32_t*>(tiled);
  p.sb_stride = sb_stride > 0 ? sb_stride : static_cast<int64_t>(k / gs) * unit_words(4, gs);
  p.N = n, p.K = k, p.M = m;
  p.out = out, p.ldo = ldo, p.out_f32 = out_f32;
  p.err = err;
  p.epi = epi, p.limit = limit;
  const int64_t tiles = static_cast<int64_t>((n + PF_COLS - 1) / PF_COLS) * ((m + 255) / 256);
  if (tiles > (1 << 24)) return fail_moe(TF_ERR_ARG, "tf_qmm_prefill: too many tiles");
  const int sms = sm_count();
  if (sms < 1) return fail_moe(TF_ERR_STATE, "tf_qmm_prefill: cannot read the SM count");
  dim3 grid(static_cast<unsigned>(tiles < sms ? tiles : sms));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (gs == 64) prefill_kernel<64, 256><<<grid, PF_THREADS, PfGeo<256>::SMEM, s>>>(map, p);
  else prefill_kernel<32, 256><<<grid, PF_THREADS, PfGeo<256>::SMEM, s>>>(map, p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_qmm_prefill");
}

extern "C" int tf_moe_experts_prefill(const void* x, int64_t ldx, int slots, const void* tiled, int64_t expert_stride,
                                      int experts, int n, int k, int gs, const int* items, const int* counts,
                                      const int* members, int pairs, int max_items, void* sorted, void* out, int64_t ldo,
                                      int out_f32, int epi, float limit, void* stream) {
  if (experts < 1) return fail_moe(TF_ERR_ARG, "tf_moe_experts_prefill: the table holds at least one expert");
  if (gs != 32 && gs != 64) return fail_moe(TF_ERR_UNSUPPORTED, "tf_moe_experts_prefill: 4-bit weights with groups of 32 or 64");
  if (n < 1 || k < gs || k % gs || k % 8 || pairs < 1 || max_items < 1 || max_items > 65535)
    return fail_moe(TF_ERR_ARG, "tf_moe_experts_prefill: bad sizes");
  if (epi < 0 || epi > 2 || (epi == 2 && n % 32) || (epi != 0 && out_f32)) return fail_moe(TF_ERR_ARG, "tf_moe_experts_prefill: bad epilogue");
  const int ncols = epi == 2 ? n / 2 : n;
  if (!x || !tiled || !items || !counts || !members || !sorted || !out || ldo < ncols || slots < 0 || ldx < k)
    return fail_moe(TF_ERR_ARG, "tf_moe_experts_prefill: null pointer or short rows");
  if (reinterpret_cast<uintptr_t>(x) % 16 || ldx % 8 || reinterpret_cast<uintptr_t>(sorted) % 16)
    return fail_moe(TF_ERR_ALIGN, "tf_moe_experts_prefill: rows must start on 16-byte boundaries");
  int* err = device_error_word();
  if (err == nullptr) return fail_moe(TF_ERR_STATE, "tf_moe_experts_prefill: tf_init has not been called for the current device");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  gather_rows_kernel<<<(pairs + 7) / 8, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, members, counts, slots, pairs, k,
                                                   static_cast<__nv_bfloat16*>(sorted));
  CUtensorMap map;
  if (int rc = encode_rows(&map, sorted, k, pairs, k, 128)) return rc;
  PrefillParams p = {};
  p.w = static_cast<const uint32_t*>(tiled);
  p.sb_stride = static_cast<int64_t>(k / gs) * unit_words(4, gs);
  p.N = n, p.K = k, p.M = pairs;
  p.out = out, p.ldo = ldo, p.out_f32 = out_f32;
  p.err = err;
  p.items = items, p.counts = counts, p.members = members;
  p.expert_stride = expert_stride;
  p.experts = experts;
  p.epi = epi, p.limit = limit;
  const int64_t tiles = static_cast<int64_t>((n + PF_COLS - 1) / PF_COLS) * max_items;   // upper bound: the plan says how many
  const int sms = sm_count();
  if (sms < 1) return fail_moe(TF_ERR_STATE, "tf_moe_experts_prefill: cannot read the SM count");
  dim3 grid(static_cast<unsigned>(tiles < sms ? tiles : sms));
  if (gs == 64) prefill_kernel<64, 128><<<grid, PF_THREADS, PfGeo<128>::SMEM, s>>>(map, p);
  else prefill_kernel<32, 128><<<grid, PF_THREADS, PfGeo<128>::SMEM, s>>>(map, p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_moe_experts_prefill");
}
