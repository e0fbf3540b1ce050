// Prefill matmul on the 5th-generation tensor cores: out[m, n] = sum_k x[m, k] * bf16(q[n, k] * s + b).
//
// Arithmetic contract (the reference's prefill form, cuda/kernels/qmm_prefill.cu:1,115-118): every weight is rounded once
// to bf16, w = bf16(fma(q, s, b)) with q exact, then ONE fp32 accumulation chain runs over all of K in 16-input steps
// (tcgen05.mma, accumulator in tensor memory).  Any chunking of the rows gives the same bits; they are not the decode
// kernel's bits (that one keeps the affine terms in fp32).
//
// Block tile = 128 output columns x 256 rows of x, "swap-AB": the dequantised weights are the MMA's A operand (M = 128),
// the rows of x its B operand (N = 256), so every dequantised weight feeds 256 rows.  Two rings decouple the latencies:
// packed units arrive from HBM (about 2000 cycles away) by bulk copies into a ring of small slots; a stage of the main
// ring holds the dequantised A tile and the x tile (a 2-D tensor-map copy with the 128-byte swizzle) of 64 inputs
// behind ONE full barrier and ONE empty barrier, because every barrier operation of the MMA-issuing thread costs about
// as much as an MMA issue and the tensor pipe idles while that thread does anything else.  Roles: warp 0 loads x,
// warp 1 owns tensor memory and issues the MMAs, warp 2 loads packed units, warps 4-19 are two groups of eight
// conversion warps that take alternate stages (a stage's conversion has a long dependent chain, so two stages are
// always in conversion) and afterwards all sixteen drain the accumulator to global memory.
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
constexpr int PF_THREADS = 640;    // 20 warps: x loads, MMA, unit loads, (idle), 2 x 8 conversion
constexpr int PF_CONV0 = 4;        // first conversion warp (a multiple of 4: tensor-memory lane groups go by warp % 4)
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
  static_assert((2 * NS + 2 * PF_NW + 1) * 8 + 16 <= PF_BAR_BYTES, "barriers fit");
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

#ifdef PF_TRACE
// debugging aid (compiled out by default): block (0, 0)'s clock at each stage's events
__device__ long long g_pf_trace[8 * 512];
#define PF_MARK(ev, i) \
  do { if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && (i) < 512) g_pf_trace[(ev) * 512 + (i)] = clock64(); } while (0)
#else
#define PF_MARK(ev, i) do { } while (0)
#endif

template <int GS, int ROWS>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_kernel(const __grid_constant__ CUtensorMap tmx, const PrefillParams p) {
  using Geo = PfGeo<ROWS>;
  constexpr int PF_ROWS = ROWS, PF_B_BYTES = Geo::B_BYTES, NS = Geo::NS;
  constexpr uint32_t PF_TMEM_COLS = ROWS;
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
  uint64_t* acc_full = w_empty + PF_NW;             // every MMA of the tile is done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sb = blockIdx.x;
  const int nstages = (p.K + PF_STAGE_K - 1) / PF_STAGE_K;
  const int total_units = p.K / GS;
  const bool grouped = p.items != nullptr;
  int m0 = blockIdx.y * PF_ROWS, rows_here, first = 0;
  const uint32_t* wroot = p.w;
  if (grouped) {
    if (static_cast<int>(blockIdx.y) >= p.counts[0]) return;               // before any barrier or tensor-memory use
    const int* item = p.items + 3 * blockIdx.y;
    wroot += static_cast<int64_t>(item[0]) * p.expert_stride;
    first = item[1];
    rows_here = min(PF_ROWS, item[2]);
    m0 = first;                                                             // row of the member-ordered input
  } else {
    rows_here = min(PF_ROWS, p.M - m0);
  }

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
    mbar_init(acc_full, 1);
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
    for (int i = 0; i < nstages && ok; ++i) {
      const int s = i % NS;
      if (i >= NS) {
        ok = mbar_wait(empty + s, (i / NS - 1) & 1, abort_flag);
        if (!ok) {
          give_up(ERR_WAIT_EMPTY);
          break;
        }
      }
      PF_MARK(0, i);
      if (lane == 0) {
#ifdef PF_DBG_NOX
        mbar_arrive(full + s);
#else
        mbar_expect_tx(full + s, PF_B_BYTES);
        tma_load_2d(b_tile(s), &tmx, i * PF_STAGE_K, m0, full + s);
#endif
      }
      __syncwarp();
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ packed units (HBM -> shared, bulk copies)
    const uint32_t* wsb = wroot + static_cast<int64_t>(sb) * p.sb_stride;
    bool ok = true;
    for (int i = 0; i < nstages && ok; ++i) {
      const int s = i % PF_NW;
      if (i >= PF_NW) {
        ok = mbar_wait(w_empty + s, (i / PF_NW - 1) & 1, abort_flag);
        if (!ok) {
          give_up(ERR_WAIT_EMPTY);
          break;
        }
      }
      PF_MARK(1, i);
      if (lane == 0) {
        const int units_here = min(UNITS, total_units - i * UNITS);
        mbar_expect_tx(w_full + s, units_here * UNITW * 4);
        bulk_load(w_slot(s), wsb + static_cast<int64_t>(i) * UNITS * UNITW, units_here * UNITW * 4, w_full + s);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue (one thread)
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((PF_ROWS >> 3) << 17) | ((PF_COLS >> 4) << 24);
    // The tensor pipe's queue is short and every instruction of this warp between two MMA issues is dead time for
    // it, so the loop is unrolled over the ring (descriptors precomputed, no index arithmetic) and the next stage's
    // full barrier is tested between this stage's MMAs, while earlier ones are still executing.
    const uint32_t leader = lane == 0 ? 1u : 0u;
    uint64_t adesc[NS], bdesc[NS];
#pragma unroll
    for (int st = 0; st < NS; ++st) {
      adesc[st] = umma_desc(smem_addr(a_tile(st)));
      bdesc[st] = umma_desc(smem_addr(b_tile(st)));
    }
    bool ok = mbar_wait(full, 0, abort_flag);
    if (!ok) give_up(ERR_WAIT_FULL);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t phase = 0;                                          // parity of the full barriers of this pass over the ring
    for (int base = 0; base < nstages && ok; base += NS, phase ^= 1u) {
#pragma unroll
      for (int st = 0; st < NS; ++st) {
        const int i = base + st;
        if (i >= nstages || !ok) break;
        const int nx = (st + 1) % NS;
        const uint32_t nx_phase = st + 1 == NS ? phase ^ 1u : phase;
        const bool more = i + 1 < nstages;
        bool next_ready = false;
        PF_MARK(4, i);
#ifndef PF_DBG_NOMMA
        umma_bf16(tmem_base, adesc[st], bdesc[st], IDESC, i > 0 ? 1u : 0u, leader);
        umma_bf16(tmem_base, adesc[st] + 2, bdesc[st] + 2, IDESC, 1u, leader);       // + 32 bytes a k16 step
        umma_bf16(tmem_base, adesc[st] + 4, bdesc[st] + 4, IDESC, 1u, leader);
        if (more) {
          next_ready = mbar_test(full + nx, nx_phase);
          if (next_ready) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        umma_bf16(tmem_base, adesc[st] + 6, bdesc[st] + 6, IDESC, 1u, leader);
#else
        if (more) next_ready = mbar_test(full + nx, nx_phase);
#endif
        PF_MARK(6, i);
        umma_commit(empty + st, leader);
        if (!more) umma_commit(acc_full, leader);
        PF_MARK(5, i);
        if (more && !next_ready) {
          ok = mbar_wait(full + nx, nx_phase, abort_flag);
          if (!ok) give_up(ERR_WAIT_FULL);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
      }
    }
  } else if (warp >= PF_CONV0) {
    // ------------------------------------------------------------------ conversion: packed codes -> swizzled bf16 A tile
    const int cw = warp - PF_CONV0, group = cw >> 3, dw = cw & 7, tp = dw & 3, h = dw >> 2, g = lane >> 2;
    const __nv_bfloat162 k128 = __floats2bfloat162_rn(128.f, 128.f);
    uint32_t row_off[4];                                        // this lane's row segment of each 16-input step of a stage
#pragma unroll
    for (int q = 0; q < 4; ++q)
      row_off[q] = (32 * tp + 16 * h + 8 * ((lane >> 3) & 1) + (lane & 7)) * 128 + (((2 * q + (lane >> 4)) ^ (lane & 7)) << 4);
    bool ok = true;
    for (int i = group; i < nstages && ok; i += 2) {
      const int sw = i % PF_NW, st = i % NS;
      ok = mbar_wait(w_full + sw, (i / PF_NW) & 1, abort_flag);
      if (ok && i >= NS) ok = mbar_wait(empty + st, (i / NS - 1) & 1, abort_flag);
      if (!ok) {
        give_up(ERR_WAIT_FULL);
        break;
      }
      if (cw == 0 || cw == 8) PF_MARK(2, i);
      const uint32_t* wst = reinterpret_cast<const uint32_t*>(w_slot(sw));
      const uint32_t at = smem_addr(a_tile(st));
      const int units_here = min(UNITS, total_units - i * UNITS);
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
          const uint2 sbw = *reinterpret_cast<const uint2*>(unit + TILE_PAIRS * 32 * WPL + tp * 32 + g * 4 + h * 2);
          const uint32_t sbv[2] = {sbw.x, sbw.y};                  // columns c0 and c0 + 8
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint32_t s2 = __byte_perm(sbv[r], 0u, 0x1010), b2 = __byte_perm(sbv[r], 0u, 0x3232);
            sc[r] = *reinterpret_cast<const __nv_bfloat162*>(&s2);
            bi[r] = *reinterpret_cast<const __nv_bfloat162*>(&b2);
          }
        }
#ifndef PF_DBG_NOCONV
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
#endif
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(full + st);
        mbar_arrive(w_empty + sw);                               // the slot's words are in registers or already used
      }
      if (cw == 0 || cw == 8) PF_MARK(3, i);
    }

    // ------------------------------------------------------------------ epilogue: tensor memory -> global
    const bool done = mbar_wait(acc_full, 0, abort_flag);
    if (!done) give_up(ERR_WAIT_FULL);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (done && *abort_flag == 0) {
      const int lg = warp & 3, part = cw >> 2;                   // this warp may touch TMEM lanes [32 lg, 32 lg + 32)
      const int n = sb * PF_COLS + lg * 32 + lane;               // the weight column this thread's lane holds
      constexpr int CHUNKS = PF_ROWS / 128;                      // 32-row chunks of this warp's quarter of the rows
#pragma unroll 1
      for (int chunk = 0; chunk < CHUNKS; ++chunk) {
        uint32_t r[32];
        const int col0 = part * (PF_ROWS / 4) + chunk * 32;
        tmem_load32(tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + col0, r);
        if (p.epi == 2) {
          // lanes 0-15 hold gate columns, lanes 16-31 the up columns of the same 16 outputs
          const int nout = sb * (PF_COLS / 2) + lg * 16 + lane;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float up = __shfl_down_sync(0xFFFFFFFFu, __uint_as_float(r[j]), 16);
            const int rr = col0 + j;
            if (lane < 16 && rr < rows_here && nout < p.N / 2) {
              const int64_t m = grouped ? p.members[first + rr] : m0 + rr;
              reinterpret_cast<__nv_bfloat16*>(p.out)[m * p.ldo + nout] =
                  __float2bfloat16_rn(pf_swiglu(__uint_as_float(r[j]), up, p.limit));
            }
          }
        } else if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int rr = col0 + j;
            if (rr < rows_here) {
              const int64_t m = grouped ? p.members[first + rr] : m0 + rr;
              float v = __uint_as_float(r[j]);
              if (p.epi == 1) {
                v = fmaxf(pf_bf16r(v), 0.f);
                v = v * v;
              }
              if (p.out_f32) reinterpret_cast<float*>(p.out)[m * p.ldo + n] = v;
              else reinterpret_cast<__nv_bfloat16*>(p.out)[m * p.ldo + n] = __float2bfloat16_rn(v);
            }
          }
        }
      }
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

#ifdef PF_TRACE
extern "C" int tf_debug_pf_trace(long long* host) {
  return cudaMemcpyFromSymbol(host, g_pf_trace, sizeof(g_pf_trace)) == cudaSuccess ? 0 : 1;
}
#endif

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
  dim3 grid((n + PF_COLS - 1) / PF_COLS, (m + 255) / 256);
  if (grid.y > 65535) return fail_moe(TF_ERR_ARG, "tf_qmm_prefill: too many rows");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (gs == 64) prefill_kernel<64, 256><<<grid, PF_THREADS, PfGeo<256>::SMEM, s>>>(map, p);
  else prefill_kernel<32, 256><<<grid, PF_THREADS, PfGeo<256>::SMEM, s>>>(map, p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_qmm_prefill");
}

extern "C" int tf_moe_experts_prefill(const void* x, int64_t ldx, int slots, const void* tiled, int64_t expert_stride, int n,
                                      int k, int gs, const int* items, const int* counts, const int* members, int pairs,
                                      int max_items, void* sorted, void* out, int64_t ldo, int out_f32, int epi, float limit,
                                      void* stream) {
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
  p.epi = epi, p.limit = limit;
  dim3 grid((n + PF_COLS - 1) / PF_COLS, max_items);
  if (gs == 64) prefill_kernel<64, 128><<<grid, PF_THREADS, PfGeo<128>::SMEM, s>>>(map, p);
  else prefill_kernel<32, 128><<<grid, PF_THREADS, PfGeo<128>::SMEM, s>>>(map, p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_moe_experts_prefill");
}
