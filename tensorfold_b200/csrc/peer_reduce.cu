// Rank-ordered all-reduce of partial sums over peer memory (NVLink / NVSwitch), one launch a rank: the ranks' buffers are
// mapped into every process; the partials of all ranks are added in rank order in fp32 ((p0 + p1) + p2 ...), rounded
// once, and every rank ends with the same bits.  Generalises the two-rank rank0.float() + rank1.float() of
// families/qwen3_5/cuda/distributed.py:249-284 (an all-gather and an add there).  The forms:
//
//   flagged words (small partials)  a rank stores its partial into a slot of every other rank's buffer as 8-byte
//       {data, epoch} words (16-byte stores of two such words; each half carries its own flag), then polls the slots
//       of its own buffer until every word shows this call's epoch, and adds.  No barrier, no fence: one trip over the
//       links.  Slots alternate with the parity of the epoch: a slot is rewritten two calls later, which the writer
//       can only reach after this rank has sent its next partial, that is, after it has finished reading this one.
//   flagged words in two hops (four and eight ranks, partials from 64 KB)  the same words, but a rank sends every other
//       rank only that rank's 1/world share, adds the shares it receives and sends the finished share to every rank.
//   shares (large partials)  ranks tell one another that their partials are in place, a rank brings its 1/world share
//       of every partial into shared memory with bulk copies (plain peer loads where a share does not split into 4 KB
//       pieces), adds, stores the sum into every rank's result, and the ranks tell one another that they are done (all
//       shares have landed; nobody still reads this rank's partial).
//   all (testing, and totals that do not split)  as shares, but every rank reads every partial whole.
//
// Each rank's buffer starts with a page of 32-bit flags, 128 bytes apart: ready[r] and done[r] (how many reductions of
// the share forms rank r has announced / finished), the calls completed in the share forms and in the flagged form (a
// launch reads its epoch there at entry and the last block bumps it at exit, so launches replayed from a CUDA graph keep
// counting), and a count of the blocks of the running launch that have finished.  Every wait has a poll limit; a wait
// that runs out sets ERR_WAIT_PEER in the device error word, the kernel skips its remaining waits and returns.
//
// In the share forms all blocks of a launch must be resident at once (the last one to finish signals for all), and in
// the flagged forms threads wait for other ranks' threads: the grids are bounded by what an SM holds.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/tensorfold_b200.h"
#include "tf_ptx.cuh"

namespace tf {

int fail_moe(int code, const char* msg);
int cuda_fail_moe(cudaError_t e, const char* what);
int* device_error_word();

namespace {

constexpr int PEER_MAX = 8;
constexpr int PEER_THREADS = 512;              // share forms
constexpr int LL_THREADS = 256;                // flagged words
constexpr int FLAG_WORDS = 32;                 // flags sit 128 bytes apart
constexpr int FLAG_READY = 0, FLAG_DONE = PEER_MAX, FLAG_CALLS = 2 * PEER_MAX, FLAG_ARRIVE = 2 * PEER_MAX + 1,
              FLAG_LL_CALLS = 2 * PEER_MAX + 2, FLAG_LL_ARRIVE = 2 * PEER_MAX + 3, FLAG_GO = 2 * PEER_MAX + 4;
constexpr size_t FLAG_BYTES = 4096;
static_assert((FLAG_GO + 1) * FLAG_WORDS * 4 <= FLAG_BYTES, "the flags fit their page");
enum Mode : int {
  MODE_ALL = 0, MODE_SHARES = 1, MODE_FLAGGED = 2, MODE_FLAGGED_PUSH = 3, MODE_FLAGGED_PULL = 4,
  MODE_HOPS = 5, MODE_HOPS_SEND = 6, MODE_HOPS_MIDDLE = 7, MODE_HOPS_COLLECT = 8,     // flagged words in two hops
};

struct PeerArgs {
  char* buf[PEER_MAX];                         // every rank's buffer as this process sees it (buf[rank] is local)
  char* mine;                                  // buf[rank]
  int rank, world;
  size_t part_off, out_off;                    // byte offsets of the partial and of the result inside every buffer
  size_t ll_off, ll_slot;                      // flagged words: 2 * world slots of ll_slot bytes from ll_off
  int64_t total;                               // elements of the partial
  int parts_bf16, out_f32, mode;
  uint32_t polls;                              // limit of every wait
  int* err;
};

__device__ __forceinline__ uint32_t* flag(char* buf, int which) { return reinterpret_cast<uint32_t*>(buf) + which * FLAG_WORDS; }

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer16(void* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile16(void* p, const uint4& v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Waits until *p has reached `target` (counters only grow; the comparison survives their wrap).  (Polling with relaxed
// loads and one fence after the last measured slower than acquiring loads: 42 us against 22 us a call on two GPUs.)
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t target, uint32_t polls) {
  for (uint32_t i = 0; i < polls; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - target) >= 0) return true;
    __nanosleep(i < 64 ? 20 : 400);
  }
  return false;
}

// Eight consecutive elements of every rank's partial, summed in rank order.
template <int WORLD, bool BF16>
__device__ __forceinline__ void sum8(const PeerArgs& a, int64_t i, float (&acc)[8]) {
  if constexpr (BF16) {
    uint4 q[WORLD];
#pragma unroll
    for (int r = 0; r < WORLD; ++r) q[r] = ld_peer16(a.buf[r] + a.part_off + i * 2);
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {
      const uint32_t u[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(u[j] << 16), hi = __uint_as_float(u[j] & 0xFFFF0000u);
        acc[2 * j] = r == 0 ? lo : acc[2 * j] + lo;
        acc[2 * j + 1] = r == 0 ? hi : acc[2 * j + 1] + hi;
      }
    }
  } else {
    uint4 q[WORLD][2];
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {
      q[r][0] = ld_peer16(a.buf[r] + a.part_off + i * 4);
      q[r][1] = ld_peer16(a.buf[r] + a.part_off + i * 4 + 16);
    }
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {
      const uint32_t u[8] = {q[r][0].x, q[r][0].y, q[r][0].z, q[r][0].w, q[r][1].x, q[r][1].y, q[r][1].z, q[r][1].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = r == 0 ? __uint_as_float(u[j]) : acc[j] + __uint_as_float(u[j]);
    }
  }
}

// Stores eight results at element i of the result inside `buf`.
__device__ __forceinline__ void store8(const PeerArgs& a, char* buf, int64_t i, const float (&acc)[8]) {
  if (a.out_f32) {
    char* o = buf + a.out_off + i * 4;
    st_peer16(o, make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3])));
    st_peer16(o + 16, make_uint4(__float_as_uint(acc[4]), __float_as_uint(acc[5]), __float_as_uint(acc[6]), __float_as_uint(acc[7])));
  } else {
    uint32_t u[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 t = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      u[j] = *reinterpret_cast<const uint32_t*>(&t);
    }
    st_peer16(buf + a.out_off + i * 2, make_uint4(u[0], u[1], u[2], u[3]));
  }
}

// The two ends of a launch of the share forms (called by every thread of every block; `s_lost`, `s_last` and `s_buf` live in
// the block's shared memory).  shares_begin: this rank's partial was written by an earlier kernel of this stream: block 0
// announces it to every rank and waits for everyone's announcement, then lets the other blocks of this launch go
// through a flag in local memory (a few threads poll across the links instead of a few thousand).
template <int WORLD>
__device__ __forceinline__ void shares_begin(const PeerArgs& a, char* const* s_buf, uint32_t target, int& s_lost) {
  const int tid = threadIdx.x;
  char* mine = a.mine;
  if (blockIdx.x == 0) {
    if (tid < WORLD) {
      add_release_sys(flag(s_buf[tid], FLAG_READY + a.rank), 1);
      if (!wait_flag(flag(mine, FLAG_READY + tid), target, a.polls)) s_lost = 1;
    }
    __syncthreads();
    if (tid == 0) st_release_gpu(flag(mine, FLAG_GO), s_lost ? target | 0x80000000u : target);   // (top bit: the wait was lost)
  } else {
    if (tid == 0) {
      // block 0 always sets the flag, after its own (bounded) waits on the other ranks: this wait gets several times
      // their limit, so that it never gives up before block 0 has
      bool seen = false;
      for (uint64_t i = 0; i < 16ull * a.polls && !seen; ++i) {
        const uint32_t v = ld_acquire_gpu(flag(mine, FLAG_GO));
        seen = (v & 0x7FFFFFFFu) == target;
        if (seen && (v >> 31)) s_lost = 1;
        if (!seen) __nanosleep(i < 64 ? 20 : 200);
      }
      if (!seen) s_lost = 1;
    }
  }
  __syncthreads();
}

// shares_end: count the blocks in; the last one tells every rank that this rank has finished reading and writing, and
// stays until every rank has said so (all shares have landed here, nobody still reads this rank's partial): the launch
// ends with it.
template <int WORLD>
__device__ __forceinline__ void shares_end(const PeerArgs& a, char* const* s_buf, uint32_t target, bool lost, int& s_lost, int& s_last) {
  const int tid = threadIdx.x;
  char* mine = a.mine;
  __threadfence_system();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(flag(mine, FLAG_ARRIVE), 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (tid < WORLD) {
      add_release_sys(flag(s_buf[tid], FLAG_DONE + a.rank), 1);
      if (!lost && !wait_flag(flag(mine, FLAG_DONE + tid), target, a.polls)) s_lost = 1;
    }
    __syncthreads();
    if (tid == 0) {
      *flag(mine, FLAG_ARRIVE) = 0;
      *reinterpret_cast<volatile uint32_t*>(flag(mine, FLAG_CALLS)) = target;
      __threadfence();
    }
  }
  if (s_lost && tid == 0) atomicCAS(a.err, 0, ERR_WAIT_PEER);
}

template <int WORLD, bool BF16>
__global__ void __launch_bounds__(PEER_THREADS) peer_reduce_kernel(const PeerArgs a) {
  __shared__ uint32_t s_target;
  __shared__ int s_lost, s_last;
  __shared__ char* s_buf[WORLD];               // the buffers by a run-time index
  const int tid = threadIdx.x;
  char* mine = a.mine;
#pragma unroll
  for (int r = 0; r < WORLD; ++r)
    if (tid == r) s_buf[r] = a.buf[r];
  if (tid == 0) {
    s_target = *reinterpret_cast<volatile uint32_t*>(flag(mine, FLAG_CALLS)) + 1;
    s_lost = 0;
  }
  __syncthreads();
  const uint32_t target = s_target;
  shares_begin<WORLD>(a, s_buf, target, s_lost);
  const bool lost = s_lost != 0;

  if (!lost) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * PEER_THREADS * 8;
    const int64_t lane0 = (static_cast<int64_t>(blockIdx.x) * PEER_THREADS + tid) * 8;
    if (a.mode == MODE_SHARES) {               // this rank sums its share and hands it to every rank
      const int64_t share = a.total / WORLD, base = share * a.rank;
      for (int64_t i = lane0; i < share; i += step) {
        float acc[8];
        sum8<WORLD, BF16>(a, base + i, acc);
#pragma unroll
        for (int r = 0; r < WORLD; ++r) store8(a, a.buf[r], base + i, acc);
      }
    } else {                                   // every rank sums everything for itself
      for (int64_t i = lane0; i < a.total; i += step) {
        float acc[8];
        sum8<WORLD, BF16>(a, i, acc);
        store8(a, mine, i, acc);
      }
    }
  }
  shares_end<WORLD>(a, s_buf, target, lost, s_lost, s_last);
}

// The share form with bulk copies: a block brings 4 KB of every rank's partial into its shared memory with one bulk
// copy a rank (three such stages in flight), adds from there and stores the sums to every rank.  Plain loads over the
// links are bounded by the outstanding misses an SM may have (16-byte loads moved about 450 GB/s a direction on eight
// ranks); a bulk copy keeps whole kilobytes in flight per request.
constexpr int BULK_THREADS = 256, BULK_CHUNK = 4096, BULK_STAGES = 3;

template <int WORLD, bool BF16>
__global__ void __launch_bounds__(BULK_THREADS) peer_reduce_bulk_kernel(const PeerArgs a) {
  extern __shared__ __align__(128) uint8_t bulk_smem[];       // [stage][rank][4 KB], then a barrier a stage and the abort word
  __shared__ uint32_t s_target;
  __shared__ int s_lost, s_last;
  __shared__ char* s_buf[WORLD];
  const int tid = threadIdx.x, lane = tid & 31;
  char* mine = a.mine;
  const uint32_t base32 = smem_addr(bulk_smem);
  const uint32_t full32 = base32 + BULK_STAGES * WORLD * BULK_CHUNK, abort32 = full32 + 8 * BULK_STAGES;
#pragma unroll
  for (int r = 0; r < WORLD; ++r)
    if (tid == r) s_buf[r] = a.buf[r];
  if (tid == 0) {
    s_target = *reinterpret_cast<volatile uint32_t*>(flag(mine, FLAG_CALLS)) + 1;
    s_lost = 0;
    for (int i = 0; i < BULK_STAGES; ++i)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full32 + 8 * i), "r"(1) : "memory");
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort32), "r"(0) : "memory");
    mbar_fence_init();
  }
  __syncthreads();
  const uint32_t target = s_target;
  shares_begin<WORLD>(a, s_buf, target, s_lost);
  const bool lost = s_lost != 0;

  if (!lost) {
    constexpr int ESIZE = BF16 ? 2 : 4, VALUES = 16 / ESIZE;  // a thread's piece: 16 bytes of every rank's chunk
    const int64_t share_bytes = a.total / WORLD * ESIZE, chunks = share_bytes / BULK_CHUNK;
    const size_t in0 = a.part_off + static_cast<size_t>(a.rank) * share_bytes;
    const int n_mine = blockIdx.x < chunks ? static_cast<int>((chunks - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    auto issue = [&](int j) {                                 // thread 0: the block's j-th chunk, one bulk copy a rank
      const int st = j % BULK_STAGES;
      const size_t at = in0 + (static_cast<size_t>(blockIdx.x) + static_cast<size_t>(j) * gridDim.x) * BULK_CHUNK;
      mbar32_expect_tx(full32 + 8 * st, WORLD * BULK_CHUNK);
#pragma unroll
      for (int r = 0; r < WORLD; ++r) bulk_load32(base32 + (st * WORLD + r) * BULK_CHUNK, a.buf[r] + at, BULK_CHUNK, full32 + 8 * st);
    };
    if (tid == 0)
      for (int j = 0; j < BULK_STAGES && j < n_mine; ++j) issue(j);
    bool dead = false;
    for (int j = 0; j < n_mine; ++j) {
      const int st = j % BULK_STAGES;
      if (!dead && !mbar32_wait(full32 + 8 * st, (j / BULK_STAGES) & 1, abort32)) {
        dead = true;                                          // (the other warps see the abort word and give up as well)
        if (lane == 0) {
          asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort32), "r"(1) : "memory");
          s_lost = 1;
        }
      }
      if (!dead) {
        float acc[VALUES];
#pragma unroll
        for (int r = 0; r < WORLD; ++r) {
          const uint4 q = lds128(base32 + (st * WORLD + r) * BULK_CHUNK + tid * 16);
          const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if constexpr (BF16) {
              const float lo = __uint_as_float(u[e] << 16), hi = __uint_as_float(u[e] & 0xFFFF0000u);
              acc[2 * e] = r == 0 ? lo : acc[2 * e] + lo;
              acc[2 * e + 1] = r == 0 ? hi : acc[2 * e + 1] + hi;
            } else {
              acc[e] = r == 0 ? __uint_as_float(u[e]) : acc[e] + __uint_as_float(u[e]);
            }
          }
        }
        // element index of the piece inside the whole partial
        const int64_t i = (static_cast<int64_t>(a.rank) * share_bytes +
                           (static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(j) * gridDim.x) * BULK_CHUNK + tid * 16) / ESIZE;
        if (a.out_f32) {
#pragma unroll
          for (int r = 0; r < WORLD; ++r) {
            char* o = a.buf[r] + a.out_off + i * 4;
            st_peer16(o, make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3])));
            if constexpr (BF16)
              st_peer16(o + 16, make_uint4(__float_as_uint(acc[4]), __float_as_uint(acc[5]), __float_as_uint(acc[6]), __float_as_uint(acc[7])));
          }
        } else {
          uint32_t u[VALUES / 2];
#pragma unroll
          for (int e = 0; e < VALUES / 2; ++e) {
            const __nv_bfloat162 t = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
            u[e] = *reinterpret_cast<const uint32_t*>(&t);
          }
#pragma unroll
          for (int r = 0; r < WORLD; ++r) {
            char* o = a.buf[r] + a.out_off + i * 2;
            if constexpr (BF16) st_peer16(o, make_uint4(u[0], u[1], u[2], u[3]));
            else asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(o), "r"(u[0]), "r"(u[1]) : "memory");
          }
        }
      }
      __syncthreads();                                        // every thread has read the stage: it may be filled again
      if (tid == 0 && !dead && j + BULK_STAGES < n_mine) issue(j + BULK_STAGES);
    }
    if (dead)
      for (int i = 0; i < 64; ++i) __nanosleep(20000);        // copies in flight land before the shared memory is released
  }
  shares_end<WORLD>(a, s_buf, target, lost, s_lost, s_last);
}

// Flagged words.  A thread owns quads of four 4-byte words of the partial (four fp32 values, or eight bf16): it stores
// them into its slot on every other rank, then collects the same quad from every other rank's slot here.
template <int WORLD, bool BF16>
__global__ void __launch_bounds__(LL_THREADS) peer_reduce_flagged_kernel(const PeerArgs a) {
  __shared__ uint32_t s_epoch;
  const int tid = threadIdx.x;
  char* mine = a.mine;
  if (tid == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(flag(mine, FLAG_LL_CALLS)) + 1;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const bool push = a.mode != MODE_FLAGGED_PULL, pull = a.mode != MODE_FLAGGED_PUSH;
  const int64_t quads = (BF16 ? a.total / 2 : a.total) / 4;
  const size_t slots = a.ll_off + static_cast<size_t>(epoch & 1) * WORLD * a.ll_slot;
  bool lost = false;
  for (int64_t q = static_cast<int64_t>(blockIdx.x) * LL_THREADS + tid; q < quads; q += static_cast<int64_t>(gridDim.x) * LL_THREADS) {
    const uint4 v = *reinterpret_cast<const uint4*>(mine + a.part_off + q * 16);
    if (push) {
      const uint4 lo = make_uint4(v.x, epoch, v.y, epoch), hi = make_uint4(v.z, epoch, v.w, epoch);
#pragma unroll
      for (int r = 0; r < WORLD; ++r)
        if (r != a.rank) {
          char* dst = a.buf[r] + slots + a.rank * a.ll_slot + q * 32;
          st_volatile16(dst, lo);
          st_volatile16(dst + 16, hi);
        }
    }
    if (!pull || lost) continue;
    uint4 got[WORLD][2];
    bool ok = false;
    for (uint32_t i = 0; i < a.polls && !ok; ++i) {
      ok = true;
#pragma unroll
      for (int r = 0; r < WORLD; ++r)
        if (r != a.rank) {
          const char* src = mine + slots + r * a.ll_slot + q * 32;
          got[r][0] = ld_volatile16(src);
          got[r][1] = ld_volatile16(src + 16);
          ok &= got[r][0].y == epoch && got[r][0].w == epoch && got[r][1].y == epoch && got[r][1].w == epoch;
        }
      if (!ok && i >= 64) __nanosleep(i < 512 ? 50 : 500);
    }
    if (!ok) {
      lost = true;
      continue;
    }
    float acc[BF16 ? 8 : 4];
#pragma unroll
    for (int r = 0; r < WORLD; ++r) {
      const bool own = r == a.rank;
      const uint32_t w[4] = {own ? v.x : got[r][0].x, own ? v.y : got[r][0].z, own ? v.z : got[r][1].x, own ? v.w : got[r][1].z};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if constexpr (BF16) {
          const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
          acc[2 * j] = r == 0 ? lo : acc[2 * j] + lo;
          acc[2 * j + 1] = r == 0 ? hi : acc[2 * j + 1] + hi;
        } else {
          acc[j] = r == 0 ? __uint_as_float(w[j]) : acc[j] + __uint_as_float(w[j]);
        }
      }
    }
    constexpr int VALUES = BF16 ? 8 : 4;
    if (a.out_f32) {
      float4* o = reinterpret_cast<float4*>(mine + a.out_off + q * VALUES * 4);
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      if constexpr (BF16) o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      uint32_t u[VALUES / 2];
#pragma unroll
      for (int j = 0; j < VALUES / 2; ++j) {
        const __nv_bfloat162 t = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        u[j] = *reinterpret_cast<const uint32_t*>(&t);
      }
      if constexpr (BF16) *reinterpret_cast<uint4*>(mine + a.out_off + q * 16) = make_uint4(u[0], u[1], u[2], u[3]);
      else *reinterpret_cast<uint2*>(mine + a.out_off + q * 8) = make_uint2(u[0], u[1]);
    }
  }
  if (lost) atomicCAS(a.err, 0, ERR_WAIT_PEER);
  if (!pull) return;                           // the pushing half of a test leaves the epoch to the pulling half
  __syncthreads();
  if (tid == 0 && atomicAdd(flag(mine, FLAG_LL_ARRIVE), 1u) == gridDim.x - 1) {
    *flag(mine, FLAG_LL_ARRIVE) = 0;
    *reinterpret_cast<volatile uint32_t*>(flag(mine, FLAG_LL_CALLS)) = epoch;
    __threadfence();
  }
}

// Flagged words in two hops, for four and eight ranks: storing a whole partial into every rank's buffer costs
// (world - 1) x 2 x its bytes on the links; here a rank sends each OTHER rank only that rank's 1/world share (hop one),
// adds the shares it received to its own in rank order, rounds, and sends the finished share to every rank (hop two):
// about (1 + out bytes / partial bytes) x 2 x the partial's bytes a rank, five times less at eight ranks.  Same flags,
// epochs and parity as the one-hop form; the first ll_slot bytes of a parity's area hold hop one's slots (source rank r
// at r * ll_slot / world), the next 2 * ll_slot bytes hop two's (owner s at s * 2 * ll_slot / world).
template <int WORLD, bool BF16>
__global__ void __launch_bounds__(LL_THREADS) peer_reduce_hops_kernel(const PeerArgs a) {
  __shared__ uint32_t s_epoch;
  __shared__ char* s_buf[WORLD];
  const int tid = threadIdx.x;
  char* mine = a.mine;
#pragma unroll
  for (int r = 0; r < WORLD; ++r)
    if (tid == r) s_buf[r] = a.buf[r];
  if (tid == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(flag(mine, FLAG_LL_CALLS)) + 1;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const bool send = a.mode == MODE_HOPS || a.mode == MODE_HOPS_SEND, middle = a.mode == MODE_HOPS || a.mode == MODE_HOPS_MIDDLE,
             collect = a.mode == MODE_HOPS || a.mode == MODE_HOPS_COLLECT;
  constexpr int VALUES = BF16 ? 8 : 4;                       // values a quad of four 4-byte words
  const int64_t quads = (BF16 ? a.total / 2 : a.total) / 4, per = quads / WORLD;
  const int vecs = (a.out_f32 ? VALUES : VALUES / 2) / 2;    // 16-byte vectors (two result words and their flags) a quad
  const size_t area = a.ll_off + static_cast<size_t>(epoch & 1) * WORLD * a.ll_slot;
  const size_t a_stride = a.ll_slot / WORLD, b_base = area + a.ll_slot, b_stride = 2 * a.ll_slot / WORLD;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * LL_THREADS + tid, tstep = static_cast<int64_t>(gridDim.x) * LL_THREADS;
  bool lost = false;

  if (send) {                                                // hop one: every quad another rank owns goes to that rank
    for (int64_t q = t0; q < quads; q += tstep) {
      const int owner = static_cast<int>(q / per);
      if (owner == a.rank) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(mine + a.part_off + q * 16);
      char* dst = s_buf[owner] + area + a.rank * a_stride + (q - owner * per) * 32;
      st_volatile16(dst, make_uint4(v.x, epoch, v.y, epoch));
      st_volatile16(dst + 16, make_uint4(v.z, epoch, v.w, epoch));
    }
  }
  if (middle) {                                              // this rank's share: collect, add in rank order, round, hand on
    for (int64_t ql = t0; ql < per; ql += tstep) {
      const int64_t q = a.rank * per + ql;
      const uint4 v = *reinterpret_cast<const uint4*>(mine + a.part_off + q * 16);
      uint4 got[WORLD][2];
      bool ok = false;
      for (uint32_t i = 0; i < a.polls && !ok; ++i) {
        ok = true;
#pragma unroll
        for (int r = 0; r < WORLD; ++r)
          if (r != a.rank) {
            const char* src = mine + area + r * a_stride + ql * 32;
            got[r][0] = ld_volatile16(src);
            got[r][1] = ld_volatile16(src + 16);
            ok &= got[r][0].y == epoch && got[r][0].w == epoch && got[r][1].y == epoch && got[r][1].w == epoch;
          }
        if (!ok && i >= 64) __nanosleep(i < 512 ? 50 : 500);
      }
      if (!ok) {
        lost = true;
        continue;
      }
      float acc[VALUES];
#pragma unroll
      for (int r = 0; r < WORLD; ++r) {
        const bool own = r == a.rank;
        const uint32_t w[4] = {own ? v.x : got[r][0].x, own ? v.y : got[r][0].z, own ? v.z : got[r][1].x, own ? v.w : got[r][1].z};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if constexpr (BF16) {
            const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
            acc[2 * j] = r == 0 ? lo : acc[2 * j] + lo;
            acc[2 * j + 1] = r == 0 ? hi : acc[2 * j + 1] + hi;
          } else {
            acc[j] = r == 0 ? __uint_as_float(w[j]) : acc[j] + __uint_as_float(w[j]);
          }
        }
      }
      uint32_t word[VALUES];                                 // the quad of the result as it lies in memory
      if (a.out_f32) {
#pragma unroll
        for (int j = 0; j < VALUES; ++j) word[j] = __float_as_uint(acc[j]);
      } else {
#pragma unroll
        for (int j = 0; j < VALUES / 2; ++j) {
          const __nv_bfloat162 t = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
          word[j] = *reinterpret_cast<const uint32_t*>(&t);
        }
      }
      uint32_t* o = reinterpret_cast<uint32_t*>(mine + a.out_off) + q * (2 * vecs);
#pragma unroll
      for (int j = 0; j < VALUES; ++j)
        if (j < 2 * vecs) o[j] = word[j];
#pragma unroll
      for (int r = 0; r < WORLD; ++r)
        if (r != a.rank) {
          char* dst = s_buf[r] + b_base + a.rank * b_stride + ql * (vecs * 16);
#pragma unroll
          for (int j = 0; j < VALUES / 2; ++j)
            if (j < vecs) st_volatile16(dst + 16 * j, make_uint4(word[2 * j], epoch, word[2 * j + 1], epoch));
        }
    }
  }
  if (collect) {                                             // hop two's other end: the shares the other ranks finished
    for (int64_t q = t0; q < quads; q += tstep) {
      const int owner = static_cast<int>(q / per);
      if (owner == a.rank) continue;
      const char* src = mine + b_base + owner * b_stride + (q - owner * per) * (vecs * 16);
      uint4 got[VALUES / 2];
      bool ok = false;
      for (uint32_t i = 0; i < a.polls && !ok; ++i) {
        ok = true;
#pragma unroll
        for (int j = 0; j < VALUES / 2; ++j)
          if (j < vecs) {
            got[j] = ld_volatile16(src + 16 * j);
            ok &= got[j].y == epoch && got[j].w == epoch;
          }
        if (!ok && i >= 64) __nanosleep(i < 512 ? 50 : 500);
      }
      if (!ok) {
        lost = true;
        continue;
      }
      uint32_t* o = reinterpret_cast<uint32_t*>(mine + a.out_off) + q * (2 * vecs);
#pragma unroll
      for (int j = 0; j < VALUES / 2; ++j)
        if (j < vecs) o[2 * j] = got[j].x, o[2 * j + 1] = got[j].z;
    }
  }
  if (lost) atomicCAS(a.err, 0, ERR_WAIT_PEER);
  if (!collect) return;                                      // the halves of a test leave the epoch to the last one
  __syncthreads();
  if (tid == 0 && atomicAdd(flag(mine, FLAG_LL_ARRIVE), 1u) == gridDim.x - 1) {
    *flag(mine, FLAG_LL_ARRIVE) = 0;
    *reinterpret_cast<volatile uint32_t*>(flag(mine, FLAG_LL_CALLS)) = epoch;
    __threadfence();
  }
}

int g_peer_plain = 0;                            // 1: the share form with plain loads only (tuning, tests)

struct DeviceFacts {
  int sms = 0, per_sm[3][2] = {};              // resident blocks of the share kernel by world (2, 4, 8) and partial type
};

template <int WORLD>
cudaError_t launch_world(const PeerArgs& a, int grid_cap, cudaStream_t s) {
  static DeviceFacts facts[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  DeviceFacts& f = facts[dev];
  if (!f.sms && (e = cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  if (a.mode >= MODE_FLAGGED) {
    const int64_t quads = (a.parts_bf16 ? a.total / 2 : a.total) / 4;
    int64_t grid = (quads + LL_THREADS - 1) / LL_THREADS;
    if (grid > 2 * f.sms) grid = 2 * f.sms;                    // every block resident: threads wait for other ranks' threads
    if (grid_cap > 0 && grid > grid_cap) grid = grid_cap;
    if (a.mode >= MODE_HOPS) {
      if constexpr (WORLD >= 4) {
        if (a.parts_bf16) peer_reduce_hops_kernel<WORLD, true><<<static_cast<unsigned>(grid), LL_THREADS, 0, s>>>(a);
        else peer_reduce_hops_kernel<WORLD, false><<<static_cast<unsigned>(grid), LL_THREADS, 0, s>>>(a);
        return cudaGetLastError();
      } else {
        return cudaErrorInvalidValue;
      }
    }
    if (a.parts_bf16) peer_reduce_flagged_kernel<WORLD, true><<<static_cast<unsigned>(grid), LL_THREADS, 0, s>>>(a);
    else peer_reduce_flagged_kernel<WORLD, false><<<static_cast<unsigned>(grid), LL_THREADS, 0, s>>>(a);
    return cudaGetLastError();
  }
  const int64_t share_bytes = a.total / WORLD * (a.parts_bf16 ? 2 : 4);
  if (a.mode == MODE_SHARES && share_bytes % BULK_CHUNK == 0 && !g_peer_plain) {
    constexpr int SMEM = BULK_STAGES * WORLD * BULK_CHUNK + 8 * BULK_STAGES + 16;
    auto go = [&](auto kernel) -> cudaError_t {
      static bool configured[64][2] = {};                      // (both kernels have one pointer type: index by the partial's type)
      if (!configured[dev][a.parts_bf16 ? 1 : 0]) {
        cudaError_t q = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (q != cudaSuccess) return q;
        configured[dev][a.parts_bf16 ? 1 : 0] = true;
      }
      // every block resident (the last one to finish signals for all): two blocks of 96 KB an SM at most
      int64_t grid = share_bytes / BULK_CHUNK;
      const int64_t resident = static_cast<int64_t>(SMEM > 100 * 1024 ? 1 : 2) * f.sms;
      if (grid > resident) grid = resident;
      if (grid_cap > 0 && grid > grid_cap) grid = grid_cap;
      kernel<<<static_cast<unsigned>(grid), BULK_THREADS, SMEM, s>>>(a);
      return cudaGetLastError();
    };
    return a.parts_bf16 ? go(peer_reduce_bulk_kernel<WORLD, true>) : go(peer_reduce_bulk_kernel<WORLD, false>);
  }
  auto run = [&](auto kernel) -> cudaError_t {
    int& per_sm = f.per_sm[WORLD == 2 ? 0 : WORLD == 4 ? 1 : 2][a.parts_bf16 ? 1 : 0];
    if (!per_sm) {
      cudaError_t q = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, PEER_THREADS, 0);
      if (q != cudaSuccess) return q;
      if (per_sm < 1) per_sm = 1;
    }
    const int64_t work = a.mode == MODE_SHARES ? a.total / a.world : a.total;
    int64_t grid = (work / 8 + PEER_THREADS - 1) / PEER_THREADS;
    // a thread that runs several pieces has the loads of one piece in flight while the stores of the piece before are
    // still on their way: both directions of the links work at once (one block an SM: measured on eight ranks)
    const int64_t resident = static_cast<int64_t>(a.mode == MODE_SHARES ? 1 : per_sm) * f.sms;
    if (grid > resident) grid = resident;
    if (grid_cap > 0 && grid > grid_cap) grid = grid_cap;
    if (grid < 1) grid = 1;
    kernel<<<static_cast<unsigned>(grid), PEER_THREADS, 0, s>>>(a);
    return cudaGetLastError();
  };
  return a.parts_bf16 ? run(peer_reduce_kernel<WORLD, true>) : run(peer_reduce_kernel<WORLD, false>);
}

}  // namespace

void peer_reduce_plain(int on) { g_peer_plain = on; }   // tf_tune("peer_plain", v)

}  // namespace tf

using namespace tf;

extern "C" {

size_t tf_peer_flag_bytes(void) { return FLAG_BYTES; }

int tf_peer_alloc(size_t bytes, void** ptr) {
  if (!ptr || bytes < FLAG_BYTES) return fail_moe(TF_ERR_ARG, "tf_peer_alloc: a buffer holds its page of flags at least");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return cuda_fail_moe(e, "tf_peer_alloc");
  if ((e = cudaMemset(p, 0, bytes)) != cudaSuccess) {
    cudaFree(p);
    return cuda_fail_moe(e, "tf_peer_alloc: clearing");
  }
  *ptr = p;
  return TF_OK;
}

int tf_peer_free(void* ptr) {
  const cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_peer_free");
}

int tf_peer_export(void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "an exported handle is 64 bytes");
  if (!ptr || !handle64) return fail_moe(TF_ERR_ARG, "tf_peer_export: null argument");
  const cudaError_t e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), ptr);
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_peer_export");
}

int tf_peer_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return fail_moe(TF_ERR_ARG, "tf_peer_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  const cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_peer_open");
}

int tf_peer_close(void* ptr) {
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_peer_close");
}

int tf_peer_reduce(void* const* bufs, int rank, int world, size_t part_off, size_t out_off, int64_t total, int parts_bf16,
                   int out_f32, int mode, size_t ll_off, size_t ll_slot, unsigned polls, int grid_cap, void* stream) {
  if (!bufs || (world != 2 && world != 4 && world != 8) || rank < 0 || rank >= world || total < 8 || mode < MODE_ALL ||
      mode > MODE_HOPS_COLLECT)
    return fail_moe(TF_ERR_ARG, "tf_peer_reduce: 2, 4 or 8 ranks, at least eight elements, a form 0..8");
  if (total % (mode == MODE_SHARES ? 8 * world : 8)) return fail_moe(TF_ERR_ARG, "tf_peer_reduce: the elements split into pieces of eight (a rank)");
  if (part_off < FLAG_BYTES || out_off < FLAG_BYTES || part_off % 16 || out_off % 16)
    return fail_moe(TF_ERR_ALIGN, "tf_peer_reduce: offsets past the flags, 16-byte aligned");
  const size_t part_bytes = static_cast<size_t>(total) * (parts_bf16 ? 2 : 4), out_bytes = static_cast<size_t>(total) * (out_f32 ? 4 : 2);
  if ((part_off < out_off ? part_off + part_bytes > out_off : out_off + out_bytes > part_off))
    return fail_moe(TF_ERR_ARG, "tf_peer_reduce: the partial and the result overlap");
  if (mode >= MODE_FLAGGED) {
    const size_t top = part_off > out_off ? part_off + part_bytes : out_off + out_bytes;
    if (ll_off % 16 || ll_slot % 16 || ll_off < top || ll_slot < 2 * part_bytes)
      return fail_moe(TF_ERR_ARG, "tf_peer_reduce: the slots lie past partial and result and hold twice the partial each");
  }
  if (mode >= MODE_HOPS) {
    if (world < 4 || total % (8 * world) || ll_slot % (16 * world))
      return fail_moe(TF_ERR_ARG, "tf_peer_reduce: two hops take 4 or 8 ranks, elements and slots that split evenly over them");
  }
  int* err = device_error_word();
  if (!err) return fail_moe(TF_ERR_STATE, "tf_peer_reduce: tf_init has not run for the current device");
  PeerArgs a = {};
  for (int r = 0; r < world; ++r) {
    if (!bufs[r] || reinterpret_cast<uintptr_t>(bufs[r]) % 256) return fail_moe(TF_ERR_ALIGN, "tf_peer_reduce: a buffer is null or not 256-byte aligned");
    a.buf[r] = static_cast<char*>(bufs[r]);
  }
  a.mine = a.buf[rank];
  a.rank = rank, a.world = world, a.part_off = part_off, a.out_off = out_off, a.ll_off = ll_off, a.ll_slot = ll_slot, a.total = total;
  a.parts_bf16 = parts_bf16, a.out_f32 = out_f32, a.mode = mode, a.polls = polls ? polls : (1u << 23), a.err = err;
  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  const cudaError_t e = world == 2 ? launch_world<2>(a, grid_cap, s) : world == 4 ? launch_world<4>(a, grid_cap, s) : launch_world<8>(a, grid_cap, s);
  return e == cudaSuccess ? TF_OK : cuda_fail_moe(e, "tf_peer_reduce");
}

}  // extern "C"
