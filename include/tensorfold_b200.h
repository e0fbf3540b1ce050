/* C ABI of libtensorfold_b200.so: the B200 (sm_100a) kernels behind TensorFold's quantized-projection entry points.
 *
 * The reference has no C ABI for this path: its boundary is a set of pybind11 functions taking torch tensors, built at
 * run time by torch.utils.cpp_extension (src/tensorfold/cuda/build.py:28-44).  Each function below names the reference
 * interface it stands in for (paths inside the reference project).  Conventions:
 *
 *   - every pointer is a DEVICE pointer unless its comment says "host";
 *   - `stream` is a cudaStream_t passed as void* (torch.cuda.current_stream().cuda_stream); nothing here synchronises;
 *   - the caller owns every buffer; no function allocates device memory;
 *   - the return value is a status: 0 = OK, TF_ERR_* < 0 for a refused argument (nothing was launched),
 *     > 0 = a cudaError_t from the launch.  tf_last_error() gives the text for the calling thread;
 *   - call tf_init(device) once per device before the first launch and before any CUDA-graph capture: it sets the
 *     kernels' shared-memory attributes and resolves the device's error word.
 */
#ifndef TENSORFOLD_B200_H
#define TENSORFOLD_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TF_OK 0
#define TF_ERR_ARG (-1)        /* bad shape, size or flag */
#define TF_ERR_ALIGN (-2)      /* pointer or stride not aligned as documented */
#define TF_ERR_UNSUPPORTED (-3)
#define TF_ERR_STATE (-4)      /* tf_init not called for the current device */

/* Library version (major * 10000 + minor * 100 + patch) and the architecture it was built for ("sm_100a"). */
int tf_version(void);
const char* tf_arch(void);
const char* tf_last_error(void);

/* Per-device set-up; replaces the lazy `static bool configured` + cudaFuncSetAttribute of
 * cuda/kernels/qmm.cu:251-255.  Idempotent. */
int tf_init(int device);

/* Reads and clears the device error word that kernels set when one of their bounded waits gave up (0 = none; 1 a stage
 * never arrived, 2 a stage was never released, 3 group sums never came, 4 a peer GPU never signalled, 5 a plan item
 * named an expert outside the table).  Synchronises `stream`.  host: *code. */
int tf_device_error(int device, void* stream, int* code);

/* Launches a wait that nothing will satisfy, with a limit of `polls` polls (1 to 4096, about a microsecond each): the
 * kernel gives up, returns, and tf_device_error then reports 1 (a stage never arrived).  This is how a host checks, on a
 * healthy GPU and without faulting anything, that a lost copy would come back as an error code and leave the context
 * usable.  No counterpart in the reference, whose kernels wait without a limit. */
int tf_selftest_lost_wait(int polls, void* stream);

/* Performance knobs that never change a result bit.  key "qmm_lanes": 128-column super-blocks a thread block streams side
 * by side (1, 2 or 4; 0 = default); "stream_lanes": the same for tf_qmm_set's persistent kernel; "stream_blocks": blocks
 * of that kernel an SM may hold (0 = as many as fit); "grouped_tiled": 1 runs tf_moe_experts through the tiled kernel
 * (one thread block a plan item and column block) instead of the persistent kernel's grouped form; "peer_plain": 1 keeps
 * tf_peer_reduce's share form on plain loads (no bulk copies into shared memory).  No counterpart
 * in the reference. */
int tf_tune(const char* key, int value);

/* ---- shape-only planning (host functions) -------------------------------------------------------------------- */

/* K slices of an (n, k) weight: cuda/kernels/qmm.py:105-111 (split_k). */
int tf_split_k(int n, int k, int gs, int target);
/* Row tile for m rows, 16/32/64, or TF_ERR_ARG for m < 1: cuda/kernels/qmm.py:114-119 (bucket). */
int tf_bucket(int m);
/* int32 words of the tiled tensor of an (n, k) weight: ceil(n / 128) * (k / gs) * (4 * gs * bits + 128). */
int64_t tf_tiled_words(int n, int k, int bits, int gs);
/* int32 words of one (128 columns, one group) unit. */
int tf_unit_words(int bits, int gs);

/* ---- load-time repack -------------------------------------------------------------------------------------- */

/* MLX rows -> tiled units.  words: [n, k * bits / 32] int32; scales, biases: [n, k / gs] bf16; tiled: tf_tiled_words.
 * Replaces the torch-indexing repack of cuda/kernels/qmm.py:55-82 (pack). */
int tf_pack(const void* words, const void* scales, const void* biases, int n, int k, int bits, int gs, void* tiled,
            void* stream);
/* Two projections of the same input packed as one weight of 2 * n_each rows that interleaves 16 rows of the first
 * (gate) with 16 rows of the second (up), so one matmul tile pair holds both halves of a SwiGLU output.  n_each % 16 == 0.
 * tiled: tf_tiled_words(2 * n_each, k, bits, gs).  Replaces the M = 2 (gate, up) interleave of cuda/experts.py:84-92 and
 * cuda/experts_pack.cu:21-41. */
int tf_pack_pair(const void* words_a, const void* scales_a, const void* biases_a, const void* words_b, const void* scales_b,
                 const void* biases_b, int n_each, int k, int bits, int gs, void* tiled, void* stream);
/* Exact inverse of tf_pack: cuda/kernels/qmm.py:85-102 (unpack). */
int tf_unpack(const void* tiled, int n, int k, int bits, int gs, void* words, void* scales, void* biases, void* stream);

/* ---- the matmul ---------------------------------------------------------------------------------------------- */

/* xs[m, g] = sum of x[m, g * gs : (g + 1) * gs] in fp32, with the bits the matmul computes for itself when it is given
 * no sums.  x: [m, k] bf16, row stride ldx elements (ldx % 2 == 0, base 4-byte aligned).  xs: [m, k / gs] fp32.
 * Replaces cuda/kernels/qmm.py:122-137 (group_sums). */
int tf_group_sums(const void* x, int64_t ldx, int m, int k, int gs, float* xs, void* stream);

/* out[m, n] = x @ dequant(w).T over the tiled layout, any m >= 1; a row's bits never depend on m.
 *   x        [m, k] bf16, base 16-byte aligned, ldx % 8 == 0 (elements)
 *   xs       optional [m, k / gs] fp32 group sums (NULL: computed in the kernel)
 *   tiled    units of the weight; sb_stride = int32 words between consecutive 128-column super-blocks
 *            (0: dense, (k / gs) * tf_unit_words)
 *   sk       K slices (>= 1, divides k / gs); sums are added in slice order
 *   out      [m, n] bf16 (out_f32 = 0) or fp32, row stride ldo elements; ignored when reduce = 0 and sk > 1
 *   part     [sk, m, n] fp32, required when reduce = 0 with sk > 1, or when sk > 8 (up to 8 slices are summed on
 *            chip; more pass through part and a second kernel), else may be NULL
 *   reduce   1: out receives the sum of the slices; 0: the slices stay in part (out untouched)
 *   pdl      1: launch with programmatic stream serialisation, so this call's weight prefetch overlaps the tail of the
 *            previous kernel in the stream (it still waits for that kernel before reading x or writing out)
 * Replaces the pybind function qmm(x, xs, w, scales, biases, out, part, n, sk, gs, bm, f32, reduce) of
 * cuda/kernels/qmm.cpp:14-44 and, for bits != 4, the Triton launch of cuda/kernels/affine.py:53-68. */
int tf_qmm(const void* x, int64_t ldx, int m, const float* xs, const void* tiled, int64_t sb_stride, int n, int k,
           int bits, int gs, int sk, void* out, int64_t ldo, int out_f32, float* part, int reduce, int pdl,
           void* stream);

/* tf_qmm for decode and verify windows (1 to 16 rows) over a SET of up to 4 projections that read the same rows of x
 * (q/k/v, gate/up, or one projection alone): one persistent launch streams all of them, and every output row has the
 * bits tf_qmm gives for the same projection and slice count.  Host arrays of nproj entries: tiled, sb_stride (entries
 * 0 or the array NULL: dense), n, sk, out, ldo.  out_f32 applies to every projection.
 *   scratch  device memory of tf_qmm_set_scratch_bytes(nproj, n, sk) bytes, 256-byte aligned: the K slices meet
 *            there (it stays in L2).  Its first 64 KB are counters that must be ZERO before the first call; every call
 *            leaves them zero (unless tf_device_error reports a lost wait: clear the scratch then).  Calls that share
 *            scratch must not overlap on the GPU: one scratch area per stream that runs sets side by side.
 * Replaces a run of the pybind qmm(...) calls of cuda/kernels/qmm.cpp:14-44 that the family engines issue for
 * projections of one input (families/qwen3_5/cuda/qmm_fast.py:49-64), with the bits of those separate calls. */
int64_t tf_qmm_set_scratch_bytes(int nproj, const int* n, const int* sk);
/* The launch geometry tf_qmm_set picks for such a set of m rows on the current device (host function; any pointer may be
 * NULL): super-blocks a thread block streams side by side, blocks an SM holds, blocks of the persistent grid.  Geometry
 * never changes a result bit.  No counterpart in the reference. */
int tf_qmm_set_geometry(int m, int bits, int gs, int nproj, const int* n, const int* sk, int* lanes, int* blocks_per_sm,
                        int* grid);
int tf_qmm_set(const void* x, int64_t ldx, int m, const float* xs, int k, int bits, int gs, int nproj,
               const void* const* tiled, const int64_t* sb_stride, const int* n, const int* sk, void* const* out,
               const int64_t* ldo, int out_f32, void* scratch, int64_t scratch_bytes, int pdl, void* stream);

/* Dense projection with an activation epilogue (one K slice): epi 1 = bf16(relu(bf16 v)^2); epi 2 = SwiGLU over a
 * tf_pack_pair weight, bf16(bf16(silu(bf16 gate)) * bf16 up) with both clipped first when limit > 0 (out then has n / 2
 * columns).  out: bf16.  The dense form of the expert epilogues of cuda/experts.cuh:57-103 (shared experts wider than the
 * routed ones run through it). */
int tf_qmm_act(const void* x, int64_t ldx, int m, const void* tiled, int64_t sb_stride, int n, int k, int bits, int gs,
               void* out, int64_t ldo, int epi, float limit, int pdl, void* stream);

/* ---- routed mixture of experts --------------------------------------------------------------------------------- */

/* Blocks of 1024 pairs a plan of `pairs` ranks: sizes the hist scratch (blocks * experts ints). */
int tf_moe_plan_blocks(int pairs);
/* Stable counting sort of the pairs by expert.  picks: [pairs] int32 expert ids; members: [pairs] pair ids grouped by
 * expert in pair order; items: [max_items][3] = (expert, first, count <= tile); counts: [2] = (items, distinct experts);
 * scratch rank: [pairs], hist: [tf_moe_plan_blocks(pairs) * experts].  Every buffer is the caller's, so a CUDA graph
 * replays it on new picks.  Replaces the pybind `plan` of cuda/experts.cpp:43-55 (cuda/experts.cu:157-334). */
int tf_moe_plan(const int* picks, int pairs, int experts, int tile, int* members, int* items, int* counts, int* rank,
                int* hist, int max_items, void* stream);
/* tf_moe_plan for callers that cannot provide scratch: same result, but rank and hist live in a 320 KB array built
 * into the library (every GPU that loads it holds that array until the process exits).  It is meant for hosts that have
 * no way to allocate at the point of the call: a serving process that has already handed all of HBM to its own pools,
 * so a late cudaMalloc would fail, or a plugin that is only given the buffers of the tensors it was called with.  This
 * entry point calls no cudaMalloc, cudaFree or any allocating library routine.
 *   limits   pairs <= 16384 and ceil(pairs / 1024) * experts <= 65536; anything larger is refused with TF_ERR_ARG and
 *            nothing is launched (use tf_moe_plan with your own scratch)
 *   set-up   tf_init(device) looks up the array's device address (and thereby loads the array, 320 KB, onto that GPU);
 *            the call itself is then a plain look-up, so it may also run under stream capture.  Without tf_init for the
 *            current device it returns TF_ERR_STATE
 *   sharing  all calls on a device use the one array and it keeps the last call's contents; nothing in it has to start
 *            at zero (every counter a call reads is written by that call first).  Two calls that overlap on the GPU
 *            (different streams, or two host threads) race on it: keep calls on a device ordered.
 * It has no counterpart in the reference, whose plan always takes caller tensors (cuda/experts.py:101-124). */
int tf_moe_plan_static(const int* picks, int pairs, int experts, int tile, int* members, int* items, int* counts,
                       int max_items, void* stream);
/* Grouped expert projection over a plan: item y = (expert, first, count) multiplies rows members[first .. first+count)
 * (row pair / slots of x when slots > 0: the token gather; row pair when slots == 0) by that expert's weight and writes
 * row `pair` of out.  tiled: [experts][ceil(n / 128)][k / gs][unit] 4-bit units, expert_stride words apart.
 * epi 0: out fp32 (out_f32 = 1) or bf16; 1: relu^2 (bf16); 2: SwiGLU over gate/up-interleaved rows (bf16, n / 2 columns).
 * tile = pairs an item may hold (8, 16, 32, 64).  experts = experts the table holds: an item that names another expert is
 * skipped (nothing is read past the table) and tf_device_error reports 5, where the reference's TORCH_CHECKs refuse a
 * plan built for another table before launching (cuda/experts.cpp:16-41).  Replaces the pybind `run` and `prefill` of
 * cuda/experts.cpp:57-82. */
int tf_moe_experts(const void* x, int64_t ldx, int slots, const void* tiled, int64_t expert_stride, int experts, int n, int k,
                   int gs, const int* items, const int* counts, const int* members, int max_items, int tile, void* out,
                   int64_t ldo, int out_f32, int epi, float limit, void* stream);
/* The same grouped projection in the prefill arithmetic (weights rounded once to bf16, one fp32 chain over K) on
 * tcgen05: the rows are first copied in member order into `sorted` ([pairs, k] bf16, caller scratch), then every item
 * (at most 128 pairs) runs as one tensor-memory tile per 128 output columns.  Plans for it use items of 128 pairs.
 * Replaces the pybind `prefill` of cuda/experts.cpp:69-82 (cuda/experts_prefill.cu:31-152). */
int tf_moe_experts_prefill(const void* x, int64_t ldx, int slots, const void* tiled, int64_t expert_stride, int experts, int n,
                           int k, int gs, const int* items, const int* counts, const int* members, int pairs, int max_items,
                           void* sorted, void* out, int64_t ldo, int out_f32, int epi, float limit, void* stream);
/* logits[r, e] = fp32 dot of bf16 rows x[r] and w[e].  Replaces the Triton `_router` of cuda/moe.py:23-55. */
int tf_moe_router(const void* x, int64_t ldx, int rows, int d, const void* w, int ne, float* out, int64_t ldo, void* stream);
/* The same logits in the prefill arithmetic: (16 rows x 16 experts) tensor-core tiles, K in order, fp32 accumulate.  A
 * row's bits do not depend on the row count, but they are not tf_moe_router's: a model keeps one form for its prompt
 * passes.  d a multiple of 16; x rows and w 4-byte aligned.  Replaces the same Triton `_router` (cuda/moe.py:23-55,
 * whose tl.dot tiles are this form). */
int tf_moe_router_tiles(const void* x, int64_t ldx, int rows, int d, const void* w, int ne, float* out, int64_t ldo,
                        void* stream);
/* Per row: top `topk` experts by fp32 logit (ties to the lower id), weights bf16(exp(l_k - l_0) / sum); with `shared`
 * one more slot, expert id `experts`, weight bf16(sigmoid(bf16(logit[experts]))).  pick, wts: [rows, topk + shared].
 * Replaces the Triton `_topk_rows` of cuda/moe.py:58-85. */
int tf_moe_topk(const float* logits, int64_t ldl, int rows, int experts, int topk, int shared, int* pick, float* wts,
                void* stream);
/* The same choice for a rank that holds experts [first, first + count) of the layer: slots of those experts carry the
 * local id (id - first) and their weight; every other slot, the shared one among them, carries id -1 and weight 0, so
 * tf_moe_plan and tf_moe_combine leave it out.  logits[.., experts] is not read.  The expert-parallel form of this
 * library; the reference splits every expert's width instead (families/nemotron_h/cuda/tp.py:38-51). */
int tf_moe_topk_local(const float* logits, int64_t ldl, int rows, int experts, int topk, int shared, int first, int count,
                      int* pick, float* wts, void* stream);
/* out[r, :] = bf16(sum over slots, in slot order, of wts[r, k] * y[r, k, :]) in fp32; y fp32 or bf16 (y_bf16).
 * Replaces the Triton `_combine` of cuda/moe.py:130-150. */
int tf_moe_combine(const void* y, int y_bf16, const float* wts, int rows, int slots, int d, void* out, void* stream);

/* ---- stored (MLX) layout helpers and the tensor-parallel reduction ------------------------------------------------ */

/* out[r, :] = q[row, :] * scale + bias in fp32 (rounded once when out is bf16) over the stored MLX words, row = ids[r]
 * (int32, or int64 with ids64) or r when ids is NULL.  meta: dtype of scales and biases, 0 bf16, 1 fp16, 2 fp32.
 * Replaces the Triton `embed` of cuda/kernels/affine_kernels.py:49-60 (cuda/kernels/affine.py:71-87) and, without ids
 * and with fp32 output, the diagnostic `dequantize` of families/qwen3_5/cuda/qmm.py:132-149. */
int tf_affine_rows(const void* ids, int ids64, int rows, const void* words, const void* scales, const void* biases, int meta,
                   int n, int k, int bits, int gs, void* out, int out_f32, void* stream);
/* out[i] = round(((p[0][i] + p[1][i]) + p[2][i]) + ...): the rank-ordered sum of `world` gathered partials (fp32, or
 * bf16 with parts_bf16), one rounding, so every rank ends with the same bits.  Generalises the two-rank
 * rank0.float() + rank1.float() of families/qwen3_5/cuda/distributed.py:281-284. */
int tf_sum_ranks(const void* parts, int world, int64_t total, int parts_bf16, void* out, int out_f32, void* stream);

/* ---- the same reduction in one launch over peer memory ------------------------------------------------------------
 * Every rank (one process a GPU, 2, 4 or 8 of them on one NVLink box) allocates one buffer of the same size with
 * tf_peer_alloc (zeroed; its first tf_peer_flag_bytes() bytes are the flags the ranks signal each other with), exports
 * it (a 64-byte handle the host passes to the other processes by any means) and opens the others'.  tf_peer_reduce
 * then sums the `total` elements at byte offset part_off of EVERY rank's buffer (fp32, or bf16 with parts_bf16) in
 * rank order, fp32 adds, one rounding, into byte offset out_off of this rank's buffer: the bits of tf_sum_ranks over
 * the gathered partials.  Every rank calls it once per reduction with the same arguments, after the kernel that wrote
 * its partial, on the same stream.  mode:
 *   2  flagged words, for small partials: a rank stores its partial as {data, epoch} words into a slot of every other
 *      rank's buffer and collects the others' from its own; no barrier between the ranks.  The 2 * world slots of
 *      ll_slot >= 2 * partial bytes each start at ll_off, past partial and result.  total a multiple of 8.
 *   1  shares, for large ones: after a barrier a rank reads its 1/world share of every partial, stores the sum into
 *      every rank's result, and a second barrier ends the call.  total a multiple of 8 * world.
 *   0  as 1 but every rank reads all partials whole (total a multiple of 8).
 *   5  flagged words in two hops, for 4 or 8 ranks: a rank sends every other rank only that rank's 1/world share,
 *      adds the shares it receives, and sends the finished share to every rank: about a fifth of mode 2's bytes at 8
 *      ranks.  Same slots (ll_slot a multiple of 16 * world); total a multiple of 8 * world.
 *   3, 4 and 6, 7, 8  the halves of modes 2 and 5 as launches of their own (a test driving all ranks from one process
 *      runs every rank's 3 then every rank's 4; every rank's 6, then 7, then 8).
 * polls: limit of each wait on a peer (0: several seconds, more than ranks drift apart while they start up; tests pass a
 * short one); a wait that runs out sets device error 4 (tf_device_error)
 * and the kernel returns; the buffers must then be freed and made anew.  grid_cap > 0 bounds the blocks (testing).
 * No counterpart in the reference, which reduces its two ranks with an all-gather and a torch add
 * (families/qwen3_5/cuda/distributed.py:249-284). */
size_t tf_peer_flag_bytes(void);
int tf_peer_alloc(size_t bytes, void** ptr);
int tf_peer_free(void* ptr);
int tf_peer_export(void* ptr, void* handle64);
int tf_peer_open(const void* handle64, void** ptr);
int tf_peer_close(void* ptr);
int tf_peer_reduce(void* const* bufs, int rank, int world, size_t part_off, size_t out_off, int64_t total, int parts_bf16,
                   int out_f32, int mode, size_t ll_off, size_t ll_slot, unsigned polls, int grid_cap, void* stream);

/* Glue that feeds the matmuls (rows contiguous, bf16, 16-byte aligned; d a multiple of gs; one block a row, so a row's
 * bits do not depend on the row count).
 * tf_add_rmsnorm: h = bf16(x + r) (r and h may be null: then h = x), y = bf16(h * inv * w) with
 * inv = 1 / sqrt(mean(h^2) + eps) in fp32, xs[row, g] = fp32 sum of y over group g (xs may be null).
 * tf_swiglu: out = bf16(g * sigmoid(g) * u) in fp32 with one rounding, xs as above.
 * Replace the Triton `_add_rmsnorm` and `_swiglu` of families/qwen3_5/cuda/glue.py:10-40,130-151. */
int tf_add_rmsnorm(const void* x, const void* r, const void* w, int rows, int d, float eps, void* h, void* y, float* xs,
                   int gs, void* stream);
int tf_swiglu(const void* gate, const void* up, int rows, int n, void* out, float* xs, int gs, void* stream);

/* Prefill matmul on tcgen05 / tensor memory: every weight rounded once to bf16, w = bf16(fma(q, s, b)), then one fp32
 * accumulation chain over K; any chunking of the rows gives the same bits (not the bits of tf_qmm).  4-bit weights,
 * groups of 32 or 64, k % 64 == 0.  x: [m, k] bf16, 16-byte aligned rows (ldx % 8 == 0); out: [m, n] bf16 or fp32.
 * Replaces the pybind function qmm_prefill(x, w, scales, biases, out, n, gs, f32, tile) of cuda/kernels/qmm.cpp:47-66
 * (cuda/kernels/qmm_prefill.cu:36-191). */
int tf_qmm_prefill(const void* x, int64_t ldx, int m, const void* tiled, int64_t sb_stride, int n, int k, int gs, void* out,
                   int64_t ldo, int out_f32, void* stream);

/* tf_qmm_prefill with the experts' activation epilogue (epi 1 relu^2, 2 SwiGLU over a tf_pack_pair weight: out then has
 * n / 2 bf16 columns): the prefill form of tf_qmm_act, used for shared experts run as dense projections. */
int tf_qmm_prefill_act(const void* x, int64_t ldx, int m, const void* tiled, int64_t sb_stride, int n, int k, int gs, void* out,
                       int64_t ldo, int out_f32, int epi, float limit, void* stream);

/* out[i] = round(part[0][i] + part[1][i] + ...), slices added in order: cuda/kernels/qmm.cu:235-243 (reduce_kernel).
 * part: [sk, total] fp32; out: [total] bf16 or fp32. */
int tf_reduce_slices(const float* part, int sk, int64_t total, void* out, int out_f32, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* TENSORFOLD_B200_H */
