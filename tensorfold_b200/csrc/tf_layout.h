// The tiled ("lane") weight layout shared by the pack kernels, the matmul kernels and the host-side layout tests.
//
// A projection (N outputs, K inputs, BITS-bit codes, one bf16 scale and bias per GS inputs) is stored as
//
//     units[N128][K / GS][UNIT_WORDS]            N128 = ceil(N / 128) super-blocks of 128 output columns
//
// so everything a thread block needs for one quantisation group of its 128 columns is one contiguous unit, and
// consecutive groups are consecutive in memory: a pipeline stage is a single bulk copy.  A unit holds
//
//     codes   [4 tile pairs][32 lanes][WPL words]     WPL = GS * BITS / 32
//     affine  [128] words, (scale bf16 | bias bf16 << 16), ordered so one lane reads its four pairs with one 16-byte load
//
// A tile pair is 32 output columns = two m16n8k16 A tiles (the weights are the A operand: 16 output columns x 16
// inputs per instruction).  A lane's words hold exactly the codes its A fragments need, as bit planes whose fields sit
// 16 bits apart, so that `(word >> shift) & mask | magic` yields a ready bf16x2 register (128 + code, 128 + code).
//
// Pair p of a lane in (tile pair, group):  p = (h * S + s) * 4 + j   with h the tile (0/1), s the 16-input step
// (S = GS / 16) and j the A-fragment register.  With lane = 4 g + t the pair holds the codes of
//     column  32 tp + 16 h + g + 8 (j & 1)          inputs  16 s + 2 t + 8 (j >> 1)  and that + 1  (low, high half).
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define TF_HD __host__ __device__ __forceinline__
#else
#define TF_HD inline
#endif

namespace tf {

constexpr int SB_COLS = 128;          // output columns of a super-block
constexpr int TILE_PAIRS = 4;         // 32-column tile pairs per super-block
constexpr int AFFINE_WORDS = 128;     // (scale, bias) words of a unit

// Bit planes of a code: plane A is the low WA bits, plane B the next WB bits (0: none).
// 8-bit codes are two nibble planes multiplied separately (low nibble by x, high nibble by 16 x).
template <int BITS> struct Fmt;
template <> struct Fmt<2> { static constexpr int WA = 2, WB = 0; static constexpr bool SPLIT = false; };
template <> struct Fmt<3> { static constexpr int WA = 2, WB = 1; static constexpr bool SPLIT = false; };
template <> struct Fmt<4> { static constexpr int WA = 4, WB = 0; static constexpr bool SPLIT = false; };
template <> struct Fmt<5> { static constexpr int WA = 4, WB = 1; static constexpr bool SPLIT = false; };
template <> struct Fmt<6> { static constexpr int WA = 4, WB = 2; static constexpr bool SPLIT = false; };
template <> struct Fmt<8> { static constexpr int WA = 4, WB = 4; static constexpr bool SPLIT = true; };

TF_HD constexpr int plane_a(int bits) { return bits == 2 || bits == 3 ? 2 : 4; }
TF_HD constexpr int plane_b(int bits) { return bits - plane_a(bits); }
TF_HD constexpr int words_per_lane(int bits, int gs) { return gs * bits / 32; }
TF_HD constexpr int unit_words(int bits, int gs) { return TILE_PAIRS * 32 * words_per_lane(bits, gs) + AFFINE_WORDS; }
TF_HD constexpr int pairs_per_lane(int gs) { return 8 * (gs / 16); }
// the constant the magic-number dequantisation adds to every code, summed over the planes as the MMAs see them
TF_HD constexpr float code_offset(int bits) { return bits == 8 ? 128.f * 17.f : 128.f; }

struct PairPos {
  int col;   // column inside the 128-column super-block
  int k;     // input inside the group, of the low half (the high half is k + 1)
};

TF_HD PairPos pair_pos(int tp, int lane, int p, int gs) {
  const int S = gs / 16, j = p & 3, s = (p >> 2) % S, h = (p >> 2) / S, g = lane >> 2, t = lane & 3;
  return PairPos{32 * tp + 16 * h + g + 8 * (j & 1), 16 * s + 2 * t + 8 * (j >> 1)};
}

// Index inside the affine words of a unit for column c of the super-block.
TF_HD int affine_index(int c) {
  const int tp = c >> 5, h = (c >> 4) & 1, r8 = (c >> 3) & 1, g = c & 7;
  return tp * 32 + g * 4 + h * 2 + r8;
}

// Code k of a stored MLX row: bits [k * BITS, k * BITS + BITS) of the little-endian word stream.
TF_HD uint32_t stored_code(const uint32_t* row, int64_t k, int bits, int64_t words) {
  const int64_t bit = k * bits, w = bit >> 5;
  const int sh = static_cast<int>(bit & 31);
  uint64_t v = row[w];
  if (sh + bits > 32 && w + 1 < words) v |= static_cast<uint64_t>(row[w + 1]) << 32;
  return static_cast<uint32_t>((v >> sh) & ((1u << bits) - 1u));
}

// Word `wi` (0 <= wi < WPL) of lane `lane` in tile pair `tp`, built from a functor code(col, k) -> stored code.
template <class CodeAt>
TF_HD uint32_t lane_word(int bits, int gs, int tp, int lane, int wi, CodeAt code) {
  const int wa = plane_a(bits), wb = plane_b(bits), np = pairs_per_lane(gs);
  const int words_a = np * wa / 16;
  int width, shift, local;
  if (wi < words_a) {
    width = wa, shift = 0, local = wi;
  } else {
    width = wb, shift = wa, local = wi - words_a;
  }
  const int ppw = 16 / width;
  uint32_t out = 0;
  for (int slot = 0; slot < ppw; ++slot) {
    const PairPos pos = pair_pos(tp, lane, local * ppw + slot, gs);
    const uint32_t mask = (1u << width) - 1u;
    const uint32_t lo = (code(pos.col, pos.k) >> shift) & mask, hi = (code(pos.col, pos.k + 1) >> shift) & mask;
    out |= lo << (slot * width);
    out |= hi << (16 + slot * width);
  }
  return out;
}

// The code a lane's words hold for pair p, half (0 low, 1 high): the inverse of lane_word, used by unpack and tests.
TF_HD uint32_t lane_code(int bits, int gs, const uint32_t* words, int p, int half) {
  const int wa = plane_a(bits), wb = plane_b(bits), np = pairs_per_lane(gs);
  const int words_a = np * wa / 16;
  const int ppa = 16 / wa;
  uint32_t v = (words[p / ppa] >> ((p % ppa) * wa + 16 * half)) & ((1u << wa) - 1u);
  if (wb) {
    const int ppb = 16 / wb;
    v |= ((words[words_a + p / ppb] >> ((p % ppb) * wb + 16 * half)) & ((1u << wb) - 1u)) << wa;
  }
  return v;
}

// The bf16x2 A-fragment register of pair p: (128 + code_low, 128 + code_high), each exact in bf16 because the code (at
// most 6 bits here) sits in the low mantissa bits of 0x4300 = 128.0.  8-bit codes come as two nibble planes: HIGH picks
// the upper nibble, which the kernel multiplies by 16 x instead of x.  With p a compile-time constant (unrolled loops)
// this is one shift and one three-input logic op per plane.
#if defined(__CUDA_ARCH__)
// (a & mask) | orv as ONE three-input logic instruction (left to itself the compiler emits an AND and an OR when both
// constants are immediates: twice the instructions in the matmul's innermost loop).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
  return r;
}
#else
inline uint32_t and_or(uint32_t a, uint32_t mask, uint32_t orv) { return (a & mask) | orv; }
#endif

template <int BITS, int GS, bool HIGH = false>
TF_HD uint32_t pair_reg(const uint32_t* wd, int p) {
  constexpr int WA = Fmt<BITS>::WA, WB = Fmt<BITS>::WB, NP = pairs_per_lane(GS), WORDS_A = NP * WA / 16, PPA = 16 / WA;
  constexpr uint32_t MAGIC = 0x43004300u, MASK_A = ((1u << WA) - 1u) * 0x00010001u;
  if constexpr (Fmt<BITS>::SPLIT) {
    const uint32_t v = wd[(HIGH ? WORDS_A : 0) + p / 4] >> ((p % 4) * 4);
    return and_or(v, 0x000F000Fu, MAGIC);
  } else {
    uint32_t r = and_or(wd[p / PPA] >> ((p % PPA) * WA), MASK_A, MAGIC);
    if constexpr (WB > 0) {
      constexpr int PPB = 16 / WB;
      constexpr uint32_t MASK_B = (((1u << WB) - 1u) << WA) * 0x00010001u;
      const int sh = (p % PPB) * WB - WA;
      const uint32_t u = wd[WORDS_A + p / PPB];
      r = and_or(sh >= 0 ? (u >> sh) : (u << (-sh)), MASK_B, r);
    }
    return r;
  }
}

// Where the code of (column c of the super-block, input kk of the group) lives: the inverse of pair_pos.
struct CodeLoc {
  int tp, lane, p, half;
};

TF_HD CodeLoc code_loc(int c, int kk, int gs) {
  const int S = gs / 16, tp = c >> 5, h = (c >> 4) & 1, r8 = (c >> 3) & 1, g = c & 7;
  const int s = kk >> 4, in = kk & 15, t = (in & 7) >> 1, j = r8 | ((in >> 3) << 1);
  return CodeLoc{tp, 4 * g + t, (h * S + s) * 4 + j, in & 1};
}

}  // namespace tf
