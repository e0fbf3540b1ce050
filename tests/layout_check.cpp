// Host check of the tiled layout: lane_word / pair_reg / lane_code / code_loc are mutually consistent for every
// format, and pair_reg yields exactly the bf16 pair (128 + code) the mma A fragment needs.  Compiled by test_layout.py.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../tensorfold_b200/csrc/tf_layout.h"

static float bf16_to_float(uint32_t half) {
  uint32_t u = half << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

template <int BITS, int GS>
static int check() {
  constexpr int WPL = tf::words_per_lane(BITS, GS), NP = tf::pairs_per_lane(GS);
  std::vector<uint32_t> codes(128 * GS);
  uint32_t state = 12345u + BITS * 131u + GS;
  for (auto& c : codes) {
    state = state * 1664525u + 1013904223u;
    c = (state >> 11) & ((1u << BITS) - 1u);
  }
  auto at = [&](int col, int k) { return codes[col * GS + k]; };
  int bad = 0;
  std::vector<int> seen(128 * GS, 0);
  for (int tp = 0; tp < 4; ++tp)
    for (int lane = 0; lane < 32; ++lane) {
      uint32_t wd[WPL];
      for (int wi = 0; wi < WPL; ++wi) wd[wi] = tf::lane_word(BITS, GS, tp, lane, wi, at);
      for (int p = 0; p < NP; ++p) {
        const tf::PairPos pos = tf::pair_pos(tp, lane, p, GS);
        for (int half = 0; half < 2; ++half) {
          const uint32_t want = at(pos.col, pos.k + half);
          float got;
          if (tf::Fmt<BITS>::SPLIT) {
            const uint32_t lo = tf::pair_reg<BITS, GS, false>(wd, p), hi = tf::pair_reg<BITS, GS, true>(wd, p);
            got = (bf16_to_float((lo >> (16 * half)) & 0xFFFF) - 128.f) +
                  16.f * (bf16_to_float((hi >> (16 * half)) & 0xFFFF) - 128.f);
          } else {
            const uint32_t r = tf::pair_reg<BITS, GS>(wd, p);
            got = bf16_to_float((r >> (16 * half)) & 0xFFFF) - 128.f;
          }
          if (got != static_cast<float>(want)) ++bad;
          if (tf::lane_code(BITS, GS, wd, p, half) != want) ++bad;
          const tf::CodeLoc loc = tf::code_loc(pos.col, pos.k + half, GS);
          if (loc.tp != tp || loc.lane != lane || loc.p != p || loc.half != half) ++bad;
          ++seen[pos.col * GS + pos.k + half];
        }
      }
    }
  for (int v : seen)
    if (v != 1) ++bad;                       // every code of the unit is held exactly once
  int hits[128] = {0};
  for (int c = 0; c < 128; ++c) ++hits[tf::affine_index(c)];
  for (int v : hits)
    if (v != 1) ++bad;
  if (bad) std::printf("bits %d gs %d: %d mismatches\n", BITS, GS, bad);
  return bad;
}

template <int BITS>
static int all_groups() { return check<BITS, 32>() + check<BITS, 64>() + check<BITS, 128>(); }

int main() {
  const int bad = all_groups<2>() + all_groups<3>() + all_groups<4>() + all_groups<5>() + all_groups<6>() + all_groups<8>();
  // stored_code against a hand-built stream: 3-bit codes 0..7 repeating
  uint32_t row[3] = {0, 0, 0};
  for (int i = 0; i < 32; ++i) {
    const uint64_t v = static_cast<uint64_t>(i % 8) << ((i * 3) % 32);
    row[(i * 3) / 32] |= static_cast<uint32_t>(v);
    if ((i * 3) % 32 + 3 > 32) row[(i * 3) / 32 + 1] |= static_cast<uint32_t>(v >> 32);
  }
  int bad2 = 0;
  for (int i = 0; i < 32; ++i)
    if (tf::stored_code(row, i, 3, 3) != static_cast<uint32_t>(i % 8)) ++bad2;
  std::printf("%s\n", bad + bad2 ? "FAIL" : "OK");
  return bad + bad2 ? 1 : 0;
}
