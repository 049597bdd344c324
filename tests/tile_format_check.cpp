// Host check of the tile-record format against the register-level decode: a record built with the offset
// functions of tile_format.cuh must decode, lane by lane, into m16n8k16 A fragments whose elements are the
// codes of the (token, coordinate) pairs the attention kernel's B operands assume.  Compiled with g++ by
// tests/test_host_logic.py (no GPU needed); prints "tile emulation OK" and returns 0 on success.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../quashkv_b200/csrc/tile_decode.cuh"

using namespace qkv;

int main() {
  srand(7);
  static int kcode[16][128], ksign[16][128], vcode[16][128];
  uint8_t krow[16][32] = {}, srow[16][16] = {}, vrow[16][48] = {};
  for (int k = 0; k < 16; ++k)
    for (int c = 0; c < 128; ++c) {
      kcode[k][c] = rand() & 3;
      ksign[k][c] = rand() & 1;
      vcode[k][c] = rand() & 7;
      krow[k][c / 4] |= kcode[k][c] << (2 * (c % 4));          // LSB-first streams of w-bit fields
      srow[k][c / 8] |= ksign[k][c] << (c % 8);
      for (int b = 0; b < 3; ++b)
        if ((vcode[k][c] >> b) & 1) vrow[k][(3 * c + b) / 8] |= 1 << ((3 * c + b) % 8);
    }
  std::vector<uint8_t> rec(tile::kBytes, 0);
  std::vector<int> cover(tile::kBytes, 0);
  std::vector<uint32_t> vbits(tile::kBytes / 4, 0);          // value bits claimed so far, per word
  for (int k = 0; k < 16; ++k)
    for (int j = 0; j < 8; ++j) {                               // the steps of the tiling kernel's thread j
      memcpy(&rec[tile::key_code_offset(k, j)], &krow[k][4 * j], 4);
      for (int b = 0; b < 4; ++b) cover[tile::key_code_offset(k, j) + b]++;
      if (j < 4) {
        memcpy(&rec[tile::key_sign_offset(k, j)], &srow[k][4 * j], 4);
        for (int b = 0; b < 4; ++b) cover[tile::key_sign_offset(k, j) + b]++;
      }
      uint64_t c48 = 0;
      memcpy(&c48, &vrow[k][6 * j], 6);
      uint32_t bits[3], mask[3];
      tile::spread_codes16(c48, tile::val_half_shift(k), bits, mask);
      const int vl = tile::val_lane(k, j), grp = tile::val_group(k);
      uint32_t back[3];
      for (int w = 0; w < 3; ++w) {                             // the atomic AND / OR of the tiling kernel
        uint32_t word;
        memcpy(&word, &rec[tile::val_word_offset(vl, 3 * grp + w)], 4);
        if (word & mask[w]) { printf("two tokens claim the same value bits\n"); return 1; }
        word = (word & ~mask[w]) | bits[w];
        memcpy(&rec[tile::val_word_offset(vl, 3 * grp + w)], &word, 4);
        vbits[tile::val_word_offset(vl, 3 * grp + w) / 4] |= mask[w];
        back[w] = word;
      }
      if (tile::gather_codes16(back, tile::val_half_shift(k)) != c48) { printf("gather_codes16 is not the inverse\n"); return 1; }
      if (j == 0)
        for (int b = 0; b < 4; ++b) { cover[tile::key_norm_offset(k) + b]++; cover[tile::val_norm_offset(k) + b]++; }
    }
  for (int i = 0; i < tile::kBytes; ++i) {
    const bool value_part = i >= tile::kOffVal16 && i < tile::kOffNorms;
    if (value_part ? vbits[i / 4] != 0xFFFFFFFFu : cover[i] != 1) { printf("byte %d of the record is not written exactly once\n", i); return 1; }
  }

  // tables of recognisable bit patterns: key entry i -> 0x1000 + i, value magnitude m -> 0x2000 + m
  const uint32_t kt_a = 0x1000u | (0x1001u << 16), kt_b = 0x1002u | (0x1003u << 16);
  int bad = 0;
  for (int lane = 0; lane < 32; ++lane) {
    const int g = lane >> 2, t = lane & 3;
    uint32_t kc[4], ks[2], va[4], vb[2];
    memcpy(kc, &rec[tile::kOffKeyCodes + 16 * lane], 16);
    memcpy(ks, &rec[tile::kOffKeySigns + 8 * lane], 8);
    memcpy(va, &rec[tile::kOffVal16 + 16 * lane], 16);
    memcpy(vb, &rec[tile::kOffVal8 + 8 * lane], 8);
    for (int h = 0; h < 2; ++h)
      for (int c = 0; c < 32; ++c)
        if (((ks[h] >> c) & 1u) != static_cast<uint32_t>(ksign[g + 8 * h][32 * t + c])) bad++;
    auto key = [&](int k, int c) { return 0x1000u + kcode[k][c]; };
    auto check_key = [&](int word, int F, const uint32_t (&af)[4]) {
      const int c = 32 * t + 16 * word + F;   // a0 | a2 cover k columns (2t, 2t+1) | (2t+8, 2t+9)
      if (af[0] != (key(g, c) | (key(g, c + 4) << 16)) || af[1] != (key(g + 8, c) | (key(g + 8, c + 4) << 16)) ||
          af[2] != (key(g, c + 8) | (key(g, c + 12) << 16)) || af[3] != (key(g + 8, c + 8) | (key(g + 8, c + 12) << 16)))
        bad++;
    };
    uint32_t af[4];
#define K(W, F) tile::key_fragment<F>(kc[W], kc[2 + W], kt_a, kt_b, af); check_key(W, F, af);
    K(0, 0) K(0, 1) K(0, 2) K(0, 3) K(1, 0) K(1, 1) K(1, 2) K(1, 3)
    // value look-ups: the table offset of field F must be 128 * (stored(token a) | stored(token b) << 3) + 4 * lane
    auto want_off = [&](int ka, int kb, int c) {
      return 128u * (tile::code_to_stored(vcode[ka][c]) | (tile::code_to_stored(vcode[kb][c]) << 3)) + 4u * lane;
    };
    uint32_t got[2][16];
#define OFF(F) got[0][F] = tile::value_table_offset<F>(va[0], va[1], va[2], 4u * lane); \
               got[1][F] = tile::value_table_offset<F>(va[3], vb[0], vb[1], 4u * lane);
    OFF(0) OFF(1) OFF(2) OFF(3) OFF(4) OFF(5) OFF(6) OFF(7) OFF(8) OFF(9) OFF(10) OFF(11) OFF(12) OFF(13) OFF(14) OFF(15)
    for (int f = 0; f < 16; ++f) {      // field f = coordinate 16 g + f; M tile i uses fields 2 i (row g) and 2 i + 1 (row g + 8)
      if (got[0][f] != want_off(2 * t, 2 * t + 1, 16 * g + f)) bad++;
      if (got[1][f] != want_off(2 * t + 8, 2 * t + 9, 16 * g + f)) bad++;
    }
  }
  if (bad) { printf("FAILED: %d fragment mismatches\n", bad); return 1; }
  printf("tile emulation OK\n");
  return 0;
}
