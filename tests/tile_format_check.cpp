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
      uint32_t mags, negs;
      tile::split_codes16(c48, mags, negs);
      if (tile::join_codes16(mags, negs) != c48) { printf("join_codes16 is not the inverse\n"); return 1; }
      for (int m = 0; m < 4; ++m) {
        rec[tile::val_mag_offset(k, j, m)] = static_cast<uint8_t>(mags >> (8 * m));
        cover[tile::val_mag_offset(k, j, m)]++;
      }
      const uint16_t ng = static_cast<uint16_t>(negs);
      memcpy(&rec[tile::val_sign_offset(k, j)], &ng, 2);
      for (int b = 0; b < 2; ++b) cover[tile::val_sign_offset(k, j) + b]++;
      if (j == 0)
        for (int b = 0; b < 4; ++b) { cover[tile::key_norm_offset(k) + b]++; cover[tile::val_norm_offset(k) + b]++; }
    }
  for (int i = 0; i < tile::kBytes; ++i)
    if (cover[i] != 1) { printf("byte %d of the record is written %d times\n", i, cover[i]); return 1; }

  // tables of recognisable bit patterns: key entry i -> 0x1000 + i, value magnitude m -> 0x2000 + m
  const uint32_t kt_a = 0x1000u | (0x1001u << 16), kt_b = 0x1002u | (0x1003u << 16);
  const uint32_t vt_a = 0x2000u | (0x2001u << 16), vt_b = 0x2002u | (0x2003u << 16);
  int bad = 0;
  for (int lane = 0; lane < 32; ++lane) {
    const int g = lane >> 2, t = lane & 3;
    uint32_t kc[4], vm[4], sg[4];
    memcpy(kc, &rec[tile::kOffKeyCodes + 16 * lane], 16);
    memcpy(vm, &rec[tile::kOffValMags + 16 * lane], 16);
    memcpy(sg, &rec[tile::kOffSigns + 16 * lane], 16);
    const uint32_t ks[2] = {sg[0], sg[1]}, vs[2] = {sg[2], sg[3]};
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
    auto val = [&](int k, int c) {
      const uint32_t u = vcode[k][c];
      return (0x2000u + tile::code_to_mag(u)) | (tile::code_to_neg(u) << 15);
    };
    auto check_val = [&](int i, const uint32_t (&a)[4]) {     // M tile i: rows g, g+8 = coordinates 16g+2i, +1
      const int c0 = 16 * g + 2 * i, c1 = c0 + 1;
      if (a[0] != (val(2 * t, c0) | (val(2 * t + 1, c0) << 16)) || a[1] != (val(2 * t, c1) | (val(2 * t + 1, c1) << 16)) ||
          a[2] != (val(2 * t + 8, c0) | (val(2 * t + 9, c0) << 16)) || a[3] != (val(2 * t + 8, c1) | (val(2 * t + 9, c1) << 16)))
        bad++;
    };
#define V(M, H) tile::value_fragment<M, H>(vm[M], vs[0], vs[1], vt_a, vt_b, af); check_val(2 * M + H, af);
    V(0, 0) V(0, 1) V(1, 0) V(1, 1) V(2, 0) V(2, 1) V(3, 0) V(3, 1)
  }
  if (bad) { printf("FAILED: %d fragment mismatches\n", bad); return 1; }
  printf("tile emulation OK\n");
  return 0;
}
