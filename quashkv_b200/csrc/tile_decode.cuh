// Register-level decode of a tile record (tile_format.cuh) into m16n8k16 fp16 A fragments.
//
// Written as host/device functions so that the index arithmetic can be checked on the CPU against the
// format definition; on the device every helper is one or two instructions.
#pragma once

#include <stdint.h>

#include "tile_format.cuh"

namespace qkv {
namespace tile {

QKV_HD uint32_t prmt_hd(uint32_t a, uint32_t b, uint32_t sel) {
#if defined(__CUDA_ARCH__)
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
#else
  const uint64_t pool = (static_cast<uint64_t>(b) << 32) | a;
  uint32_t d = 0;
  for (int i = 0; i < 4; ++i) {
    const uint32_t n = (sel >> (4 * i)) & 0xFu;
    uint32_t byte = static_cast<uint32_t>(pool >> (8 * (n & 7u))) & 0xFFu;
    if (n & 8u) byte = (byte & 0x80u) ? 0xFFu : 0u;
    d |= byte << (8 * i);
  }
  return d;
#endif
}

// Four 2-bit codes, one per byte of `w` at bits 2 f .. 2 f + 1, become two PRMT selectors: the table of
// four fp16 values sits in two registers as (lo, hi) byte pairs, so selector byte 0x10 + 0x22 * code
// picks a whole fp16: one multiply-add builds four selector bytes.  `lo` selects for the codes of bytes
// 0 and 1, `hi` for bytes 2 and 3 (PRMT reads the low 16 bits of a selector).  (Right shifts written
// as high-word multiplications, to move them off the logic pipe, measured 10 % slower.)
template <int F>
QKV_HD void selectors(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t y = (F == 0 ? w : w >> (2 * F)) & 0x03030303u;
  lo = y * 0x22u + 0x10101010u;
  hi = lo >> 16;
}

// Key codes of one k-step.  w0 / w1: the same code word of the tokens in rows g and g + 8.  Step
// (word, F) covers the lane's coordinates 16 word + {F, 4 + F | 8 + F, 12 + F} (k columns 2t, 2t+1 | 2t+8, 2t+9).
template <int F>
QKV_HD void key_fragment(uint32_t w0, uint32_t w1, uint32_t tab_a, uint32_t tab_b, uint32_t (&af)[4]) {
  uint32_t l0, h0, l1, h1;
  selectors<F>(w0, l0, h0);
  selectors<F>(w1, l1, h1);
  af[0] = prmt_hd(tab_a, tab_b, l0);
  af[1] = prmt_hd(tab_a, tab_b, l1);
  af[2] = prmt_hd(tab_a, tab_b, h0);
  af[3] = prmt_hd(tab_a, tab_b, h1);
}

// Byte offset, inside a 64-entry value table whose entry e of lane L sits at 128 e + 4 L (every lane reads its
// own bank), of field F (0..15) of a 96-bit group w[0..2]: two instructions, a (funnel) shift that brings the
// field to bits 7..12 and one logic operation that masks it and merges the lane's offset.
template <int F>
QKV_HD uint32_t value_table_offset(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t lane4) {
  constexpr int bit = 6 * F, word = bit >> 5, sh = bit & 31;
  const uint32_t lo = word == 0 ? w0 : (word == 1 ? w1 : w2);
  const uint32_t hi = word == 0 ? w1 : w2;               // only read when the field straddles two words
  uint32_t t;
  if (sh + 6 > 32) {
#if defined(__CUDA_ARCH__)
    t = __funnelshift_r(lo, hi, sh - 7);
#else
    t = static_cast<uint32_t>(((static_cast<uint64_t>(hi) << 32) | lo) >> (sh - 7));
#endif
  } else if (sh >= 7) {
    t = lo >> (sh - 7);
  } else {
    t = lo << (7 - sh);
  }
  return (t & (0x3Fu << 7)) | lane4;
}

}  // namespace tile
}  // namespace qkv
