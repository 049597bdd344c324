// The tile record: storage format of the d = 128, 3-bit-key / 3-bit-value cache that the tensor-core
// decode kernel reads (attention_tiled.cu) and the tiling kernels write (tiling.cu).
//
// One record holds 16 consecutive tokens of one (batch, kv head) — or one 16-token slice of a page of a
// paged pool — in 1664 bytes, the same 104 bytes per token as the five row-major planes
// (reference packing.py:22-94 rows of 32 + 16 + 48 bytes and two fp32 norms).  The bytes are arranged
// in the order in which the lanes of a warp consume them as m16n8k16 fragments, so that a lane
// fetches its share with five vector loads and the whole record arrives with one bulk copy.
//
// Lane L = 4 g + t (g = 0..7, t = 0..3):
//   [   0,  512)  key codes     16 B per lane: tokens g and g+8, coordinates 32 t .. 32 t + 31 each
//                               (bytes 8 t .. 8 t + 7 of the token's 32-byte 2-bit row, unchanged)
//   [ 512,  768)  key signs      8 B per lane: tokens g and g+8, coordinates 32 t .. 32 t + 31 (bytes 4 t ..
//                               4 t + 3 of the token's 16-byte sign row, unchanged)
//   [ 768, 1536)  values        24 B per lane, as two groups of 96 bits: group h = 0, 1 belongs to the token
//                               pair (2 t + 8 h, 2 t + 8 h + 1) and holds sixteen 6-bit fields; field f (bits
//                               6 f .. 6 f + 5 of the group) is coordinate 16 g + f: the first token's value in
//                               its low three bits, the second token's in its high three.  Words 0..3 of a
//                               lane (group 0 and the first word of group 1) sit in [768, 1280), 16 B per lane;
//                               words 4, 5 in [1280, 1536), 8 B per lane.
//   [1536, 1664)  norms         16 B per g: key norm of tokens g, g+8, value norm of tokens g, g+8
//
// A value is stored as magnitude index and sign, (neg << 2) | mag, instead of the reference's 3-bit code u
// (0..7, ascending centroid): neg = !(u >> 2), mag = u & 3 for u >= 4 and 3 - u below, which is a bijection,
// so the reference's packed rows are recovered exactly (qkv_untile_rows).  A 6-bit field is the index of a
// 64-entry table of ready fp16 pairs in the decode kernel, which presumes centroid[7 - i] = -centroid[i]
// (true of Lloyd-Max tables of a symmetric density).
//
// A token owns whole bytes of the key part.  In the value part the two tokens of a pair share words, so the
// tiling kernel updates a token's bits with atomic AND / OR: tokens can still be written independently, in
// any order, by different threads or calls.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define QKV_HD __host__ __device__ __forceinline__
#else
#define QKV_HD inline
#endif

namespace qkv {
namespace tile {

constexpr int kTokens = 16;
constexpr int kBytes = 1664;
constexpr int kOffKeyCodes = 0, kOffKeySigns = 512, kOffVal16 = 768, kOffVal8 = 1280, kOffNorms = 1536;
constexpr int kKeyRowBytes = 32, kSignRowBytes = 16, kValRowBytes = 48;

// ---- where a token's bytes live ----------------------------------------------------------------------
// key codes: 4-byte piece j (0..7) of token k's 32-byte row
QKV_HD int key_code_offset(int k, int j) { return kOffKeyCodes + 16 * (4 * (k & 7) + (j >> 1)) + 8 * (k >> 3) + 4 * (j & 1); }
// key signs: 4-byte piece t (0..3) of token k's 16-byte row
QKV_HD int key_sign_offset(int k, int t) { return kOffKeySigns + 8 * (4 * (k & 7) + t) + 4 * (k >> 3); }
// values: byte offset of word w (0..5) of lane L's 24 bytes
QKV_HD int val_word_offset(int L, int w) { return w < 4 ? kOffVal16 + 16 * L + 4 * w : kOffVal8 + 8 * L + 4 * (w - 4); }
// values: token k, coordinate group g (coordinates 16 g .. 16 g + 15) -> lane, group, and the shift of the token's
// three bits inside a 6-bit field
QKV_HD int val_lane(int k, int g) { return 4 * g + ((k & 7) >> 1); }
QKV_HD int val_group(int k) { return k >> 3; }
QKV_HD int val_half_shift(int k) { return 3 * (k & 1); }
QKV_HD int key_norm_offset(int k) { return kOffNorms + 16 * (k & 7) + 4 * (k >> 3); }
QKV_HD int val_norm_offset(int k) { return kOffNorms + 16 * (k & 7) + 8 + 4 * (k >> 3); }

// ---- 3-bit value code <-> stored form (neg << 2) | mag ---------------------------------------------------
QKV_HD uint32_t code_to_stored(uint32_t u) { return (u & 4u) ? (u & 3u) : (4u | (~u & 3u)); }
QKV_HD uint32_t stored_to_code(uint32_t v) { return (v & 4u) ? 3u - (v & 3u) : 4u + (v & 3u); }

// 16 three-bit codes of one token (48 bits, coordinate p at bits 3 p ..) -> the token's bits of a 96-bit group:
// stored value of coordinate p at bits 6 p + half_shift .. + 2.  Also the mask of those bit positions.
QKV_HD void spread_codes16(uint64_t codes48, int half_shift, uint32_t (&bits)[3], uint32_t (&mask)[3]) {
  bits[0] = bits[1] = bits[2] = 0;
  mask[0] = mask[1] = mask[2] = 0;
#pragma unroll
  for (int p = 0; p < 16; ++p) {
    const uint32_t v = code_to_stored(static_cast<uint32_t>(codes48 >> (3 * p)) & 7u);
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      const int pos = 6 * p + half_shift + b;
      bits[pos >> 5] |= ((v >> b) & 1u) << (pos & 31);
      mask[pos >> 5] |= 1u << (pos & 31);
    }
  }
}

QKV_HD uint64_t gather_codes16(const uint32_t (&w)[3], int half_shift) {
  uint64_t codes48 = 0;
#pragma unroll
  for (int p = 0; p < 16; ++p) {
    uint32_t v = 0;
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      const int pos = 6 * p + half_shift + b;
      v |= ((w[pos >> 5] >> (pos & 31)) & 1u) << b;
    }
    codes48 |= static_cast<uint64_t>(stored_to_code(v)) << (3 * p);
  }
  return codes48;
}

}  // namespace tile
}  // namespace qkv
