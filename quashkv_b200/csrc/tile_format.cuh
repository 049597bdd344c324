// The tile record: storage format of the d = 128, 3-bit-key / 3-bit-value cache that the tensor-core
// decode kernel reads (attention_tiled.cu) and the tiling kernels write (tiling.cu).
//
// One record holds 16 consecutive tokens of one (batch, kv head) — or one 16-token slice of a page of a
// paged pool — in 1664 bytes, the same 104 bytes per token as the five row-major planes
// (reference packing.py:22-94 rows of 32 + 16 + 48 bytes and two fp32 norms).  The bytes are arranged
// in the order in which the lanes of a warp consume them as m16n8k16 fragments, so that a lane
// fetches its share with four vector loads and the whole record arrives with one bulk copy.
//
// Lane L = 4 g + t (g = 0..7, t = 0..3):
//   [   0,  512)  key codes     16 B per lane: tokens g and g+8, coordinates 32 t .. 32 t + 31 each
//                               (bytes 8 t .. 8 t + 7 of the token's 32-byte 2-bit row, unchanged)
//   [ 512, 1024)  value mags    16 B per lane: words m = 0..3; byte b of a word belongs to token
//                               2 t + (b & 1) + 8 (b >> 1); its 2-bit field f to coordinate 16 g + 4 m + f
//   [1024, 1536)  sign bits     16 B per lane:
//                   key signs   8 B: tokens g and g+8, coordinates 32 t .. 32 t + 31 (bytes 4 t .. 4 t + 3
//                               of the token's 16-byte sign row, unchanged)
//                   value signs 8 B: word h = 0, 1; its low half belongs to token 2 t + 8 h, its high half
//                               to token 2 t + 1 + 8 h; bit p to coordinate 16 g + p
//   [1536, 1664)  norms         16 B per g: key norm of tokens g, g+8, value norm of tokens g, g+8
//
// Values are stored as sign and magnitude instead of the reference's 3-bit code u (0..7, ascending
// centroid): negative = !(u >> 2), magnitude index = u & 3 for u >= 4 and 3 - u below, which is a
// bijection, so the reference's packed rows are recovered exactly (qkv_untile_rows).  The decode
// kernel looks the magnitude up in a four-entry table and flips the sign bit, which presumes
// centroid[7 - i] = -centroid[i] (true of Lloyd-Max tables of a symmetric density).
//
// Every token owns whole bytes of a record (no two tokens share a byte), so tokens can be written
// independently, in any order, by different threads or calls.
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
constexpr int kOffKeyCodes = 0, kOffValMags = 512, kOffSigns = 1024, kOffNorms = 1536;
constexpr int kKeyRowBytes = 32, kSignRowBytes = 16, kValRowBytes = 48;

// ---- where a token's bytes live ----------------------------------------------------------------------
// key codes: 4-byte piece j (0..7) of token k's 32-byte row
QKV_HD int key_code_offset(int k, int j) { return kOffKeyCodes + 16 * (4 * (k & 7) + (j >> 1)) + 8 * (k >> 3) + 4 * (j & 1); }
// key signs: 4-byte piece t (0..3) of token k's 16-byte row
QKV_HD int key_sign_offset(int k, int t) { return kOffSigns + 16 * (4 * (k & 7) + t) + 4 * (k >> 3); }
// value magnitudes: byte of token k in word m of coordinate group g (coordinates 16 g + 4 m .. + 3)
QKV_HD int val_mag_offset(int k, int g, int m) {
  return kOffValMags + 16 * (4 * g + ((k & 7) >> 1)) + 4 * m + (k & 1) + 2 * (k >> 3);
}
// value signs: 16-bit piece of token k for coordinate group g (bit p = coordinate 16 g + p)
QKV_HD int val_sign_offset(int k, int g) { return kOffSigns + 16 * (4 * g + ((k & 7) >> 1)) + 8 + 4 * (k >> 3) + 2 * (k & 1); }
QKV_HD int key_norm_offset(int k) { return kOffNorms + 16 * (k & 7) + 4 * (k >> 3); }
QKV_HD int val_norm_offset(int k) { return kOffNorms + 16 * (k & 7) + 8 + 4 * (k >> 3); }

// ---- 3-bit value code <-> (negative, magnitude index) ---------------------------------------------------
QKV_HD uint32_t code_to_mag(uint32_t u) { return (u & 4u) ? (u & 3u) : (~u & 3u); }
QKV_HD uint32_t code_to_neg(uint32_t u) { return ((u >> 2) & 1u) ^ 1u; }
QKV_HD uint32_t signmag_to_code(uint32_t neg, uint32_t mag) { return neg ? 3u - mag : 4u + mag; }

// 16 three-bit codes (48 bits, coordinate p at bits 3 p ..) -> four magnitude bytes (byte m holds
// coordinates 4 m .. 4 m + 3 as 2-bit fields) and 16 sign bits.
QKV_HD void split_codes16(uint64_t codes48, uint32_t& mags, uint32_t& negs) {
  mags = 0;
  negs = 0;
#pragma unroll
  for (int p = 0; p < 16; ++p) {
    const uint32_t u = static_cast<uint32_t>(codes48 >> (3 * p)) & 7u;
    mags |= code_to_mag(u) << (2 * p);
    negs |= code_to_neg(u) << p;
  }
}

QKV_HD uint64_t join_codes16(uint32_t mags, uint32_t negs) {
  uint64_t codes48 = 0;
#pragma unroll
  for (int p = 0; p < 16; ++p)
    codes48 |= static_cast<uint64_t>(signmag_to_code((negs >> p) & 1u, (mags >> (2 * p)) & 3u)) << (3 * p);
  return codes48;
}

}  // namespace tile
}  // namespace qkv
