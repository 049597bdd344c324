// Decode fast path of the packed-cache attention: head_dim 128, 3-bit keys (2-bit codes + sign
// bit), 3-bit values, up to 8 query rows per KV head (grouped-query heads x q_len).
//
// The generic kernel spends ~150 warp instructions per token-head on scalar unpack + FMA; the
// HBM roofline leaves room for about 18.  Here every warp owns 16-token tiles and
//   * loads its slice of the packed rows straight into registers (a quad of lanes covers one
//     32-byte code row, so a warp load is a run of whole rows),
//   * decodes codes to fp16 IN REGISTERS, directly in mma.sync fragment layout, using PRMT as
//     a byte look-up table (2-bit codes: 4-entry table; 3-bit codes: spread to nibbles, then
//     an 8-entry table) and one LOP3 per pair of sign bits,
//   * scores 8 query columns with m16n8k16 MMAs (tokens are the M dimension, the rotated
//     query and the sign weights are register-resident B operands),
//   * runs the online softmax on the accumulator fragment, transposes the weights with
//     movmatrix, and accumulates values (coordinates as M, tokens as K) in fp32.
// Nothing is staged through shared memory in the token loop.  fp16 operands carry 11
// significant bits; products are exact and accumulate in fp32.
//
// Output: the same per-split partials (max, sum, rotated accumulator) as the generic kernel,
// merged and un-rotated by merge_splits_kernel.
#include <math.h>
#include <stdlib.h>

#include "attention_common.cuh"
#include "mma_decode.cuh"

namespace qkv {

constexpr int kMmaWarps = 4;
constexpr int kTile = 16;                 // tokens per warp step
constexpr float kLog2e = 1.4426950408889634f;

constexpr int kStages = 4;                  // tiles in flight per warp (3 ahead of the one in use)
constexpr int kStageBytes = 512 + 256 + 768 + 64 + 64;   // codes, signs, value codes, 2 x 16 norms
constexpr int kOffKs = 512, kOffV = 768, kOffKn = 1536, kOffVn = 1600;

struct TileRegs {
  uint2 kc[2];      // key codes: this lane's 8 bytes of rows gid, gid+8
  uint32_t ks[2];   // sign words of the same rows
  float kn[2], vn[2];
  uint32_t v[4][2]; // value words of tokens 2tig, 2tig+1, 2tig+8, 2tig+9
};

struct MmaPtrs {
  const uint8_t* kcode; const uint8_t* ksign; const uint8_t* vcode; const float* knorm; const float* vnorm;
};

template <bool PAGED>
__global__ void __launch_bounds__(kMmaWarps * 32, 4) attend_decode_mma_kernel(AttnArgs a) {
  constexpr int D = 128;
  __shared__ float q_s[8][2 * D];                    // [query row][q_rot*scale | sign weights]
  // the per-warp staging rings of the token loop and the end-of-kernel reduction share storage
  constexpr int kRingBytes = kMmaWarps * kStages * kStageBytes;
  constexpr int kRedBytes = kMmaWarps * 8 * (D + 2) * 4;
  __shared__ __align__(16) unsigned char pool[kRingBytes > kRedBytes ? kRingBytes : kRedBytes];
  float (*red)[8][D + 2] = reinterpret_cast<float (*)[8][D + 2]>(pool);   // [warp][query][max, sum, acc]
  __shared__ float wsum[8];                          // sum of the sign weights per query row
  __shared__ uint2 bop[24][32];                      // B operands per k-step and lane: 8 query-high, 8 query-low, 8 sign

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int split = blockIdx.z, seg = blockIdx.x;     // splits are the slowest dimension: longest first
  const int b = seg / a.Hkv, hkv = seg % a.Hkv;
  // Query rows of a (batch, kv head) are numbered g * q_len + position; a CTA takes eight of them
  // (blockIdx.y), so decode (one tile) and prefill (many) run through the same code.
  const int r0 = 8 * blockIdx.y;
  // a paged cache has its own token count per batch entry; a.kv_len is then only their upper bound
  int64_t kv_len = a.kv_len;
  if (PAGED) kv_len = min(static_cast<int64_t>(max(a.seq_lens[b], 0)), a.kv_len);
  const int nq_all = a.G * a.q_len;
  const int nq = nq_all - r0 < 8 ? nq_all - r0 : 8;

  // Every (batch entry's) length is divided over the splits in whole 128-token chunks, unequal shares, longest
  // first; a short sequence of a paged batch so keeps all its CTAs busy for a short time.
  const int64_t chunks = (kv_len + 127) / 128;
  const int64_t t_begin = 128 * split_begin_chunk(split, a.n_splits, chunks, a.skew);
  int64_t t_end = 128 * split_begin_chunk(split + 1, a.n_splits, chunks, a.skew);
  if (t_end > kv_len) t_end = kv_len;
  if (a.causal) {                      // tokens past the last position any row of this tile may see are skipped
    int last = 0;
    for (int r = 0; r < nq; ++r) last = max(last, (r0 + r) % a.q_len);
    const int64_t visible = kv_len - a.q_len + last + 1;
    if (t_end > visible) t_end = visible;
  }
  const int n_valid = static_cast<int>(t_end - t_begin);        // tokens of this split
  // A split without tokens (past the end of a short sequence of a paged batch, or above the diagonal of a
  // causal prefill) skips the operand set-up and goes straight to its neutral partial result.
  const bool has_work = n_valid > 0;

  // contiguous cache: first row of this (batch, kv head); paged cache: this head's rows inside block 0
  const int64_t seg_row0 = PAGED ? static_cast<int64_t>(hkv) * a.block_size : static_cast<int64_t>(seg) * a.cache.capacity;
  MmaPtrs p;
  p.kcode = a.cache.k_codes + seg_row0 * 32;
  p.ksign = a.cache.k_signs + seg_row0 * 16;
  p.vcode = a.cache.v_codes + seg_row0 * 48;
  p.knorm = a.cache.k_norms + seg_row0;
  p.vnorm = a.cache.v_norms + seg_row0;

  // ---- cp.async ring: each lane copies up to four 16-byte chunks of a tile (104 chunks) ----------
  const int64_t t_first = t_begin + static_cast<int64_t>(warp) * kTile;
  constexpr int kStep = kMmaWarps * kTile;                       // tokens between a warp's tiles
  const int first_rel = warp * kTile;
  const int n_it = first_rel < n_valid ? (n_valid - first_rel + kStep - 1) / kStep : 0;
  unsigned char* ring = pool + warp * (kStages * kStageBytes);
  // Chunk sources: src0 is the chunk's address in tile 0 (paged: in the first tile of block 0) and stride the
  // bytes between this warp's consecutive tiles (paged: the bytes of one row, a tile's first row being looked
  // up in the block table).
  const unsigned char* src0[4];
  int dst_off[4], tok_off[4], stride[4];
  const int64_t t_src = PAGED ? 0 : t_first;
  constexpr int kRowStep = PAGED ? 1 : kStep;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = lane + 32 * k;
    if (c < 32) {            // key codes: two chunks per token row
      tok_off[k] = c >> 1; stride[k] = kRowStep * 32; dst_off[k] = c * 16;
      src0[k] = p.kcode + (t_src + (c >> 1)) * 32 + (c & 1) * 16;
    } else if (c < 48) {     // sign bits: one chunk per token
      const int r = c - 32;
      tok_off[k] = r; stride[k] = kRowStep * 16; dst_off[k] = kOffKs + r * 16;
      src0[k] = p.ksign + (t_src + r) * 16;
    } else if (c < 96) {     // value codes: three chunks per token
      const int i = c - 48;
      tok_off[k] = i / 3; stride[k] = kRowStep * 48; dst_off[k] = kOffV + i * 16;
      src0[k] = p.vcode + (t_src + i / 3) * 48 + (i % 3) * 16;
    } else {                 // norms: four tokens per chunk (c < 104 holds data)
      const int j = (c - 96) & 3, which = (c - 96) >> 2;
      tok_off[k] = 4 * j; stride[k] = kRowStep * 4;
      dst_off[k] = (which ? kOffVn : kOffKn) + j * 16;
      src0[k] = reinterpret_cast<const unsigned char*>((which ? p.vnorm : p.knorm) + t_src + 4 * j);
    }
  }
  // paged: the block of the tile that the next issue() copies, read one call ahead of its use
  const int32_t* bt = PAGED ? a.block_table + static_cast<int64_t>(b) * a.max_blocks : nullptr;
  auto block_of = [&](int it) -> int {
    const unsigned t = static_cast<unsigned>(t_first) + static_cast<unsigned>(it) * kStep;   // kv_len < 2^31
    return it < n_it ? __ldg(bt + t / static_cast<unsigned>(a.block_size)) : 0;
  };
  int blk_next = PAGED ? block_of(0) : 0;
  auto issue = [&](int it) {                                // called with it = 0, 1, 2, ... in order
    if (it < n_it) {
      const int rel = first_rel + it * kStep;
      unsigned char* stage = ring + (it % kStages) * kStageBytes;
      int64_t step = it;                                    // multiplies stride[k]
      if (PAGED) {                                          // first row of the tile inside the pool, less this head's offset
        const unsigned t = static_cast<unsigned>(t_first) + static_cast<unsigned>(it) * kStep;
        step = static_cast<int64_t>(blk_next) * a.Hkv * a.block_size + t % static_cast<unsigned>(a.block_size);
      }
      if (rel + kTile <= n_valid) {                         // warp-uniform: the whole tile lies inside the split
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (k < 3 || lane < 8) cp_async16(stage + dst_off[k], src0[k] + step * stride[k], 16);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (k < 3 || lane < 8) {
            const bool ok = rel + tok_off[k] < n_valid;    // rows past the split are zero-filled, not read
            cp_async16(stage + dst_off[k], ok ? src0[k] + step * stride[k] : src0[k], ok ? 16 : 0);
          }
        }
      }
    }
    if (PAGED) blk_next = block_of(it + 1);
    cp_async_commit();                                      // one group per tile slot, even when empty
  };
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) issue(i);

  // Everything above read only the cache planes and the block table, which no kernel of this call writes: when
  // the launch allows it (programmatic dependent launch), this grid starts while the query-rotation kernel is
  // still running and its first tiles are already on their way.  From here on the rotated queries, the look-up
  // tables and the zeroed arrival counters are needed: wait for that kernel to have completed.
  asm volatile("griddepcontrol.wait;\n" ::: "memory");


  for (int idx = threadIdx.x; has_work && idx < 8 * 2 * D; idx += blockDim.x) {
    const int r = idx / (2 * D), e = idx % (2 * D);
    float v = 0.f;
    if (r < nq) {
      const int g = (r0 + r) / a.q_len, qi = (r0 + r) % a.q_len;
      const int64_t qrow = (static_cast<int64_t>(b) * a.Hq + hkv * a.G + g) * a.q_len + qi;
      v = a.qk[qrow * 2 * D + e];
    }
    q_s[r][e] = v;
  }
  __syncthreads();
  if (has_work) {                   // a warp sums the sign weights of two query rows
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float* w = q_s[2 * warp + h] + D;
      float t = (w[lane] + w[lane + 32]) + (w[lane + 64] + w[lane + 96]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(QKV_FULL_MASK, t, o);
      if (lane == 0) wsum[2 * warp + h] = t * kLog2e;
    }
  }
  __syncthreads();

  // ---- register-resident B operands for query column n = gid ---------------------------------
  // Key-code k-step s = 4*word + grp covers this lane's coordinates base + {o, o+2 | o+4, o+6},
  // base = 32 tig + 16 word, o = 8*(grp&1) + (grp>>1): the order in which the PRMT decode below
  // produces them.  Sign k-step s covers 32 tig + {2s, 2s+16 | 2s+1, 2s+17}.
  const float inv_sk = __uint_as_float(a.tables[6]), inv_sv = __uint_as_float(a.tables[7]);
  if (has_work) {                   // the operands depend on the lane only: each warp builds two k-steps
    const float qf = kLog2e * inv_sk;
    const float* q = q_s[gid];
    const float* w = q_s[gid] + D;
#pragma unroll
    for (int s = warp; s < 8; s += kMmaWarps) {
      const int word = s >> 2, grp = s & 3;
      const int c0 = 32 * tig + 16 * word + grp;        // k-step s: coordinates c0 + {0, 4 | 8, 12}
      float v[4], r[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[e] = q[c0 + 4 * e] * qf;
        r[e] = v[e] - __half2float(__float2half_rn(v[e]));
      }
      bop[s][lane] = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
      bop[8 + s][lane] = make_uint2(pack_half2(r[0], r[1]), pack_half2(r[2], r[3]));
      uint32_t wq[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {           // pairs t = 2s, 2s+1 of this lane's 32 coordinates
        const int t = 2 * s + h, j = 32 * tig + sign_coord(t);
        const float f = 2.f * kLog2e / sign_v1(sign_pos(t));
        wq[h] = pack_half2(w[j] * f, w[j + 16] * f);
      }
      bop[16 + s][lane] = make_uint2(wq[0], wq[1]);
    }
  }
  __syncthreads();
  // ---- PRMT look-up tables: low and high bytes of the fp16 centroids ---------------------------
  const uint32_t kt_a = a.tables[0], kt_b = a.tables[1];     // fp16 key centroids 0,1 | 2,3
  const uint32_t vt_lo[2] = {a.tables[2], a.tables[3]}, vt_hi[2] = {a.tables[4], a.tables[5]};
  // causal limits of this lane's two query columns (2 tig, 2 tig + 1)
  int lim[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = 2 * tig + e;
    lim[e] = (r < nq) ? (a.causal ? static_cast<int>(kv_len - a.q_len + (r0 + r) % a.q_len) : 0x7fffffff) : -1;
  }


  // positions relative to the split start, as 32-bit values
  int lim_rel[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int64_t d = static_cast<int64_t>(lim[e]) - t_begin;
    lim_rel[e] = lim[e] == 0x7fffffff ? 0x7fffffff : (d < -1 ? -1 : static_cast<int>(d));
  }

  float O[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f;
  // reference exponents start at a finite "nothing seen yet" value (any finite score raises them at once), so that
  // the token loop needs no test for minus infinity; the value written out below turns it back into -inf
  constexpr float kNone = -1e30f;
  float m[2] = {kNone, kNone}, l[2] = {0.f, 0.f};
  const int odd16 = (gid & 1) * 16;
  const float ci0 = -wsum[2 * tig], ci1 = -wsum[2 * tig + 1];   // accumulator start: -sum of sign weights

  auto fetch = [&](TileRegs& T, int it) {                  // this lane's fragment slice of a staged tile
    const unsigned char* stage = ring + (it % kStages) * kStageBytes;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      T.kc[h] = *reinterpret_cast<const uint2*>(stage + (gid + 8 * h) * 32 + tig * 8);
      T.ks[h] = *reinterpret_cast<const uint32_t*>(stage + kOffKs + (gid + 8 * h) * 16 + tig * 4);
      T.kn[h] = *reinterpret_cast<const float*>(stage + kOffKn + (gid + 8 * h) * 4);
      T.vn[h] = *reinterpret_cast<const float*>(stage + kOffVn + (gid + 8 * h) * 4);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int tok = 2 * tig + (k & 1) + 8 * (k >> 1);
      const uint32_t* row = reinterpret_cast<const uint32_t*>(stage + kOffV + tok * 48) + ((3 * gid) >> 1);
      T.v[k][0] = row[0];
      T.v[k][1] = row[1];
    }
  };

  // 8 three-bit fields (24 bits) -> 8 nibbles, sum c_k 8^k -> sum c_k 16^k, in three halving steps
  auto spread = [](uint32_t g) {
    g = g + 15u * (g & 0xFFF000u);          // 12-bit halves to 16-bit stride
    g = g + 3u * (g & 0x0FC00FC0u);         // 6-bit pairs to 8-bit stride
    return g + (g & 0x38383838u);           // 3-bit fields to 4-bit stride
  };

  auto process = [&](const TileRegs& cur, int it) {
    const int rel = first_rel + it * kStep;
    const bool masked = a.causal || rel + kTile > n_valid;      // warp-uniform
    // ---- scores: 8 MMAs on key codes, 8 on sign bits --------------------------------------------
    float c[4] = {ci0, ci1, ci0, ci1};
#pragma unroll
    for (int word = 0; word < 2; ++word) {
      const uint32_t w0 = word ? cur.kc[0].y : cur.kc[0].x;
      const uint32_t w1 = word ? cur.kc[1].y : cur.kc[1].x;
      // Codes r, 4+r, 8+r, 12+r of a word sit in its four bytes after a shift by 2r.  The 2-bit table
      // fits PRMT's 8 source bytes as (lo,hi) pairs, so selector byte 0x10 + 0x22*code picks a whole
      // fp16: one multiply-add builds four selector bytes, one PRMT yields a half2 operand.
#pragma unroll
      for (int grp = 0; grp < 4; ++grp) {
        const uint32_t y0 = (w0 >> (2 * grp)) & 0x03030303u, y1 = (w1 >> (2 * grp)) & 0x03030303u;
        const uint32_t sl0 = y0 * 0x22u + 0x10101010u, sh0 = sl0 >> 16;
        const uint32_t sl1 = y1 * 0x22u + 0x10101010u, sh1 = sl1 >> 16;
        uint32_t af[4];
        af[0] = prmt(kt_a, kt_b, sl0);
        af[1] = prmt(kt_a, kt_b, sl1);
        af[2] = prmt(kt_a, kt_b, sh0);
        af[3] = prmt(kt_a, kt_b, sh1);
        const uint2 bh = bop[word * 4 + grp][lane], bl = bop[8 + word * 4 + grp][lane];
        mma16816(c, af, bh.x, bh.y);
        mma16816(c, af, bl.x, bl.y);
      }
    }
    {
      const uint32_t cp0[4] = {cur.ks[0], cur.ks[0] << 7, cur.ks[0] >> 1, cur.ks[0] << 13};
      const uint32_t cp1[4] = {cur.ks[1], cur.ks[1] << 7, cur.ks[1] >> 1, cur.ks[1] << 13};
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        uint32_t af[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int t = 2 * s + h;
          const int cpy = t < 7 ? 0 : (t < 14 ? 1 : t - 12);
          const uint32_t mask = 0x00010001u << sign_pos(t);
          af[2 * h] = cp0[cpy] & mask;
          af[2 * h + 1] = cp1[cpy] & mask;
        }
        const uint2 bw = bop[16 + s][lane];
        mma16816(c, af, bw.x, bw.y);
      }
    }

    // ---- online softmax on the accumulator fragment (log2 domain) ------------------------------
    float sc[4] = {c[0] * cur.kn[0], c[1] * cur.kn[0], c[2] * cur.kn[1], c[3] * cur.kn[1]};
    if (masked) {
      const int tokA = rel + gid, tokB = tokA + 8;
      if (!(tokA < n_valid && tokA <= lim_rel[0])) sc[0] = -INFINITY;
      if (!(tokA < n_valid && tokA <= lim_rel[1])) sc[1] = -INFINITY;
      if (!(tokB < n_valid && tokB <= lim_rel[0])) sc[2] = -INFINITY;
      if (!(tokB < n_valid && tokB <= lim_rel[1])) sc[3] = -INFINITY;
    }
    // m is a reference exponent, not the exact running maximum: it is raised (to the exact maximum of the tile,
    // over the eight token lanes of a query column) only when a score of this tile exceeds it by more than
    // kSlack, so that most tiles need one vote instead of three shuffle rounds.  Weights stay below 2^kSlack,
    // far inside fp16 once multiplied by a value norm, and the merge of the splits only needs l and the
    // accumulators to be relative to the m that is written out.
    constexpr float kSlack = 4.f;
    float mx[2] = {fmaxf(sc[0], sc[2]), fmaxf(sc[1], sc[3])};
    if (__any_sync(QKV_FULL_MASK, mx[0] > m[0] + kSlack || mx[1] > m[1] + kSlack)) {
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(QKV_FULL_MASK, mx[0], o));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(QKV_FULL_MASK, mx[1], o));
      }
      float al[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        al[e] = (mx[e] > m[e]) ? ex2(m[e] - mx[e]) : 1.f;     // ex2(kNone - x) = 0 on the first tile
        m[e] = fmaxf(m[e], mx[e]);
        l[e] *= al[e];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        O[i][0] *= al[0]; O[i][1] *= al[1]; O[i][2] *= al[0]; O[i][3] *= al[1];
      }
    }
    const float p0 = ex2(sc[0] - m[0]), p1 = ex2(sc[1] - m[1]);   // masked scores are -inf: weight 0
    const float p2 = ex2(sc[2] - m[0]), p3 = ex2(sc[3] - m[1]);
    l[0] += p0 + p2;
    l[1] += p1 + p3;
    // weights times value norm, transposed into the B layout (tokens as K, query = gid as N)
    const uint32_t pb0 = movmatrix_trans(pack_half2(p0 * cur.vn[0], p1 * cur.vn[0]));
    const uint32_t pb1 = movmatrix_trans(pack_half2(p2 * cur.vn[1], p3 * cur.vn[1]));

    // ---- values: spread 3-bit codes to nibbles, PRMT look-up, 8 MMAs -----------------------------
    uint32_t nib[4][2];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t lo = __funnelshift_r(cur.v[k][0], cur.v[k][1], odd16);
      const uint32_t hi = cur.v[k][1] >> odd16;
      nib[k][0] = spread(lo & 0xFFFFFFu);
      nib[k][1] = spread(__funnelshift_r(lo, hi, 24) & 0xFFFFFFu);
    }
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t pick = i | ((4 + i) << 4);
        const uint32_t sAB = prmt(nib[0][grp], nib[1][grp], pick);
        const uint32_t sCD = prmt(nib[2][grp], nib[3][grp], pick);
        const uint32_t loAB = prmt(vt_lo[0], vt_lo[1], sAB), hiAB = prmt(vt_hi[0], vt_hi[1], sAB);
        const uint32_t loCD = prmt(vt_lo[0], vt_lo[1], sCD), hiCD = prmt(vt_hi[0], vt_hi[1], sCD);
        uint32_t af[4];
        af[0] = prmt(loAB, hiAB, 0x6240);
        af[1] = prmt(loAB, hiAB, 0x7351);
        af[2] = prmt(loCD, hiCD, 0x6240);
        af[3] = prmt(loCD, hiCD, 0x7351);
        mma16816(O[grp * 4 + i], af, pb0, pb1);
      }
    }
  };

  for (int it = 0; it < n_it; ++it) {
    issue(it + kStages - 1);              // refills the slot that tile it-1 used
    cp_async_wait<kStages - 1>();         // this lane's chunks of tile `it` have landed
    __syncwarp();                         // ... and every other lane's
    TileRegs cur;
    fetch(cur, it);
    __syncwarp();                         // all reads of the slot are done before it is refilled
    process(cur, it);
  }
  cp_async_wait<0>();
  __syncthreads();                        // the reduction buffer below reuses the ring storage

  // ---- per-warp results to shared memory: column sums over the token lanes, then all warps ------
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l[0] += __shfl_xor_sync(QKV_FULL_MASK, l[0], o);
    l[1] += __shfl_xor_sync(QKV_FULL_MASK, l[1], o);
  }
  constexpr float kLn2 = 0.6931471805599453f;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    float* dst = red[warp][2 * tig + e];
    if (gid == 0) {
      dst[0] = m[e] == kNone ? -INFINITY : m[e] * kLn2;   // natural-log units, as the merge expects; -inf = no token
      dst[1] = l[e];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {   // M-tile i holds coordinates 16 gid + 2 i, +1
      dst[2 + 16 * gid + 2 * i] = O[i][e] * inv_sv;
      dst[2 + 16 * gid + 2 * i + 1] = O[i][2 + e] * inv_sv;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nq * (D + 2); idx += blockDim.x) {
    const int r = idx / (D + 2), e = idx % (D + 2);
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) M = fmaxf(M, red[w][r][0]);
    float v = 0.f;
    if (e == 0) {
      v = M;
    } else {
#pragma unroll
      for (int w = 0; w < kMmaWarps; ++w) {
        const float f = (red[w][r][0] == -INFINITY) ? 0.f : expf(red[w][r][0] - M);
        v += f * red[w][r][e];
      }
    }
    const int g = (r0 + r) / a.q_len, qi = (r0 + r) % a.q_len;
    const int64_t qrow = (static_cast<int64_t>(b) * a.Hq + hkv * a.G + g) * a.q_len + qi;
    a.part[(qrow * a.n_splits + split) * (D + 2) + e] = v;
  }

  // ---- the CTA that finishes a (batch, kv head) last merges its splits and applies Pi ----------------
  __shared__ bool last_split;
  __threadfence();                                   // this CTA's partials are visible device-wide
  __syncthreads();
  if (threadIdx.x == 0)
    last_split = atomicAdd(a.arrivals + seg * gridDim.y + blockIdx.y, 1u) == static_cast<unsigned>(a.n_splits - 1);
  __syncthreads();
  if (!last_split) return;
  __threadfence();                                   // ... and so are everyone else's, now
  float* vec = reinterpret_cast<float*>(pool);       // [8][D] merged, normalised accumulators
  float* wgt = vec + 8 * D;                          // [8][kMaxSplits] weights of the splits
  float* invl = wgt + 8 * kMaxSplits;                // [8]
  for (int r = warp; r < nq; r += kMmaWarps) {       // a warp per query row
    const int g = (r0 + r) / a.q_len, qi = (r0 + r) % a.q_len;
    const int64_t qrow = (static_cast<int64_t>(b) * a.Hq + hkv * a.G + g) * a.q_len + qi;
    const float* pp = a.part + qrow * a.n_splits * (D + 2);
    float M = -INFINITY;
    for (int sp = lane; sp < a.n_splits; sp += 32) M = fmaxf(M, __ldcg(pp + sp * (D + 2)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(QKV_FULL_MASK, M, o));
    float L = 0.f;
    for (int sp = lane; sp < a.n_splits; sp += 32) {
      const float mm = __ldcg(pp + sp * (D + 2));
      const float f = (mm == -INFINITY) ? 0.f : expf(mm - M);
      wgt[r * kMaxSplits + sp] = f;
      L += f * __ldcg(pp + sp * (D + 2) + 1);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(QKV_FULL_MASK, L, o);
    if (lane == 0) invl[r] = 1.f / fmaxf(L, 1e-30f);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nq * D; idx += blockDim.x) {
    const int r = idx / D, j = idx % D;
    const int g = (r0 + r) / a.q_len, qi = (r0 + r) % a.q_len;
    const int64_t qrow = (static_cast<int64_t>(b) * a.Hq + hkv * a.G + g) * a.q_len + qi;
    const float* pp = a.part + qrow * a.n_splits * (D + 2);
    float v = 0.f;
    for (int sp = 0; sp < a.n_splits; ++sp) v += wgt[r * kMaxSplits + sp] * __ldcg(pp + sp * (D + 2) + 2 + j);
    vec[r * D + j] = v * invl[r];
  }
  __syncthreads();
  {
    const int i = threadIdx.x;                       // output coordinate (blockDim.x == D)
    float o[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) o[r] = 0.f;
#pragma unroll 8
    for (int j = 0; j < D; ++j) {
      const float mval = __ldg(a.Pi + j * D + i);
#pragma unroll
      for (int r = 0; r < 8; ++r) o[r] = fmaf(vec[r * D + j], mval, o[r]);
    }
    for (int r = 0; r < nq; ++r) {
      const int g = (r0 + r) / a.q_len, qi = (r0 + r) % a.q_len;
      const int64_t qrow = (static_cast<int64_t>(b) * a.Hq + hkv * a.G + g) * a.q_len + qi;
      a.out[qrow * D + i] = o[r];
    }
  }
}

bool mma_path_ok(int d, int key_bits, int val_bits, int group, int q_len) {
  (void)group; (void)q_len;            // any number of query rows: tiles of eight
  return d == 128 && key_bits == 3 && val_bits == 3;
}

int launch_attend_mma(const AttnArgs& a, cudaStream_t st) {
  const dim3 grid(a.B * a.Hkv, (a.G * a.q_len + 7) / 8, a.n_splits);
  // Programmatic dependent launch: the grid may start while the kernel before it in the stream (the query
  // rotation, which releases its dependents at once) is still running; the kernel waits for that kernel's
  // completion before it reads anything that kernel writes.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kMmaWarps * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t err = a.block_table ? cudaLaunchKernelEx(&cfg, attend_decode_mma_kernel<true>, a)
                                        : cudaLaunchKernelEx(&cfg, attend_decode_mma_kernel<false>, a);
  if (err != cudaSuccess) return QKV_ELAUNCH;
  return check_launch();
}

}  // namespace qkv
