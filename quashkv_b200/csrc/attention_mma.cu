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

#include "attention_common.cuh"

namespace qkv {

constexpr int kMmaWarps = 4;
constexpr int kTile = 16;                 // tokens per warp step
constexpr float kLog2e = 1.4426950408889634f;

// Sign bits become MMA operands without a per-pair shift: a masked single bit at position p of a
// 16-bit half IS an fp16 number (0 when clear, v1(p) when set: 2, 2^-7, 2^-11, 2^-13, 2^-14 and
// the subnormals 2^-15, 2^-16 for p = 14..8), so `word & mask` is the operand and the weight
// carries 2 / v1(p); the constant -sum(w) goes into the accumulator's initial value.  Bit 15 (the
// fp16 sign) cannot be used, so four copies of the word (as is, <<7, >>1, <<13) bring all 16
// bit pairs (j, j+16) to positions 8..14.  Pair t of a 32-coordinate slice:
//   t 0..6 : word,      p = 8+t,  coordinates (8+t, 24+t)      t 14: word>>1,  p = 14, (15, 31)
//   t 7..13: word<<7,   p = 1+t,  coordinates (t-6, t+10)      t 15: word<<13, p = 13, (0, 16)
__host__ __device__ constexpr int sign_pos(int t) { return t < 7 ? 8 + t : (t < 14 ? 1 + t : (t == 14 ? 14 : 13)); }
__host__ __device__ constexpr int sign_coord(int t) { return t < 7 ? 8 + t : (t < 14 ? t - 6 : (t == 14 ? 15 : 0)); }
__host__ __device__ constexpr float sign_v1(int p) {
  return p == 14 ? 2.f : (p == 13 ? 0.0078125f : (p == 12 ? 4.8828125e-4f : 1.f / static_cast<float>(1 << (24 - p))));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// 8 three-bit fields (24 bits) -> 8 nibbles: sum c_k 8^k  ->  sum c_k 16^k.
__device__ __forceinline__ uint32_t spread3to4(uint32_t g) {
  g = g + 15u * (g & 0xFFF000u);          // 12-bit halves to 16-bit stride
  g = g + 3u * (g & 0x0FC00FC0u);         // 6-bit pairs to 8-bit stride
  return g + (g & 0x38383838u);           // 3-bit fields to 4-bit stride
}

struct TileRegs {
  uint2 kc[2];      // key codes: this lane's 8 bytes of rows gid, gid+8
  uint32_t ks[2];   // sign words of the same rows
  float kn[2], vn[2];
  uint32_t v[4][2]; // value words of tokens 2tig, 2tig+1, 2tig+8, 2tig+9
};

struct MmaPtrs {
  const uint8_t* kcode; const uint8_t* ksign; const uint8_t* vcode; const float* knorm; const float* vnorm;
};

__device__ __forceinline__ void load_tile(TileRegs& r, const MmaPtrs& p, int64_t t0, int64_t t_end, int gid,
                                          int tig) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int64_t tok = t0 + gid + 8 * h;
    if (tok < t_end) {
      r.kc[h] = __ldg(reinterpret_cast<const uint2*>(p.kcode + tok * 32) + tig);
      r.ks[h] = __ldg(reinterpret_cast<const uint32_t*>(p.ksign + tok * 16) + tig);
      r.kn[h] = __ldg(p.knorm + tok);
      r.vn[h] = __ldg(p.vnorm + tok);
    } else {
      r.kc[h] = make_uint2(0u, 0u);
      r.ks[h] = 0u;
      r.kn[h] = 0.f;
      r.vn[h] = 0.f;
    }
  }
  const int wo = (3 * gid) >> 1;           // first word of this lane's 48 bits (coords 16 gid ..)
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int64_t tok = t0 + 2 * tig + (k & 1) + 8 * (k >> 1);
    if (tok < t_end) {
      const uint32_t* row = reinterpret_cast<const uint32_t*>(p.vcode + tok * 48);
      r.v[k][0] = __ldg(row + wo);
      r.v[k][1] = __ldg(row + wo + 1);
    } else {
      r.v[k][0] = 0u;
      r.v[k][1] = 0u;
    }
  }
}

// One warp: for a table of n centroids find the scale s in [1,2) (2048 candidates) that makes the
// largest relative fp16 rounding error of s*c_i smallest, so that the systematic error of the
// fp16 operand tables drops well below 2^-12.
__device__ float best_fp16_scale(const float* cent, int n, int lane) {
  float best_err = 1e30f, best_s = 1.f;
  for (int k = 0; k < 64; ++k) {
    const float s = 1.f + static_cast<float>(lane + 32 * k) * (1.f / 2048.f);
    float err = 0.f;
    for (int i = 0; i < n; ++i) {
      const float v = cent[i] * s;
      if (v != 0.f) err = fmaxf(err, fabsf(__half2float(__float2half_rn(v)) - v) / fabsf(v));
    }
    if (err < best_err) { best_err = err; best_s = s; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float e2 = __shfl_xor_sync(QKV_FULL_MASK, best_err, o);
    const float s2 = __shfl_xor_sync(QKV_FULL_MASK, best_s, o);
    if (e2 < best_err || (e2 == best_err && s2 < best_s)) { best_err = e2; best_s = s2; }
  }
  return best_s;
}

// tables[0..1] key low/high bytes, [2..3] value low bytes, [4..5] value high bytes,
// [6] 1/key scale, [7] 1/value scale (floats).
__global__ void prepare_tables_kernel(const float* __restrict__ kcent, const float* __restrict__ vcent,
                                      uint32_t* __restrict__ tables) {
  const int lane = threadIdx.x;
  const float sk = best_fp16_scale(kcent, 4, lane), sv = best_fp16_scale(vcent, 8, lane);
  if (lane != 0) return;
  uint32_t t[6] = {0, 0, 0, 0, 0, 0};
  for (int i = 0; i < 4; ++i) {
    const uint32_t h = __half_as_ushort(__float2half_rn(kcent[i] * sk));
    t[0] |= (h & 0xFFu) << (8 * i);
    t[1] |= (h >> 8) << (8 * i);
  }
  for (int i = 0; i < 8; ++i) {
    const uint32_t h = __half_as_ushort(__float2half_rn(vcent[i] * sv));
    t[2 + (i >> 2)] |= (h & 0xFFu) << (8 * (i & 3));
    t[4 + (i >> 2)] |= (h >> 8) << (8 * (i & 3));
  }
  for (int i = 0; i < 6; ++i) tables[i] = t[i];
  tables[6] = __float_as_uint(1.f / sk);
  tables[7] = __float_as_uint(1.f / sv);
}

__global__ void __launch_bounds__(kMmaWarps * 32, 3) attend_decode_mma_kernel(AttnArgs a) {
  constexpr int D = 128;
  __shared__ float q_s[8][2 * D];                    // [query row][q_rot*scale | sign weights]
  __shared__ float red[kMmaWarps][8][D + 2];         // per warp and query: max, sum, accumulator
  __shared__ float wsum[8];                          // sum of the sign weights per query row

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int split = blockIdx.x, seg = blockIdx.z;
  const int b = seg / a.Hkv, hkv = seg % a.Hkv;
  const int nq = a.G * a.q_len;

  for (int idx = threadIdx.x; idx < 8 * 2 * D; idx += blockDim.x) {
    const int r = idx / (2 * D), e = idx % (2 * D);
    float v = 0.f;
    if (r < nq) {
      const int g = r / a.q_len, qi = r % a.q_len;
      const int64_t qrow = (static_cast<int64_t>(b) * a.Hq + hkv * a.G + g) * a.q_len + qi;
      v = a.qk[qrow * 2 * D + e];
    }
    q_s[r][e] = v;
  }
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = 0.f;
    for (int j = 0; j < D; ++j) t += q_s[threadIdx.x][D + j];
    wsum[threadIdx.x] = t * kLog2e;
  }
  __syncthreads();

  // ---- register-resident B operands for query column n = gid ---------------------------------
  // Key-code k-step s = 4*word + grp covers this lane's coordinates base + {o, o+2 | o+4, o+6},
  // base = 32 tig + 16 word, o = 8*(grp&1) + (grp>>1): the order in which the PRMT decode below
  // produces them.  Sign k-step s covers 32 tig + {2s, 2s+16 | 2s+1, 2s+17}.
  const float inv_sk = __uint_as_float(a.tables[6]), inv_sv = __uint_as_float(a.tables[7]);
  uint32_t qb[8][2], ql[8][2], wb[8][2];      // query high part, low part (q - fp16(q)), sign weights
  {
    const float qf = kLog2e * inv_sk;
    const float* q = q_s[gid];
    const float* w = q_s[gid] + D;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const int word = s >> 2, grp = s & 3;
      const int c0 = 32 * tig + 16 * word + 8 * (grp & 1) + (grp >> 1);
      float v[4], r[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[e] = q[c0 + 2 * e] * qf;
        r[e] = v[e] - __half2float(__float2half_rn(v[e]));
      }
      qb[s][0] = pack_half2(v[0], v[1]);
      qb[s][1] = pack_half2(v[2], v[3]);
      ql[s][0] = pack_half2(r[0], r[1]);
      ql[s][1] = pack_half2(r[2], r[3]);
#pragma unroll
      for (int h = 0; h < 2; ++h) {           // pairs t = 2s, 2s+1 of this lane's 32 coordinates
        const int t = 2 * s + h, j = 32 * tig + sign_coord(t);
        const float f = 2.f * kLog2e / sign_v1(sign_pos(t));
        wb[s][h] = pack_half2(w[j] * f, w[j + 16] * f);
      }
    }
  }
  // ---- PRMT look-up tables: low and high bytes of the fp16 centroids ---------------------------
  const uint32_t kt_lo = a.tables[0], kt_hi = a.tables[1];
  const uint32_t vt_lo[2] = {a.tables[2], a.tables[3]}, vt_hi[2] = {a.tables[4], a.tables[5]};
  // causal limits of this lane's two query columns (2 tig, 2 tig + 1)
  int lim[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = 2 * tig + e;
    lim[e] = (r < nq) ? (a.causal ? static_cast<int>(a.kv_len - a.q_len + r % a.q_len) : 0x7fffffff) : -1;
  }

  const int64_t seg_row0 = static_cast<int64_t>(seg) * a.cache.capacity;
  MmaPtrs p;
  p.kcode = a.cache.k_codes + seg_row0 * 32;
  p.ksign = a.cache.k_signs + seg_row0 * 16;
  p.vcode = a.cache.v_codes + seg_row0 * 48;
  p.knorm = a.cache.k_norms + seg_row0;
  p.vnorm = a.cache.v_norms + seg_row0;

  const int64_t t_begin = split * a.split_len;
  int64_t t_end = t_begin + a.split_len;
  if (t_end > a.kv_len) t_end = a.kv_len;

  float O[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int odd16 = (gid & 1) * 16;

  const float ci0 = -wsum[2 * tig], ci1 = -wsum[2 * tig + 1];   // accumulator start: -sum of sign weights
  TileRegs cur, nxt;
  int64_t t0 = t_begin + static_cast<int64_t>(warp) * kTile;
  if (t0 < t_end) load_tile(cur, p, t0, t_end, gid, tig);
  for (; t0 < t_end; t0 += kMmaWarps * kTile) {
    const int64_t tn = t0 + kMmaWarps * kTile;
    if (tn < t_end) load_tile(nxt, p, tn, t_end, gid, tig);

    // ---- scores: 8 MMAs on key codes, 8 on sign bits --------------------------------------------
    float c[4] = {ci0, ci1, ci0, ci1};
#pragma unroll
    for (int word = 0; word < 2; ++word) {
      const uint32_t w0 = word ? cur.kc[0].y : cur.kc[0].x;
      const uint32_t w1 = word ? cur.kc[1].y : cur.kc[1].x;
      const uint32_t x0 = w0 & 0x33333333u, y0 = (w0 >> 2) & 0x33333333u;
      const uint32_t x1 = w1 & 0x33333333u, y1 = (w1 >> 2) & 0x33333333u;
#pragma unroll
      for (int grp = 0; grp < 4; ++grp) {
        const uint32_t s0 = (grp >> 1 ? y0 : x0) >> (16 * (grp & 1));
        const uint32_t s1 = (grp >> 1 ? y1 : x1) >> (16 * (grp & 1));
        const uint32_t lo0 = prmt(kt_lo, kt_hi, s0), hi0 = prmt(kt_hi, kt_lo, s0);
        const uint32_t lo1 = prmt(kt_lo, kt_hi, s1), hi1 = prmt(kt_hi, kt_lo, s1);
        uint32_t af[4];
        af[0] = prmt(lo0, hi0, 0x5140);
        af[1] = prmt(lo1, hi1, 0x5140);
        af[2] = prmt(lo0, hi0, 0x7362);
        af[3] = prmt(lo1, hi1, 0x7362);
        mma16816(c, af, qb[word * 4 + grp][0], qb[word * 4 + grp][1]);
        mma16816(c, af, ql[word * 4 + grp][0], ql[word * 4 + grp][1]);
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
        mma16816(c, af, wb[s][0], wb[s][1]);
      }
    }

    // ---- online softmax on the accumulator fragment (log2 domain) ------------------------------
    const int64_t tokA = t0 + gid, tokB = tokA + 8;
    float sc[4];
    sc[0] = (tokA < t_end && tokA <= lim[0]) ? c[0] * cur.kn[0] : -INFINITY;
    sc[1] = (tokA < t_end && tokA <= lim[1]) ? c[1] * cur.kn[0] : -INFINITY;
    sc[2] = (tokB < t_end && tokB <= lim[0]) ? c[2] * cur.kn[1] : -INFINITY;
    sc[3] = (tokB < t_end && tokB <= lim[1]) ? c[3] * cur.kn[1] : -INFINITY;
    float mx[2] = {fmaxf(sc[0], sc[2]), fmaxf(sc[1], sc[3])};
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      mx[0] = fmaxf(mx[0], __shfl_xor_sync(QKV_FULL_MASK, mx[0], o));
      mx[1] = fmaxf(mx[1], __shfl_xor_sync(QKV_FULL_MASK, mx[1], o));
    }
    if (__any_sync(QKV_FULL_MASK, mx[0] > m[0] || mx[1] > m[1])) {
      float al[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        al[e] = (mx[e] > m[e]) ? ex2(m[e] - mx[e]) : 1.f;     // ex2(-inf) = 0 on the first tile
        m[e] = fmaxf(m[e], mx[e]);
        l[e] *= al[e];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        O[i][0] *= al[0]; O[i][1] *= al[1]; O[i][2] *= al[0]; O[i][3] *= al[1];
      }
    }
    const float ms[2] = {m[0] == -INFINITY ? 0.f : m[0], m[1] == -INFINITY ? 0.f : m[1]};
    const float p0 = ex2(sc[0] - ms[0]), p1 = ex2(sc[1] - ms[1]);
    const float p2 = ex2(sc[2] - ms[0]), p3 = ex2(sc[3] - ms[1]);
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
      nib[k][0] = spread3to4(lo & 0xFFFFFFu);
      nib[k][1] = spread3to4(__funnelshift_r(lo, hi, 24) & 0xFFFFFFu);
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
    cur = nxt;
  }

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
      dst[0] = m[e] * kLn2;       // natural-log units, as the merge kernel expects (-inf stays -inf)
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
    const int g = r / a.q_len, qi = r % a.q_len;
    const int64_t qrow = (static_cast<int64_t>(b) * a.Hq + hkv * a.G + g) * a.q_len + qi;
    a.part[(qrow * a.n_splits + split) * (D + 2) + e] = v;
  }
}

bool mma_path_ok(int d, int key_bits, int val_bits, int group, int q_len) {
  return d == 128 && key_bits == 3 && val_bits == 3 && group * q_len <= 8;
}

int launch_prepare_tables(const float* kcent, const float* vcent, uint32_t* tables, cudaStream_t st) {
  prepare_tables_kernel<<<1, 32, 0, st>>>(kcent, vcent, tables);
  return check_launch();
}

int launch_attend_mma(const AttnArgs& a, cudaStream_t st) {
  const dim3 grid(a.n_splits, 1, a.B * a.Hkv);
  attend_decode_mma_kernel<<<grid, kMmaWarps * 32, 0, st>>>(a);
  return check_launch();
}

}  // namespace qkv
