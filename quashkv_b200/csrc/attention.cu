// Attention over the packed compressed cache (generic path: any key/value bit width,
// d in {32,64,96,128}, grouped-query heads, q_len >= 1, optional causal mask).
//
// Three kernels per call:
//   1. rotate_queries: q_rot = q @ Pi^T once per query row; stores q_rot*scale and
//      qjl_scale*scale*|q_rot|*S so that the streaming loop needs no other constants.
//   2. attend_split: grid (split, query tile, batch*kv_head).  A warp step covers 8 tokens
//      (d>=96) / 16 (d=64) / 32 (d=32): lane = (token, 32-coordinate slot).  Each lane reads
//      its slot's words of the key-code, sign and value-code rows (adjacent lanes read
//      adjacent words, so a warp load covers whole contiguous rows), scores 4 query rows in
//      the rotated domain, runs an online softmax and accumulates sum_k p_k * v_norm_k *
//      c_V[code] in the ROTATED domain in registers.  Per split it writes (max, sum, acc[d]).
//   3. merge_splits: combines the splits of a query row and applies Pi once
//      (out = (acc / sum) @ Pi), which equals un-rotating every value first because the
//      rotation is linear.
#include <math.h>
#include <stdlib.h>

#include "attention_common.cuh"
#include "mma_decode.cuh"

namespace qkv {

// q_rot = q @ Pi^T for 4 query rows per CTA.  A warp takes eight rows of Pi at a time, a lane four columns of
// each (coalesced 16-byte loads, all eight in flight), against the four query rows; the 32 partial sums of a
// lane are reduced over the warp by a butterfly of 31 exchanges, after which lane L holds the total of Pi row
// (L >> 2) of the eight and query row L & 3.
constexpr int kRowsPerCta = 4;

// Rows i0 .. i0 + 7 of Pi (d columns, d a multiple of 4, at most 128) against four vectors held as the lane's
// four columns each: on return v[0] of lane L is <Pi[i0 + (L >> 2)], vector L & 3>.
__device__ __forceinline__ void rotate_eight_rows(const float* __restrict__ Pi, int d, int i0, int lane,
                                                  const float4 (&x)[kRowsPerCta], float (&v)[32]) {
  float4 m[8];
#pragma unroll
  for (int o = 0; o < 8; ++o)
    m[o] = (i0 + o < d && 4 * lane < d) ? __ldg(reinterpret_cast<const float4*>(Pi + static_cast<int64_t>(i0 + o) * d) + lane)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int o = 0; o < 8; ++o)
#pragma unroll
    for (int r = 0; r < kRowsPerCta; ++r)
      v[4 * o + r] = fmaf(m[o].x, x[r].x, fmaf(m[o].y, x[r].y, fmaf(m[o].z, x[r].z, m[o].w * x[r].w)));
#pragma unroll
  for (int s = 16, n = 32; s >= 1; s >>= 1, n >>= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int k = 0; k < n / 2; ++k) {
      const float send = upper ? v[k] : v[k + n / 2];
      const float keep = upper ? v[k + n / 2] : v[k];
      v[k] = keep + __shfl_xor_sync(QKV_FULL_MASK, send, s);
    }
  }
}
// Four rows of Pi already in registers (`m`, this lane's four columns of rows i0 .. i0 + 3) against eight vectors:
// on return v[0] of lane L is <Pi[i0 + (L >> 3)], vector L & 7>.
__device__ __forceinline__ void rotate_four_rows_eight(const float4 (&m)[4], const float4 (&x)[8], float (&v)[32]) {
#pragma unroll
  for (int o = 0; o < 4; ++o)
#pragma unroll
    for (int r = 0; r < 8; ++r)
      v[8 * o + r] = fmaf(m[o].x, x[r].x, fmaf(m[o].y, x[r].y, fmaf(m[o].z, x[r].z, m[o].w * x[r].w)));
#pragma unroll
  for (int s = 16, n = 32; s >= 1; s >>= 1, n >>= 1) {
    const bool upper = (threadIdx.x & s) != 0;
#pragma unroll
    for (int k = 0; k < n / 2; ++k) {
      const float send = upper ? v[k] : v[k + n / 2];
      const float keep = upper ? v[k + n / 2] : v[k];
      v[k] = keep + __shfl_xor_sync(QKV_FULL_MASK, send, s);
    }
  }
}

__global__ void __launch_bounds__(128) rotate_queries_kernel(const void* __restrict__ q, int q_dtype, int64_t rows,
                                                             int d, const float* __restrict__ Pi,
                                                             const float* __restrict__ S, float qjl_scale,
                                                             float scale, float* __restrict__ qk,
                                                             const float* __restrict__ kcent,
                                                             const float* __restrict__ vcent,
                                                             uint32_t* __restrict__ tables, int n_counters) {
  // The attention kernel that follows may be launched as a programmatic dependent: let it start right away (it
  // waits for this grid's completion before it reads the rotated queries, the tables or the counters).
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  if (tables != nullptr && blockIdx.x == gridDim.x - 1) {   // one extra CTA: look-up tables of the
    unsigned* arrivals = reinterpret_cast<unsigned*>(reinterpret_cast<unsigned char*>(tables) + kAttnHeaderBytes);
    for (int i = threadIdx.x; i < n_counters; i += blockDim.x) arrivals[i] = 0u;   // tensor-core path,
    prepare_tables_cta(kcent, vcent, tables);                                        // and its counters
    return;
  }
  __shared__ __align__(16) float x_s[kRowsPerCta][kMaxD];
  const int i = threadIdx.x;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * kRowsPerCta;
  for (int idx = threadIdx.x; idx < kRowsPerCta * kMaxD; idx += blockDim.x) {
    const int r = idx / kMaxD, j = idx % kMaxD;
    x_s[r][j] = (row0 + r < rows && j < d) ? load_float(q, q_dtype, (row0 + r) * d + j) : 0.f;
  }
  __syncthreads();
  const int lane = i & 31, warp = i >> 5;
  float4 x[kRowsPerCta];
#pragma unroll
  for (int r = 0; r < kRowsPerCta; ++r) x[r] = *reinterpret_cast<const float4*>(&x_s[r][4 * lane]);   // zero beyond d
  for (int i0 = 8 * warp; i0 < d; i0 += 32) {
    float v[32];
    rotate_eight_rows(Pi, d, i0, lane, x, v);
    const int io = i0 + (lane >> 2), ro = lane & 3;
    if (io < d && row0 + ro < rows) {
      qk[(row0 + ro) * 2 * d + io] = v[0] * scale;
      qk[(row0 + ro) * 2 * d + d + io] = (qjl_scale * scale) * (fabsf(v[0]) * S[io]);
    }
  }
}


// Query rotation for the tiled attention with scores from bit planes (head_dim 128, up to four query rows per
// KV head): CTA k rotates the rows of (batch, kv head) k, 128 threads per row, and builds plane image k; one
// extra CTA prepares the look-up tables and zeroes the arrival counters.
//
// Element (plane, coordinate j) of a token is a bit worth 2^p in its operand byte: p = 2 (j & 3) + plane for
// the code planes (plane 0 / 1: low / high bit of the 2-bit key code, coordinates four to a byte), p = j & 7
// for the sign plane.  With the key table written as c(u) = g0 + g1 (u & 1) + g2 (u >> 1) the bit weighs
// log2e g1 q_j, log2e g2 q_j, or 2 log2e w_j for a sign bit (in the score before the key norm, log2 domain).
// The B operand holds y = weight * s / 2^p, s per query row bringing the largest |y| to 127, in radix 128 as
// t1 + t2 / 128 + t3 / 128^2 + t4 / 128^3 (signed bytes): columns n and n + 4 of the first accumulator chain
// take t1, t2 of row n, those of the second chain t3, t4.  Lane L = 4 n' + t of k-step s holds, in byte b of
// register r, the element that the attention kernel cuts out of the lane's word with 0x01010101 << (2 f + r):
// code word s >> 2, f = s & 3, coordinate 32 t + 16 (s >> 2) + 4 b + f for s < 8; sign word, f = s - 8,
// coordinate 32 t + 8 b + 2 f + r for s >= 8.
__global__ void __launch_bounds__(512) rotate_planes_kernel(const void* __restrict__ q, int q_dtype, int64_t rows,
                                                            const float* __restrict__ Pi, const float* __restrict__ S,
                                                            float qjl_scale, float scale, float* __restrict__ qk,
                                                            const float* __restrict__ kcent,
                                                            const float* __restrict__ vcent,
                                                            uint32_t* __restrict__ tables, int n_counters,
                                                            int rows_per_cta, PlaneImage* __restrict__ planes) {
  // Launched as a programmatic dependent itself: when the kernel before it in the stream releases its dependents
  // early (the scan of the previous decode step does), this grid is already resident when that kernel ends.
  // Nothing is read or written before the wait.
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  if (blockIdx.x == gridDim.x - 1) {
    unsigned* arrivals = reinterpret_cast<unsigned*>(reinterpret_cast<unsigned char*>(tables) + kAttnHeaderBytes);
    for (int i = threadIdx.x; i < n_counters; i += blockDim.x) arrivals[i] = 0u;
    prepare_tables_cta(kcent, vcent, tables);
    return;
  }
  constexpr int D = 128;
  constexpr float kL2e = 1.4426950408889634f;
  __shared__ __align__(16) float x_s[kRowsPerCta][D];
  __shared__ float q_s[kRowsPerCta][D], w_s[kRowsPerCta][D];
  __shared__ float red_s[kRowsPerCta][4][3];
  __shared__ float scale_s[kRowsPerCta];
  const int r = threadIdx.x >> 7, i = threadIdx.x & 127, lane = threadIdx.x & 31, wr = (threadIdx.x >> 5) & 3;
  const int warp = threadIdx.x >> 5;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
  {
    const int64_t row = row0 + r;
    x_s[r][i] = (r < rows_per_cta && row < rows) ? load_float(q, q_dtype, row * D + i) : 0.f;
  }
  const float g0 = kcent[0], g1 = kcent[1] - kcent[0], g2 = kcent[2] - kcent[0];
  // Rotation: warp w takes rows 8 w .. 8 w + 7 of Pi (rotate_eight_rows).
  __syncthreads();
  float v[32];
  {
    float4 x[kRowsPerCta];
#pragma unroll
    for (int rr = 0; rr < kRowsPerCta; ++rr) x[rr] = *reinterpret_cast<const float4*>(&x_s[rr][4 * lane]);
    rotate_eight_rows(Pi, D, 8 * warp, lane, x, v);
  }
  {
    const int io = 8 * warp + (lane >> 2), ro = lane & 3;            // this lane's output: coordinate, query row
    const int64_t row = row0 + ro;
    const bool live = ro < rows_per_cta && row < rows;
    const float acc = v[0];
    const float qo = live ? acc * scale : 0.f;
    const float wo = live ? (qjl_scale * scale) * (fabsf(acc) * S[io]) : 0.f;
    if (live) {
      qk[row * 2 * D + io] = qo;
      qk[row * 2 * D + D + io] = wo;
    }
    q_s[ro][io] = qo;
    w_s[ro][io] = wo;
  }
  __syncthreads();
  const float qv = q_s[r][i], wv = w_s[r][i];
  {
    const float e0 = 1.f / static_cast<float>(1 << (2 * (i & 3))), e2 = 1.f / static_cast<float>(1 << (i & 7));
    float mx = fmaxf(fmaxf(fabsf(qv * g1) * e0, fabsf(qv * g2) * (0.5f * e0)), 2.f * fabsf(wv) * e2);
    float sq = qv, sw = wv;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(QKV_FULL_MASK, mx, o));
      sq += __shfl_xor_sync(QKV_FULL_MASK, sq, o);
      sw += __shfl_xor_sync(QKV_FULL_MASK, sw, o);
    }
    if (lane == 0) { red_s[r][wr][0] = mx; red_s[r][wr][1] = sq; red_s[r][wr][2] = sw; }
  }
  __syncthreads();
  PlaneImage* img = planes + blockIdx.x;
  if (threadIdx.x < kRowsPerCta) {
    const int n = threadIdx.x;
    float mx = 0.f, sq = 0.f, sw = 0.f;
    for (int w = 0; w < 4; ++w) { mx = fmaxf(mx, red_s[n][w][0]); sq += red_s[n][w][1]; sw += red_s[n][w][2]; }
    mx *= kL2e;
    scale_s[n] = mx > 0.f ? 127.f / mx : 0.f;
    img->inv[n] = mx * (1.f / 127.f);
    img->cst[n] = kL2e * (g0 * sq - sw);
  }
  __syncthreads();
  if (threadIdx.x < 12 * 32) {
    const int item = threadIdx.x;
    const int s = item >> 5, L = item & 31, t = L & 3, n = (L >> 2) & 3, hi = L >> 4;
    const float sc = scale_s[n];
    uint32_t ra[2] = {0u, 0u}, rb[2] = {0u, 0u};
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        int p; float x;
        if (s < 8) {
          p = 2 * (s & 3) + rr;
          x = kL2e * (rr ? g2 : g1) * q_s[n][32 * t + 16 * (s >> 2) + 4 * b + (s & 3)];
        } else {
          p = 2 * (s - 8) + rr;
          x = 2.f * kL2e * w_s[n][32 * t + 8 * b + p];
        }
        const float y = x * sc * (1.f / static_cast<float>(1 << p));
        const float t1 = fminf(fmaxf(rintf(y), -127.f), 127.f);
        const float r1 = (y - t1) * 128.f;
        const float t2 = fminf(fmaxf(rintf(r1), -127.f), 127.f);
        const float r2 = (r1 - t2) * 128.f;
        const float t3 = fminf(fmaxf(rintf(r2), -127.f), 127.f);
        const float r3 = (r2 - t3) * 128.f;
        const float t4 = fminf(fmaxf(rintf(r3), -127.f), 127.f);
        const int ba = static_cast<int>(hi ? t2 : t1), bb = static_cast<int>(hi ? t4 : t3);
        ra[rr] |= (static_cast<uint32_t>(ba) & 0xFFu) << (8 * b);
        rb[rr] |= (static_cast<uint32_t>(bb) & 0xFFu) << (8 * b);
      }
    }
    img->bop[s][L] = make_uint4(ra[0], ra[1], rb[0], rb[1]);
  }
}

// Query rotation for the tiled attention with fp16 scores (head_dim 128).  A CTA rotates kGroupsPerCta
// consecutive groups of eight query rows of a (batch, kv head) (rows n0 .. n0 + 7 of the head's G * q_len rows;
// with `lo4` four rows, columns 4..7 carrying the fp16 rounding residual of columns 0..3), every four rows of Pi
// being loaded once for all of them, and builds their GroupImages: the B operands in the order the scan's MMAs
// consume them.  Key-code k-step s = 4 * word + f covers a lane's coordinates 32 t + 16 word + {f, 4 + f | 8 + f,
// 12 + f}; sign k-step s covers 32 t + {2s, 2s + 16 | 2s + 1, 2s + 17} through sign_coord / sign_pos
// (mma_decode.cuh).  One extra CTA prepares the look-up tables and the counters.
constexpr int kGroupsPerCta = 2;
__global__ void __launch_bounds__(128) rotate_groups_kernel(const void* __restrict__ q, int q_dtype,
                                                            const float* __restrict__ Pi, const float* __restrict__ S,
                                                            float qjl_scale, float scale,
                                                            const float* __restrict__ kcent,
                                                            const float* __restrict__ vcent,
                                                            uint32_t* __restrict__ tables, int n_counters,
                                                            int nq_all, int groups_per_seg, int n_groups, int lo4,
                                                            GroupImage* __restrict__ groups) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  if (blockIdx.x == gridDim.x - 1) {
    unsigned* arrivals = reinterpret_cast<unsigned*>(reinterpret_cast<unsigned char*>(tables) + kAttnHeaderBytes);
    for (int i = threadIdx.x; i < n_counters; i += blockDim.x) arrivals[i] = 0u;
    prepare_tables_cta(kcent, vcent, tables);
    return;
  }
  constexpr int D = 128, NGC = kGroupsPerCta;
  constexpr float kL2e = 1.4426950408889634f;
  __shared__ __align__(16) float x_s[NGC][8][D];
  __shared__ float q_s[NGC][8][D], w_s[NGC][8][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
  const int g_first = NGC * blockIdx.x;
  for (int idx = threadIdx.x; idx < NGC * 8 * D; idx += blockDim.x) {
    const int gl = idx / (8 * D), r = (idx >> 7) & 7, j = idx & 127;
    const int g_idx = g_first + gl;
    float v = 0.f;
    if (g_idx < n_groups) {
      const int seg = g_idx / groups_per_seg, n0 = 8 * (g_idx % groups_per_seg);
      const int rq = lo4 ? (r & 3) : r;
      if (n0 + rq < nq_all)                              // the head's rows are consecutive query rows
        v = load_float(q, q_dtype, (static_cast<int64_t>(seg) * nq_all + n0 + rq) * D + j);
    }
    x_s[gl][r][j] = v;
  }
  const float inv_sk = 1.f / best_fp16_scale_cta(kcent, 4);      // the scale the table CTA gives the key table (syncs)
  const float qf = kL2e * inv_sk;
  for (int i0 = 4 * warp; i0 < D; i0 += 16) {          // a warp takes four rows of Pi at a time
    float4 m[4];
#pragma unroll
    for (int o = 0; o < 4; ++o) m[o] = __ldg(reinterpret_cast<const float4*>(Pi + static_cast<int64_t>(i0 + o) * D) + lane);
#pragma unroll
    for (int gl = 0; gl < NGC; ++gl) {
      float4 x[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) x[r] = *reinterpret_cast<const float4*>(&x_s[gl][r][4 * lane]);
      float v[32];
      rotate_four_rows_eight(m, x, v);
      const int io = i0 + (lane >> 3), ro = lane & 7;
      q_s[gl][ro][io] = v[0] * scale;
      w_s[gl][ro][io] = (qjl_scale * scale) * (fabsf(v[0]) * S[io]);
    }
  }
  __syncthreads();
#pragma unroll 1
  for (int gl = 0; gl < NGC; ++gl) {
    const int g_idx = g_first + gl;
    if (g_idx >= n_groups) break;
    GroupImage* img = groups + g_idx;
#pragma unroll
    for (int h = 0; h < 2; ++h) {           // a warp sums the sign weights of two query columns
      const int col = 2 * warp + h;
      const float* w = w_s[gl][col];
      float t = (w[lane] + w[lane + 32]) + (w[lane + 64] + w[lane + 96]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(QKV_FULL_MASK, t, o);
      if (lane == 0) img->wsum[col] = (lo4 && col >= 4) ? 0.f : t * kL2e;
    }
    const float* qv = q_s[gl][gid];
    const float* w = w_s[gl][gid];
    const bool resid = lo4 && gid >= 4;
#pragma unroll
    for (int s = warp; s < 8; s += 4) {
      const int word = s >> 2, f = s & 3;
      const int c0 = 32 * tig + 16 * word + f;
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[e] = qv[c0 + 4 * e] * qf;
        if (resid) v[e] -= __half2float(__float2half_rn(v[e]));
      }
      reinterpret_cast<uint2*>(&img->bop[s >> 1][lane])[s & 1] = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
      uint32_t wq[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {           // pairs t = 2s, 2s+1 of this lane's 32 coordinates
        const int t = 2 * s + h, j = 32 * tig + sign_coord(t);
        const float fs = resid ? 0.f : 2.f * kL2e / sign_v1(sign_pos(t));
        wq[h] = pack_half2(w[j] * fs, w[j + 16] * fs);
      }
      reinterpret_cast<uint2*>(&img->bop[4 + (s >> 1)][lane])[s & 1] = make_uint2(wq[0], wq[1]);
    }
  }
}

// Field c (compile-time) of a W-bit stream held in words w[0..W).
template <int W>
__device__ __forceinline__ uint32_t field32(const uint32_t (&w)[W], int c) {
  const int bit = c * W, wi = bit >> 5, sh = bit & 31;
  uint32_t v = w[wi] >> sh;
  if (sh + W > 32) v |= w[(wi + 1 < W) ? wi + 1 : wi] << (32 - sh);
  return v & ((1u << W) - 1u);
}

template <int WK, int WV>
__global__ void __launch_bounds__(kAttnWarps * 32) attend_split_kernel(AttnArgs a) {
  __shared__ float4 qa[4 * 33];
  __shared__ float4 wa[4 * 33];
  __shared__ float kc_s[16];
  __shared__ float vc_s[16];
  __shared__ float red_m[kAttnWarps][kQT];
  __shared__ float red_l[kAttnWarps][kQT];
  __shared__ float red_acc[kAttnWarps][kQT][kMaxD];

  const int d = a.d;
  const int nsp = d >= 96 ? 4 : (d == 64 ? 2 : 1);     // lanes per token
  const int tps = 32 / nsp;                            // tokens per warp step
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slot = lane % nsp, ts = lane / nsp;
  const bool slot_live = slot * 32 < d;

  const int split = blockIdx.x, qtile = blockIdx.y;
  const int seg = blockIdx.z;                 // b * Hkv + hkv
  const int b = seg / a.Hkv, hkv = seg % a.Hkv;
  const int nq = a.G * a.q_len;
  // a paged cache has its own token count per batch entry; a.kv_len is then only their upper bound
  const bool paged = a.block_table != nullptr;
  int64_t kv_len = a.kv_len;
  if (paged) kv_len = min(static_cast<int64_t>(max(a.seq_lens[b], 0)), a.kv_len);

  // ---- stage the query tile: qa[slot*33 + c] = (q0, q1, q2, q3) of coordinate slot*32+c ----
  int64_t qrow[kQT];
  int limit[kQT];
#pragma unroll
  for (int q = 0; q < kQT; ++q) {
    const int r = qtile * kQT + q;
    if (r < nq) {
      const int g = r / a.q_len, qi = r % a.q_len;
      qrow[q] = (static_cast<int64_t>(b) * a.Hq + hkv * a.G + g) * a.q_len + qi;
      limit[q] = a.causal ? static_cast<int>(kv_len - a.q_len + qi) : static_cast<int>(kv_len - 1);
    } else {
      qrow[q] = -1;
      limit[q] = -1;
    }
  }
  for (int j = threadIdx.x; j < 128; j += blockDim.x) {
    float qv[kQT], wv[kQT];
#pragma unroll
    for (int q = 0; q < kQT; ++q) {
      const bool ok = qrow[q] >= 0 && j < d;
      qv[q] = ok ? a.qk[qrow[q] * 2 * d + j] : 0.f;
      wv[q] = ok ? a.qk[qrow[q] * 2 * d + d + j] : 0.f;
    }
    const int jj = (j >> 5) * 33 + (j & 31);
    qa[jj] = make_float4(qv[0], qv[1], qv[2], qv[3]);
    wa[jj] = make_float4(wv[0], wv[1], wv[2], wv[3]);
  }
  if (threadIdx.x < 16) {
    kc_s[threadIdx.x] = threadIdx.x < (1 << WK) ? a.kcent[threadIdx.x] : 0.f;
    vc_s[threadIdx.x] = threadIdx.x < (1 << WV) ? a.vcent[threadIdx.x] : 0.f;
  }
  __syncthreads();

  int64_t split_len = a.split_len;
  if (paged) {                         // a paged batch entry divides its own length over the splits
    const int64_t per = ((kv_len + a.n_splits - 1) / a.n_splits + 127) / 128 * 128;
    split_len = per < 128 ? 128 : per;
  }
  const int64_t t_begin = split * split_len;
  int64_t t_end = t_begin + split_len;
  if (t_end > kv_len) t_end = kv_len;

  const int words_k = (d >> 5) * WK, words_v = (d >> 5) * WV, words_s = d >> 5;
  // contiguous cache: first row of this (batch, kv head); paged cache: this head's rows inside block 0
  const int64_t seg_row0 = paged ? static_cast<int64_t>(hkv) * a.block_size : static_cast<int64_t>(seg) * a.cache.capacity;
  const int32_t* bt = paged ? a.block_table + static_cast<int64_t>(b) * a.max_blocks : nullptr;
  const uint32_t* kcode = reinterpret_cast<const uint32_t*>(a.cache.k_codes) + seg_row0 * words_k;
  const uint32_t* ksign = reinterpret_cast<const uint32_t*>(a.cache.k_signs) + seg_row0 * words_s;
  const uint32_t* vcode = reinterpret_cast<const uint32_t*>(a.cache.v_codes) + seg_row0 * words_v;
  const float* knorm = a.cache.k_norms + seg_row0;
  const float* vnorm = a.cache.v_norms + seg_row0;

  float m_run[kQT], l_run[kQT], acc[kQT][32];
#pragma unroll
  for (int q = 0; q < kQT; ++q) {
    m_run[q] = -INFINITY;
    l_run[q] = 0.f;
#pragma unroll
    for (int c = 0; c < 32; ++c) acc[q][c] = 0.f;
  }

  for (int64_t t0 = t_begin + static_cast<int64_t>(warp) * tps; t0 < t_end;
       t0 += static_cast<int64_t>(kAttnWarps) * tps) {
    const int64_t pos = t0 + ts;               // token position; `tok` is its row relative to seg_row0
    int64_t tok = pos;
    if (paged && pos < t_end) {
      const unsigned up = static_cast<unsigned>(pos), bs = static_cast<unsigned>(a.block_size);
      tok = static_cast<int64_t>(__ldg(bt + up / bs)) * a.Hkv * a.block_size + up % bs;
    }
    const bool live = pos < t_end && slot_live;
    uint32_t kw[WK], vw[WV], sw = 0;
    float kn = 0.f, vn = 0.f;
#pragma unroll
    for (int i = 0; i < WK; ++i) kw[i] = live ? __ldg(kcode + tok * words_k + slot * WK + i) : 0u;
#pragma unroll
    for (int i = 0; i < WV; ++i) vw[i] = live ? __ldg(vcode + tok * words_v + slot * WV + i) : 0u;
    if (live) sw = __ldg(ksign + tok * words_s + slot);
    if (pos < t_end) {                       // every lane of a token, so the softmax stays warp-uniform
      kn = __ldg(knorm + tok);
      vn = __ldg(vnorm + tok);
    }
    // ---- partial scores over this lane's 32 coordinates -----------------------------------
    float s[kQT] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float kc = kc_s[field32<WK>(kw, c)];
        const float4 qv = qa[slot * 33 + c];
        const float4 wv = wa[slot * 33 + c];
        const bool pos = (sw >> c) & 1u;
        s[0] = fmaf(qv.x, kc, s[0]) + (pos ? wv.x : -wv.x);
        s[1] = fmaf(qv.y, kc, s[1]) + (pos ? wv.y : -wv.y);
        s[2] = fmaf(qv.z, kc, s[2]) + (pos ? wv.z : -wv.z);
        s[3] = fmaf(qv.w, kc, s[3]) + (pos ? wv.w : -wv.w);
      }
    }
    for (int o = 1; o < nsp; o <<= 1) {
#pragma unroll
      for (int q = 0; q < kQT; ++q) s[q] += __shfl_xor_sync(QKV_FULL_MASK, s[q], o);
    }
    // ---- online softmax --------------------------------------------------------------------
    float sc[kQT], mx[kQT];
    bool grew = false;
#pragma unroll
    for (int q = 0; q < kQT; ++q) {
      const bool vis = pos < t_end && pos <= limit[q];
      sc[q] = vis ? kn * s[q] : -INFINITY;
      mx[q] = sc[q];
    }
    for (int o = nsp; o < 32; o <<= 1) {
#pragma unroll
      for (int q = 0; q < kQT; ++q) mx[q] = fmaxf(mx[q], __shfl_xor_sync(QKV_FULL_MASK, mx[q], o));
    }
#pragma unroll
    for (int q = 0; q < kQT; ++q) grew |= mx[q] > m_run[q];
    if (grew) {                                   // warp-uniform: mx and m_run are
#pragma unroll
      for (int q = 0; q < kQT; ++q) {
        if (mx[q] > m_run[q]) {
          const float alpha = (m_run[q] == -INFINITY) ? 0.f : expf(m_run[q] - mx[q]);
          m_run[q] = mx[q];
          l_run[q] *= alpha;
#pragma unroll
          for (int c = 0; c < 32; ++c) acc[q][c] *= alpha;
        }
      }
    }
    float pv[kQT];
#pragma unroll
    for (int q = 0; q < kQT; ++q) {
      const float p = (sc[q] == -INFINITY) ? 0.f : expf(sc[q] - m_run[q]);
      l_run[q] += p;
      pv[q] = p * vn;
    }
    // ---- values: acc[q][c] += p * v_norm * c_V[code] ------------------------------------------
    if (live) {
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float vc = vc_s[field32<WV>(vw, c)];
#pragma unroll
        for (int q = 0; q < kQT; ++q) acc[q][c] = fmaf(pv[q], vc, acc[q][c]);
      }
    }
  }

  // ---- reduce over the token lanes of the warp, then over warps -------------------------------
  for (int o = nsp; o < 32; o <<= 1) {
#pragma unroll
    for (int q = 0; q < kQT; ++q) {
      l_run[q] += __shfl_xor_sync(QKV_FULL_MASK, l_run[q], o);
#pragma unroll
      for (int c = 0; c < 32; ++c) acc[q][c] += __shfl_xor_sync(QKV_FULL_MASK, acc[q][c], o);
    }
  }
  if (ts == 0) {
#pragma unroll
    for (int q = 0; q < kQT; ++q) {
      if (slot == 0) { red_m[warp][q] = m_run[q]; red_l[warp][q] = l_run[q]; }
      if (slot_live) {
#pragma unroll
        for (int c = 0; c < 32; ++c) red_acc[warp][q][slot * 32 + c] = acc[q][c];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < kQT * (d + 2); idx += blockDim.x) {
    const int q = idx / (d + 2), e = idx % (d + 2);
    if (qrow[q] < 0) continue;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, red_m[w][q]);
    float v = 0.f;
    if (e == 0) {
      v = M;
    } else {
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) {
        const float f = (red_m[w][q] == -INFINITY) ? 0.f : expf(red_m[w][q] - M);
        v += f * (e == 1 ? red_l[w][q] : red_acc[w][q][e - 2]);
      }
    }
    a.part[(qrow[q] * a.n_splits + split) * (d + 2) + e] = v;
  }
}

// A few query rows per CTA: combine the splits of each row, normalise, then un-rotate; thread i owns output
// coordinate i and reads row j of Pi coalesced, each element feeding every row of the CTA.
__global__ void __launch_bounds__(128) merge_splits_kernel(const float* __restrict__ part, int64_t rows,
                                                           int n_splits, int d, const float* __restrict__ Pi,
                                                           float* __restrict__ out) {
  __shared__ float vec[kRowsPerCta][kMaxD];
  __shared__ float wsplit[kRowsPerCta][kMaxSplits];
  __shared__ float inv_l[kRowsPerCta];
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * kRowsPerCta;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = warp; r < kRowsPerCta; r += blockDim.x >> 5) {     // a warp per row: weights of its splits
    if (row0 + r >= rows) continue;
    const float* p = part + (row0 + r) * n_splits * (d + 2);
    float M = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, p[s * (d + 2)]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(QKV_FULL_MASK, M, o));
    float L = 0.f;
    for (int s = lane; s < n_splits; s += 32) {
      const float m = p[s * (d + 2)];
      const float f = (m == -INFINITY) ? 0.f : expf(m - M);
      wsplit[r][s] = f;
      L += f * p[s * (d + 2) + 1];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(QKV_FULL_MASK, L, o);
    if (lane == 0) inv_l[r] = 1.f / fmaxf(L, 1e-30f);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < kRowsPerCta * d; idx += blockDim.x) {
    const int r = idx / d, j = idx % d;
    float v = 0.f;
    if (row0 + r < rows) {
      const float* p = part + (row0 + r) * n_splits * (d + 2);
      for (int s = 0; s < n_splits; ++s) v += wsplit[r][s] * p[s * (d + 2) + 2 + j];
      v *= inv_l[r];
    }
    vec[r][j] = v;
  }
  __syncthreads();
  const int i = threadIdx.x;
  if (i < d) {
    float o[kRowsPerCta];
#pragma unroll
    for (int r = 0; r < kRowsPerCta; ++r) o[r] = 0.f;
#pragma unroll 8
    for (int j = 0; j < d; ++j) {
      const float m = __ldg(Pi + j * d + i);
#pragma unroll
      for (int r = 0; r < kRowsPerCta; ++r) o[r] = fmaf(vec[r][j], m, o[r]);
    }
#pragma unroll
    for (int r = 0; r < kRowsPerCta; ++r)
      if (row0 + r < rows) out[(row0 + r) * d + i] = o[r];
  }
}

// Host-side launcher shared with the index scan.
static int launch_rotate(const void* q, int q_dtype, int64_t rows, int d, const float* Pi, const float* S,
                         float qjl_scale, float scale, float* qk, const float* kcent, const float* vcent,
                         uint32_t* tables, int n_counters, cudaStream_t st) {
  const unsigned ctas = static_cast<unsigned>((rows + kRowsPerCta - 1) / kRowsPerCta) + (tables ? 1u : 0u);
  rotate_queries_kernel<<<ctas, 128, 0, st>>>(q, q_dtype, rows, d, Pi, S, qjl_scale, scale, qk, kcent, vcent,
                                              tables, n_counters);
  return check_launch();
}

int launch_rotate_with_tables(const void* q, int q_dtype, int64_t rows, int d, const float* Pi, const float* S,
                              float qjl_scale, float scale, float* qk, const float* kcent, const float* vcent,
                              uint32_t* tables, cudaStream_t st) {
  return launch_rotate(q, q_dtype, rows, d, Pi, S, qjl_scale, scale, qk, kcent, vcent, tables, 0, st);
}

int launch_rotate_queries(const void* q, int q_dtype, int64_t rows, int d, const float* Pi, const float* S,
                          float qjl_scale, float scale, float* qk, cudaStream_t st) {
  return launch_rotate(q, q_dtype, rows, d, Pi, S, qjl_scale, scale, qk, nullptr, nullptr, nullptr, 0, st);
}

typedef void (*AttnKernel)(AttnArgs);

template <int WK>
static AttnKernel pick_v(int wv) {
  switch (wv) {
    case 1: return attend_split_kernel<WK, 1>;
    case 2: return attend_split_kernel<WK, 2>;
    case 3: return attend_split_kernel<WK, 3>;
    default: return attend_split_kernel<WK, 4>;
  }
}

static AttnKernel pick(int wk, int wv) {
  switch (wk) {
    case 1: return pick_v<1>(wv);
    case 2: return pick_v<2>(wv);
    default: return pick_v<3>(wv);
  }
}

}  // namespace qkv

using namespace qkv;

extern "C" size_t qkv_attention_workspace_bytes(int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d) {
  if (B < 1 || Hq < 1 || Hkv < 1 || q_len < 1 || kv_len < 1 || d < 32) return 0;
  const AttnPlan p = make_plan(B, Hq, Hkv, q_len, kv_len, d);
  return p.hdr_bytes + p.qk_bytes + p.part_bytes;
}

namespace {
struct PagedInfo {
  const int32_t* block_table; const int32_t* seq_lens;
  int max_blocks, block_size;
};

int attention_run(const void* q, int q_dtype, qkv_cache_t cache, const uint8_t* records, const PagedInfo* paged,
                  int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d,
                  int key_bits, int val_bits,
                  const float* Pi, const float* key_centroids, const float* val_centroids,
                  const float* S, float qjl_scale, float scale, int causal,
                  float* out, void* workspace, size_t workspace_bytes, void* stream) {
  const bool tiled = records != nullptr;
  if (!q || !Pi || !key_centroids || !val_centroids || !S || !out || !workspace) return QKV_ENULL;
  if (!tiled && (!cache.k_codes || !cache.k_signs || !cache.k_norms || !cache.v_codes || !cache.v_norms))
    return QKV_ENULL;
  if (q_dtype != QKV_F32 && q_dtype != QKV_BF16 && q_dtype != QKV_F16) return QKV_EDTYPE;
  if (d < 32 || d > kMaxD || (d & 31)) return QKV_EDIM;
  if (B < 1 || Hq < 1 || Hkv < 1 || q_len < 1 || kv_len < 1 || (!paged && kv_len > cache.capacity) ||
      kv_len > 0x7fffffff || Hq % Hkv != 0)
    return QKV_EDIM;
  if (key_bits < 2 || key_bits > 4 || val_bits < 1 || val_bits > 4) return QKV_EBITS;
  if (causal && q_len > kv_len) return QKV_EARG;
  if (paged) {
    if (!paged->block_table || !paged->seq_lens) return QKV_ENULL;
    if (paged->block_size < 1 || paged->max_blocks < 1 ||
        static_cast<int64_t>(paged->max_blocks) * paged->block_size < kv_len)
      return QKV_EARG;
  }
  const uintptr_t al = reinterpret_cast<uintptr_t>(cache.k_codes) | reinterpret_cast<uintptr_t>(cache.k_signs) |
                       reinterpret_cast<uintptr_t>(cache.v_codes) | reinterpret_cast<uintptr_t>(workspace) |
                       reinterpret_cast<uintptr_t>(records);
  if (al & 15u) return QKV_EALIGN;
  if (tiled) {           // records exist for head_dim 128 at 3/3 bits only, in whole 16-token tiles
    if (!tiled_path_ok(d, key_bits, val_bits)) return QKV_EBITS;
    if (paged ? (paged->block_size & 15) != 0 : (cache.capacity & 15) != 0) return QKV_EARG;
  }
  const AttnPlan p = make_plan(B, Hq, Hkv, q_len, kv_len, d);
  if (workspace_bytes < p.hdr_bytes + p.qk_bytes + p.part_bytes) return QKV_EWORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  uint32_t* tables = reinterpret_cast<uint32_t*>(ws);
  float* qk = reinterpret_cast<float*>(ws + p.hdr_bytes);
  float* part = reinterpret_cast<float*>(ws + p.hdr_bytes + p.qk_bytes);
  // QUASHKV_B200_GENERIC_ATTENTION=1 routes every call to the generic kernel (for A/B checks).
  const char* env = getenv("QUASHKV_B200_GENERIC_ATTENTION");
  const bool force_generic = env && env[0] == '1';
  // the tensor-core path copies 16-byte chunks of every plane, norms included
  // (a paged tile of 16 tokens must also lie inside one block)
  const bool chunks_ok = (paged ? paged->block_size % 16 == 0 : cache.capacity % 4 == 0) &&
      ((reinterpret_cast<uintptr_t>(cache.k_norms) | reinterpret_cast<uintptr_t>(cache.v_norms)) & 15u) == 0;
  const bool use_mma = tiled || (mma_path_ok(d, key_bits, val_bits, Hq / Hkv, q_len) && chunks_ok && !force_generic);
  // tile records with up to four query rows per KV head: scores from bit planes, operands built by the rotation
  const bool from_planes = tiled && tiled_scores_from_planes(Hq / Hkv, q_len);
  PlaneImage* planes = from_planes ? reinterpret_cast<PlaneImage*>(ws + p.img_off) : nullptr;
  // ... otherwise fp16 scores from operand images per group of eight query rows, built by the rotation as well
  GroupImage* groups = (tiled && !from_planes) ? reinterpret_cast<GroupImage*>(ws + p.img_off) : nullptr;
  int rc;
  if (groups) {
    const int nq_all = (Hq / Hkv) * q_len, gps = (nq_all + 7) / 8;
    const int n_groups = B * Hkv * gps;
    rotate_groups_kernel<<<static_cast<unsigned>((n_groups + kGroupsPerCta - 1) / kGroupsPerCta + 1), 128, 0, st>>>(
        q, q_dtype, Pi, S, qjl_scale, scale, key_centroids, val_centroids, tables, n_groups, nq_all, gps, n_groups,
        nq_all <= 4 ? 1 : 0, groups);
    rc = check_launch();
  } else if (from_planes) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(B * Hkv + 1));
    cfg.blockDim = dim3(512);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, rotate_planes_kernel, q, q_dtype, p.rows, Pi, S, qjl_scale, scale, qk, key_centroids,
                           val_centroids, tables, B * Hkv, (Hq / Hkv) * q_len, planes) != cudaSuccess)
      return QKV_ELAUNCH;
    rc = check_launch();
  } else {
    rc = launch_rotate(q, q_dtype, p.rows, d, Pi, S, qjl_scale, scale, qk, key_centroids, val_centroids,
                       use_mma ? tables : nullptr, B * Hkv * (((Hq / Hkv) * q_len + 7) / 8), st);
  }
  if (rc) return rc;

  AttnArgs a{};
  a.cache = cache; a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.G = Hq / Hkv; a.q_len = q_len; a.d = d;
  a.causal = causal; a.kv_len = kv_len; a.qk = qk; a.kcent = key_centroids; a.vcent = val_centroids;
  a.part = part; a.n_splits = p.n_splits; a.split_len = p.split_len;
  if (paged) {
    a.block_table = paged->block_table; a.seq_lens = paged->seq_lens;
    a.max_blocks = paged->max_blocks; a.block_size = paged->block_size;
  }
  if (use_mma) {          // one launch: the last split of every (batch, kv head) merges and un-rotates
    a.tables = tables;
    const int64_t grid_ctas = static_cast<int64_t>(B) * Hkv * (((Hq / Hkv) * q_len + 7) / 8) * p.n_splits;
    a.skew = grid_ctas >= 2 * 4 * kNumSMs ? kSplitSkew : 0.f;
    a.arrivals = reinterpret_cast<unsigned*>(ws + kAttnHeaderBytes);
    a.Pi = Pi;
    a.out = out;
    a.records = records;
    a.planes = planes;
    a.groups = groups;
    return tiled ? launch_attend_tiled(a, st) : launch_attend_mma(a, st);
  } else {
    const dim3 grid(p.n_splits, p.n_qtiles, B * Hkv);
    pick(key_bits - 1, val_bits)<<<grid, kAttnWarps * 32, 0, st>>>(a);
  }
  merge_splits_kernel<<<static_cast<unsigned>((p.rows + kRowsPerCta - 1) / kRowsPerCta), 128, 0, st>>>(
      part, p.rows, p.n_splits, d, Pi, out);
  return check_launch();
}
}  // namespace

extern "C" int qkv_attention(const void* q, int q_dtype, qkv_cache_t cache,
                             int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d,
                             int key_bits, int val_bits,
                             const float* Pi, const float* key_centroids, const float* val_centroids,
                             const float* S, float qjl_scale, float scale, int causal,
                             float* out, void* workspace, size_t workspace_bytes, void* stream) {
  return attention_run(q, q_dtype, cache, nullptr, nullptr, B, Hq, Hkv, q_len, kv_len, d, key_bits, val_bits, Pi,
                       key_centroids, val_centroids, S, qjl_scale, scale, causal, out, workspace, workspace_bytes,
                       stream);
}

extern "C" int qkv_attention_paged(const void* q, int q_dtype, qkv_paged_cache_t pool,
                                   int B, int Hq, int Hkv, int q_len, int64_t max_kv_len, int d,
                                   int key_bits, int val_bits,
                                   const float* Pi, const float* key_centroids, const float* val_centroids,
                                   const float* S, float qjl_scale, float scale, int causal,
                                   float* out, void* workspace, size_t workspace_bytes, void* stream) {
  qkv_cache_t planes{};
  planes.k_codes = pool.k_codes; planes.k_signs = pool.k_signs; planes.k_norms = pool.k_norms;
  planes.v_codes = pool.v_codes; planes.v_norms = pool.v_norms;
  planes.capacity = 0;
  const PagedInfo info{pool.block_table, pool.seq_lens, pool.max_blocks, pool.block_size};
  return attention_run(q, q_dtype, planes, nullptr, &info, B, Hq, Hkv, q_len, max_kv_len, d, key_bits, val_bits, Pi,
                       key_centroids, val_centroids, S, qjl_scale, scale, causal, out, workspace, workspace_bytes,
                       stream);
}

extern "C" int qkv_attention_tiled(const void* q, int q_dtype, qkv_tiled_cache_t cache,
                                   int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d,
                                   int key_bits, int val_bits,
                                   const float* Pi, const float* key_centroids, const float* val_centroids,
                                   const float* S, float qjl_scale, float scale, int causal,
                                   float* out, void* workspace, size_t workspace_bytes, void* stream) {
  if (!cache.records) return QKV_ENULL;
  qkv_cache_t planes{};
  planes.capacity = cache.capacity;
  const PagedInfo info{cache.block_table, cache.seq_lens, cache.max_blocks, cache.block_size};
  return attention_run(q, q_dtype, planes, cache.records, cache.block_table ? &info : nullptr, B, Hq, Hkv, q_len,
                       kv_len, d, key_bits, val_bits, Pi, key_centroids, val_centroids, S, qjl_scale, scale, causal,
                       out, workspace, workspace_bytes, stream);
}

// ---- attention without a caller-provided workspace ------------------------------------------------
// The scratch array is part of the library image, so no allocation call is ever made for it.  In
// host code the symbol is only a handle: its device address comes from cudaGetSymbolAddress, asked
// once per device (with that device current) and kept in a small table.
namespace {
__device__ __align__(256) unsigned char g_attention_scratch[QKV_ATTENTION_STATIC_SCRATCH_BYTES];
constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
}  // namespace

extern "C" int qkv_attention_static_scratch(const void* q, int q_dtype, qkv_cache_t cache,
                                            int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d,
                                            int key_bits, int val_bits,
                                            const float* Pi, const float* key_centroids,
                                            const float* val_centroids, const float* S, float qjl_scale,
                                            float scale, int causal, float* out, void* stream) {
  if (B < 1 || Hq < 1 || Hkv < 1 || q_len < 1 || kv_len < 1 || d < 32 || d > kMaxD) return QKV_EDIM;
  const size_t need = qkv_attention_workspace_bytes(B, Hq, Hkv, q_len, kv_len, d);
  if (need == 0 || need > QKV_ATTENTION_STATIC_SCRATCH_BYTES) return QKV_EWORKSPACE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return QKV_EARG;
  void* ptr = __atomic_load_n(&g_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (ptr == nullptr) {   // first call on this device; concurrent first calls all obtain the same address
    if (cudaGetSymbolAddress(&ptr, g_attention_scratch) != cudaSuccess || ptr == nullptr) return QKV_ELAUNCH;
    __atomic_store_n(&g_scratch_addr[dev], ptr, __ATOMIC_RELEASE);
  }
  return qkv_attention(q, q_dtype, cache, B, Hq, Hkv, q_len, kv_len, d, key_bits, val_bits, Pi, key_centroids,
                       val_centroids, S, qjl_scale, scale, causal, out, ptr, QKV_ATTENTION_STATIC_SCRATCH_BYTES,
                       stream);
}
