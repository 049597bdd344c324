// Declarations shared by the generic and the tensor-core attention kernels.
#pragma once

#include <cuda_fp16.h>
#include <stddef.h>
#include <stdlib.h>

#include "common.cuh"

namespace qkv {

constexpr int kQT = 4;          // query rows per CTA
constexpr int kAttnWarps = 4;
constexpr int kMaxSplits = 64;

// Bit-plane scores of the tiled path (up to four query rows per KV head): what a CTA needs of its (batch, kv head)
// besides the records, built once by the query-rotation kernel and fetched with one bulk copy.
struct PlaneImage {
  uint4 bop[12][32];    // B operands per k-step and lane: both accumulator chains
  float inv[4];         // score units per unit of the first term, per query row
  float cst[4];         // the score of a token whose bits are all clear, per query row
};
static_assert(sizeof(PlaneImage) % 16 == 0, "fetched with a bulk copy");

// fp16 scores of the tiled path: the B operands of one group of eight query rows of a (batch, kv head), built once
// by the query-rotation kernel (the CTAs of the scan fetch them with bulk copies instead of rebuilding them).
struct GroupImage {
  uint4 bop[8][32];     // per lane: two k-steps per entry, 8 key-code steps, then 8 sign steps
  float wsum[8];        // log2e * sum of the sign weights per query column (0 for the residual columns)
};
static_assert(sizeof(GroupImage) % 16 == 0 && offsetof(GroupImage, wsum) % 16 == 0, "fetched with bulk copies");

struct AttnArgs {
  qkv_cache_t cache;
  int B, Hq, Hkv, G, q_len, d, causal;
  int64_t kv_len;
  const float* qk;      // [rows][2][d]
  const float* kcent; const float* vcent;
  float* part;          // [rows][n_splits][d+2]
  const uint32_t* tables;   // tensor-core path: fp16 look-up tables and their scales (8 words)
  unsigned* arrivals;       // tensor-core path: splits finished per (batch, kv head); zeroed by the rotation kernel
  const float* Pi;          // tensor-core path: the last split of a head merges and un-rotates
  float* out;
  int n_splits; int64_t split_len;
  // Paged cache (block_table != nullptr): the planes are a pool of blocks of block_size rows per kv head,
  // row (block * Hkv + hkv) * block_size + offset; token t of batch entry b lives in block
  // block_table[b * max_blocks + t / block_size] and the entry has seq_lens[b] tokens (kv_len bounds them).
  const int32_t* block_table; const int32_t* seq_lens;
  int max_blocks, block_size;
  float skew;               // tensor-core path: how unequal the splits are (split_begin_chunk)
  // Tiled cache (records != nullptr): 16-token tile records (tile_format.cuh) instead of the five planes;
  // contiguous: cache.capacity / 16 records per (batch, kv head); paged: block_size / 16 records per
  // (block, kv head).
  const uint8_t* records;
  const PlaneImage* planes; // tiled path, bit-plane scores: one image per (batch, kv head), else nullptr
  const GroupImage* groups; // tiled path, fp16 scores: one image per (batch, kv head, group of eight query rows)
};

// Tensor-core path: the KV range is cut into splits of UNEQUAL length, in 128-token chunks, the longest first:
// split k gets a share proportional to 1 + kSkew (1 - 2k/(n-1)).  Splits are dispatched longest first (the split
// index is the slowest grid dimension), so CTAs that share an SM end at different times instead of all running
// their set-up and reduction phases together, and the last CTAs to start are the shortest.  The skew is only
// used when the grid is at least two waves of resident CTAs: with fewer CTAs everything runs at once and the
// longest split would set the time (measured on the benchmark shape: 0 -> 1.89, 0.4 -> 1.93, 0.8 -> 1.96 TB/s).
constexpr float kSplitSkew = 0.8f;
__host__ __device__ inline int64_t split_begin_chunk(int k, int n, int64_t chunks, float skew) {
  if (k <= 0) return 0;
  if (k >= n) return chunks;
  const float kf = static_cast<float>(k);
  const float f = (kf + skew * (kf - kf * (kf - 1.f) / static_cast<float>(n - 1))) / static_cast<float>(n);
  const int64_t c = static_cast<int64_t>(f * static_cast<float>(chunks) + 0.5f);
  return c < 0 ? 0 : (c > chunks ? chunks : c);
}

constexpr size_t kAttnHeaderBytes = 256;   // workspace header: look-up tables of the tensor-core path

struct AttnPlan {
  int n_splits; int64_t split_len; int n_qtiles; int64_t rows;
  size_t hdr_bytes;     // look-up tables (first 256 bytes), the arrival counters of the tensor-core path, plane images
  size_t img_off;       // offset of the plane images (one per batch entry and kv head) inside the header
  size_t qk_bytes, part_bytes;
};

inline AttnPlan make_plan(int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d) {
  AttnPlan p;
  const int G = Hq / (Hkv > 0 ? Hkv : 1);
  const int nq = G * q_len;
  p.n_qtiles = (nq + kQT - 1) / kQT;
  p.rows = static_cast<int64_t>(B) * Hq * q_len;
  (void)d;
  const int64_t chunk = 128;   // a multiple of every kernel's tokens per CTA pass (32..128)
  const int64_t ctas = static_cast<int64_t>(B) * Hkv * p.n_qtiles;
  // Number of KV splits.  A grid runs in waves of four resident CTAs per SM and every CTA carries a fixed cost
  // (set-up, pipeline fill, reduction, the merge by the last CTA of a head: about 15 us), so the plan is the
  // SMALLEST count, from one that fills a single wave up to four times that, whose CTA total fills whole waves
  // within 3 % of the best: few long CTAs beat many short ones.  Measured on 32 sequences x 32768 tokens:
  // 1 KV head 18 splits (one wave) 89 us against 100 us for 37 (two waves); 2 heads 9 splits 132 us against
  // 142 us for 18; 4 heads 9 splits 226 us (best 224 us at 13); 8 heads 9 splits 397 us (best 393 us at 4).
  const int64_t max_by_len = (kv_len + 4 * chunk - 1) / (4 * chunk);
  int64_t cap = max_by_len < kMaxSplits ? max_by_len : kMaxSplits;
  if (cap < 1) cap = 1;
  const int64_t wave = 4 * kNumSMs;
  int64_t lo = wave / (ctas > 0 ? ctas : 1);
  if (lo < 1) lo = 1;
  if (lo > cap) lo = cap;
  int64_t hi = 4 * lo + 1;
  if (hi > cap) hi = cap;
  double best = -1.0;
  for (int64_t n = lo; n <= hi; ++n) {
    const double waves = static_cast<double>(ctas * n) / static_cast<double>(wave);
    const double whole = static_cast<double>(static_cast<int64_t>(waves + 0.999999));
    const double eff = waves / (whole > 0 ? whole : 1.0);
    if (eff > best) best = eff;
  }
  int64_t want = lo;
  for (int64_t n = lo; n <= hi; ++n) {
    const double waves = static_cast<double>(ctas * n) / static_cast<double>(wave);
    const double whole = static_cast<double>(static_cast<int64_t>(waves + 0.999999));
    if (waves / (whole > 0 ? whole : 1.0) >= best - 0.03) { want = n; break; }
  }
  if (const char* e = getenv("QUASHKV_B200_SPLITS")) {      // experiments: a fixed number of splits
    const int64_t n = atoll(e);
    if (n >= 1 && n <= cap) want = n;
  }
  int64_t len = (kv_len + want - 1) / want;
  len = (len + chunk - 1) / chunk * chunk;
  if (len < chunk) len = chunk;
  p.split_len = len;
  p.n_splits = static_cast<int>((kv_len + len - 1) / len);
  if (p.n_splits < 1) p.n_splits = 1;
  // arrival counters: one per (batch, kv head, tile of eight query rows) of the tensor-core path
  p.img_off = (kAttnHeaderBytes + static_cast<size_t>(B) * Hkv * ((nq + 7) / 8) * sizeof(unsigned) + 255) / 256 * 256;
  p.hdr_bytes = p.img_off;
  if (d == 128) {       // operand images of the tiled path: bit planes (up to four rows) or fp16 groups of eight rows
    const size_t planes = nq <= 4 ? static_cast<size_t>(B) * Hkv * sizeof(PlaneImage) : 0;
    const size_t groups = static_cast<size_t>(B) * Hkv * ((nq + 7) / 8) * sizeof(GroupImage);
    p.hdr_bytes = (p.img_off + (planes > groups ? planes : groups) + 255) / 256 * 256;
  }
  p.qk_bytes = static_cast<size_t>(p.rows) * 2 * d * sizeof(float);
  p.qk_bytes = (p.qk_bytes + 255) / 256 * 256;
  p.part_bytes = static_cast<size_t>(p.rows) * p.n_splits * (d + 2) * sizeof(float);
  return p;
}


// Tensor-core decode path (attention_mma.cu): usable when mma_path_ok() holds.
bool mma_path_ok(int d, int key_bits, int val_bits, int group, int q_len);
int launch_attend_mma(const AttnArgs& a, cudaStream_t st);

// Tensor-core path over tile records (attention_tiled.cu).
bool tiled_path_ok(int d, int key_bits, int val_bits);
bool tiled_scores_from_planes(int group, int q_len);      // up to four query rows per KV head (and not switched off)
int launch_attend_tiled(const AttnArgs& a, cudaStream_t st);
unsigned int bulk_copy_timeouts();        // bounded waits on a record copy that ran out (device-wide counter)

// Look-up tables of the tensor-core path, built by one CTA of 128 threads.  For each table the scale
// s in [1,2) (512 candidates, 4 per thread) is chosen that makes the largest relative fp16 rounding
// error of s*c_i smallest, so the systematic error of the fp16 operands drops well below 2^-12.
// tables[0..1] key centroids as fp16 pairs, [2..3] value low bytes, [4..5] value high bytes,
// [6] 1/key scale, [7] 1/value scale (floats), [8..9] the four value magnitudes (entries 4..7 of the
// value table, the positive half of a symmetric table) as fp16 pairs for the sign-and-magnitude records,
// [10] contract flags (bit 0: the value table is not symmetric, bit 1: the key table is not affine in the two
// bits of its code), [11..13] g0, g1, g2 of the key table written as c(u) = g0 + g1 (u & 1) + g2 (u >> 1).
// The scale in [1, 2) of a table of n <= 8 values: a CTA-wide call (first 128 threads search four candidates each,
// everyone passes the barriers), every thread gets the result.  Deterministic: smallest error, then smallest scale.
__device__ inline float best_fp16_scale_cta(const float* __restrict__ cent, int n) {
  __shared__ float cand_err[4];
  __shared__ float cand_s[4];
  __shared__ float chosen;
  const int tid = threadIdx.x;
  if (tid < 128) {
    float c[8];
    for (int i = 0; i < 8; ++i) c[i] = i < n ? cent[i] : 0.f;
    float best_err = 1e30f, best_s = 1.f;
    for (int k = 0; k < 4; ++k) {
      const float s = 1.f + static_cast<float>(tid + 128 * k) * (1.f / 512.f);
      float err = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float v = c[i] * s;
        if (v != 0.f) err = fmaxf(err, fabsf(__half2float(__float2half_rn(v)) - v) / fabsf(v));
      }
      if (err < best_err) { best_err = err; best_s = s; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float e2 = __shfl_xor_sync(0xffffffffu, best_err, o), s2 = __shfl_xor_sync(0xffffffffu, best_s, o);
      if (e2 < best_err || (e2 == best_err && s2 < best_s)) { best_err = e2; best_s = s2; }
    }
    if ((tid & 31) == 0) { cand_err[tid >> 5] = best_err; cand_s[tid >> 5] = best_s; }
  }
  __syncthreads();
  if (tid == 0) {
    float e = 1e30f, s = 1.f;
    for (int i = 0; i < 4; ++i)
      if (cand_err[i] < e || (cand_err[i] == e && cand_s[i] < s)) { e = cand_err[i]; s = cand_s[i]; }
    chosen = s;
  }
  __syncthreads();
  const float r = chosen;
  __syncthreads();                          // the scratch may be reused by the next call
  return r;
}

__device__ inline void prepare_tables_cta(const float* __restrict__ kcent, const float* __restrict__ vcent,
                                          uint32_t* __restrict__ tables) {
  const int tid = threadIdx.x;
  float sc[2];
  sc[0] = best_fp16_scale_cta(kcent, 4);
  sc[1] = best_fp16_scale_cta(vcent, 8);
  if (tid != 0) return;
  uint32_t t[6] = {0, 0, 0, 0, 0, 0};
  for (int i = 0; i < 4; ++i) {   // whole fp16 values: entries 0,1 in word 0, entries 2,3 in word 1
    const uint32_t h = __half_as_ushort(__float2half_rn(kcent[i] * sc[0]));
    t[i >> 1] |= h << (16 * (i & 1));
  }
  for (int i = 0; i < 8; ++i) {
    const uint32_t h = __half_as_ushort(__float2half_rn(vcent[i] * sc[1]));
    t[2 + (i >> 2)] |= (h & 0xFFu) << (8 * (i & 3));
    t[4 + (i >> 2)] |= (h >> 8) << (8 * (i & 3));
  }
  for (int i = 0; i < 6; ++i) tables[i] = t[i];
  uint32_t mg[2] = {0, 0};
  for (int i = 0; i < 4; ++i) {
    const uint32_t h = __half_as_ushort(__float2half_rn(vcent[4 + i] * sc[1]));
    mg[i >> 1] |= h << (16 * (i & 1));
  }
  tables[8] = mg[0];
  tables[9] = mg[1];
  tables[6] = __float_as_uint(1.f / sc[0]);
  tables[7] = __float_as_uint(1.f / sc[1]);
  float kmax = 0.f, vmax = 0.f, vasym = 0.f;
  for (int i = 0; i < 4; ++i) kmax = fmaxf(kmax, fabsf(kcent[i]));
  for (int i = 0; i < 8; ++i) vmax = fmaxf(vmax, fabsf(vcent[i]));
  for (int i = 0; i < 4; ++i) vasym = fmaxf(vasym, fabsf(vcent[i] + vcent[7 - i]));
  const float kbend = fabsf((kcent[3] - kcent[2]) - (kcent[1] - kcent[0]));
  tables[10] = (vasym > 1e-5f * vmax ? 1u : 0u) | (kbend > 1e-5f * kmax ? 2u : 0u);
  tables[11] = __float_as_uint(kcent[0]);
  tables[12] = __float_as_uint(kcent[1] - kcent[0]);
  tables[13] = __float_as_uint(kcent[2] - kcent[0]);
}

}  // namespace qkv
