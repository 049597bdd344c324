// Decode / prefill attention over a cache of tile records (tile_format.cuh): head_dim 128, 3-bit keys
// (2-bit codes + sign bit), 3-bit values, eight (prefill: sixteen) query rows of a KV head per CTA.
// Semantics: QuashKVEngine.attention (reference engine.py:204-299).
//
// A warp owns 16-token tiles of its split.  One elected lane fetches a whole record (1664 bytes) with
// ONE bulk copy into the warp's ring of four stages; an mbarrier per stage counts the bytes in, every
// wait on it is bounded.  Each lane then reads its share with five vector loads and feeds mma.sync:
//   scores   tokens = M, queries = N, coordinates = K
//   values   coordinates = M, tokens = K, queries = N, accumulated in the ROTATED domain; a value operand
//            register is one look-up per pair of tokens in a 64-entry table of ready fp16 pairs in shared memory,
//            laid out so that every lane reads its own bank: 8 MMAs per group of eight query columns
// with an online softmax in between (log2 domain, lazily raised reference exponent).  Per split the
// CTA writes (max, sum, accumulator); the last CTA of a (batch, kv head) to finish merges the splits
// and applies Pi once, which equals un-rotating every value (engine.py:284-287) because the rotation
// is linear.  With a single split the rows go straight through the un-rotation.
// Everything the scores need of the queries (B operands, constants) is built once per (batch, kv head) by the
// query-rotation kernel (attention.cu) and fetched with bulk copies.
//
// Scores, up to four query rows per KV head (decode with up to four query heads per KV head): on the INTEGER
// tensor cores from bit planes (MODE 2).  A 4-level key table that is affine in
// the two bits of its code, c(u) = g0 + g1 b0 + g2 b1 (true of every table with c0 + c3 = c1 + c2, so of
// every symmetric one), turns the score into a constant plus a weighted sum over single bits: of the two code
// bits and of the sign bit of every coordinate.  `word & (0x01010101 << p)` IS an unsigned 8-bit A operand
// (four elements, each 0 or 2^p) of mma.m16n8k32.u8.s8, so a register of four operand elements costs one
// logic instruction and no shift, against three instructions per TWO elements of the fp16 path; the query
// side carries weight / 2^p as four signed 8-bit terms (radix 128, a common scale per query), two per
// accumulator chain in the column pairs (n, n + 4), which is exact integer arithmetic to 2^-21 of the largest
// weight: 24 MMAs per tile.  The accumulators start at the bit pattern of 1.5 * 2^23, so the integer sums read
// back as floats with one subtraction.  (The fp16 form of the same idea, MODE 1, puts the fp16 rounding residual
// of the queries into columns 4..7; it is kept for comparison, QUASHKV_B200_SCORES=fp16.)
//
// Scores, more rows (MODE 0: five to eight; MODE 3: sixteen as two groups of eight columns, for prefill): fp16
// m16n8k16, key codes decoded in registers with one PRMT per pair of codes, sign bits with one LOP3 per pair
// (tile_decode.cuh, mma_decode.cuh): 8 MMAs on the key codes and 8 on the sign bits per group; in MODE 3 every
// decoded key and value fragment feeds both groups.
#include <math.h>
#include <stdlib.h>

#include "attention_common.cuh"
#include "mma_decode.cuh"
#include "tile_decode.cuh"
#include "umma.cuh"

namespace qkv {

namespace {

constexpr int kWarps = 4;
// Ring slots per warp: three records in flight while one is worked on.  (Five or six resident CTAs per SM,
// 96 / 80 registers, measured 6 % / 10 % slower than four at their best split counts.)
constexpr int kRing = 4;
constexpr float kLog2e = 1.4426950408889634f;

__device__ unsigned int g_bulk_timeouts = 0;   // bounded waits on a bulk copy that ran out

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(umma::smem_u32(bar)), "r"(bytes)
               : "memory");
}

// global -> shared bulk copy of this GPU's own memory; completion is counted on `bar` in bytes
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   umma::smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(umma::smem_u32(bar))
               : "memory");
}

struct TileRegs {
  uint4 kc;       // key codes: token g words 0, 1; token g + 8 words 0, 1
  uint2 ks;       // key sign words of tokens g, g + 8
  uint4 va;       // values: the three words of token pair (2t, 2t+1), then the first word of pair (2t+8, 2t+9)
  uint2 vb;       // values: the other two words of pair (2t+8, 2t+9)
  float4 nrm;     // key norms of tokens g, g + 8; value norms of tokens g, g + 8
};

// u8 x s8 -> s32, m16n8k32
__device__ __forceinline__ void imma16832(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MODE 0: up to eight query rows, fp16 scores.  MODE 1: up to four rows, fp16 scores with the residual of the
// queries in columns 4..7.  MODE 2: up to four rows, scores from bit planes on the integer tensor cores.
// MODE 3: up to sixteen query rows as two groups of eight columns (prefill): every decoded key and value
// fragment feeds two MMAs, so the decode work and the cache traffic per query row halve; fp16 scores.
template <bool PAGED, int MODE>
__global__ void __launch_bounds__(kWarps * 32, MODE == 3 ? 3 : 4) attend_tiled_kernel(AttnArgs a) {
  constexpr bool LO4 = MODE == 1 || MODE == 2;       // query columns n and n + 4 belong to the same query row
  constexpr bool PLANES = MODE == 2;
  constexpr int NG = MODE == 3 ? 2 : 1;              // groups of eight query columns
  constexpr int kRows = 8 * NG;                      // query rows per CTA
  constexpr int D = 128;
  constexpr int kTile = tile::kTokens;
  // the per-warp record rings of the token loop and the end-of-kernel reduction share storage
  constexpr int kRingBytes = kWarps * kRing * tile::kBytes;
  constexpr int kRedBytes = kWarps * 8 * (D + 2) * 4;
  __shared__ __align__(128) unsigned char pool[kRingBytes > kRedBytes ? kRingBytes : kRedBytes];
  float (*red)[8][D + 2] = reinterpret_cast<float (*)[8][D + 2]>(pool);   // [warp][query][max, sum, acc]
  __shared__ __align__(8) uint64_t bars[kWarps][kRing];
  __shared__ __align__(16) float wsum[kRows];        // fp16 scores: sum of the sign weights per query column
  // B operands per lane.  fp16 scores: two k-steps per entry, 8 key-code steps, then 8 sign steps.  Bit planes:
  // the image that the rotation kernel built for this (batch, kv head): one k-step per entry (both accumulator
  // chains), 8 steps on the code words, then 4 on the sign words, followed by the constants of the query rows.
  __shared__ __align__(16) unsigned char opbuf[PLANES ? sizeof(PlaneImage) : NG * 8 * 32 * sizeof(uint4)];   // [group][k-steps / 2][lane]
  uint4 (*bop)[32] = reinterpret_cast<uint4 (*)[32]>(opbuf);
  __shared__ __align__(8) uint64_t img_bar;
  __shared__ uint32_t vtab[64][32];                  // value table: entry (6-bit field) x lane, an fp16 pair each

  // A kernel launched behind this one as a programmatic dependent (the rotation of the next decode step) may take
  // free CTA slots from now on; it reads and writes nothing before this grid has completed.
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  // Splits are the slowest grid dimension: longest first.  (The splits of a head in consecutive CTAs, so that the
  // CTAs sharing an SM differ in length, measured 5-15 % slower.)
  const int split = blockIdx.z, seg = blockIdx.x;
  const int b = seg / a.Hkv, hkv = seg % a.Hkv;
  // Query rows of a (batch, kv head) are numbered g * q_len + position; a CTA takes eight (sixteen) of them
  // (blockIdx.y), so decode (one tile) and prefill (many) run through the same code.
  const int r0 = kRows * blockIdx.y;
  int64_t kv_len = a.kv_len;
  if (PAGED) kv_len = min(static_cast<int64_t>(max(a.seq_lens[b], 0)), a.kv_len);
  const int nq_all = a.G * a.q_len;
  const int nq = nq_all - r0 < kRows ? nq_all - r0 : kRows;

  // Every (batch entry's) length is divided over the splits in whole 128-token chunks, unequal shares,
  // longest first (split_begin_chunk).
  const int64_t chunks = (kv_len + 127) / 128;
  const int64_t t_begin = 128 * split_begin_chunk(split, a.n_splits, chunks, a.skew);
  int64_t t_end = 128 * split_begin_chunk(split + 1, a.n_splits, chunks, a.skew);
  if (t_end > kv_len) t_end = kv_len;
  if (a.causal) {                      // tokens past the last position any row of this tile may see are skipped
    // rows r0 .. r0 + nq - 1 are consecutive positions of one query head unless they run past its end
    const int p_first = r0 % a.q_len;
    const int last = p_first + nq - 1 >= a.q_len ? a.q_len - 1 : p_first + nq - 1;
    const int64_t visible = kv_len - a.q_len + last + 1;
    if (t_end > visible) t_end = visible;
  }
  const int n_valid = static_cast<int>(t_end - t_begin);        // tokens of this split
  const bool has_work = n_valid > 0;

  // ---- record ring: lane 0 of a warp issues one bulk copy per tile --------------------------------------
  constexpr int kStep = kWarps * kTile;                          // tokens between a warp's tiles
  const int first_rel = warp * kTile;
  const int n_it = first_rel < n_valid ? (n_valid - first_rel + kStep - 1) / kStep : 0;
  unsigned char* ring = pool + warp * (kRing * tile::kBytes);
  uint64_t* bar = bars[warp];
  const int64_t tile_first = (t_begin >> 4) + warp;              // this warp's first tile of the sequence
  // contiguous cache: records of this (batch, kv head); paged: the pool, indexed through the block table
  const int tiles_per_block = PAGED ? a.block_size >> 4 : 1;
  const uint8_t* rec0 = PAGED ? a.records
                              : a.records + (static_cast<int64_t>(seg) * (a.cache.capacity >> 4) + tile_first) * tile::kBytes;
  const int32_t* bt = PAGED ? a.block_table + static_cast<int64_t>(b) * a.max_blocks : nullptr;
  // Paged: position of the tile the next issue() fetches, as (entry of the block table, tile inside the block),
  // advanced by kWarps tiles per issue without a division in the loop; the block id is read one issue ahead.
  int pg_entry = 0, pg_off = 0, pg_step_q = 0, pg_step_r = 0, blk_next = 0;
  if (PAGED) {
    const unsigned tpb = static_cast<unsigned>(tiles_per_block);
    pg_entry = static_cast<int>(static_cast<unsigned>(tile_first) / tpb);
    pg_off = static_cast<int>(static_cast<unsigned>(tile_first) % tpb);
    pg_step_q = static_cast<int>(kWarps / tpb);
    pg_step_r = static_cast<int>(kWarps % tpb);
    blk_next = n_it > 0 ? __ldg(bt + pg_entry) : 0;
  }
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kRing; ++s) umma::mbar_init(bar + s, 1);
    if (warp == 0) umma::mbar_init(&img_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  auto issue = [&](int it, int slot) {                // called with it = 0, 1, 2, ... in order; slot = it % kRing
    if (it < n_it && lane == 0) {
      const uint8_t* src;
      if (PAGED) {
        src = rec0 + ((static_cast<int64_t>(blk_next) * a.Hkv + hkv) * tiles_per_block + pg_off) * tile::kBytes;
      } else {
        src = rec0 + static_cast<int64_t>(it) * (kWarps * tile::kBytes);
      }
      uint64_t* bs = bar + slot;
      mbar_expect_tx(bs, tile::kBytes);
      bulk_load(ring + slot * tile::kBytes, src, tile::kBytes, bs);
    }
    if (PAGED) {                                      // on to tile it + 1 of this warp
      pg_entry += pg_step_q;
      pg_off += pg_step_r;
      if (pg_off >= tiles_per_block) { pg_off -= tiles_per_block; ++pg_entry; }
      blk_next = it + 1 < n_it ? __ldg(bt + pg_entry) : 0;
    }
  };
#pragma unroll
  for (int i = 0; i < kRing; ++i) issue(i, i);

  // Everything above read only the records and the block table, which no kernel of this call writes: when
  // the launch allows it (programmatic dependent launch), this grid starts while the query-rotation kernel is
  // still running and its first records are already on their way.  From here on the rotated queries, the
  // look-up tables and the zeroed arrival counters are needed: wait for that kernel to have completed.
  asm volatile("griddepcontrol.wait;\n" ::: "memory");

  // Everything the scores need of the queries was built by the rotation kernel: the bit-plane image of this
  // (batch, kv head), or the fp16 operand images of this CTA's groups of eight query rows.  One thread fetches
  // them with bulk copies; they land while the value table is built.
  const int groups_per_seg = (nq_all + 7) / 8;
  if (PLANES) {
    if (has_work && threadIdx.x == 0) {
      mbar_expect_tx(&img_bar, sizeof(PlaneImage));
      bulk_load(opbuf, a.planes + seg, sizeof(PlaneImage), &img_bar);
    }
  } else if (has_work) {
    int n_live = 0;
#pragma unroll
    for (int grp = 0; grp < NG; ++grp) n_live += (NG * static_cast<int>(blockIdx.y) + grp < groups_per_seg) ? 1 : 0;
    if (threadIdx.x == 0) {
      mbar_expect_tx(&img_bar, n_live * static_cast<uint32_t>(sizeof(GroupImage)));
#pragma unroll
      for (int grp = 0; grp < NG; ++grp) {
        const int gi = NG * static_cast<int>(blockIdx.y) + grp;
        if (gi < groups_per_seg) {
          const GroupImage* src = a.groups + static_cast<int64_t>(seg) * groups_per_seg + gi;
          bulk_load(opbuf + grp * sizeof(src->bop), src->bop, sizeof(src->bop), &img_bar);
          bulk_load(wsum + 8 * grp, src->wsum, sizeof(src->wsum), &img_bar);
        }
      }
    }
#pragma unroll
    for (int grp = 0; grp < NG; ++grp) {               // a group past the head's last row: neutral operands
      if (NG * static_cast<int>(blockIdx.y) + grp >= groups_per_seg) {
        for (int i = threadIdx.x; i < 8 * 32; i += blockDim.x) bop[8 * grp + (i >> 5)][i & 31] = make_uint4(0u, 0u, 0u, 0u);
        if (threadIdx.x < 8) wsum[8 * grp + threadIdx.x] = 0.f;
      }
    }
  }
  const float inv_sv = __uint_as_float(a.tables[7]);
  const uint32_t kt_a = a.tables[0], kt_b = a.tables[1];     // fp16 key centroids 0,1 | 2,3
  if (has_work) {
    // value table: entry e holds the fp16 values of two stored codes (neg << 2 | mag), the first token's in the
    // low half; every entry is repeated for the 32 lanes (entry e of lane L at word 32 e + L), so that a warp's
    // look-ups never meet in a bank
    const uint32_t mg0 = a.tables[8], mg1 = a.tables[9];        // fp16 value magnitudes 0,1 | 2,3
    auto value_bits = [&](int v) { return ((((v & 2) ? mg1 : mg0) >> (16 * (v & 1))) & 0xFFFFu) | ((v & 4) ? 0x8000u : 0u); };
#pragma unroll
    for (int k = 0; k < 64 / kWarps; ++k) {
      const int e = warp + kWarps * k;
      vtab[e][lane] = value_bits(e & 7) | (value_bits(e >> 3) << 16);
    }
  }
  __syncthreads();
  const unsigned char* vt_base = reinterpret_cast<const unsigned char*>(&vtab[0][0]);
  const uint32_t lane4 = 4u * lane;
  // causal limits of this lane's query columns (2 tig, 2 tig + 1 of every group), relative to the split start
  int lim_rel[NG][2];
#pragma unroll
  for (int grp = 0; grp < NG; ++grp) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int col = 2 * tig + e;
      const int r = 8 * grp + (LO4 ? (col & 3) : col);
      int lim = (r < nq) ? (a.causal ? static_cast<int>(kv_len - a.q_len + (r0 + r) % a.q_len) : 0x7fffffff) : -1;
      const int64_t dlt = static_cast<int64_t>(lim) - t_begin;
      lim_rel[grp][e] = lim == 0x7fffffff ? 0x7fffffff : (dlt < -1 ? -1 : static_cast<int>(dlt));
    }
  }

  float O[NG][8][4];
#pragma unroll
  for (int grp = 0; grp < NG; ++grp)
#pragma unroll
    for (int i = 0; i < 8; ++i) O[grp][i][0] = O[grp][i][1] = O[grp][i][2] = O[grp][i][3] = 0.f;
  // reference exponents start at a finite "nothing seen yet" value (any finite score raises them at once), so that
  // the token loop needs no test for minus infinity; the value written out below turns it back into -inf
  constexpr float kNone = -1e30f;
  float m[NG][2], l[NG][2];
#pragma unroll
  for (int grp = 0; grp < NG; ++grp) { m[grp][0] = m[grp][1] = kNone; l[grp][0] = l[grp][1] = 0.f; }
  // fp16 scores: the accumulators start at -sum of the sign weights.  Bit planes: columns 2 tig, 2 tig + 1 hold
  // terms (t1, t3) of queries 2 tig + e for tig < 2, terms (t2, t4) of queries 2 (tig - 2) + e otherwise; kA, kB
  // turn the two integer sums into score units and ci is the constant of the query (counted once, by tig < 2).
  float ci[NG][2], kA[2] = {0.f, 0.f}, kB[2] = {0.f, 0.f};
#pragma unroll
  for (int grp = 0; grp < NG; ++grp) ci[grp][0] = ci[grp][1] = 0.f;
  bool img_failed = false;
  // the image copies were issued before the value table was built: they have normally landed by now
  if (has_work) img_failed = !__all_sync(QKV_FULL_MASK, umma::mbar_wait(&img_bar, 0));
  if (PLANES) {
    if (has_work) {
      const PlaneImage* img = reinterpret_cast<const PlaneImage*>(opbuf);
      const int hi = tig >> 1;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float u = img->inv[(2 * tig + e) & 3];
        kA[e] = hi ? u * (1.f / 128.f) : u;
        kB[e] = hi ? u * (1.f / 2097152.f) : u * (1.f / 16384.f);
      }
      ci[0][0] = (hi ? 0.f : img->cst[(2 * tig) & 3]) - 12582912.f * kB[0];
      ci[0][1] = (hi ? 0.f : img->cst[(2 * tig + 1) & 3]) - 12582912.f * kB[1];
    }
  } else {
#pragma unroll
    for (int grp = 0; grp < NG; ++grp) {
      ci[grp][0] = -wsum[8 * grp + 2 * tig];
      ci[grp][1] = -wsum[8 * grp + 2 * tig + 1];
    }
  }

  auto process = [&](const TileRegs& cur, int rel) {
    const bool masked = a.causal || rel + kTile > n_valid;      // warp-uniform
    float c[NG][4];
    if constexpr (PLANES) {
      // ---- scores from bit planes: 12 k-steps of 32 single-bit elements, two integer accumulator chains ----
      constexpr int kMagic = 0x4B400000;                         // bit pattern of 1.5 * 2^23
      int ia[4] = {kMagic, kMagic, kMagic, kMagic}, ib[4] = {kMagic, kMagic, kMagic, kMagic};
      uint32_t af[4];
      uint4 bq;
#define QKV_PLANE_STEP(S, W0, W1, P)                                    \
  bq = bop[S][lane];                                                    \
  af[0] = (W0) & (0x01010101u << (P));                                  \
  af[1] = (W1) & (0x01010101u << (P));                                  \
  af[2] = (W0) & (0x01010101u << ((P) + 1));                            \
  af[3] = (W1) & (0x01010101u << ((P) + 1));                            \
  imma16832(ia, af, bq.x, bq.y);                                        \
  imma16832(ib, af, bq.z, bq.w);
      QKV_PLANE_STEP(0, cur.kc.x, cur.kc.z, 0) QKV_PLANE_STEP(1, cur.kc.x, cur.kc.z, 2)
      QKV_PLANE_STEP(2, cur.kc.x, cur.kc.z, 4) QKV_PLANE_STEP(3, cur.kc.x, cur.kc.z, 6)
      QKV_PLANE_STEP(4, cur.kc.y, cur.kc.w, 0) QKV_PLANE_STEP(5, cur.kc.y, cur.kc.w, 2)
      QKV_PLANE_STEP(6, cur.kc.y, cur.kc.w, 4) QKV_PLANE_STEP(7, cur.kc.y, cur.kc.w, 6)
      QKV_PLANE_STEP(8, cur.ks.x, cur.ks.y, 0) QKV_PLANE_STEP(9, cur.ks.x, cur.ks.y, 2)
      QKV_PLANE_STEP(10, cur.ks.x, cur.ks.y, 4) QKV_PLANE_STEP(11, cur.ks.x, cur.ks.y, 6)
#undef QKV_PLANE_STEP
      // The sums are below 2^22 in magnitude, so the first chain comes out exactly with one subtraction.  The
      // second chain weighs 2^-14 of the first: its offset is taken out with the constant (ci holds
      // -1.5 * 2^23 * kB), the rounding of that product being 2^-38 of the largest weight.
      constexpr float kMagicF = 12582912.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float fa = __int_as_float(ia[e]) - kMagicF;
        c[0][e] = fmaf(fa, kA[e & 1], fmaf(__int_as_float(ib[e]), kB[e & 1], ci[0][e & 1]));
      }
    } else {
      // ---- scores: 8 MMAs on key codes, 8 on sign bits, per group of eight query columns ----------------
#pragma unroll
      for (int grp = 0; grp < NG; ++grp) {
        c[grp][0] = ci[grp][0]; c[grp][1] = ci[grp][1]; c[grp][2] = ci[grp][0]; c[grp][3] = ci[grp][1];
      }
      {
        uint32_t af[4];
        uint4 bq[NG];
#define QKV_KEY_STEPS(W0, W1, WORD, F)                                                      \
  _Pragma("unroll") for (int grp = 0; grp < NG; ++grp) bq[grp] = bop[8 * grp + (WORD) * 2 + (F) / 2][lane];   \
  tile::key_fragment<F>(W0, W1, kt_a, kt_b, af);                                            \
  _Pragma("unroll") for (int grp = 0; grp < NG; ++grp) mma16816(c[grp], af, bq[grp].x, bq[grp].y);            \
  tile::key_fragment<F + 1>(W0, W1, kt_a, kt_b, af);                                        \
  _Pragma("unroll") for (int grp = 0; grp < NG; ++grp) mma16816(c[grp], af, bq[grp].z, bq[grp].w);
        QKV_KEY_STEPS(cur.kc.x, cur.kc.z, 0, 0) QKV_KEY_STEPS(cur.kc.x, cur.kc.z, 0, 2)
        QKV_KEY_STEPS(cur.kc.y, cur.kc.w, 1, 0) QKV_KEY_STEPS(cur.kc.y, cur.kc.w, 1, 2)
#undef QKV_KEY_STEPS
      }
      {
        const uint32_t cp0[4] = {cur.ks.x, cur.ks.x << 7, cur.ks.x >> 1, cur.ks.x << 13};
        const uint32_t cp1[4] = {cur.ks.y, cur.ks.y << 7, cur.ks.y >> 1, cur.ks.y << 13};
#pragma unroll
        for (int s2 = 0; s2 < 4; ++s2) {
          uint4 bw[NG];
#pragma unroll
          for (int grp = 0; grp < NG; ++grp) bw[grp] = bop[8 * grp + 4 + s2][lane];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int s = 2 * s2 + u;
            uint32_t af[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int t = 2 * s + h;
              const int cpy = t < 7 ? 0 : (t < 14 ? 1 : t - 12);
              const uint32_t mask = 0x00010001u << sign_pos(t);
              af[2 * h] = cp0[cpy] & mask;
              af[2 * h + 1] = cp1[cpy] & mask;
            }
#pragma unroll
            for (int grp = 0; grp < NG; ++grp)
              mma16816(c[grp], af, u ? bw[grp].z : bw[grp].x, u ? bw[grp].w : bw[grp].y);
          }
        }
      }
    }
    if (LO4) {                      // column n + 4 holds the other part of column n: add the two
#pragma unroll
      for (int e = 0; e < 4; ++e) c[0][e] += __shfl_xor_sync(QKV_FULL_MASK, c[0][e], 2);
    }

    // ---- online softmax on the accumulator fragment (log2 domain) ------------------------------
    // t = score - m, in one multiply-add per entry.  m is a reference exponent, not the exact running maximum:
    // it is raised (to the exact maximum of the tile, over the eight token lanes of a query column) only when a
    // score of this tile exceeds it by more than kSlack, so that most tiles need one vote instead of three
    // shuffle rounds.  Weights stay below 2^kSlack, far inside fp16 once multiplied by a value norm, and the
    // merge of the splits only needs l and the accumulators to be relative to the m that is written out.
    constexpr float kSlack = 4.f;
    const float kn0 = cur.nrm.x, kn1 = cur.nrm.y;
    float vn0 = cur.nrm.z, vn1 = cur.nrm.w;
    const int tokA = rel + gid, tokB = tokA + 8;
    if (masked) {
      if (tokA >= n_valid) vn0 = 0.f;         // rows past the end of the sequence hold no data
      if (tokB >= n_valid) vn1 = 0.f;
    }
    uint32_t pb[NG][2];             // weights times value norm, in the B layout (tokens as K, query = gid as N)
#pragma unroll
    for (int grp = 0; grp < NG; ++grp) {
      float t[4] = {fmaf(c[grp][0], kn0, -m[grp][0]), fmaf(c[grp][1], kn0, -m[grp][1]),
                    fmaf(c[grp][2], kn1, -m[grp][0]), fmaf(c[grp][3], kn1, -m[grp][1])};
      if (masked) {
        if (!(tokA < n_valid && tokA <= lim_rel[grp][0])) t[0] = -INFINITY;
        if (!(tokA < n_valid && tokA <= lim_rel[grp][1])) t[1] = -INFINITY;
        if (!(tokB < n_valid && tokB <= lim_rel[grp][0])) t[2] = -INFINITY;
        if (!(tokB < n_valid && tokB <= lim_rel[grp][1])) t[3] = -INFINITY;
      }
      if (__any_sync(QKV_FULL_MASK, fmaxf(fmaxf(t[0], t[2]), fmaxf(t[1], t[3])) > kSlack)) {
        // (rare after the first tiles) exact scores again: against the start value of m, t has lost them
        float sc[4] = {c[grp][0] * kn0, c[grp][1] * kn0, c[grp][2] * kn1, c[grp][3] * kn1};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (t[e] == -INFINITY) sc[e] = -INFINITY;
        float mx[2] = {fmaxf(sc[0], sc[2]), fmaxf(sc[1], sc[3])};
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          mx[0] = fmaxf(mx[0], __shfl_xor_sync(QKV_FULL_MASK, mx[0], o));
          mx[1] = fmaxf(mx[1], __shfl_xor_sync(QKV_FULL_MASK, mx[1], o));
        }
        float al[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          al[e] = (mx[e] > m[grp][e]) ? ex2(m[grp][e] - mx[e]) : 1.f;     // ex2(kNone - x) = 0 on the first tile
          m[grp][e] = fmaxf(m[grp][e], mx[e]);
          l[grp][e] *= al[e];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          O[grp][i][0] *= al[0]; O[grp][i][1] *= al[1]; O[grp][i][2] *= al[0]; O[grp][i][3] *= al[1];
        }
        t[0] = sc[0] - m[grp][0]; t[1] = sc[1] - m[grp][1]; t[2] = sc[2] - m[grp][0]; t[3] = sc[3] - m[grp][1];
      }
      const float p0 = ex2(t[0]), p1 = ex2(t[1]), p2 = ex2(t[2]), p3 = ex2(t[3]);   // masked entries: weight 0
      l[grp][0] += p0 + p2;
      l[grp][1] += p1 + p3;
      pb[grp][0] = movmatrix_trans(pack_half2(p0 * vn0, p1 * vn0));
      pb[grp][1] = movmatrix_trans(pack_half2(p2 * vn1, p3 * vn1));
    }

    // ---- values: one table look-up per pair of tokens, 8 MMAs per group --------------------------------
    {
      uint32_t af[4];
      auto vt = [&](uint32_t off) { return *reinterpret_cast<const uint32_t*>(vt_base + off); };
#define QKV_VAL_STEP(I)                                                                                   \
  af[0] = vt(tile::value_table_offset<2 * (I)>(cur.va.x, cur.va.y, cur.va.z, lane4));                     \
  af[1] = vt(tile::value_table_offset<2 * (I) + 1>(cur.va.x, cur.va.y, cur.va.z, lane4));                 \
  af[2] = vt(tile::value_table_offset<2 * (I)>(cur.va.w, cur.vb.x, cur.vb.y, lane4));                     \
  af[3] = vt(tile::value_table_offset<2 * (I) + 1>(cur.va.w, cur.vb.x, cur.vb.y, lane4));                 \
  _Pragma("unroll") for (int grp = 0; grp < NG; ++grp) mma16816(O[grp][I], af, pb[grp][0], pb[grp][1]);
      QKV_VAL_STEP(0) QKV_VAL_STEP(1) QKV_VAL_STEP(2) QKV_VAL_STEP(3)
      QKV_VAL_STEP(4) QKV_VAL_STEP(5) QKV_VAL_STEP(6) QKV_VAL_STEP(7)
#undef QKV_VAL_STEP
    }
  };

  // The loop over this warp's tiles is unrolled over the ring, so that stage addresses and barrier addresses are
  // constants of each copy of the body.
  int it_failed = -1;
  {
    int it = 0, rel = first_rel;
    uint32_t parity = 0;
    while (it < n_it && it_failed < 0) {
#pragma unroll
      for (int slot = 0; slot < kRing; ++slot) {
        if (it < n_it && it_failed < 0) {
          if (__all_sync(QKV_FULL_MASK, umma::mbar_wait(bar + slot, parity))) {
            const unsigned char* stage = ring + slot * tile::kBytes;
            TileRegs cur;
            cur.kc = *reinterpret_cast<const uint4*>(stage + tile::kOffKeyCodes + 16 * lane);
            cur.ks = *reinterpret_cast<const uint2*>(stage + tile::kOffKeySigns + 8 * lane);
            cur.va = *reinterpret_cast<const uint4*>(stage + tile::kOffVal16 + 16 * lane);
            cur.vb = *reinterpret_cast<const uint2*>(stage + tile::kOffVal8 + 8 * lane);
            cur.nrm = *reinterpret_cast<const float4*>(stage + tile::kOffNorms + 16 * gid);
            process(cur, rel);
            // The slot is refilled only now.  A warp issues its instructions in order and an instruction issues
            // only once its source registers hold their values, so at this point every lane's loads from the
            // slot have returned (process() consumed all of them): the copy cannot overwrite bytes that are still
            // to be read.  Issuing it straight after the loads, before their values are used, lost that
            // guarantee: with records coming from L2 and the load queue of the SM full, a copy was seen to land
            // before a queued load.
            __syncwarp();
            issue(it + kRing, slot);
            ++it;
            rel += kStep;
          } else {
            it_failed = it;
          }
        }
      }
      parity ^= 1u;
    }
  }
  if (it_failed >= 0) {
    // A copy never arrived (not seen in practice; a hardware fault would look like this).  Count it, give the
    // copies that are still in flight a last bounded chance to land, so that nothing writes this CTA's shared
    // memory once it is reused below, and go on: the result of this split is then meaningless, and the
    // counter behind qkv_tensor_core_timeouts() tells the caller so.
    if (lane == 0) atomicAdd(&g_bulk_timeouts, 1u);
    for (int it = it_failed + 1; it < n_it && it < it_failed + kRing; ++it)
      umma::mbar_wait(bar + it % kRing, (it / kRing) & 1);
  }
  if (img_failed && lane == 0) atomicAdd(&g_bulk_timeouts, 1u);   // same for the operand image (its storage is not reused)
  __syncthreads();                        // the reduction buffer below reuses the ring storage

  // out rows = vec @ Pi for up to eight rows `vec[r][D]` in shared memory.  Warp w takes rows 32 w .. 32 w + 31 of
  // Pi, a lane four output coordinates, so that the 32 loads of a thread are independent (two rounds of 16); the
  // four warps' partial sums meet in `psum` ([kWarps][8][D], shared memory that nobody else is reading).
  // A table that breaks what the record format (symmetric value table) or the bit planes (key table affine in
  // its code bits) presume would give wrong numbers silently: NaN instead.
  const bool broken = (a.tables[10] & (PLANES ? 3u : 1u)) != 0u;
  auto unrotate = [&](const float* vec, float* psum, int n_rows, const int64_t* qrow) {
    float4 o[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) o[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4* prow = reinterpret_cast<const float4*>(a.Pi + static_cast<int64_t>(32 * warp) * D) + lane;
#pragma unroll 16
    for (int jj = 0; jj < 32; ++jj) {
      const float4 mval = __ldg(prow + jj * (D / 4));
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float x = vec[r * D + 32 * warp + jj];
        o[r].x = fmaf(x, mval.x, o[r].x);
        o[r].y = fmaf(x, mval.y, o[r].y);
        o[r].z = fmaf(x, mval.z, o[r].z);
        o[r].w = fmaf(x, mval.w, o[r].w);
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) *reinterpret_cast<float4*>(psum + (warp * 8 + r) * D + 4 * lane) = o[r];
    __syncthreads();
    const int i = threadIdx.x;                       // output coordinate (blockDim.x == D)
    for (int r = 0; r < n_rows; ++r) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) v += psum[(w * 8 + r) * D + i];
      a.out[qrow[r] * D + i] = broken ? __int_as_float(0x7fc00000) : v;
    }
  };
  // With a single split there is nothing to merge: the rows go from the reduction buffer straight through the
  // un-rotation, without the round trip through the partials in global memory, the fence and the arrival counter.
  const bool single = a.n_splits == 1;
  float* vec1 = reinterpret_cast<float*>(pool + kRedBytes);     // [8][D] behind the reduction buffer
  static_assert(kRedBytes + 8 * D * 4 <= sizeof(pool) && kWarps * 8 * D * 4 <= kRedBytes, "single-split buffers fit");

  // ---- per-warp results to shared memory: column sums over the token lanes, then all warps; a group of eight
  // query columns at a time through the same buffer ------------------------------------------------------------
  constexpr float kLn2 = 0.6931471805599453f;
  // weights of the four warps' results per query row, and where the row's partials go: once per row, not per entry
  __shared__ float fw_s[kWarps][8], mrow_s[8];
  __shared__ int64_t qrow_s[kRows];
  if (threadIdx.x < kRows) {
    const int r = threadIdx.x;
    const int g = (r0 + r) / a.q_len, qi = (r0 + r) % a.q_len;
    qrow_s[r] = (static_cast<int64_t>(b) * a.Hq + hkv * a.G + g) * a.q_len + qi;
  }
#pragma unroll
  for (int grp = 0; grp < NG; ++grp) {
    if (grp > 0) __syncthreads();                     // the previous group's rows have been read
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l[grp][0] += __shfl_xor_sync(QKV_FULL_MASK, l[grp][0], o);
      l[grp][1] += __shfl_xor_sync(QKV_FULL_MASK, l[grp][1], o);
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float* dst = red[warp][2 * tig + e];
      if (gid == 0) {
        dst[0] = m[grp][e] == kNone ? -INFINITY : m[grp][e] * kLn2;   // natural-log units, as the merge expects; -inf = no token
        dst[1] = l[grp][e];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {   // M-tile i holds coordinates 16 gid + 2 i, +1
        dst[2 + 16 * gid + 2 * i] = O[grp][i][e] * inv_sv;
        dst[2 + 16 * gid + 2 * i + 1] = O[grp][i][2 + e] * inv_sv;
      }
    }
    __syncthreads();
    if (threadIdx.x < 8 * kWarps) {
      const int w = threadIdx.x >> 3, r = threadIdx.x & 7;
      float M = -INFINITY;
#pragma unroll
      for (int u = 0; u < kWarps; ++u) M = fmaxf(M, red[u][r][0]);
      fw_s[w][r] = (red[w][r][0] == -INFINITY) ? 0.f : expf(red[w][r][0] - M);
      if (w == 0) mrow_s[r] = M;
    }
    __syncthreads();
    const int nqg = nq - 8 * grp < 8 ? nq - 8 * grp : 8;
    if (single) {
#pragma unroll
      for (int r = 0; r < 8; ++r) {                  // a thread per coordinate
        float v = 0.f, sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          v = fmaf(fw_s[w][r], red[w][r][2 + threadIdx.x], v);
          sum = fmaf(fw_s[w][r], red[w][r][1], sum);
        }
        vec1[r * D + threadIdx.x] = r < nqg ? v / fmaxf(sum, 1e-30f) : 0.f;
      }
      __syncthreads();                               // rows complete; the reduction buffer is free for the sums
      unrotate(vec1, reinterpret_cast<float*>(pool), nqg, qrow_s + 8 * grp);
      continue;
    }
    for (int r = 0; r < nqg; ++r) {                  // a thread per coordinate; threads 0, 1 also write max and sum
      float* dst = a.part + (qrow_s[8 * grp + r] * a.n_splits + split) * (D + 2);
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) v = fmaf(fw_s[w][r], red[w][r][2 + threadIdx.x], v);
      dst[2 + threadIdx.x] = v;
      if (threadIdx.x == 0) dst[0] = mrow_s[r];
      if (threadIdx.x == 1) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) sum = fmaf(fw_s[w][r], red[w][r][1], sum);
        dst[1] = sum;
      }
    }
  }

  if (single) return;

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
  static_assert((8 * D + 8 * kMaxSplits + 8 + kWarps * 8 * D) * 4 <= sizeof(pool), "merge buffers fit the ring storage");
  for (int grp = 0; grp < NG; ++grp) {               // eight query rows at a time through the merge buffers
  const int nqg = nq - 8 * grp < 8 ? nq - 8 * grp : 8;
  if (grp > 0) __syncthreads();
  // This tail runs once per (batch, kv head) at the very end of the call, so it is written for latency: every
  // round of loads is issued before the first result is used.
  for (int r = warp; r < nqg; r += kWarps) {          // a warp per query row; a lane takes splits lane, lane + 32
    const float* pp = a.part + qrow_s[8 * grp + r] * a.n_splits * (D + 2);
    float mm[2], ll[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int sp = lane + 32 * h;
      const bool live = sp < a.n_splits;
      mm[h] = live ? __ldcg(pp + sp * (D + 2)) : -INFINITY;
      ll[h] = live ? __ldcg(pp + sp * (D + 2) + 1) : 0.f;
    }
    float M = fmaxf(mm[0], mm[1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(QKV_FULL_MASK, M, o));
    float L = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int sp = lane + 32 * h;
      const float f = (mm[h] == -INFINITY) ? 0.f : expf(mm[h] - M);
      if (sp < a.n_splits) wgt[r * kMaxSplits + sp] = f;
      L += f * ll[h];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(QKV_FULL_MASK, L, o);
    if (lane == 0) invl[r] = 1.f / fmaxf(L, 1e-30f);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nqg * (D / 2); idx += blockDim.x) {     // a thread per pair of coordinates
    const int r = idx / (D / 2), j = 2 * (idx % (D / 2));
    const float* pp = a.part + qrow_s[8 * grp + r] * a.n_splits * (D + 2) + 2 + j;  // 8-byte aligned: rows of 130 floats
    const float* w = wgt + r * kMaxSplits;
    float2 acc = make_float2(0.f, 0.f);
    for (int sp = 0; sp < a.n_splits; sp += 16) {                         // sixteen splits per round of loads
      float2 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        v[u] = sp + u < a.n_splits ? __ldcg(reinterpret_cast<const float2*>(pp + (sp + u) * (D + 2))) : make_float2(0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const float wu = sp + u < a.n_splits ? w[sp + u] : 0.f;
        acc.x = fmaf(wu, v[u].x, acc.x);
        acc.y = fmaf(wu, v[u].y, acc.y);
      }
    }
    vec[r * D + j] = acc.x * invl[r];
    vec[r * D + j + 1] = acc.y * invl[r];
  }
  __syncthreads();
  unrotate(vec, invl + 8, nqg, qrow_s + 8 * grp);   // partial sums behind vec, wgt and invl
  }
}

}  // namespace

unsigned int bulk_copy_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_bulk_timeouts, sizeof(v));
  return v;
}


bool tiled_path_ok(int d, int key_bits, int val_bits) { return d == 128 && key_bits == 3 && val_bits == 3; }

// QUASHKV_B200_SCORES=fp16 keeps the fp16 scores everywhere (for comparison).
bool tiled_scores_from_planes(int group, int q_len) {
  if (group * q_len > 4) return false;
  const char* e = getenv("QUASHKV_B200_SCORES");
  return !(e && e[0] == 'f');
}

// QUASHKV_B200_PREFILL_ROWS=8 keeps eight query rows per CTA for longer query blocks too (for comparison).
static bool sixteen_rows(int nq_all) {
  if (nq_all <= 8) return false;
  const char* e = getenv("QUASHKV_B200_PREFILL_ROWS");
  return !(e && e[0] == '8');
}

int launch_attend_tiled(const AttnArgs& a_in, cudaStream_t st) {
  const int nq_all = a_in.G * a_in.q_len;
  // up to four query rows: scores from bit planes on the integer tensor cores, when the caller had the rotation
  // kernel build the operand images, else the fp16 form; five to eight rows: one group of eight columns; more:
  // sixteen rows per CTA
  const int mode = nq_all <= 4 ? (a_in.planes ? 2 : 1) : (sixteen_rows(nq_all) ? 3 : 0);
  const int rows = mode == 3 ? 16 : 8;
  const dim3 grid(a_in.B * a_in.Hkv, (nq_all + rows - 1) / rows, a_in.n_splits);
  // Programmatic dependent launch: the grid may start while the kernel before it in the stream (the query
  // rotation, which releases its dependents at once) is still running; the kernel waits for that kernel's
  // completion before it reads anything that kernel writes.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const AttnArgs& a = a_in;
  cudaError_t err;
  if (a.block_table)
    err = mode == 3 ? cudaLaunchKernelEx(&cfg, attend_tiled_kernel<true, 3>, a)
        : mode == 2 ? cudaLaunchKernelEx(&cfg, attend_tiled_kernel<true, 2>, a)
        : mode == 1 ? cudaLaunchKernelEx(&cfg, attend_tiled_kernel<true, 1>, a)
                    : cudaLaunchKernelEx(&cfg, attend_tiled_kernel<true, 0>, a);
  else
    err = mode == 3 ? cudaLaunchKernelEx(&cfg, attend_tiled_kernel<false, 3>, a)
        : mode == 2 ? cudaLaunchKernelEx(&cfg, attend_tiled_kernel<false, 2>, a)
        : mode == 1 ? cudaLaunchKernelEx(&cfg, attend_tiled_kernel<false, 1>, a)
                    : cudaLaunchKernelEx(&cfg, attend_tiled_kernel<false, 0>, a);
  if (err != cudaSuccess) return QKV_ELAUNCH;
  return check_launch();
}

}  // namespace qkv
