// Decompress at d = 128 with the un-rotation on the fifth-generation tensor cores (tcgen05).
//
// out = norm * (v @ Pi) with v_i = c[code_i] (+ qjl_scale * S_i * (2 sign_i - 1) for keys): a 128 x 128 x 128
// contraction per tile of 128 vectors with A = the decoded rows and B = Pi^T.  One CTA per SM; the fp32
// accumulator lives in tensor memory (two accumulators alternate) and completion arrives on an mbarrier.
//
//   * Exact fp32 from fp16 MMAs.  Both operands are scaled by a power of two that puts their largest magnitude
//     just below 2^14 and split into TWO fp16 terms, x = h + m with |m| <= ulp(h) / 2: 22 significand bits, and
//     the scaling keeps m out of the subnormal range for every value that matters.  Three products (m*h, h*m,
//     h*h, smallest first: 24 MMAs of 128 x 128 x 16 per tile; m*m is below 2^-22) accumulate in fp32; the power
//     of two leaves with the norm.  B (two planes of Pi^T, 128-byte swizzled K-major) is staged once per CTA.
//   * Decode by pairs, straight into tensor memory.  With S = +-1 (what the quantiser generates) a pair of
//     neighbouring coordinates takes one of 2^(2 bits [+ 2]) values, and the packed row holds the two codes side
//     by side: the field (and the two sign bits) index a shared-memory table of READY operand words (h0 | h1,
//     m0 | m1), repeated per lane so that every lane of a half warp reads its own banks.  A pair costs a shift,
//     a mask (a shift and a merge more for the sign bits) and one 8-byte load, and its two words ARE 32-bit
//     columns of the two A planes in tensor memory (lane = row): sixteen pairs leave as one tcgen05.st per
//     plane, and the MMA reads A from tensor memory, so the tensor core's shared-memory traffic is B alone.
//   * Roles.  Warp 0 only issues: its first lane waits until every worker thread has arrived on the "A(i) is
//     written" barrier, issues the 24 MMAs and commits them (the issuing thread is held for about as long as the
//     MMAs execute; as a worker it held the whole CTA back by that time).  Warps 4-11 are the workers: two per
//     lane quadrant of tensor memory, 2 x 32 columns per thread.  There is no CTA barrier in the loop; two A
//     buffers, so tile i+1 is decoded while tile i is multiplied.
//   * Output.  A worker issues the read of tile i-1's accumulator, decodes tile i while it travels, then scales
//     its 64 values by the norm.  fp32: the 256 bytes go to a staging row of the thread's own and leave with ONE
//     bulk copy (shared -> global); bf16: a warp transposition and stores of 4 rows x 128 bytes.
//   * The packed words and the norm of a tile are fetched one tile ahead of their use.
//
// Every wait on the tensor core is bounded; if one runs out the CTA stops using the tensor core, counts the
// event and derives its remaining tiles with the fp32 chain alone (slow, still correct).
#include <cuda_fp16.h>

#include <cstdlib>

#include <type_traits>

#include "rotate_exact.cuh"
#include "umma.cuh"

namespace qkv {

__device__ unsigned int g_dec_umma_timeouts = 0;

namespace {

constexpr int kDTile = 128;                       // vectors per tile = MMA M
constexpr int kDFirstWorker = 4;                  // warps 4 .. 11 decode and store; warp 0 issues the MMAs
constexpr int kDWorkers = 256;                    // two worker threads per vector: 2 x 32 coordinates each
constexpr int kDThreads = 32 * kDFirstWorker + kDWorkers;
constexpr uint32_t kDPlaneBytes = 128 * 128 * 2;  // one fp16 plane of Pi^T (two 64-wide K blocks)
constexpr uint32_t kDTmemCols = 512;              // accumulators [0, 256), A operands [256, 512)
constexpr uint32_t kDTmemA = 256;                 // A[buffer][term]: 64 columns each (128 fp16 per row)
constexpr uint32_t kDTableBytes = 32768;          // pair tables (mixed precision: two halves)
constexpr int kDProducts = 3;                     // of m*m, m*h, h*m, h*h the last three: the first is below 2^-22
constexpr uint32_t kDStageRow = 272;              // staging row of a worker thread: 256 bytes + 16
constexpr int kDTopExp = 14;                      // operands are scaled to a largest magnitude in [2^13, 2^14)

__host__ __device__ constexpr int ilog2(int v) { return v <= 1 ? 0 : 1 + ilog2(v >> 1); }

// A pair table has one entry per (code, code [, sign, sign]) of two neighbouring coordinates and is repeated
// `replicas` times, entry e of replica r at element e * replicas + r: with 16 replicas the 16 lanes of a half
// warp (an 8-byte load is served per half warp) never meet in a bank whatever entries they read.
template <int BW, bool SIGNS>
__host__ __device__ constexpr int pair_entries() { return 1 << (2 * (BW + (SIGNS ? 1 : 0))); }
template <int BW, bool SIGNS, bool MIXED>
__host__ __device__ constexpr int pair_replicas() {
  constexpr int cap = static_cast<int>((MIXED ? kDTableBytes / 2 : kDTableBytes) / 8) / pair_entries<BW, SIGNS>();
  return cap >= 16 ? 16 : cap;
}

struct DecSmem {
  unsigned char* scratch;   // output staging: a row of kDStageRow bytes per worker thread (fp32 out) or 32 lines of
                            // 128 bytes per worker warp (bf16 out); 4 planes, which also keeps the CTA alone on its
                            // SM (it owns all of tensor memory)
  unsigned char* b;         // Pi^T planes h, m
  unsigned char* tab;       // pair tables
  uint64_t* mbar;           // [4]: accumulator 0 / 1 complete, A buffer 0 / 1 written
  uint32_t* tmem_slot;
  int* dead;
};

constexpr size_t dec_smem_bytes() { return 1024 + 6 * kDPlaneBytes + kDTableBytes + 4 * 8 + 16; }

__device__ __forceinline__ DecSmem carve_dec(unsigned char* raw) {
  DecSmem s;
  unsigned char* p = raw + ((1024u - (umma::smem_u32(raw) & 1023u)) & 1023u);
  s.scratch = p; p += 4 * kDPlaneBytes;
  s.b = p; p += 2 * kDPlaneBytes;
  s.tab = p; p += kDTableBytes;
  s.mbar = reinterpret_cast<uint64_t*>(p); p += 32;
  s.tmem_slot = reinterpret_cast<uint32_t*>(p);
  s.dead = reinterpret_cast<int*>(p + 4);
  return s;
}

// x = h + m to 22 bits, each term an fp16 (round to nearest at both steps; x - h is exact in fp32).
__device__ __forceinline__ void split2h(float x, __half& h, __half& m) {
  h = __float2half_rn(x);
  m = __float2half_rn(x - __half2float(h));
}

// One arrival (release at CTA scope) on a CTA-local barrier; the thread does not wait.
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_u32(bar)) : "memory");
}

// Bulk copy shared -> global of `bytes` (a multiple of 16; both addresses 16-byte aligned), tracked by the
// thread's bulk groups.
__device__ __forceinline__ void bulk_store(void* dst, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dst),
               "r"(umma::smem_u32(src_smem)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// All of this thread's bulk groups have read their source / have completed.
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_h(__half lo, __half hi) {
  return static_cast<uint32_t>(__half_as_ushort(lo)) | (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
}

// Power of two that brings a largest magnitude of `mx` into [2^(kDTopExp-1), 2^kDTopExp); 0 for 0, inf, nan.
__device__ __forceinline__ int scale_exponent(float mx) {
  if (!(mx > 0.f) || !(mx < 3.0e38f)) return 0;
  int e;
  frexpf(mx, &e);                                   // mx = f * 2^e, f in [0.5, 1)
  const int k = kDTopExp - e;
  return k < -60 ? -60 : (k > 60 ? 60 : k);
}

// y = Pi^T-rotation of one decoded row by the fp32 chain (only used after a tensor-core timeout).
__device__ __noinline__ float decompress_chain(const float* vrow, const float* Pi, int col) {
  float z = 0.f;
  for (int i = 0; i < kRD; ++i) z = fmaf(vrow[i], __ldg(Pi + i * kRD + col), z);
  return z;
}

// BITS1 != 0: mixed precision (no sign term).  The K dimension runs in STREAM order (outlier channels first):
// A column k' is stream position k' and B row k' is Pi[perm[k']], so each block of 32 coordinates belongs to
// one table; needs the outlier count to be a multiple of 32, otherwise the CTA returns and the CUDA-core
// kernel launched behind it does the work (same device-side test, inverted).
//
// Warps: 0 = the issuing warp (its first lane waits for "A(i) is written", issues the 24 MMAs of tile i and
// commits them to the accumulator's barrier), 1-3 take part in the set-up only, 4-11 = workers.  Worker warp w
// owns rows 32 (w & 3) .. + 31 (the tensor-memory lanes its warp may read) and columns 64 ((w - 4) >> 2) .. + 63
// as two blocks of 32; a worker thread decodes and later stores 2 x 32 coordinates of ONE row.  Workers never wait
// for each other inside the loop: they arrive on the "written" barrier and go on to the epilogue of the previous
// tile, so the decode of some warps overlaps the stores of others.  (The thread that issues the MMAs is blocked
// for about as long as they execute, the queue being short; as a worker it held the whole CTA back by that time
// at the next barrier.)
template <int BITS, bool SIGNS, int BITS1 = 0>
__global__ void __launch_bounds__(kDThreads, 1) decompress_umma_kernel(DecompressArgs a) {
  constexpr bool MIXED = BITS1 != 0;
  constexpr int BMAX = BITS > BITS1 ? BITS : BITS1;
  constexpr int R0 = pair_replicas<BITS, SIGNS, MIXED>();
  constexpr int R1 = pair_replicas<(MIXED ? BITS1 : BITS), SIGNS, MIXED>();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float cent_s[2][16], qs_s[kRD];
  __shared__ uint32_t smask_s[4];           // bit c of word w: S[32 w + c] < 0 (mixed: channel is an outlier)
  __shared__ uint32_t red_s[3];             // bit patterns of max |Pi|, max |centroid|, max |S|
  __shared__ uint8_t perm_s[kRD];
  const DecSmem s = carve_dec(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool worker = warp >= kDFirstWorker;
  const int trow = 32 * (warp & 3) + lane;
  const int blk0 = worker ? 2 * ((warp - kDFirstWorker) >> 2) : 0;     // first of this thread's two column blocks
  const uint32_t* codes = reinterpret_cast<const uint32_t*>(a.codes);
  const uint32_t* signs = reinterpret_cast<const uint32_t*>(a.signs);

  int n_out = MIXED ? 0 : kRD;                      // K positions below n_out use table 0
  if (MIXED) {
    bool o = false;
    if (tid < kRD) {
      o = a.is_outlier[tid] != 0;
      const uint32_t m = __ballot_sync(QKV_FULL_MASK, o);
      if (lane == 0) smask_s[warp] = m;
    }
    __syncthreads();
    int before = 0;
    for (int w = 0; w < 4; ++w) {
      const int c = __popc(smask_s[w]);
      n_out += c;
      if (w < warp) before += c;
    }
    if (n_out & 31) return;                         // every thread of every CTA: left to the CUDA-core kernel
    if (tid < kRD) {
      before += __popc(smask_s[warp] & ((1u << lane) - 1u));
      perm_s[o ? before : n_out + (tid - before)] = static_cast<uint8_t>(tid);
    }
    __syncthreads();
  }
  const int m_out = n_out >> 5;
  const int row_words = MIXED ? m_out * BITS + (4 - m_out) * BITS1 : 4 * BITS;
  int cls[2], word_off[2], bits_c[2];               // per column block: table, first packed word, bit width
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int blk = blk0 + u;
    cls[u] = blk >= m_out ? 1 : 0;
    word_off[u] = cls[u] ? m_out * BITS + (blk - m_out) * BITS1 : blk * BITS;
    bits_c[u] = cls[u] ? BITS1 : BITS;
  }

  // ---- one-time setup: small tables, operand scales, Pi^T planes, pair tables, barriers, TMEM --------------
  if (tid < 3) red_s[tid] = 0u;
  if (tid < 16) {
    cent_s[0][tid] = tid < (1 << BITS) ? a.cents0[tid] : 0.f;
    cent_s[1][tid] = (MIXED && tid < (1 << BITS1)) ? a.cents1[tid] : 0.f;
  }
  bool pm1 = true;
  float s_abs = 0.f;
  if (tid < kRD) {
    const float sv = SIGNS ? a.S[tid] : 1.f;
    qs_s[tid] = SIGNS ? a.qjl_scale * sv : 0.f;
    pm1 = fabsf(sv) == 1.f;
    s_abs = SIGNS ? fabsf(sv) : 0.f;
    const uint32_t neg = __ballot_sync(QKV_FULL_MASK, sv < 0.f);
    if (lane == 0) smask_s[warp] = neg;
  }
  const bool table_ok = __syncthreads_and(pm1) != 0;     // S = +-1 everywhere: the pair table applies
  {
    float pi_abs = 0.f;
    for (int idx = tid; idx < kRD * kRD; idx += kDThreads) pi_abs = fmaxf(pi_abs, fabsf(__ldg(a.Pi + idx)));
    float c_abs = tid < 32 ? fabsf(cent_s[tid >> 4][tid & 15]) : 0.f;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      pi_abs = fmaxf(pi_abs, __shfl_xor_sync(QKV_FULL_MASK, pi_abs, o));
      c_abs = fmaxf(c_abs, __shfl_xor_sync(QKV_FULL_MASK, c_abs, o));
      s_abs = fmaxf(s_abs, __shfl_xor_sync(QKV_FULL_MASK, s_abs, o));
    }
    if (lane == 0) {                                // non-negative floats order like their bit patterns
      atomicMax(&red_s[0], __float_as_uint(pi_abs));
      if (warp == 0) atomicMax(&red_s[1], __float_as_uint(c_abs));
      if (SIGNS && warp < 4) atomicMax(&red_s[2], __float_as_uint(s_abs));
    }
  }
  __syncthreads();
  const int kb = scale_exponent(__uint_as_float(red_s[0]));
  const int ka = scale_exponent(__uint_as_float(red_s[1]) + fabsf(a.qjl_scale) * __uint_as_float(red_s[2]));
  const float scale_a = ldexpf(1.f, ka), scale_b = ldexpf(1.f, kb), descale = ldexpf(1.f, -(ka + kb));

  for (int idx = tid; idx < kRD * kRD; idx += kDThreads) {      // B[n = output j][k] = Pi[channel of k][j]
    const int i = idx >> 7, j = idx & 127;
    __half h, m;
    split2h(a.Pi[(MIXED ? perm_s[i] : i) * kRD + j] * scale_b, h, m);
    const uint32_t off = umma::sw128_offset(j, i, 128);
    *reinterpret_cast<__half*>(s.b + off) = h;
    *reinterpret_cast<__half*>(s.b + kDPlaneBytes + off) = m;
  }
  auto build_pairs = [&](auto bw_tag, auto rep_tag, uint2* tab, const float* cent) {
    constexpr int BW = decltype(bw_tag)::value, R = decltype(rep_tag)::value;
    constexpr int E = pair_entries<BW, SIGNS>();
    constexpr uint32_t CM = (1u << BW) - 1u;
    for (int idx = tid; idx < E * R; idx += kDThreads) {
      const uint32_t e = static_cast<uint32_t>(idx / R);
      float x0 = cent[e & CM], x1 = cent[(e >> BW) & CM];
      if (SIGNS) {
        x0 += (e >> (2 * BW)) & 1u ? a.qjl_scale : -a.qjl_scale;
        x1 += (e >> (2 * BW + 1)) & 1u ? a.qjl_scale : -a.qjl_scale;
      }
      __half h0, m0, h1, m1;
      split2h(x0 * scale_a, h0, m0);
      split2h(x1 * scale_a, h1, m1);
      tab[idx] = make_uint2(pack_h(h0, h1), pack_h(m0, m1));
    }
  };
  uint2* const tab0 = reinterpret_cast<uint2*>(s.tab);
  uint2* const tab1 = reinterpret_cast<uint2*>(s.tab + kDTableBytes / 2);
  build_pairs(std::integral_constant<int, BITS>{}, std::integral_constant<int, R0>{}, tab0, cent_s[0]);
  if (MIXED)
    build_pairs(std::integral_constant<int, (MIXED ? BITS1 : BITS)>{}, std::integral_constant<int, R1>{}, tab1, cent_s[1]);
  const unsigned char* tabl[2];
  uint32_t smask[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    tabl[u] = cls[u] ? reinterpret_cast<const unsigned char*>(tab1 + (lane & (R1 - 1)))
                     : reinterpret_cast<const unsigned char*>(tab0 + (lane & (R0 - 1)));
    smask[u] = SIGNS ? smask_s[blk0 + u] : 0u;
  }
  if (tid == 0) {
    umma::mbar_init(&s.mbar[0], 1);                  // accumulator 0 / 1 complete (one commit)
    umma::mbar_init(&s.mbar[1], 1);
    umma::mbar_init(&s.mbar[2], kDWorkers);          // A buffer 0 / 1 written (every worker thread)
    umma::mbar_init(&s.mbar[3], kDWorkers);
    *s.dead = 0;
  }
  if (warp == 0) umma::tmem_alloc(s.tmem_slot, kDTmemCols);
  umma::fence_smem_to_async();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem_base = *s.tmem_slot;
  const int64_t n_tiles = (a.n_vec + kDTile - 1) / kDTile;
  const bool one_segment = a.rows.seg_len >= a.n_vec;           // rows are n + seg_off: no division
  auto row_of = [&](int64_t n) -> int64_t { return one_segment ? n + a.rows.seg_off : map_row(a.rows, n); };

  // ---- warp 0: per tile, wait until every worker has written A(i), then four products, smallest first --------
  if (warp == 0) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma::instr_desc(umma::kFmtF16, 128, 128);
      // terms of A and of B per product: m*m (left out with three products), m*h, h*m, h*h
      constexpr int pa[4] = {1, 1, 0, 0}, pb[4] = {1, 0, 1, 0};
      uint32_t full_phase[2] = {0u, 0u};
      int i = 0;
      for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++i) {
        const int bf = i & 1;
        if (*reinterpret_cast<volatile int*>(s.dead)) break;
        if (!umma::mbar_wait(&s.mbar[2 + bf], full_phase[bf])) {     // a worker gave up (or never came)
          *reinterpret_cast<volatile int*>(s.dead) = 1;
          atomicAdd(&g_dec_umma_timeouts, 1u);
          break;
        }
        full_phase[bf] ^= 1u;
        if (*reinterpret_cast<volatile int*>(s.dead)) break;
        if (a.test_drop_mma && blockIdx.x == 0 && i == 1) continue;   // test hook: this tile is never multiplied
        umma::fence_after_sync();
        const uint32_t d = tmem_base + bf * 128;
        bool acc = false;
#pragma unroll
        for (int pr = 4 - kDProducts; pr < 4; ++pr) {
          const uint32_t a_tmem = tmem_base + kDTmemA + (2 * bf + pa[pr]) * 64;
          const uint32_t b_addr = umma::smem_u32(s.b) + pb[pr] * kDPlaneBytes;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = (ks >> 2) * (128 * 128) + (ks & 3) * 32;
            umma::mma_f16_ts(d, a_tmem + 8 * ks, umma::smem_desc_sw128(b_addr + off), idesc, acc);
            acc = true;
          }
        }
        umma::commit(&s.mbar[bf]);
      }
    }
    __syncwarp();
  }

  if (worker) {
    // Packed words (and the norm) of this thread's part of a row, fetched one tile ahead of their use.
    uint32_t nw[2][BMAX + 1], nsw[2] = {0u, 0u};
    float nnorm = 0.f;
    auto fetch = [&](int64_t tile) {
      const int64_t n = tile * kDTile + trow;
      const bool live = tile < n_tiles && n < a.n_vec;
      const int64_t row = live ? row_of(n) : 0;
      if (MIXED) {
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int q = 0; q < BMAX; ++q)
            nw[u][q] = (live && q < bits_c[u]) ? __ldg(codes + row * row_words + word_off[u] + q) : 0u;
      } else {
        // the two blocks are 2 BITS consecutive words: the widest loads their alignment allows (a warp's rows are
        // 16 BITS bytes apart, so every load instruction touches the same lines whatever its width)
        const uint32_t* src = codes + row * row_words + word_off[0];
        uint32_t w[2 * BITS];
        if (BITS % 2 == 0) {
#pragma unroll
          for (int q = 0; q < BITS / 2; ++q) {
            const uint4 t = live ? __ldg(reinterpret_cast<const uint4*>(src) + q) : make_uint4(0u, 0u, 0u, 0u);
            w[4 * q] = t.x; w[4 * q + 1] = t.y; w[4 * q + 2] = t.z; w[4 * q + 3] = t.w;
          }
        } else {
#pragma unroll
          for (int q = 0; q < BITS; ++q) {
            const uint2 t = live ? __ldg(reinterpret_cast<const uint2*>(src) + q) : make_uint2(0u, 0u);
            w[2 * q] = t.x; w[2 * q + 1] = t.y;
          }
        }
#pragma unroll
        for (int q = 0; q < BITS; ++q) { nw[0][q] = w[q]; nw[1][q] = w[BITS + q]; }
      }
      nw[0][BMAX] = 0u;
      nw[1][BMAX] = 0u;
      if (SIGNS) {
        const uint2 t = live ? __ldg(reinterpret_cast<const uint2*>(signs + row * (kRD / 32) + blk0)) : make_uint2(0u, 0u);
        nsw[0] = t.x; nsw[1] = t.y;
      }
      nnorm = live ? __ldg(a.norms + row) : 0.f;
    };

    // this warp's lanes of the A operands in tensor memory (lane = row of the tile)
    const uint32_t a_tmem_row = tmem_base + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + kDTmemA;

    // Decode block u (32 coordinates of row trow) into the two operand planes of A[bf] through the pair table.
    auto decode_table = [&](auto bw_tag, auto rep_tag, int u, int bf) {
      constexpr int BW = decltype(bw_tag)::value, R = decltype(rep_tag)::value;
      constexpr int L = 3 + ilog2(R);                   // an entry index becomes a byte offset by << L
      constexpr uint32_t FM = ((1u << (2 * BW)) - 1u) << L, SM = 3u << (2 * BW + L);
      const uint32_t sx = nsw[u] ^ smask[u];            // bit c: add (1) or subtract (0) qjl_scale
      uint32_t hcol[16], mcol[16];                      // a pair is one 32-bit column of each term
#pragma unroll
      for (int p = 0; p < 16; ++p) {
        const int bit = 2 * BW * p, wi = bit >> 5, sh = bit & 31;
        uint32_t off;
        if (sh + 2 * BW > 32) off = __funnelshift_r(nw[u][wi], nw[u][wi + 1], sh - L);
        else off = sh >= L ? nw[u][wi] >> (sh - L) : nw[u][wi] << (L - sh);
        off &= FM;
        if (SIGNS) {
          const int ss = 2 * p - (2 * BW + L);          // the pair's two sign bits go right above the codes
          off |= (ss >= 0 ? sx >> ss : sx << -ss) & SM;
        }
        const uint2 e = *reinterpret_cast<const uint2*>(tabl[u] + off);
        hcol[p] = e.x;
        mcol[p] = e.y;
      }
      const uint32_t ta = a_tmem_row + 2 * bf * 64 + 16 * (blk0 + u);
      umma::tmem_st16(ta, hcol);
      umma::tmem_st16(ta + 64, mcol);
    };
    auto decode_block = [&](int u, int bf) {
      if (MIXED) {
        if (cls[u]) decode_table(std::integral_constant<int, (MIXED ? BITS1 : BITS)>{}, std::integral_constant<int, R1>{}, u, bf);
        else decode_table(std::integral_constant<int, BITS>{}, std::integral_constant<int, R0>{}, u, bf);
        return;
      }
      if (table_ok) {
        decode_table(std::integral_constant<int, BITS>{}, std::integral_constant<int, R0>{}, u, bf);
        return;
      }
      // S with other magnitudes than 1: every coordinate by arithmetic
      uint32_t hcol[16], mcol[16];
#pragma unroll
      for (int p = 0; p < 16; ++p) {
        float v[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = 2 * p + h;
          const int bit = BITS * c, wi = bit >> 5, sh = bit & 31;
          uint32_t code = nw[u][wi] >> sh;
          if (sh + BITS > 32) code |= nw[u][wi + 1] << (32 - sh);
          code &= (1u << BITS) - 1u;
          float x = cent_s[0][code];
          if (SIGNS) {
            const float q = qs_s[32 * (blk0 + u) + c];
            x += ((nsw[u] >> c) & 1u) ? q : -q;
          }
          v[h] = x * scale_a;
        }
        __half h0, m0, h1, m1;
        split2h(v[0], h0, m0);
        split2h(v[1], h1, m1);
        hcol[p] = pack_h(h0, h1);
        mcol[p] = pack_h(m0, m1);
      }
      const uint32_t ta = a_tmem_row + 2 * bf * 64 + 16 * (blk0 + u);
      umma::tmem_st16(ta, hcol);
      umma::tmem_st16(ta + 64, mcol);
    };

    // Scale this thread's 2 x 32 outputs of row trow by the norm and store them.  A thread holds consecutive outputs
    // of ONE row; stored as they are, a warp instruction would touch 32 rows.
    // fp32: the thread writes its 256 bytes to a staging row of its own (rows 272 bytes apart, so that the eight
    // lanes served together never meet in a bank) and hands the row to the bulk-copy engine (shared -> global, one
    // copy per thread and tile): no transposition, no store instruction per 16 bytes, and nobody else ever touches
    // the staging row; the thread only has to know that its previous copy has been READ before it writes the row
    // again.  bf16: a row is 128 bytes per thread, and at that size the number of copies binds; the warp
    // transposes through 32 lines of 128 bytes of its own (16-byte chunk c of row r at position c ^ (r & 7):
    // conflict-free both ways) and stores 4 rows x 128 contiguous bytes per instruction, whole lines.
    const int rbase = 32 * (warp & 3);
    unsigned char* const stage = s.scratch + ((warp - kDFirstWorker) * 32 + lane) * kDStageRow;
    unsigned char* const lines = s.scratch + (warp - kDFirstWorker) * (32 * 128);
    const int rr = lane >> 3, rc = lane & 7;           // read side of the transposition: row 4 j + rr, chunk rc
    auto line_off = [&](int row, int c) -> uint32_t { return static_cast<uint32_t>(row * 128 + ((c ^ (row & 7)) << 4)); };
    // The accumulator read is issued early (before the decode of the next tile) and waited for here.
    auto epilogue = [&](int64_t tile, int ab, float nrm, bool use_tmem, uint32_t (&v)[64]) {   // ab: accumulator of the tile
      const int64_t n = tile * kDTile + trow;
      const bool live = n < a.n_vec;
      if (!use_tmem) {                                     // tensor core timed out: fp32 chain from the packed row,
        if (live) {                                        // stored value by value (kept apart from the registers of
          const int64_t row = row_of(n);                   // the normal path, which must never be indexed by a variable)
          float vrow[kRD];
          for (int i = 0; i < kRD; ++i) {                  // i = stream position; channel = perm[i] when mixed
            const int ci = i >= n_out ? 1 : 0;
            const int bit = ci ? n_out * BITS + (i - n_out) * BITS1 : i * BITS;
            const uint32_t code = read_field(a.codes + row * (row_words * 4), bit, ci ? BITS1 : BITS, row_words * 4);
            float x = cent_s[ci][code];
            if (SIGNS) x += ((signs[row * (kRD / 32) + (i >> 5)] >> (i & 31)) & 1u) ? qs_s[i] : -qs_s[i];
            vrow[MIXED ? perm_s[i] : i] = x;
          }
#pragma unroll 1
          for (int c = 0; c < 64; ++c)
            store_float(a.out, a.out_dtype, n * a.out_pitch + 32 * blk0 + c, decompress_chain(vrow, a.Pi, 32 * blk0 + c) * nrm);
        }
        return;
      }
      umma::tmem_ld64_wait(v);
      float f = nrm * descale;
      if (!(fabsf(f) >= 1e-30f && fabsf(f) <= 1e30f)) {    // the product would lose bits: take the power of two first
#pragma unroll
        for (int c = 0; c < 64; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * descale);
        f = nrm;
      }
      if (a.out_dtype == QKV_F32) {
        bulk_wait_read();                                  // the copy of the previous tile has left the staging row
#pragma unroll
        for (int c = 0; c < 16; ++c)
          *reinterpret_cast<float4*>(stage + 16 * c) =
              make_float4(__uint_as_float(v[4 * c]) * f, __uint_as_float(v[4 * c + 1]) * f,
                          __uint_as_float(v[4 * c + 2]) * f, __uint_as_float(v[4 * c + 3]) * f);
        umma::fence_smem_to_async();                       // the row is visible to the copy engine
        if (live) bulk_store(reinterpret_cast<float*>(a.out) + n * a.out_pitch + 32 * blk0, stage, 256u);
        bulk_commit();
      } else if (a.out_dtype == QKV_BF16) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 2 * e]) * f,
                                                            __uint_as_float(v[8 * c + 2 * e + 1]) * f);
            pk[e] = *reinterpret_cast<const uint32_t*>(&b2);
          }
          *reinterpret_cast<uint4*>(lines + line_off(lane, c)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        __syncwarp();
        const int64_t n0 = tile * kDTile + rbase;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = 4 * j + rr;
          const uint4 o = *reinterpret_cast<const uint4*>(lines + line_off(r, rc));
          if (n0 + r < a.n_vec)
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.out) + (n0 + r) * a.out_pitch + 32 * blk0 + 8 * rc) = o;
        }
        __syncwarp();
      } else if (live) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          store_float(a.out, a.out_dtype, n * a.out_pitch + 32 * blk0 + c, __uint_as_float(v[c]) * f);
      }
    };
    // Wait for the products of the tile in accumulator `acc_buf`; false once the tensor core has been given up.
    uint32_t phase[2] = {0u, 0u};
    auto wait_products = [&](int acc_buf) -> bool {
      bool ok = *reinterpret_cast<volatile int*>(s.dead) == 0;
      if (ok) {
        ok = umma::mbar_wait(&s.mbar[acc_buf], phase[acc_buf]);
        phase[acc_buf] ^= 1u;
        if (!ok) { *reinterpret_cast<volatile int*>(s.dead) = 1; atomicAdd(&g_dec_umma_timeouts, 1u); }
      }
      umma::fence_after_sync();
      return ok;
    };

    // ---- workers: wait(i-1); decode(i); arrive; epilogue(i-1)   (decode overlaps the MMAs of tile i-1) ---------
    // A(i+1) goes into the buffer of tile i-1, whose products this thread has waited for; accumulator (i+1) & 1 is
    // overwritten only after every worker has arrived for tile i+1, that is after its epilogue of tile i-1.
    int64_t prev_tile = -1;
    int i = 0;
    float norm_cur = 0.f, norm_prev = 0.f;
    const uint32_t acc_row = tmem_base + (static_cast<uint32_t>(rbase) << 16) + 32 * blk0;
    // The accumulator read of tile i-1 is issued before the decode of tile i and waited for after it, which hides
    // its latency (fp32 output +7 %; bf16 output -3 %, the same whether or not that case keeps the read next to
    // its use, so there is one order for both).
    fetch(blockIdx.x);
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++i) {
      const int bf = i & 1;                   // A buffer and accumulator of tile i
      uint32_t v[64];
      bool ok = true;
      if (prev_tile >= 0) {                   // the products of tile i-1 were issued a whole decode + epilogue ago
        ok = wait_products(bf ^ 1);
        if (ok) umma::tmem_ld64_issue(acc_row + (bf ^ 1) * 128, v);
      }
      decode_block(0, bf);
      decode_block(1, bf);
      norm_prev = norm_cur;
      norm_cur = nnorm;
      fetch(tile + gridDim.x);                // the next tile's words travel while this one is multiplied and stored
      umma::tmem_st_wait();                   // this thread's part of A(i) is in tensor memory
      umma::fence_before_sync();
      mbar_arrive(&s.mbar[2 + bf]);
      if (prev_tile >= 0) epilogue(prev_tile, bf ^ 1, norm_prev, ok, v);
      prev_tile = tile;
    }
    if (prev_tile >= 0) {
      const int bf = (i - 1) & 1;
      uint32_t v[64];
      const bool ok = wait_products(bf);
      if (ok) umma::tmem_ld64_issue(acc_row + bf * 128, v);
      epilogue(prev_tile, bf, norm_cur, ok, v);
    }
    bulk_wait_all();
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem_base, kDTmemCols);
}

template <int BITS, bool SIGNS, int BITS1 = 0>
int launch_t(const DecompressArgs& a, cudaStream_t st) {
  constexpr size_t smem = dec_smem_bytes();
  if (cudaFuncSetAttribute(decompress_umma_kernel<BITS, SIGNS, BITS1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return QKV_ELAUNCH;
  const int64_t tiles = (a.n_vec + kDTile - 1) / kDTile;
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);
  decompress_umma_kernel<BITS, SIGNS, BITS1><<<grid, kDThreads, smem, st>>>(a);
  return check_launch();
}

}  // namespace

unsigned int decompress_umma_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_dec_umma_timeouts, sizeof(v));
  return v;
}

bool decompress_umma_ok(const DecompressArgs& a) {
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.codes) | reinterpret_cast<uintptr_t>(a.out) |
                       (a.signs ? reinterpret_cast<uintptr_t>(a.signs) : 0);
  if (a.mode == MODE_MIXED) {   // the common width pairs; rows are whole 4-byte words (36 B at 32 x 3 + 96 x 2 bits)
    const bool pair = (a.bits0 == 3 && a.bits1 == 2) || (a.bits0 == 4 && a.bits1 == 3) || (a.bits0 == 4 && a.bits1 == 2);
    return pair && a.d == kRD && a.packed && a.n_vec >= 1024 && (a.out_pitch & 7) == 0 &&
           ((reinterpret_cast<uintptr_t>(a.out) & 15u) | (reinterpret_cast<uintptr_t>(a.codes) & 3u)) == 0;
  }
  return a.d == kRD && a.packed && a.n_vec >= 1024 && (a.out_pitch & 7) == 0 && (al & 15u) == 0;
}

int launch_decompress_umma(const DecompressArgs& a_in, cudaStream_t st) {
  // QUASHKV_B200_TEST_DROP_MMA=1 (tests only): one tile's tensor-core work is never issued, which makes the
  // bounded wait on it run out and exercises the recovery path without anything faulting or hanging.
  DecompressArgs a = a_in;
  const char* hook = getenv("QUASHKV_B200_TEST_DROP_MMA");
  a.test_drop_mma = hook && hook[0] == '1';
  if (a.mode == MODE_MIXED) {
    if (a.bits0 == 3) return launch_t<3, false, 2>(a, st);
    return a.bits1 == 3 ? launch_t<4, false, 3>(a, st) : launch_t<4, false, 2>(a, st);
  }
  const bool sg = a.signs != nullptr;
  switch (a.bits0) {
    case 1: return sg ? launch_t<1, true>(a, st) : launch_t<1, false>(a, st);
    case 2: return sg ? launch_t<2, true>(a, st) : launch_t<2, false>(a, st);
    case 3: return sg ? launch_t<3, true>(a, st) : launch_t<3, false>(a, st);
    default: return sg ? launch_t<4, true>(a, st) : launch_t<4, false>(a, st);
  }
}

}  // namespace qkv
