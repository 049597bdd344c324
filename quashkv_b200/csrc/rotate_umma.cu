// Compress at d = 128 with the rotation on the fifth-generation tensor cores (tcgen05).
//
// One CTA per SM walks over tiles of 128 vectors.  The rotation y = x @ Pi^T of a tile is a
// 128 x 128 x 128 contraction issued by ONE thread as tcgen05.mma instructions (M = 128, N = 128,
// K = 16 each) whose operands are read from shared memory through matrix descriptors and whose fp32
// accumulator lives in tensor memory:
//   * B = Pi, split exactly into three bf16 planes (h + m + l), staged once per CTA in the 128-byte
//     swizzled K-major layout (96 KB);
//   * A = the raw vectors.  bf16 input is its own exact single term, so the tile is copied from
//     global memory straight into the operand layout by cp.async (no register staging, double
//     buffered); products A*l, A*m, A*h accumulate smallest first: 24 MMAs per tile;
//   * two accumulators (2 x 128 tensor-memory columns) alternate, so the MMAs of tile t run while
//     the threads classify tile t-1.
// Four threads then share one vector (512 threads per CTA): a thread reads 32 columns of its row of the
// accumulator with tcgen05.ld, scales by 1/norm (fp64 sum of squares, as in the CUDA-core kernel), classifies
// every coordinate through the bucket table, packs the 32 codes into whole words and stores its part of the
// packed row.  A coordinate whose bucket holds a decision boundary is classified exactly from a register copy
// (tensor memory is re-read only for threads with several such coordinates); coordinates within kRecheckEps of a
// boundary go to a per-warp queue and are recomputed with the sequential fp32 FMA chain, exactly as in the
// mma.sync kernel, so the bytes are identical to the CUDA-core kernel's.  The queues are emptied by all warps
// together (a flag out of the tile barrier), and the products of a tile are issued one at a time between the
// phases of the loop, because the issuing thread is held for about as long as its MMAs execute.
//
// Every wait on the tensor core is bounded; if one runs out the CTA stops using the tensor core,
// counts the event and derives its remaining tiles with the fp32 chain alone (slow, still exact).
#include <type_traits>

#include "rotate_exact.cuh"
#include "mma_decode.cuh"
#include "umma.cuh"

namespace qkv {

__device__ unsigned int g_umma_timeouts = 0;

constexpr int kUTile = 128;                       // vectors per tile = MMA M
constexpr int kUThreads = 512;                    // four threads per vector: 32 output coordinates each
constexpr int kUWarps = kUThreads / 32;
constexpr uint32_t kUPlaneBytes = 128 * 128 * 2;  // one bf16 operand tile (two 64-wide K blocks)
constexpr uint32_t kUTmemCols = 256;

// Bucket table of this kernel: LUTN buckets of width 2 / LUTN over [-1, 1) (32768 where shared memory allows:
// bf16 input, uniform width; else 16384).  The low nibble of an entry is
// the code of the bucket; bit 7 flags a bucket whose coordinates need a second look, of kind
// 0x40 = decision boundary number (entry & 15) lies in or within the recheck margin of the bucket
//        (code = that number, +1 if y is above it),
// 0x20 = a centroid does (the sign bit needs the residual test),
// 0x60 = anything else (edge buckets, two features in one bucket): generic path.
template <int LUTN>
__device__ __forceinline__ int bucket_fine(float v, float scale) {          // scale = (LUTN / 2) / norm
  return __float_as_int(fmaf(v, scale, static_cast<float>(LUTN / 2) + 8388608.f)) & (LUTN - 1);
}

template <int BITS, bool IP, int LUTN>
__device__ __forceinline__ void build_fine_lut(uint8_t* lut, const float* bnd, const float* cent) {
  constexpr int NB = (1 << BITS) - 1;
  constexpr float kHalf = static_cast<float>(LUTN / 2), kInv = 1.f / kHalf;
  for (int k = threadIdx.x; k < LUTN; k += blockDim.x) {
    const float lo = (static_cast<float>(k) - kHalf - 0.5f) * kInv;
    const float hi = (static_cast<float>(k) - kHalf + 0.5f) * kInv;
    const float margin = kRecheckEps + 2e-6f;
    int n_b = 0, which = 0, n_c = 0;
    for (int b = 0; b < NB; ++b)
      if (bnd[b] >= lo - margin && bnd[b] <= hi + margin) { ++n_b; which = b; }
    if (IP)
      for (int c = 0; c <= NB; ++c) n_c += (cent[c] >= lo - margin && cent[c] <= hi + margin) ? 1 : 0;
    const float mid = (static_cast<float>(k) - kHalf) * kInv;
    uint32_t v = count_bounds<BITS>(bnd, mid);
    if (k == 0 || k == LUTN - 1 || n_b > 1 || n_c > 1 || (n_b && n_c)) v |= 0xE0u;
    else if (n_b) v = static_cast<uint32_t>(which) | 0xC0u;
    else if (n_c) v |= 0xA0u;
    lut[k] = static_cast<uint8_t>(v);
  }
}

// NT = bf16 terms of the A operand: 1 for bf16 input (two tile buffers), 3 for fp32 / fp16 input (one
// buffer of three planes; together with Pi's three planes that is 192 KB).
template <int NT> __host__ __device__ constexpr int queue_cap() { return NT == 1 ? 64 : 32; }

struct UmmaSmem {
  unsigned char* a[2][3];   // A tiles [buffer][term] (bf16, swizzled), 1024-byte aligned
  unsigned char* b[3];      // Pi planes h, m, l
  uint4* queue;             // [warps][kUQueueCap]
  double* ssq;              // [2 tiles][4 quarters][128 rows] partial sums of squares
  uint32_t* smask;          // [4] bit c of word w: S[32 w + c] < 0
  int* qcount;              // [warps]
  uint64_t* mbar;           // [2]
  uint32_t* tmem_slot;
  int* dead;
};

// dynamic part; the bucket table and the small tables are static shared arrays (constant addresses)
template <int NT>
constexpr size_t umma_smem_bytes() {
  return 1024 + (NT == 1 ? 5 : 6) * kUPlaneBytes + kUWarps * queue_cap<NT>() * 16 + 2 * 4 * 128 * 8 + 16 +
         kUWarps * 4 + 2 * 8 + 16;
}

template <int NT>
__device__ __forceinline__ UmmaSmem carve_umma(unsigned char* raw) {
  UmmaSmem s;
  unsigned char* p = raw + ((1024u - (umma::smem_u32(raw) & 1023u)) & 1023u);
  for (int bf = 0; bf < 2; ++bf)
    for (int t = 0; t < 3; ++t) s.a[bf][t] = nullptr;
  if (NT == 1) {
    s.a[0][0] = p; s.a[1][0] = p + kUPlaneBytes; p += 2 * kUPlaneBytes;
  } else {
    for (int t = 0; t < 3; ++t) { s.a[0][t] = p; p += kUPlaneBytes; }
  }
  for (int t = 0; t < 3; ++t) { s.b[t] = p; p += kUPlaneBytes; }
  s.queue = reinterpret_cast<uint4*>(p); p += kUWarps * queue_cap<NT>() * 16;
  s.ssq = reinterpret_cast<double*>(p); p += 2 * 4 * 128 * 8;
  s.smask = reinterpret_cast<uint32_t*>(p); p += 16;
  s.mbar = reinterpret_cast<uint64_t*>(p); p += 16;
  s.qcount = reinterpret_cast<int*>(p); p += kUWarps * 4;
  s.tmem_slot = reinterpret_cast<uint32_t*>(p);
  s.dead = reinterpret_cast<int*>(p + 4);
  return s;
}

// BITS1 != 0: mixed precision.  Channels flagged in is_outlier use table 0 at BITS, the others table 1 at
// BITS1, and the packed row is the outlier channels' stream followed by the regular channels' stream.
// The rows of Pi are staged in THAT order (B row n' = Pi[perm[n']]), so accumulator column n' is
// stream position n' and every 32-column block belongs to one table; this needs the number of
// outlier channels to be a multiple of 32 (otherwise the CTA returns at once and the CUDA-core
// kernel, launched behind it with the same test inverted, does the work).
template <int BITS, bool IP, int NT, int BITS1 = 0>
__global__ void __launch_bounds__(kUThreads, 1) compress_umma_kernel(CompressArgs a) {
  constexpr bool MIXED = BITS1 != 0;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LUTN = (NT == 1 && !MIXED) ? 2 * kLutSize : kLutSize;
  __shared__ int8_t lut_s[MIXED ? 2 : 1][LUTN];
  __shared__ float bnd_s[2][16], cent_s[16], sgn_s[kRD];
  __shared__ uint8_t perm_s[kRD];
  const UmmaSmem s = carve_umma<NT>(smem_raw);
  constexpr int kUQueueCap = queue_cap<NT>();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int trow = 32 * (warp & 3) + lane;          // vector of the tile = tensor-memory lane
  const int blk = warp >> 2;                        // output coordinates 32 blk .. 32 blk + 31
  constexpr int NB = (1 << BITS) - 1;
  const __nv_bfloat16* xg = reinterpret_cast<const __nv_bfloat16*>(a.x);

  // ---- mixed precision: stream order of the channels -------------------------------------------------------
  int n_out = MIXED ? 0 : kRD;                      // columns below n_out use table 0
  if (MIXED) {
    bool o = false;
    if (tid < kRD) {
      o = a.is_outlier[tid] != 0;
      const uint32_t m = __ballot_sync(QKV_FULL_MASK, o);
      if (lane == 0) s.smask[warp] = m;
    }
    __syncthreads();
    int before = 0;
    for (int w = 0; w < 4; ++w) {
      const int c = __popc(s.smask[w]);
      n_out += c;
      if (w < warp) before += c;
    }
    if (n_out & 31) return;                         // every thread of every CTA: left to the CUDA-core kernel
    if (tid < kRD) {
      before += __popc(s.smask[warp] & ((1u << lane) - 1u));            // outlier channels below this one
      perm_s[o ? before : n_out + (tid - before)] = static_cast<uint8_t>(tid);
    }
    __syncthreads();
  }
  const int m_out = n_out >> 5;                     // 32-column blocks of table 0
  const int row_words = MIXED ? m_out * BITS + (4 - m_out) * BITS1 : 4 * BITS;

  // ---- one-time setup: Pi planes, tables, barriers, tensor memory -------------------------------------
  for (int idx = tid; idx < kRD * kRD; idx += kUThreads) {
    const int n = idx >> 7, k = idx & 127;
    __nv_bfloat16 h, m, l;
    split3(a.Pi[(MIXED ? perm_s[n] : n) * kRD + k], h, m, l);
    const uint32_t off = umma::sw128_offset(n, k, 128);
    *reinterpret_cast<__nv_bfloat16*>(s.b[0] + off) = h;
    *reinterpret_cast<__nv_bfloat16*>(s.b[1] + off) = m;
    *reinterpret_cast<__nv_bfloat16*>(s.b[2] + off) = l;
  }
  if (tid < 16) {
    bnd_s[0][tid] = tid < NB ? a.bounds0[tid] : INFINITY;
    bnd_s[1][tid] = (MIXED && tid < (1 << BITS1) - 1) ? a.bounds1[tid] : INFINITY;
    cent_s[tid] = (IP && tid < (1 << BITS)) ? a.centroids[tid] : 0.f;
  }
  if (tid < kRD) {
    const float sv = IP ? a.S[tid] : 0.f;
    sgn_s[tid] = sv;
    const uint32_t m = __ballot_sync(QKV_FULL_MASK, sv < 0.f);
    if (lane == 0) s.smask[warp] = m;
  }
  if (tid < kUWarps) s.qcount[tid] = 0;
  if (tid == 0) {
    umma::mbar_init(&s.mbar[0], 1);
    umma::mbar_init(&s.mbar[1], 1);
    *s.dead = 0;
  }
  __syncthreads();
  build_fine_lut<BITS, IP, LUTN>(reinterpret_cast<uint8_t*>(lut_s[0]), bnd_s[0], cent_s);
  if (MIXED)
    build_fine_lut<(MIXED ? BITS1 : 1), false, LUTN>(reinterpret_cast<uint8_t*>(lut_s[MIXED ? 1 : 0]), bnd_s[1], cent_s);
  if (warp == 0) umma::tmem_alloc(s.tmem_slot, kUTmemCols);
  umma::fence_smem_to_async();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem_base = *s.tmem_slot;
  const uint32_t smask = s.smask[blk];

  uint4* queue = s.queue + warp * kUQueueCap;
  uint32_t* out_codes = reinterpret_cast<uint32_t*>(a.codes);
  uint32_t* out_signs = reinterpret_cast<uint32_t*>(a.signs);

  // Recompute queued elements with the fp32 FMA chain, one per lane; patch changed codes / signs.
  auto drain = [&](int count) {
    __threadfence();
    __syncwarp();
    for (int base = 0; base < count; base += 32) {
      const int i = base + lane;
      if (i < count) {
        const uint4 it = queue[i];
        const int64_t n = it.x;
        const int col = it.y & 0xFF;
        const uint32_t old_code = (it.y >> 8) & 0xFF, old_sign = (it.y >> 16) & 1u;
        const int cls = col >= n_out ? 1 : 0;
        const int bits_c = cls ? BITS1 : BITS;
        const float z = exact_chain_s(a.x, a.x_dtype, a.x_pitch, a.Pi, n, MIXED ? perm_s[col] : col,
                                      __uint_as_float(it.z));
        uint32_t code = 0;
        for (int b = 0; b < (1 << bits_c) - 1; ++b) code += z > bnd_s[cls][b] ? 1u : 0u;
        const int64_t row = map_row(a.rows, n);
        const uint32_t diff = code ^ old_code;
        if (diff) {
          const int bit = cls ? n_out * BITS + (col - n_out) * BITS1 : col * BITS, w = bit >> 5, sh = bit & 31;
          atomicXor(out_codes + row * row_words + w, diff << sh);
          if (sh + bits_c > 32) atomicXor(out_codes + row * row_words + w + 1, diff >> (32 - sh));
        }
        if (IP) {
          const uint32_t sign = ((z - cent_s[code]) * sgn_s[col] >= 0.f) ? 1u : 0u;
          if (sign != old_sign) atomicXor(out_signs + row * (kRD / 32) + (col >> 5), 1u << (col & 31));
        }
      }
    }
    __syncwarp();
  };
  const int cls_blk = blk >= m_out ? 1 : 0;         // table of this thread's 32 columns
  const int word_off = cls_blk ? m_out * BITS + (blk - m_out) * BITS1 : blk * BITS;

  const int64_t n_tiles = (a.n_vec + kUTile - 1) / kUTile;

  // cp.async of one tile into A[buf]: 2048 chunks of 16 bytes, 8 per thread, coalesced along rows.
  auto load_tile = [&](int64_t tile, int buf) {
    const int64_t v0 = tile * kUTile;
#pragma unroll
    for (int j = 0; j < 2048 / kUThreads; ++j) {
      const int p = tid + kUThreads * j;
      const int r = p >> 4, c16 = p & 15;
      const int64_t n = v0 + r;
      const bool live = n < a.n_vec;
      const __nv_bfloat16* src = xg + (live ? n : 0) * a.x_pitch + c16 * 8;
      cp_async16(s.a[buf][0] + umma::sw128_offset(r, c16 * 8, 128), src, live ? 16 : 0);
    }
    cp_async_commit();
  };

  // fp64 sum of squares of this thread's 32 coordinates of row trow of A[buf], left in shared memory.
  auto part_squares = [&](int buf) {
    double ss = 0.0;
#pragma unroll
    for (int c8 = 0; c8 < 4; ++c8) {
      const uint4 v = *reinterpret_cast<const uint4*>(s.a[buf][0] + umma::sw128_offset(trow, 32 * blk + c8 * 8, 128));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const double lo = static_cast<double>(__uint_as_float(w[i] << 16));
        const double hi = static_cast<double>(__uint_as_float(w[i] & 0xFFFF0000u));
        ss += lo * lo + hi * hi;
      }
    }
    s.ssq[(buf * 4 + blk) * 128 + trow] = ss;
  };
  // fp32 / fp16 input: this thread's 32 coordinates of row trow, split exactly into three bf16 terms and
  // written to the three A planes; their squares go to the partial sums of tile parity `par`.
  auto load_split_tile = [&](int64_t tile, int par) {
    const int64_t n = tile * kUTile + trow;
    const bool live = n < a.n_vec;
    double ss = 0.0;
#pragma unroll
    for (int c8 = 0; c8 < 4; ++c8) {
      float v[8];
      if (a.x_dtype == QKV_F32) {
        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.x) +
                                                            (live ? n : 0) * a.x_pitch + 32 * blk + 8 * c8);
        const float4 u0 = live ? __ldg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 u1 = live ? __ldg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
        v[0] = u0.x; v[1] = u0.y; v[2] = u0.z; v[3] = u0.w; v[4] = u1.x; v[5] = u1.y; v[6] = u1.z; v[7] = u1.w;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          v[e] = live ? load_float(a.x, a.x_dtype, n * a.x_pitch + 32 * blk + 8 * c8 + e) : 0.f;
      }
      uint32_t pk[3][4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        __nv_bfloat16 h0, m0, l0, h1, m1, l1;
        split3(v[2 * p], h0, m0, l0);
        split3(v[2 * p + 1], h1, m1, l1);
        pk[0][p] = pack_bf16(h0, h1); pk[1][p] = pack_bf16(m0, m1); pk[2][p] = pack_bf16(l0, l1);
        ss += static_cast<double>(v[2 * p]) * static_cast<double>(v[2 * p]) +
              static_cast<double>(v[2 * p + 1]) * static_cast<double>(v[2 * p + 1]);
      }
      const uint32_t off = umma::sw128_offset(trow, 32 * blk + 8 * c8, 128);
#pragma unroll
      for (int t = 0; t < 3; ++t)
        *reinterpret_cast<uint4*>(s.a[0][t] + off) = make_uint4(pk[t][0], pk[t][1], pk[t][2], pk[t][3]);
    }
    s.ssq[(par * 4 + blk) * 128 + trow] = ss;
  };
  auto row_norm = [&](int buf) {
    const double* q = s.ssq + buf * 4 * 128 + trow;
    return fmaxf(static_cast<float>(sqrt((q[0] + q[128]) + (q[256] + q[384]))), 1e-8f);
  };

  // Thread 0: the MMAs of one tile, smallest products first (bf16 input: A*l, A*m, A*h; split input:
  // m*m, l*h, h*l, m*h, h*m, h*h), then the completion arrival on the accumulator's barrier.  The queue in
  // front of the tensor core is short: the thread that issues a whole tile's MMAs in one go is held for about
  // as long as they execute, and its warp then reaches the next barrier that much later than the others.  So
  // the products are issued one at a time (`slice` = 0 .. n_prod - 1, the last one commits) at points of the
  // loop that lie far enough apart for the queue to drain in between.
  constexpr int n_prod = NT == 1 ? 3 : 6;
  auto issue_mmas = [&](int abuf, int acc_buf, int slice) {
    constexpr uint32_t idesc = umma::instr_desc(umma::kFmtBF16, 128, 128);
    const uint32_t d = tmem_base + acc_buf * 128;
    constexpr int pa1[3] = {0, 0, 0}, pb1[3] = {2, 1, 0};
    constexpr int pa3[6] = {1, 2, 0, 1, 0, 0}, pb3[6] = {1, 0, 2, 0, 1, 0};
#pragma unroll
    for (int pr = 0; pr < n_prod; ++pr) {
      if (pr != slice) continue;
      bool acc = pr != 0;
      const int ta = NT == 1 ? pa1[pr] : pa3[pr], tb = NT == 1 ? pb1[pr] : pb3[pr];
      const uint32_t a_addr = umma::smem_u32(s.a[abuf][ta]), b_addr = umma::smem_u32(s.b[tb]);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = (ks >> 2) * (128 * 128) + (ks & 3) * 32;
        umma::mma_f16(d, umma::smem_desc_sw128(a_addr + off), umma::smem_desc_sw128(b_addr + off), idesc, acc);
        acc = true;
      }
    }
    if (slice == n_prod - 1) umma::commit(&s.mbar[acc_buf]);
  };

  // Classify / pack / store this thread's 32 coordinates of row trow of a finished tile.  use_tmem ==
  // false: every coordinate by the fp32 chain.  The common path is branch-free: 32 independent table
  // look-ups whose flag bits are collected in a mask, packing by shifted adds.  Then the warp walks
  // over the columns in which any of its lanes was flagged (usually one or two): the column is
  // re-read from tensor memory and the flagged lanes classify it exactly and patch their words.
  auto epilogue_t = [&](auto bits_tag, int64_t tile, int buf, float nrm, bool use_tmem) {
    constexpr int BW = decltype(bits_tag)::value;   // bit width of this thread's columns
    constexpr int NBW = (1 << BW) - 1;
    const int8_t* lut_c = lut_s[MIXED ? cls_blk : 0];
    const float* bnd_c = bnd_s[cls_blk];
    const int64_t n = tile * kUTile + trow;
    const bool live = n < a.n_vec;
    const int64_t row = live ? map_row(a.rows, n) : 0;
    const float iv = 1.f / nrm, scale = iv * static_cast<float>(LUTN / 2);
    const int col0 = 32 * blk;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + buf * 128 + col0;
    uint32_t fmask = 0, fval = 0, R = 0;
    uint32_t wb[BW + 1];
#pragma unroll
    for (int w = 0; w <= BW; ++w) wb[w] = 0u;
    if (use_tmem) {
      uint32_t v[32];
      umma::tmem_ld32(taddr, v);
      uint32_t fm = 0;                           // flag of coordinate c ends up at bit 31 - c
      float fl_raw = 0.f;                        // the last flagged coordinate of this thread, kept in registers:
      int fl_c = 0;                              // nearly always its only one
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float raw = __uint_as_float(v[c]);
        const int e = lut_c[bucket_fine<LUTN>(raw, scale)];             // sign-extended: negative when flagged
        fm = __funnelshift_l(static_cast<uint32_t>(e), fm, 1);
        if (e < 0) { fl_raw = raw; fl_c = c; }
        const uint32_t code = static_cast<uint32_t>(e) & 15u;
        const int bit = BW * c, w = bit >> 5, sh = bit & 31;
        wb[w] += code << sh;                                       // fields are disjoint: add == or
        if (sh + BW > 32) wb[w + 1] += code >> (32 - sh);
        if (IP) R = __funnelshift_l(__float_as_uint(raw * iv - cent_s[code]), R, 1);
      }
      // A flagged coordinate gets the exact classification from its accumulator value: boundary test, sign of the
      // residual, and a place in the queue when it lies within the recheck margin.
      auto resolve = [&](int c, float raw) {
        const int col = col0 + c;
        const float y = raw * iv;
        const uint32_t ec = static_cast<uint8_t>(lut_c[bucket_fine<LUTN>(raw, scale)]);
        uint32_t code = ec & 15u, sign = 0;
        bool near = false;
        if ((ec & 0x60u) == 0x60u) {                 // edge bucket or two features: generic classification
          const uint32_t r = classify_slow(bnd_c, cent_s, IP ? sgn_s[col] : 0.f, y, NBW, IP ? 1 : 0);
          code = r & 0xFFu; sign = (r >> 8) & 1u; near = (r >> 16) != 0;
        } else {
          if (ec & 0x40u) {                          // one boundary in reach: code = its number, +1 above it
            const float b = bnd_c[code];
            near = fabsf(y - b) < kRecheckEps;
            code += y > b ? 1u : 0u;
          }
          if (IP) {
            const float resid = y - cent_s[code];
            sign = (resid * sgn_s[col] >= 0.f) ? 1u : 0u;
            near |= fabsf(resid) < kRecheckEps;
          }
        }
        if (near && live) {
          const int slot = atomicAdd(&s.qcount[warp], 1);
          if (slot < kUQueueCap) {
            queue[slot] = make_uint4(static_cast<uint32_t>(n), col | (code << 8) | (sign << 16),
                                     __float_as_uint(nrm), 0u);
          } else {
            const float z = exact_chain_s(a.x, a.x_dtype, a.x_pitch, a.Pi, n, MIXED ? perm_s[col] : col, nrm);
            code = count_bounds<BW>(bnd_c, z);
            if (IP) sign = ((z - cent_s[code]) * sgn_s[col] >= 0.f) ? 1u : 0u;
          }
        }
        fmask |= 1u << c;
        fval |= sign << c;
        const uint32_t diff = code ^ (ec & 15u);
        const int bit = BW * c, w = bit >> 5, sh = bit & 31;
#pragma unroll
        for (int q = 0; q <= BW; ++q) {
          if (q == w) wb[q] ^= diff << sh;
          if (q == w + 1 && sh + BW > 32) wb[q] ^= diff >> (32 - sh);
        }
      };
      uint32_t mine = __brev(fm);
      if (__popc(mine) == 1) {                     // the usual case: resolved from the registers, no second read
        resolve(fl_c, fl_raw);
        mine = 0u;
      }
      __syncwarp();
      // Threads with several flagged coordinates (rare): the warp walks over the columns concerned, re-reads each
      // from tensor memory (up to four per round, so that the reads overlap) and the flagged lanes resolve it.
      uint32_t cols = __reduce_or_sync(QKV_FULL_MASK, mine);
      while (cols) {
        int cc[4]; uint32_t ta[4], rv[4];
        int n_c = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          cc[j] = cols ? __ffs(cols) - 1 : 0;
          if (cols) { ++n_c; cols &= cols - 1; }
          ta[j] = taddr + cc[j];
        }
        umma::tmem_ld1x4(ta, rv);
#pragma unroll 1
        for (int j = 0; j < n_c; ++j) {
          const int c = j == 0 ? cc[0] : (j == 1 ? cc[1] : (j == 2 ? cc[2] : cc[3]));
          const float raw = __uint_as_float(j == 0 ? rv[0] : (j == 1 ? rv[1] : (j == 2 ? rv[2] : rv[3])));
          if ((mine >> c) & 1u) resolve(c, raw);
          __syncwarp();
        }
      }
    } else {
#pragma unroll 1
      for (int c = 0; c < 32; ++c) {
        const int col = col0 + c;
        const float z = live ? exact_chain_s(a.x, a.x_dtype, a.x_pitch, a.Pi, n, MIXED ? perm_s[col] : col, nrm) : 0.f;
        const uint32_t code = count_bounds<BW>(bnd_c, z);
        if (IP) fval |= (((z - cent_s[code]) * sgn_s[col] >= 0.f) ? 1u : 0u) << c;
        const int bit = BW * c, w = bit >> 5, sh = bit & 31;
#pragma unroll
        for (int q = 0; q <= BW; ++q) {
          if (q == w) wb[q] |= code << sh;
          if (q == w + 1 && sh + BW > 32) wb[q] |= code >> (32 - sh);
        }
      }
      fmask = 0xFFFFFFFFu;
    }
    if (live) {
      uint32_t* dst = out_codes + row * row_words + word_off;
      if (!MIXED && BW == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(wb[0], wb[1], wb[2], wb[BW - 1]);
      else if (!MIXED && BW == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(wb[0], wb[1]);
      else {
#pragma unroll
        for (int w = 0; w < BW; ++w) dst[w] = wb[w];
      }
      if (IP) {
        // unflagged coordinates: sign = residual >= 0 exclusive-or S < 0 (a zero residual is always flagged)
        const uint32_t sw = ~(__brev(R) ^ smask);
        out_signs[row * (kRD / 32) + blk] = (sw & ~fmask) | fval;
      }
      if (blk == 0) a.norms[row] = nrm;
    }
    __syncwarp();
  };
  // The queues are emptied by all warps together: a warp that re-derives its queued coordinates takes a few
  // thousand cycles, which the others would spend waiting at the next barrier anyway, so one such pause serves
  // sixteen queues.  `any` comes out of the barrier at the top of the loop (some queue is at least half full);
  // a queue that overflows before that is handled element by element where it happens.
  auto drain_all = [&](int any) {
    if (!any) return;
    const int queued = s.qcount[warp];
    if (queued > 0) drain(queued < kUQueueCap ? queued : kUQueueCap);
    __syncwarp();
    if (lane == 0) s.qcount[warp] = 0;
    __syncwarp();
  };
  auto epilogue = [&](int64_t tile, int buf, float nrm, bool use_tmem) {
    if (MIXED && cls_blk) epilogue_t(std::integral_constant<int, (MIXED ? BITS1 : BITS)>{}, tile, buf, nrm, use_tmem);
    else epilogue_t(std::integral_constant<int, BITS>{}, tile, buf, nrm, use_tmem);
  };

  // ---- pipeline over this CTA's tiles ------------------------------------------------------------------
  uint32_t phase[2] = {0u, 0u};
  int64_t prev_tile = -1;
  int i = 0;
  auto wait_acc = [&](int acc_buf) {      // bounded wait for the MMAs that write accumulator acc_buf
    bool ok = *s.dead == 0;
    if (ok) {
      ok = umma::mbar_wait(&s.mbar[acc_buf], phase[acc_buf]);
      phase[acc_buf] ^= 1u;
      if (!ok) { *s.dead = 1; atomicAdd(&g_umma_timeouts, 1u); }
    }
    umma::fence_after_sync();
    return ok;
  };
  if (NT == 1) {
    // iteration i: wait A(i); issue MMAs(i); squares(i); [wait MMAs(i-1); prefetch A(i+1); epilogue(i-1)]
    if (blockIdx.x < n_tiles) load_tile(blockIdx.x, 0);
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++i) {
      const int buf = i & 1;
      cp_async_wait<0>();
      umma::fence_smem_to_async();
      umma::fence_before_sync();
      // A(i) complete and visible; epilogue(i-2) has left accumulator `buf`
      const int any = __syncthreads_or(s.qcount[warp] >= kUQueueCap / 2);
      const bool issuer = tid == 0 && *s.dead == 0 && !(a.test_drop_mma && blockIdx.x == 0 && i == 1);
      if (issuer) {
        umma::fence_after_sync();
        issue_mmas(buf, buf, 0);
      }
      // The MMAs of tile i-1 were issued a whole iteration ago: their barrier is normally complete, so the
      // copy of tile i+1 into the buffer they read starts right away and travels during everything below.
      const int64_t next = tile + gridDim.x;
      bool ok = true;
      if (prev_tile >= 0) ok = wait_acc(buf ^ 1);
      if (next < n_tiles) load_tile(next, buf ^ 1);
      const float norm_prev = prev_tile >= 0 ? row_norm(buf ^ 1) : 1.f;   // squares(i-1) were left before the barrier
      if (issuer) issue_mmas(buf, buf, 1);
      drain_all(any);
      // the fp64 sums of half the warps go before the epilogue and of the other half after it, so that the
      // sixteen warps do not queue for the fp64 pipe at the same moment
      if (blk < 2) part_squares(buf);
      if (issuer) issue_mmas(buf, buf, 2);
      if (prev_tile >= 0) epilogue(prev_tile, buf ^ 1, norm_prev, ok);
      if (blk >= 2) part_squares(buf);
      prev_tile = tile;
    }
  } else {
    // iteration i: wait MMAs(i-1) (they read the only A buffer); load + split A(i); issue MMAs(i); epilogue(i-1)
    bool prev_ok = true;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++i) {
      const int par = i & 1;
      if (prev_tile >= 0) prev_ok = wait_acc(par ^ 1);
      load_split_tile(tile, par);
      umma::fence_smem_to_async();
      umma::fence_before_sync();
      // A(i) and its squares complete; epilogue(i-2) has left accumulator `par`
      const int any = __syncthreads_or(s.qcount[warp] >= kUQueueCap / 2);
      if (tid == 0 && *s.dead == 0 && !(a.test_drop_mma && blockIdx.x == 0 && i == 1)) {
        umma::fence_after_sync();
#pragma unroll
        for (int sl = 0; sl < n_prod; ++sl) issue_mmas(0, par, sl);
      }
      // the norm is read before anything slow: a warp that runs ahead overwrites these partial sums with those
      // of tile i+1 as soon as it has passed its own epilogue
      const float norm_prev = prev_tile >= 0 ? row_norm(par ^ 1) : 1.f;
      drain_all(any);
      if (prev_tile >= 0) epilogue(prev_tile, par ^ 1, norm_prev, prev_ok);
      prev_tile = tile;
    }
  }
  if (prev_tile >= 0) {
    const int buf = (i - 1) & 1;
    __syncthreads();                      // squares of the last tile
    const float norm_last = row_norm(buf);
    const bool ok = wait_acc(buf);
    epilogue(prev_tile, buf, norm_last, ok);
  }
  __syncwarp();
  const int queued = s.qcount[warp];
  if (queued > 0) drain(queued < kUQueueCap ? queued : kUQueueCap);
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem_base, kUTmemCols);
}

bool compress_umma_ok(const CompressArgs& a) {
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.codes) |
                       (a.mode == MODE_IP ? reinterpret_cast<uintptr_t>(a.signs) : 0);
  if (a.mode == MODE_MIXED) {   // bf16 input, the common width pairs; row of 4-byte words (36 B at 32x3 + 96x2)
    const bool pair = (a.bits0 == 3 && a.bits1 == 2) || (a.bits0 == 4 && a.bits1 == 3) || (a.bits0 == 4 && a.bits1 == 2);
    if (!pair || a.x_dtype != QKV_BF16) return false;
    return a.d == kRD && a.packed && a.n_vec >= 1024 && a.n_vec < (int64_t(1) << 31) && (a.x_pitch & 7) == 0 &&
           ((reinterpret_cast<uintptr_t>(a.x) & 15u) | (reinterpret_cast<uintptr_t>(a.codes) & 3u)) == 0;
  }
  return a.d == kRD && a.packed && a.n_vec >= 1024 && a.n_vec < (int64_t(1) << 31) &&
         (a.x_pitch & 7) == 0 && (al & 15u) == 0;
}

template <int BITS, bool IP, int NT>
static int launch_compress_umma_n(const CompressArgs& a, cudaStream_t st) {
  constexpr size_t smem = umma_smem_bytes<NT>();
  if (cudaFuncSetAttribute(compress_umma_kernel<BITS, IP, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return QKV_ELAUNCH;
  const int64_t tiles = (a.n_vec + kUTile - 1) / kUTile;
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);
  compress_umma_kernel<BITS, IP, NT><<<grid, kUThreads, smem, st>>>(a);
  return check_launch();
}

template <int BITS, bool IP>
static int launch_compress_umma_t(const CompressArgs& a, cudaStream_t st) {
  return a.x_dtype == QKV_BF16 ? launch_compress_umma_n<BITS, IP, 1>(a, st) : launch_compress_umma_n<BITS, IP, 3>(a, st);
}

template <int B0, int B1>
static int launch_compress_umma_mixed(const CompressArgs& a, cudaStream_t st) {
  constexpr size_t smem = umma_smem_bytes<1>();
  if (cudaFuncSetAttribute(compress_umma_kernel<B0, false, 1, B1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return QKV_ELAUNCH;
  const int64_t tiles = (a.n_vec + kUTile - 1) / kUTile;
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);
  compress_umma_kernel<B0, false, 1, B1><<<grid, kUThreads, smem, st>>>(a);
  return check_launch();
}

int launch_compress_umma(const CompressArgs& a_in, cudaStream_t st) {
  // QUASHKV_B200_TEST_DROP_MMA=1 (tests only): one tile's tensor-core work is never issued, which makes the
  // bounded wait on it run out and exercises the recovery path without anything faulting or hanging.
  CompressArgs a = a_in;
  const char* hook = getenv("QUASHKV_B200_TEST_DROP_MMA");
  a.test_drop_mma = hook && hook[0] == '1';
  if (a.mode == MODE_MIXED) {
    if (a.bits0 == 3) return launch_compress_umma_mixed<3, 2>(a, st);
    return a.bits1 == 3 ? launch_compress_umma_mixed<4, 3>(a, st) : launch_compress_umma_mixed<4, 2>(a, st);
  }
  const bool ip = a.mode == MODE_IP;
  switch (a.bits0) {
    case 1: return ip ? launch_compress_umma_t<1, true>(a, st) : launch_compress_umma_t<1, false>(a, st);
    case 2: return ip ? launch_compress_umma_t<2, true>(a, st) : launch_compress_umma_t<2, false>(a, st);
    case 3: return ip ? launch_compress_umma_t<3, true>(a, st) : launch_compress_umma_t<3, false>(a, st);
    default: return ip ? launch_compress_umma_t<4, true>(a, st) : launch_compress_umma_t<4, false>(a, st);
  }
}

unsigned int decompress_umma_timeouts();           // decompress_umma.cu keeps its own counter

unsigned int umma_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_umma_timeouts, sizeof(v));
  return v + decompress_umma_timeouts();
}


}  // namespace qkv
