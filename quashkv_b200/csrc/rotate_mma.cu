// Tensor-core rotation for compress and decompress at d = 128 (uniform bit width).
//
// The rotation x_unit @ Pi^T is the only dense contraction of the path.  Both operands are split
// exactly into three bf16 terms (8+8+8 = 24 significant bits: x = h + m + l), and the six products
// that matter (hH, hM, mH, hL, lH, mM; the rest is below 2^-32 relative) run as bf16 m16n8k16 MMAs
// with fp32 accumulation, smallest terms first.  That reproduces an fp32 dot product to a few
// units in the last place.
//
// Codes must equal the fp32 result of the reference bit for bit, and a code flips when a rotated
// coordinate crosses a decision boundary.  So every coordinate whose tensor-core value lies within
// kRecheckEps of a boundary (or, for the sign bit, whose residual lies within it of zero) is
// recomputed with the sequential fp32 FMA chain of the CUDA-core kernel, which is the arithmetic
// the parity tests pinned to the reference; about one coordinate in 2000 takes that path.  Norms
// use the CUDA-core kernel's exact summation order.
//
// CTA = 8 warps = 4 groups of 32 vectors x 2 halves of the 128 output coordinates; Pi's three bf16
// planes (padded, 104 KB) stay in shared memory for the CTA's lifetime; a 128-vector tile of
// x_unit (fp32, 70 KB) is staged per iteration.
#include "rotate_exact.cuh"

namespace qkv {

constexpr int kRTile = 128;                 // vectors per CTA tile
constexpr int kPiStride = kRD + 8;          // bf16 elements per padded Pi row (conflict-free B loads)
constexpr int kXStride = kRD + 8;           // fp32 elements per padded x row (conflict-free A loads)

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct RotSmem {
  __nv_bfloat16* pi[3];      // [128][kPiStride] each: B operand rows (output coordinate), k contiguous
  float* x;                  // [128][kXStride] staged A operand (fp32)
  uint8_t* codes;            // [128][128] codes of the tile
  uint8_t* signs;            // [128][128] sign bits of the tile (IP mode)
  float* tab;                // [16] boundaries / centroids
  float* cent;               // [16]
  float* sgn;                // [128]
  float* norm;               // [128]
};

__device__ __forceinline__ RotSmem carve_rot(unsigned char* raw) {
  RotSmem s;
  __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(raw);
  for (int t = 0; t < 3; ++t) s.pi[t] = p + t * kRD * kPiStride;
  s.x = reinterpret_cast<float*>(p + 3 * kRD * kPiStride);
  s.codes = reinterpret_cast<uint8_t*>(s.x + kRTile * kXStride);
  s.signs = s.codes + kRTile * kRD;
  s.tab = reinterpret_cast<float*>(s.signs + kRTile * kRD);
  s.cent = s.tab + 16;
  s.sgn = s.cent + 16;
  s.norm = s.sgn + kRD;
  return s;
}

constexpr size_t kRotSmemBytes = 3 * kRD * kPiStride * 2 + kRTile * kXStride * 4 + 2 * kRTile * kRD +
                                 (16 + 16 + kRD + kRTile) * 4;

// Split a (128 x 128) fp32 matrix into three bf16 planes in shared memory.  transpose == false:
// plane[n][k] = M[n][k] (compress: B[k][n] = Pi[n][k]); true: plane[n][k] = M[k][n] (decompress).
__device__ __forceinline__ void stage_matrix(__nv_bfloat16* const (&pi)[3], const float* __restrict__ M,
                                             bool transpose) {
  for (int idx = threadIdx.x; idx < kRD * kRD; idx += blockDim.x) {
    const int r = idx >> 7, c = idx & 127;                // coalesced read of M[r][c]
    __nv_bfloat16 h, m, l;
    split3(M[idx], h, m, l);
    const int n = transpose ? c : r, k = transpose ? r : c;
    pi[0][n * kPiStride + k] = h;
    pi[1][n * kPiStride + k] = m;
    pi[2][n * kPiStride + k] = l;
  }
}

// acc[mt][nt][4] += A(32 rows of s.x, fp32 split on the fly) x B(64 output coordinates of the planes).
__device__ __forceinline__ void rotate_tile(const RotSmem& s, int row0, int col0, int gid, int tig,
                                            float (&acc)[2][8][4]) {
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
#pragma unroll 1
  for (int k0 = 0; k0 < kRD; k0 += 16) {
    uint32_t ah[2][4], am[2][4], al[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {       // fragment register q: row gid + 8 (q&1), k = k0 + 2 tig + 8 (q>>1)
        const int r = row0 + 16 * mt + gid + 8 * (q & 1), k = k0 + 2 * tig + 8 * (q >> 1);
        const float2 v = *reinterpret_cast<const float2*>(s.x + r * kXStride + k);
        __nv_bfloat16 h0, m0, l0, h1, m1, l1;
        split3(v.x, h0, m0, l0);
        split3(v.y, h1, m1, l1);
        ah[mt][q] = pack_bf16(h0, h1);
        am[mt][q] = pack_bf16(m0, m1);
        al[mt][q] = pack_bf16(l0, l1);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int n = col0 + 8 * nt + gid;
      uint32_t bh[2], bm[2], bl[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {       // B register q: k = k0 + 2 tig + 8 q, n = gid
        const int off = n * kPiStride + k0 + 2 * tig + 8 * q;
        bh[q] = *reinterpret_cast<const uint32_t*>(s.pi[0] + off);
        bm[q] = *reinterpret_cast<const uint32_t*>(s.pi[1] + off);
        bl[q] = *reinterpret_cast<const uint32_t*>(s.pi[2] + off);
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {    // smallest products first
        mma_bf16(acc[mt][nt], am[mt], bm[0], bm[1]);
        mma_bf16(acc[mt][nt], al[mt], bh[0], bh[1]);
        mma_bf16(acc[mt][nt], ah[mt], bl[0], bl[1]);
        mma_bf16(acc[mt][nt], am[mt], bh[0], bh[1]);
        mma_bf16(acc[mt][nt], ah[mt], bm[0], bm[1]);
        mma_bf16(acc[mt][nt], ah[mt], bh[0], bh[1]);
      }
    }
  }
}

// ---- compress ------------------------------------------------------------------------------------
// Each warp owns 32 vectors x 64 output coordinates and runs without block-wide barriers: it streams
// its rows from global memory straight into A fragments (bf16 input needs no split and three
// products; fp32 input is split and takes six), accumulates the fp64 sum of squares of the same
// values for the norm, classifies the accumulators through a 16K-entry bucket table in shared memory
// (bucket = round(4096 y) + 4096; a bucket that could contain a decision boundary is "ambiguous"),
// packs the codes of its quad with two shuffles per word and stores whole words.  Elements that are
// really within kRecheckEps of a boundary go to a per-warp queue and are recomputed 32 at a time (one
// per lane) with the fp32 FMA chain; a changed code is patched into the packed row with atomicXor.

struct CompSmem {
  __nv_bfloat16* pi[3];
  uint8_t* lut;        // [kLutSize]: code | 0x80 when ambiguous
  float* bnd;          // [16] boundaries (+inf padded)
  float* cent;         // [16]
  float* sgn;          // [128]
  uint4* queue;        // [warps][kQueueCap]: n, col | code<<8 | sign<<16, norm bits, unused
  int* qcount;         // [warps]
};

template <int WARPS>
__device__ __forceinline__ CompSmem carve_comp(unsigned char* raw) {
  CompSmem s;
  __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(raw);
  for (int t = 0; t < 3; ++t) s.pi[t] = p + t * kRD * kPiStride;
  s.queue = reinterpret_cast<uint4*>(p + 3 * kRD * kPiStride);
  s.lut = reinterpret_cast<uint8_t*>(s.queue + WARPS * kQueueCap);
  s.bnd = reinterpret_cast<float*>(s.lut + kLutSize);
  s.cent = s.bnd + 16;
  s.sgn = s.cent + 16;
  s.qcount = reinterpret_cast<int*>(s.sgn + kRD);
  return s;
}

template <int WARPS>
constexpr size_t comp_smem_bytes() {
  return 3 * kRD * kPiStride * 2 + WARPS * kQueueCap * 16 + kLutSize + (16 + 16 + kRD) * 4 + WARPS * 4;
}

// OR-combine the quad's partial words and store them: lane tig writes words tig, tig+4, ...
template <int NW>
__device__ __forceinline__ void quad_store(uint32_t (&W)[NW], uint32_t* dst, int tig, bool live) {
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    W[w] |= __shfl_xor_sync(QKV_FULL_MASK, W[w], 1);
    W[w] |= __shfl_xor_sync(QKV_FULL_MASK, W[w], 2);
  }
#pragma unroll
  for (int w = 0; w < NW; ++w)
    if (live && (w & 3) == tig) dst[w] = W[w];
}

template <int BITS, bool IP, int NTERM, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) compress_mma_kernel(CompressArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const CompSmem s = carve_comp<WARPS>(smem_raw);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int row0 = 32 * (warp >> 1), col0 = 64 * (warp & 1);
  constexpr int NB = (1 << BITS) - 1;
  constexpr int kRows = (WARPS / 2) * 32;          // vectors per CTA pass
  constexpr int row_words = (BITS == 3 ? 3 * (kRD / 8) : kRD * BITS / 8) / 4;

  stage_matrix(s.pi, a.Pi, false);
  if (threadIdx.x < 16) {
    s.bnd[threadIdx.x] = threadIdx.x < NB ? a.bounds0[threadIdx.x] : INFINITY;
    s.cent[threadIdx.x] = (IP && threadIdx.x < (1 << BITS)) ? a.centroids[threadIdx.x] : 0.f;
  }
  if (threadIdx.x < kRD) s.sgn[threadIdx.x] = IP ? a.S[threadIdx.x] : 0.f;
  if (threadIdx.x < WARPS) s.qcount[threadIdx.x] = 0;
  __syncthreads();
  build_bucket_lut<BITS, IP>(s.lut, s.bnd, s.cent);
  __syncthreads();

  uint4* queue = s.queue + warp * kQueueCap;
  uint32_t* out_codes = reinterpret_cast<uint32_t*>(a.codes);
  uint32_t* out_signs = reinterpret_cast<uint32_t*>(a.signs);

  // Recompute queued elements with the fp32 FMA chain (x/norm, ascending coordinate), one per lane.
  auto drain = [&](int count) {
    __threadfence();                       // this warp's packed words are visible before they are patched
    __syncwarp();
    for (int base = 0; base < count; base += 32) {
      const int i = base + lane;
      if (i < count) {
        const uint4 it = queue[i];
        const int64_t n = it.x;
        const int col = it.y & 0xFF;
        const uint32_t old_code = (it.y >> 8) & 0xFF, old_sign = (it.y >> 16) & 1u;
        const float norm = __uint_as_float(it.z);
        const float z = exact_chain(a, n, col, norm);
        const uint32_t code = count_bounds<BITS>(s.bnd, z);
        const int64_t row = map_row(a.rows, n);
        const uint32_t diff = code ^ old_code;
        if (diff) {
          const int bit = col * BITS, w = bit >> 5, sh = bit & 31;
          atomicXor(out_codes + row * row_words + w, diff << sh);
          if (sh + BITS > 32) atomicXor(out_codes + row * row_words + w + 1, diff >> (32 - sh));
        }
        if (IP) {
          const uint32_t sign = ((z - s.cent[code]) * s.sgn[col] >= 0.f) ? 1u : 0u;
          if (sign != old_sign) atomicXor(out_signs + row * (kRD / 32) + (col >> 5), 1u << (col & 31));
        }
      }
    }
    __syncwarp();
  };

  const int64_t n_pass = (a.n_vec + kRows - 1) / kRows;
  for (int64_t pass = blockIdx.x; pass < n_pass; pass += gridDim.x) {
    const int64_t v0 = pass * kRows + row0;
    if (v0 >= a.n_vec) continue;             // warp-uniform: nothing left for this warp
    // rows of this lane: v0 + 16 mt + gid + 8 h; rows past the end re-read the last vector (discarded)
    int64_t nrow[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t n = v0 + 16 * mt + gid + 8 * h;
        nrow[mt][h] = n < a.n_vec ? n : a.n_vec - 1;
      }
    float acc[2][8][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
    double ss[2][2] = {{0.0, 0.0}, {0.0, 0.0}};

    // raw A registers of one k-step: bf16 pairs as loaded, or fp32 pairs; the next step's are fetched
    // while this step's MMAs run
    constexpr int RAW = NTERM == 1 ? 1 : 2;
    uint32_t raw[2][4][RAW], nxt[2][4][RAW];
    auto fetch = [&](uint32_t (&dst)[2][4][RAW], int k0) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int q = 0; q < 4; ++q) {       // register q: row gid + 8 (q&1), k = k0 + 2 tig + 8 (q>>1)
          const int64_t off = nrow[mt][q & 1] * a.x_pitch + k0 + 2 * tig + 8 * (q >> 1);
          if (NTERM == 1) {
            dst[mt][q][0] = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(a.x) + off));
          } else if (a.x_dtype == QKV_F32) {
            const float2 v = __ldg(reinterpret_cast<const float2*>(reinterpret_cast<const float*>(a.x) + off));
            dst[mt][q][0] = __float_as_uint(v.x);
            dst[mt][q][RAW - 1] = __float_as_uint(v.y);
          } else {
            dst[mt][q][0] = __float_as_uint(load_float(a.x, a.x_dtype, off));
            dst[mt][q][RAW - 1] = __float_as_uint(load_float(a.x, a.x_dtype, off + 1));
          }
        }
    };
    fetch(raw, 0);
#pragma unroll 1
    for (int k0 = 0; k0 < kRD; k0 += 16) {
      if (k0 + 16 < kRD) fetch(nxt, k0 + 16);
      uint32_t af[NTERM][2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float v0f, v1f;
          if (NTERM == 1) {
            af[0][mt][q] = raw[mt][q][0];
            v0f = __uint_as_float(raw[mt][q][0] << 16);
            v1f = __uint_as_float(raw[mt][q][0] & 0xFFFF0000u);
          } else {
            v0f = __uint_as_float(raw[mt][q][0]);
            v1f = __uint_as_float(raw[mt][q][RAW - 1]);
            __nv_bfloat16 h0, m0, l0, h1, m1, l1;
            split3(v0f, h0, m0, l0);
            split3(v1f, h1, m1, l1);
            af[0][mt][q] = pack_bf16(h0, h1);
            af[NTERM > 1 ? 1 : 0][mt][q] = pack_bf16(m0, m1);
            af[NTERM > 2 ? 2 : 0][mt][q] = pack_bf16(l0, l1);
          }
          ss[mt][q & 1] += static_cast<double>(v0f) * static_cast<double>(v0f) +
                           static_cast<double>(v1f) * static_cast<double>(v1f);
        }
      }
      // two n-tiles at a time; within a product term the four MMAs are independent, so an
      // accumulator is revisited only after three others were issued
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bh[2][2], bm[2][2], bl[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = col0 + 8 * (2 * np + j) + gid;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int off = n * kPiStride + k0 + 2 * tig + 8 * q;
            bh[j][q] = *reinterpret_cast<const uint32_t*>(s.pi[0] + off);
            bm[j][q] = *reinterpret_cast<const uint32_t*>(s.pi[1] + off);
            bl[j][q] = *reinterpret_cast<const uint32_t*>(s.pi[2] + off);
          }
        }
#define QKV_TERM(A, B)                                                             \
  _Pragma("unroll") for (int j = 0; j < 2; ++j) _Pragma("unroll") for (int mt = 0; mt < 2; ++mt) \
      mma_bf16(acc[mt][2 * np + j], A[mt], B[j][0], B[j][1]);
        if (NTERM == 1) {                       // smallest products first
          QKV_TERM(af[0], bl) QKV_TERM(af[0], bm) QKV_TERM(af[0], bh)
        } else {
          QKV_TERM(af[NTERM > 1 ? 1 : 0], bm) QKV_TERM(af[NTERM > 2 ? 2 : 0], bh) QKV_TERM(af[0], bl)
          QKV_TERM(af[NTERM > 1 ? 1 : 0], bh) QKV_TERM(af[0], bm) QKV_TERM(af[0], bh)
        }
#undef QKV_TERM
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int r = 0; r < RAW; ++r) raw[mt][q][r] = nxt[mt][q][r];
    }

    // ---- norms: the quad holds a row's squares ----------------------------------------------------------
    float norm[2][2], inv[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        double t = ss[mt][h];
        t += __shfl_xor_sync(QKV_FULL_MASK, t, 1);
        t += __shfl_xor_sync(QKV_FULL_MASK, t, 2);
        norm[mt][h] = fmaxf(static_cast<float>(sqrt(t)), 1e-8f);
        inv[mt][h] = 1.f / norm[mt][h];
      }

    // ---- classify, pack per quad, store; queue the elements that need the exact chain.  One loop
    //      iteration per (m-tile, row half) keeps the code small enough for the instruction cache; the
    //      16 accumulators of the iteration are picked with selects. ------------------------------------
#pragma unroll 1
    for (int it = 0; it < 4; ++it) {
      const int mt = it >> 1, h = it & 1;
      float yv[8][2];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e)
          yv[nt][e] = it == 0 ? acc[0][nt][e] : (it == 1 ? acc[0][nt][2 + e] : (it == 2 ? acc[1][nt][e] : acc[1][nt][2 + e]));
      const float nrm = it == 0 ? norm[0][0] : (it == 1 ? norm[0][1] : (it == 2 ? norm[1][0] : norm[1][1]));
      const float iv = it == 0 ? inv[0][0] : (it == 1 ? inv[0][1] : (it == 2 ? inv[1][0] : inv[1][1]));
      const int64_t n = v0 + 16 * mt + gid + 8 * h;
      const bool live = n < a.n_vec;
      const int64_t row = live ? map_row(a.rows, n) : 0;
      uint32_t W[2 * BITS], SW[2] = {0u, 0u};
#pragma unroll
      for (int w = 0; w < 2 * BITS; ++w) W[w] = 0u;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        uint32_t pair = 0, spair = 0;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = col0 + 8 * nt + 2 * tig + e;
          const float y = yv[nt][e] * iv;
          const uint32_t v = s.lut[bucket_of(y)];
          uint32_t code = v & 0x7Fu, sign = 0;
          if (IP) sign = ((y - s.cent[code]) * s.sgn[col] >= 0.f) ? 1u : 0u;
          if (v & 0x80u) {                 // rare: exact classification of the estimate, and the near test
            const uint32_t r = classify_slow(s.bnd, s.cent, IP ? s.sgn[col] : 0.f, y, NB, IP ? 1 : 0);
            code = r & 0xFFu;
            sign = (r >> 8) & 1u;
            if ((r >> 16) && live) {
              const int slot = atomicAdd(&s.qcount[warp], 1);
              if (slot < kQueueCap) {
                queue[slot] = make_uint4(static_cast<uint32_t>(n), col | (code << 8) | (sign << 16),
                                         __float_as_uint(nrm), 0u);
              } else {                      // queue full (degenerate input, e.g. all-zero vectors): do it now
                const float z = exact_chain(a, n, col, nrm);
                code = count_bounds<BITS>(s.bnd, z);
                if (IP) sign = ((z - s.cent[code]) * s.sgn[col] >= 0.f) ? 1u : 0u;
              }
            }
          }
          pair |= code << (BITS * e);
          spair |= sign << e;
        }
        const uint32_t g = pair << (2 * BITS * tig);
        constexpr int kGroupBits = 8 * BITS;
        const int pos = kGroupBits * nt, w = pos >> 5, sh = pos & 31;
        W[w] |= g << sh;
        if (sh + kGroupBits > 32) W[w + 1] |= g >> (32 - sh);
        if (IP) SW[nt >> 2] |= (spair << (2 * tig)) << (8 * (nt & 3));
      }
      quad_store<2 * BITS>(W, out_codes + row * row_words + (col0 / 64) * 2 * BITS, tig, live);
      if (IP) quad_store<2>(SW, out_signs + row * (kRD / 32) + (col0 / 64) * 2, tig, live);
      if (live && col0 == 0 && tig == 0) a.norms[row] = nrm;
    }
    // ---- drain the queue when a batch is full (or it might overflow on the next pass) -----------------
    __syncwarp();
    const int queued = s.qcount[warp];
    if (queued >= 32) {
      drain(queued < kQueueCap ? queued : kQueueCap);
      __syncwarp();
      if (lane == 0) s.qcount[warp] = 0;
      __syncwarp();
    }
  }
  __syncwarp();
  const int queued = s.qcount[warp];
  if (queued > 0) drain(queued < kQueueCap ? queued : kQueueCap);
}

bool compress_mma_ok(const CompressArgs& a) {
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.codes) |
                       (a.mode == MODE_IP ? reinterpret_cast<uintptr_t>(a.signs) : 0);
  return a.d == kRD && a.mode != MODE_MIXED && a.packed && a.n_vec >= 256 && a.n_vec < (int64_t(1) << 31) &&
         (a.x_pitch & 3) == 0 && (al & 15u) == 0;
}

template <int BITS, bool IP, int NTERM>
static int launch_compress_mma_t(const CompressArgs& a, cudaStream_t st) {
  constexpr int WARPS = 8;
  constexpr size_t smem = comp_smem_bytes<WARPS>();
  if (cudaFuncSetAttribute(compress_mma_kernel<BITS, IP, NTERM, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return QKV_ELAUNCH;
  const int64_t passes = (a.n_vec + (WARPS / 2) * 32 - 1) / ((WARPS / 2) * 32);
  const int grid = static_cast<int>(passes < kNumSMs ? passes : kNumSMs);
  compress_mma_kernel<BITS, IP, NTERM, WARPS><<<grid, WARPS * 32, smem, st>>>(a);
  return check_launch();
}

template <int BITS, bool IP>
static int launch_compress_mma_n(const CompressArgs& a, cudaStream_t st) {
  return a.x_dtype == QKV_BF16 ? launch_compress_mma_t<BITS, IP, 1>(a, st) : launch_compress_mma_t<BITS, IP, 3>(a, st);
}

int launch_compress_mma(const CompressArgs& a, cudaStream_t st) {
  const bool ip = a.mode == MODE_IP;
  switch (a.bits0) {
    case 1: return ip ? launch_compress_mma_n<1, true>(a, st) : launch_compress_mma_n<1, false>(a, st);
    case 2: return ip ? launch_compress_mma_n<2, true>(a, st) : launch_compress_mma_n<2, false>(a, st);
    case 3: return ip ? launch_compress_mma_n<3, true>(a, st) : launch_compress_mma_n<3, false>(a, st);
    default: return ip ? launch_compress_mma_n<4, true>(a, st) : launch_compress_mma_n<4, false>(a, st);
  }
}

// out = (c[codes] (+ qjl_scale * S * (2 sign - 1))) @ Pi * norm on the same machinery; no bit-exact
// output here, so no recheck: the result equals an fp32 matmul to a few units in the last place.
__global__ void __launch_bounds__(256, 1) decompress_mma_kernel(DecompressArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const RotSmem s = carve_rot(smem_raw);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int row0 = 32 * (warp >> 1), col0 = 64 * (warp & 1);

  stage_matrix(s.pi, a.Pi, true);
  if (threadIdx.x < 16) s.tab[threadIdx.x] = threadIdx.x < (1 << a.bits0) ? a.cents0[threadIdx.x] : 0.f;
  if (threadIdx.x < kRD) s.sgn[threadIdx.x] = a.signs ? a.S[threadIdx.x] : 0.f;

  const int row_bytes = packed_row_bytes(kRD, a.bits0);
  const int64_t n_tiles = (a.n_vec + kRTile - 1) / kRTile;
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t v0 = tile * kRTile;
    __syncthreads();
    for (int rr = 0; rr < 16; ++rr) {
      const int r = 16 * warp + rr;
      const int64_t n = v0 + r;
      const bool live = n < a.n_vec;
      const int64_t row = live ? map_row(a.rows, n) : 0;
      if (lane == 0) s.norm[r] = live ? a.norms[row] : 0.f;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int j = lane + 32 * t;
        float y = 0.f;
        if (live) {
          const uint32_t c = a.packed ? read_field(a.codes + row * row_bytes, j * a.bits0, a.bits0, row_bytes)
                                      : a.codes[row * kRD + j];
          y = s.tab[c];
          if (a.signs) {
            const uint32_t sb = a.packed ? ((a.signs[row * (kRD / 8) + (j >> 3)] >> (j & 7)) & 1u)
                                         : a.signs[row * kRD + j];
            y += a.qjl_scale * (s.sgn[j] * (sb ? 1.f : -1.f));
          }
        }
        s.x[r * kXStride + j] = y;
      }
    }
    __syncthreads();
    float acc[2][8][4];
    rotate_tile(s, row0, col0, gid, tig, acc);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = row0 + 16 * mt + gid + 8 * h;
        const int64_t n = v0 + r;
        if (n >= a.n_vec) continue;
        const float nrm = s.norm[r];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const int col = col0 + 8 * nt + 2 * tig;
          store_float(a.out, a.out_dtype, n * a.out_pitch + col, acc[mt][nt][2 * h] * nrm);
          store_float(a.out, a.out_dtype, n * a.out_pitch + col + 1, acc[mt][nt][2 * h + 1] * nrm);
        }
      }
    }
  }
}

bool decompress_mma_ok(const DecompressArgs& a) {
  return a.d == kRD && a.mode != MODE_MIXED && a.n_vec >= 2 * kRTile;
}

int launch_decompress_mma(const DecompressArgs& a, cudaStream_t st) {
  if (cudaFuncSetAttribute(decompress_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kRotSmemBytes)) != cudaSuccess)
    return QKV_ELAUNCH;
  const int64_t tiles = (a.n_vec + kRTile - 1) / kRTile;
  const int grid = static_cast<int>(tiles < kNumSMs ? tiles : kNumSMs);
  decompress_mma_kernel<<<grid, 256, kRotSmemBytes, st>>>(a);
  return check_launch();
}

}  // namespace qkv
