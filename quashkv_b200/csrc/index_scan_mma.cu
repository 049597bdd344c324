// Tensor-core index scan for dim 128, 3 bits (2-bit codes + sign bit).
//
// score[m,n] = norm_n * (q_rot_m . c[code_n] + qjl_scale * sum |q_rot_m| S (2 sign_n - 1)) for every
// (query, database row) pair is a dense contraction whose one operand is decoded on the fly, so it
// belongs on the tensor cores: database rows are the M dimension (16 per warp tile, decoded in
// registers exactly like the keys of the decode attention), 32 queries per CTA are the N dimension
// (ready B fragments in shared memory: the unit-normalised rotated query in fp16 and its sign
// weights), K = 256: 64 MMAs per tile.
//
// The fp16 scores only PROPOSE candidates; the result is exact.  With queries normalised to unit
// length the approximate score of a row is within kEps * norm_row of its fp32 score (fp16 rounding
// of the query, of the four centroids and of the sign weights; products and sums are fp32).  Each
// accumulator starts at kEps - sum(w), so what the kernel compares and stores is the OPTIMISTIC
// score u = s~ + kEps * norm.  A row can only belong to the true top-k if u >= T, where T is any
// lower bound of the k-th best PESSIMISTIC score; the kernel uses T = (k-th best u) - 2 kEps *
// (largest norm seen), which only ever rises.  Every warp keeps its own candidate buffers (no CTA
// barrier in the streaming loop); T is shared between the warps of a CTA through a racy maximum.
// The survivors are re-scored with the fp32 arithmetic of the CUDA-core scan kernel and merged by
// exact score (ties by lower id).  A query whose candidates do not fit (more than the list holds
// within the bound of the k-th score: many equal rows), or whose norm is zero or not finite, is
// flagged, and the CUDA-core scan redoes exactly the flagged queries.
#include <math.h>

#include <stdlib.h>

#include "index_candidates.cuh"

namespace qkv {

template <int CAPW>
__global__ void __launch_bounds__(kIWarps * 32, CAPW <= 32 ? 4 : (CAPW <= 48 ? 3 : 2))
index_scan_mma_kernel(ScanMmaArgs a) {
  constexpr int D = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* ring_s = smem_raw;                                             // per-warp staging rings
  uint2 (*bop)[kIQ / 8][32] = reinterpret_cast<uint2 (*)[kIQ / 8][32]>(ring_s + kIWarps * kIStages * kIStageBytes);
  float* buf_u = reinterpret_cast<float*>(bop + 16);                            // [query][warp][CAPW]
  uint16_t* buf_r = reinterpret_cast<uint16_t*>(buf_u + kIWarps * kIQ * CAPW);  // [query][warp][CAPW]
  __shared__ float init_c[kIQ];          // kEps - sum of the sign weights of the unit query
  __shared__ float thr[kIQ];             // lower bound of the k-th best pessimistic score
  __shared__ int cnt[kIWarps][kIQ];
  __shared__ float quart[kIWarps][kIQ];  // per warp: lower bound of its ceil(k/4)-th best pessimistic score
  __shared__ float nmax_w[kIWarps];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int slice = blockIdx.x, q0 = blockIdx.y * kIQ;
  const float inv_sk = __uint_as_float(a.tables[6]);
  const uint32_t kt_a = a.tables[0], kt_b = a.tables[1];

  // ---- B fragments: warp w builds n-tile w (query q0 + 8 w + gid; lane tig covers coordinates 32 tig..) ----
  {
    const int nt = warp;
    const int m = q0 + 8 * nt + gid;
    const float* q = a.qk + static_cast<int64_t>(m < a.M ? m : 0) * 2 * D;
    float q2 = 0.f, ws = 0.f;
    for (int j = 32 * tig; j < 32 * tig + 32; ++j) { q2 = fmaf(q[j], q[j], q2); ws += q[D + j]; }
    q2 += __shfl_xor_sync(QKV_FULL_MASK, q2, 1); ws += __shfl_xor_sync(QKV_FULL_MASK, ws, 1);
    q2 += __shfl_xor_sync(QKV_FULL_MASK, q2, 2); ws += __shfl_xor_sync(QKV_FULL_MASK, ws, 2);
    const float qn = sqrtf(q2);
    const bool usable = m < a.M && qn > 0.f && qn < INFINITY;
    const float inv = usable ? 1.f / qn : 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const int word = s >> 2, grp = s & 3;
      const int c0 = 32 * tig + 16 * word + grp;
      const float f = inv * inv_sk;
      bop[s][nt][lane] = make_uint2(pack_half2(q[c0] * f, q[c0 + 4] * f), pack_half2(q[c0 + 8] * f, q[c0 + 12] * f));
      uint32_t wq[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int t = 2 * s + h, j = 32 * tig + sign_coord(t);
        const float g = 2.f / sign_v1(sign_pos(t)) * inv;
        wq[h] = pack_half2(q[D + j] * g, q[D + j + 16] * g);
      }
      bop[8 + s][nt][lane] = make_uint2(wq[0], wq[1]);
    }
    if (tig == 0) {
      init_c[8 * nt + gid] = kEps - ws * inv;
      thr[8 * nt + gid] = usable ? -INFINITY : INFINITY;      // unusable queries collect nothing
      if (m < a.M && !usable) a.flags[m] = 1;
    }
  }
  cnt[warp][lane] = 0;
  quart[warp][lane] = -INFINITY;
  __syncthreads();
  const int k4 = (a.k + 3) / 4;

  const int64_t n_begin = slice * a.slice_len;
  int64_t n_end = n_begin + a.slice_len;
  if (n_end > a.N) n_end = a.N;
  const int n_valid = static_cast<int>(n_end - n_begin);
  constexpr int kStep = kIWarps * 16;
  const int n_it = (n_valid + kStep - 1) / kStep;          // every warp takes one 16-row tile per step
  const int first_rel = warp * 16;
  constexpr int QS = kIWarps * CAPW;          // slots per query; this warp's CAPW start at warp * CAPW
  float* my_u = buf_u + warp * CAPW;
  uint16_t* my_r = buf_r + warp * CAPW;
  float my_nmax = 0.f;

  // ---- cp.async ring: 52 chunks of 16 bytes per tile (32 code, 16 sign, 4 norm) ------------------------
  unsigned char* ring = ring_s + warp * (kIStages * kIStageBytes);
  const unsigned char* src0[2];
  int dst_off[2], tok_off[2], stride[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int c = lane + 32 * k;
    const int64_t t_first = n_begin + first_rel;
    if (c < 32) {
      tok_off[k] = c >> 1; stride[k] = kStep * 32; dst_off[k] = c * 16;
      src0[k] = a.codes + (t_first + (c >> 1)) * 32 + (c & 1) * 16;
    } else if (c < 48) {
      const int r = c - 32;
      tok_off[k] = r; stride[k] = kStep * 16; dst_off[k] = 512 + r * 16;
      src0[k] = a.signs + (t_first + r) * 16;
    } else {
      const int j = (c - 48) & 3;
      tok_off[k] = 4 * j; stride[k] = kStep * 4; dst_off[k] = 768 + j * 16;
      src0[k] = reinterpret_cast<const unsigned char*>(a.norms + t_first + 4 * j);
    }
  }
  auto issue = [&](int it) {
    if (it < n_it) {
      const int rel = first_rel + it * kStep;
      unsigned char* stage = ring + (it % kIStages) * kIStageBytes;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        if (k == 0 || lane < 20) {
          const int left = n_valid - (rel + tok_off[k]);            // rows of this chunk inside the slice
          const bool ok = left > 0;
          const int bytes = (lane + 32 * k < 48 || left >= 4) ? 16 : 4 * left;   // a norm chunk holds 4 rows
          cp_async16(stage + dst_off[k], ok ? src0[k] + static_cast<int64_t>(it) * stride[k] : a.codes,
                     ok ? bytes : 0);
        }
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int i = 0; i < kIStages - 1; ++i) issue(i);
  for (int it = 0; it < n_it; ++it) {
    issue(it + kIStages - 1);
    cp_async_wait<kIStages - 1>();
    __syncwarp();
    const unsigned char* stage = ring + (it % kIStages) * kIStageBytes;
    uint2 kc[2]; uint32_t ks[2]; float kn[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      kc[h] = *reinterpret_cast<const uint2*>(stage + (gid + 8 * h) * 32 + tig * 8);
      ks[h] = *reinterpret_cast<const uint32_t*>(stage + 512 + (gid + 8 * h) * 16 + tig * 4);
      kn[h] = *reinterpret_cast<const float*>(stage + 768 + (gid + 8 * h) * 4);
    }
    __syncwarp();
    my_nmax = fmaxf(my_nmax, fmaxf(kn[0], kn[1]));

    float c[kIQ / 8][4];
#pragma unroll
    for (int nt = 0; nt < kIQ / 8; ++nt) {
      const float2 i2 = *reinterpret_cast<const float2*>(&init_c[8 * nt + 2 * tig]);
      c[nt][0] = c[nt][2] = i2.x;
      c[nt][1] = c[nt][3] = i2.y;
    }
    {   // sign part first: its operands need no table look-up
      const uint32_t cp0[4] = {ks[0], ks[0] << 7, ks[0] >> 1, ks[0] << 13};
      const uint32_t cp1[4] = {ks[1], ks[1] << 7, ks[1] >> 1, ks[1] << 13};
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
#pragma unroll
        for (int nt = 0; nt < kIQ / 8; ++nt) {
          const uint2 bw = bop[8 + s][nt][lane];
          mma16816(c[nt], af, bw.x, bw.y);
        }
      }
    }
#pragma unroll
    for (int word = 0; word < 2; ++word) {
      const uint32_t w0 = word ? kc[0].y : kc[0].x, w1 = word ? kc[1].y : kc[1].x;
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
#pragma unroll
        for (int nt = 0; nt < kIQ / 8; ++nt) {
          const uint2 bh = bop[word * 4 + grp][nt][lane];
          mma16816(c[nt], af, bh.x, bh.y);
        }
      }
    }
    // ---- the other slices' progress: lane = query --------------------------------------------------------------
    if ((it & 3) == 0 && q0 + lane < a.M) {
      const float g = *reinterpret_cast<const volatile float*>(a.gthr + q0 + lane);
      if (g > thr[lane] && thr[lane] != INFINITY) raise_threshold(&thr[lane], g);
    }
    __syncwarp();
    // ---- candidates: optimistic score at or above the query's threshold ---------------------------------
    const int rel = first_rel + it * kStep;
#pragma unroll
    for (int nt = 0; nt < kIQ / 8; ++nt) {
      const float2 t2 = *reinterpret_cast<const float2*>(&thr[8 * nt + 2 * tig]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int q = 8 * nt + 2 * tig + (e & 1), r = rel + gid + 8 * (e >> 1);
        const float u = c[nt][e] * kn[e >> 1];
        if (u >= ((e & 1) ? t2.y : t2.x) && r < n_valid) {
          const int pos = atomicAdd(&cnt[warp][q], 1);
          if (pos < CAPW) {
            my_u[q * QS + pos] = u; my_r[q * QS + pos] = static_cast<uint16_t>(r);
          } else {                                  // full before it could be pruned (see the prune mark): redo the query
            if (q0 + q < a.M) a.flags[q0 + q] = 1;
            thr[q] = INFINITY;
          }
        }
      }
    }
    __syncwarp();
    // ---- shrink the buffers that could overflow on the next tile ------------------------------------------
    unsigned need = __ballot_sync(QKV_FULL_MASK, cnt[warp][lane] > CAPW - kIRoom);
    if (need) {
      float nm = my_nmax;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) nm = fmaxf(nm, __shfl_xor_sync(QKV_FULL_MASK, nm, o));
      while (need) {
        const int q = __ffs(need) - 1;
        need &= need - 1;
        const int n = cnt[warp][q] < CAPW ? cnt[warp][q] : CAPW;
        // Two valid lower bounds of the CTA's k-th best pessimistic score: this warp's own k-th best, and
        // the smallest of the four warps' ceil(k/4)-th best (each warp then has that many rows at or
        // above it, and the warps' rows are disjoint).  The second is the tight one: a quarter of the
        // rows yields the k/4-th best at about the height of the whole CTA's k-th best.
        float T, T4;
        const int kept = select_sorted<CAPW>(my_u + q * QS, my_r + q * QS, n, a.k, 2.f * kEps * nm,
                                             CAPW - kIRoom, thr[q], k4, T, T4, lane);
        if (lane == 0) {
          if (kept > CAPW - kIRoom) {             // more rows within the bound than a buffer holds
            if (q0 + q < a.M) a.flags[q0 + q] = 1;
            thr[q] = INFINITY;
            cnt[warp][q] = 0;
          } else {
            cnt[warp][q] = kept;
            quart[warp][q] = fmaxf(quart[warp][q], T4);
            const float all4 = fminf(fminf(*reinterpret_cast<volatile float*>(&quart[0][q]),
                                           *reinterpret_cast<volatile float*>(&quart[1][q])),
                                     fminf(*reinterpret_cast<volatile float*>(&quart[2][q]),
                                           *reinterpret_cast<volatile float*>(&quart[3][q])));
            const float bound = fmaxf(T, all4);
            raise_threshold(&thr[q], bound);
            if (q0 + q < a.M && bound > -INFINITY) publish_bound(a.gthr + q0 + q, bound);
          }
        }
      }
      __syncwarp();
    }
  }
  cp_async_wait<0>();
  {
    float nm = my_nmax;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) nm = fmaxf(nm, __shfl_xor_sync(QKV_FULL_MASK, nm, o));
    if (lane == 0) nmax_w[warp] = nm;
  }
  __syncthreads();

  // ---- per (query, slice): union of the four warps' candidates, bounded once more, to the list -------------
  constexpr int ENT = (CAPW + 31) / 32;
  const int out_k = a.k + kIExtra;
  const float nm_cta = fmaxf(fmaxf(nmax_w[0], nmax_w[1]), fmaxf(nmax_w[2], nmax_w[3]));
  for (int q = warp; q < kIQ; q += kIWarps) {
    if (q0 + q >= a.M) continue;
    const int64_t o = (static_cast<int64_t>(q0 + q) * a.n_slices + slice) * out_k;
    const float T0 = thr[q];
    float u[kIWarps][ENT]; int r[kIWarps][ENT]; bool live[kIWarps][ENT];
#pragma unroll
    for (int w = 0; w < kIWarps; ++w) {
      const int n_w = cnt[w][q] < CAPW ? cnt[w][q] : CAPW;
#pragma unroll
      for (int e = 0; e < ENT; ++e) {
        const int slot = lane + 32 * e;
        u[w][e] = slot < n_w ? buf_u[q * QS + w * CAPW + slot] : -INFINITY;
        r[w][e] = slot < n_w ? buf_r[q * QS + w * CAPW + slot] : 0;
        live[w][e] = slot < n_w && u[w][e] >= T0;
      }
    }
    __syncwarp();
    int total = 0;
    float* bu = buf_u + q * QS;                // the query's four buffers, as one, now hold the union
    uint16_t* br = buf_r + q * QS;
#pragma unroll
    for (int w = 0; w < kIWarps; ++w) {
#pragma unroll
      for (int e = 0; e < ENT; ++e) {
        const unsigned m = __ballot_sync(QKV_FULL_MASK, live[w][e]);
        const int dst = total + __popc(m & ((1u << lane) - 1u));
        if (live[w][e]) { bu[dst] = u[w][e]; br[dst] = static_cast<uint16_t>(r[w][e]); }
        total += __popc(m);
      }
    }
    __syncwarp();
    bool redo = T0 == INFINITY;
    int kept = 0;
    if (!redo) {
      float T, T4;
      kept = select_sorted<QS>(bu, br, total, a.k, 2.f * kEps * nm_cta, out_k, T0, 1, T, T4, lane);
      redo = kept > out_k;
    }
    if (redo) { kept = 0; if (lane == 0) a.flags[q0 + q] = 1; }
    for (int s = lane; s < out_k; s += 32) {
      a.list_scores[o + s] = s < kept ? bu[s] : -INFINITY;
      a.list_ids[o + s] = s < kept ? n_begin + br[s] : -1;       // row inside the index; the re-scoring adds id_base
    }
  }
}

// Exact fp32 score of every candidate, with the arithmetic (and order) of the CUDA-core scan kernel.
__global__ void index_rescore_kernel(const float* __restrict__ qk, int64_t n_entries, int per_query,
                                     const uint32_t* __restrict__ codes, const uint32_t* __restrict__ signs,
                                     const float* __restrict__ norms, const float* __restrict__ cent,
                                     int64_t id_base, float* __restrict__ scores, int64_t* __restrict__ ids) {
  const int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (e >= n_entries) return;
  const int64_t n = ids[e];
  if (n < 0) return;
  const float* q = qk + (e / per_query) * 256;
  const float k0 = cent[0], k1 = cent[1], k2 = cent[2], k3 = cent[3];
  float acc = 0.f;
  for (int g = 0; g < 4; ++g) {
    const uint32_t w0 = __ldg(codes + n * 8 + 2 * g), w1 = __ldg(codes + n * 8 + 2 * g + 1);
    const uint32_t sw = __ldg(signs + n * 4 + g);
#pragma unroll 8
    for (int c = 0; c < 32; ++c) {
      const uint32_t code = ((c < 16 ? w0 : w1) >> (2 * (c & 15))) & 3u;
      const float sg = ((sw >> c) & 1u) ? 1.f : -1.f;
      const int j = 32 * g + c;
      const float kc = code & 2u ? (code & 1u ? k3 : k2) : (code & 1u ? k1 : k0);
      acc = fmaf(sg, __ldg(q + 128 + j), fmaf(__ldg(q + j), kc, acc));
    }
  }
  scores[e] = acc * __ldg(norms + n);
  ids[e] = n + id_base;
}

template <int CAPW>
constexpr size_t scan_mma_smem() {
  return kIWarps * kIStages * kIStageBytes + 16 * (kIQ / 8) * 32 * 8 + static_cast<size_t>(kIWarps) * kIQ * CAPW * 6;
}

// Buffer size by k: a warp buffer keeps at most CAPW - kIRoom rows between tiles, and the list of a
// (query, slice) holds k + kIExtra rows, which must fit one buffer.
static int capw_for(int k) { return k <= 12 ? 32 : (k <= 28 ? 48 : 80); }
constexpr int kIMaxK = 48;

struct ScanMmaPlan {
  int n_slices; int64_t slice_len; int n_qtiles;
  size_t hdr_bytes, flag_bytes, qk_bytes, ls_bytes, li_bytes, fallback_bytes;
  size_t total() const { return hdr_bytes + flag_bytes + qk_bytes + ls_bytes + li_bytes + fallback_bytes; }
};

// The tcgen05 scan (index_scan_umma.cu) gives the same results and is the faster one where it applies (k <= 12);
// QUASHKV_B200_INDEX_TCGEN05=0 keeps the mma.sync scan (A/B checks, tests).
static bool scan_on_tcgen05(int k) {
  const char* e = getenv("QUASHKV_B200_INDEX_TCGEN05");
  return index_umma_ok(k) && !(e && e[0] == '0');
}

static ScanMmaPlan make_mma_plan(int64_t N, int M, int k, bool tcgen05) {
  ScanMmaPlan p;
  p.n_qtiles = tcgen05 ? index_umma_qtiles(M) : (M + kIQ - 1) / kIQ;
  const int capw = capw_for(k);
  const int ctas_per_sm = capw <= 32 ? 4 : (capw <= 48 ? 3 : 2);
  int64_t want = tcgen05 ? (2 * kNumSMs) / p.n_qtiles                             // one CTA per SM, two rounds
                         : (ctas_per_sm * kNumSMs * 2 + p.n_qtiles - 1) / p.n_qtiles;   // about two waves
  const int64_t chunk = 256;
  const int64_t max_by_len = (N + 8 * chunk - 1) / (8 * chunk);
  const int64_t min_by_len = (N + kIMaxSlice - 1) / kIMaxSlice;
  if (want > max_by_len) want = max_by_len;
  if (want < min_by_len) want = min_by_len;
  if (want < 1) want = 1;
  int64_t len = (N + want - 1) / want;
  len = (len + chunk - 1) / chunk * chunk;
  p.slice_len = len;
  p.n_slices = static_cast<int>((N + len - 1) / len);
  const size_t per = static_cast<size_t>(M) * p.n_slices * (k + kIExtra);
  p.hdr_bytes = 256;
  p.flag_bytes = 2 * ((static_cast<size_t>(M) * sizeof(int) + 255) / 256 * 256);      // flags, then the shared bounds
  p.qk_bytes = (static_cast<size_t>(M) * 256 * sizeof(float) + 255) / 256 * 256;
  p.ls_bytes = (per * sizeof(float) + 255) / 256 * 256;
  p.li_bytes = (per * sizeof(int64_t) + 255) / 256 * 256;
  p.fallback_bytes = index_flagged_list_bytes(N, M, k);
  return p;
}

bool index_mma_ok(int d, int bits, int64_t N, int k, const void* codes, const void* signs, const void* norms) {
  const uintptr_t al = reinterpret_cast<uintptr_t>(codes) | reinterpret_cast<uintptr_t>(signs) |
                       reinterpret_cast<uintptr_t>(norms);
  return d == 128 && bits == 3 && N >= 4096 && k <= kIMaxK && (al & 15u) == 0;
}

size_t index_mma_workspace_bytes(int64_t N, int M, int k) {
  const int kk = k < kIMaxK ? k : kIMaxK;
  const size_t a = make_mma_plan(N, M, kk, false).total();
  const size_t b = index_umma_ok(kk) ? make_mma_plan(N, M, kk, true).total() : 0;
  return a > b ? a : b;                      // the environment may select either kernel
}

template <int CAPW>
static int launch_scan_mma(const ScanMmaArgs& a, dim3 grid, cudaStream_t st) {
  if (cudaFuncSetAttribute(index_scan_mma_kernel<CAPW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(scan_mma_smem<CAPW>())) != cudaSuccess)
    return QKV_ELAUNCH;
  index_scan_mma_kernel<CAPW><<<grid, kIWarps * 32, scan_mma_smem<CAPW>(), st>>>(a);
  return QKV_OK;
}

// Look-up tables into the workspace header, rotate the queries, scan on the tensor cores, re-score
// the candidates, merge; then the CUDA-core scan and a second merge for the flagged queries only.
int launch_index_scan_mma(const float* queries, int M, const uint8_t* codes, const uint8_t* signs,
                          const float* norms, int64_t N, const float* Pi, const float* cent, const float* S,
                          float qjl_scale, int k, int64_t id_base, float* out_scores, int64_t* out_ids,
                          void* workspace, size_t workspace_bytes, cudaStream_t st) {
  const bool tcgen05 = scan_on_tcgen05(k);
  const ScanMmaPlan p = make_mma_plan(N, M, k, tcgen05);
  if (workspace_bytes < p.total()) return QKV_EWORKSPACE;
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  uint32_t* tables = reinterpret_cast<uint32_t*>(ws);
  int* flags = reinterpret_cast<int*>(ws + p.hdr_bytes);
  float* qk = reinterpret_cast<float*>(ws + p.hdr_bytes + p.flag_bytes);
  unsigned char* lists = ws + p.hdr_bytes + p.flag_bytes + p.qk_bytes;
  float* gthr = reinterpret_cast<float*>(ws + p.hdr_bytes + p.flag_bytes / 2);
  index_init_kernel<<<(M + 255) / 256, 256, 0, st>>>(flags, gthr, M);
  int rc = launch_rotate_with_tables(queries, QKV_F32, M, 128, Pi, S, qjl_scale, 1.f, qk, cent, cent, tables, st);
  if (rc) return rc;
  ScanMmaArgs a{};
  a.qk = qk; a.M = M; a.k = k; a.codes = codes; a.signs = signs; a.norms = norms; a.N = N;
  a.slice_len = p.slice_len; a.n_slices = p.n_slices; a.tables = tables; a.flags = flags; a.gthr = gthr;
  a.list_scores = reinterpret_cast<float*>(lists);
  a.list_ids = reinterpret_cast<int64_t*>(lists + p.ls_bytes);
  const dim3 grid(p.n_slices, p.n_qtiles);
  if (tcgen05) {
    rc = launch_index_scan_umma(a, p.n_qtiles, st);
  } else {
    switch (capw_for(k)) {
      case 32: rc = launch_scan_mma<32>(a, grid, st); break;
      case 48: rc = launch_scan_mma<48>(a, grid, st); break;
      default: rc = launch_scan_mma<80>(a, grid, st); break;
    }
  }
  if (rc) return rc;
  const int per_query = p.n_slices * (k + kIExtra);
  const int64_t entries = static_cast<int64_t>(M) * per_query;
  index_rescore_kernel<<<static_cast<unsigned>((entries + 255) / 256), 256, 0, st>>>(
      qk, entries, per_query, reinterpret_cast<const uint32_t*>(codes), reinterpret_cast<const uint32_t*>(signs),
      norms, cent, id_base, a.list_scores, a.list_ids);
  if ((rc = check_launch())) return rc;
  if ((rc = qkv_topk_merge(a.list_scores, a.list_ids, M, per_query, k, out_scores, out_ids, st))) return rc;
  return launch_scan_flagged(qk, M, k, codes, signs, norms, N, cent, id_base, flags,
                             lists + p.ls_bytes + p.li_bytes, out_scores, out_ids, st);
}

}  // namespace qkv
