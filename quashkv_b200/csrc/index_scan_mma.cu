// Tensor-core index scan for dim 128, 3 bits (2-bit codes + sign bit).
//
// score[m,n] = norm_n * (q_rot_m . c[code_n] + qjl_scale * sum |q_rot_m| S (2 sign_n - 1)) for every
// (query, database row) pair is a dense contraction whose one operand is decoded on the fly, so it
// belongs on the tensor cores: database rows are the M dimension (16 per warp tile, decoded in
// registers exactly like the keys of the decode attention), 32 queries per CTA are the N dimension
// (their fp16 high + low parts and sign weights sit in shared memory as ready B fragments), K = 256.
// The fp16 high/low split keeps the approximate score within ~1e-5 relative of the fp32 value.
//
// Exact top-k: the scan keeps, per query, every row whose approximate score is within a small
// slack of the k-th best approximate score (a superset of the true top-k), the candidates are
// re-scored with the fp32 arithmetic of the CUDA-core scan kernel, and the merge kernel picks the
// final k by exact score (ties by lower id).
#include <math.h>

#include "attention_common.cuh"
#include "mma_decode.cuh"

namespace qkv {

constexpr int kIQ = 32;                 // queries per CTA
constexpr int kIWarps = 4;
constexpr int kICap = 128;              // candidate slots per query in shared memory
constexpr int kIStages = 4;
constexpr int kIStageBytes = 512 + 256 + 64;     // 16 rows: codes, signs, norms
constexpr int kIExtra = 16;             // candidates kept beyond k per (query, slice)
constexpr float kRelSlack = 2e-4f, kAbsSlack = 1e-6f;

struct ScanMmaArgs {
  const float* qk;       // [M][2][128] rotated queries (scale 1)
  int M, k;
  const uint8_t* codes; const uint8_t* signs; const float* norms;
  int64_t N; int64_t slice_len; int n_slices;
  const uint32_t* tables;              // key table (fp16 pairs) and 1/scale
  int64_t id_base;
  float* list_scores; int64_t* list_ids;   // [M][n_slices][k + kIExtra]
};

__device__ __forceinline__ bool better(float sa, int ia, float sb, int ib) {
  return sa > sb || (sa == sb && ia < ib);
}

__global__ void __launch_bounds__(kIWarps * 32, 3) index_scan_mma_kernel(ScanMmaArgs a) {
  constexpr int D = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* ring_s = smem_raw;                                             // per-warp staging rings
  uint2 (*bop)[kIQ / 8][32] = reinterpret_cast<uint2 (*)[kIQ / 8][32]>(ring_s + kIWarps * kIStages * kIStageBytes);
  float (*buf_s)[kICap] = reinterpret_cast<float (*)[kICap]>(bop + 24);        // candidate scores per query
  int (*buf_i)[kICap] = reinterpret_cast<int (*)[kICap]>(buf_s + kIQ);          // candidate rows per query
  __shared__ float wsum[kIQ];
  __shared__ float thr[kIQ];
  __shared__ int cnt[kIQ];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int slice = blockIdx.x, q0 = blockIdx.y * kIQ;
  const float inv_sk = __uint_as_float(a.tables[6]);
  const uint32_t kt_a = a.tables[0], kt_b = a.tables[1];

  // ---- B fragments of the 32 queries (query column n = gid of n-tile nt is query q0 + 8 nt + gid) ----
  for (int nt = warp; nt < kIQ / 8; nt += kIWarps) {
    const int m = q0 + 8 * nt + gid;
    const float* q = a.qk + static_cast<int64_t>(m < a.M ? m : 0) * 2 * D;
    const float live = m < a.M ? 1.f : 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const int word = s >> 2, grp = s & 3;
      const int c0 = 32 * tig + 16 * word + grp;
      float v[4], r[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[e] = q[c0 + 4 * e] * inv_sk * live;
        r[e] = v[e] - __half2float(__float2half_rn(v[e]));
      }
      bop[s][nt][lane] = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
      bop[8 + s][nt][lane] = make_uint2(pack_half2(r[0], r[1]), pack_half2(r[2], r[3]));
      uint32_t wq[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int t = 2 * s + h, j = 32 * tig + sign_coord(t);
        const float f = 2.f / sign_v1(sign_pos(t)) * live;
        wq[h] = pack_half2(q[D + j] * f, q[D + j + 16] * f);
      }
      bop[16 + s][nt][lane] = make_uint2(wq[0], wq[1]);
    }
  }
  if (threadIdx.x < kIQ) {
    const int m = q0 + threadIdx.x;
    float t = 0.f;
    if (m < a.M)
      for (int j = 0; j < D; ++j) t += a.qk[static_cast<int64_t>(m) * 2 * D + D + j];
    wsum[threadIdx.x] = t;
    thr[threadIdx.x] = m < a.M ? -INFINITY : INFINITY;     // padding queries never collect candidates
    cnt[threadIdx.x] = 0;
  }
  __syncthreads();

  const int64_t n_begin = slice * a.slice_len;
  int64_t n_end = n_begin + a.slice_len;
  if (n_end > a.N) n_end = a.N;
  const int n_valid = static_cast<int>(n_end - n_begin);
  constexpr int kStep = kIWarps * 16;
  const int n_it = (n_valid + kStep - 1) / kStep;          // CTA passes; every warp takes one tile per pass
  const int first_rel = warp * 16;

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
          cp_async16(stage + dst_off[k], ok ? src0[k] + static_cast<int64_t>(it) * stride[k] : src0[k],
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

    float c[kIQ / 8][4];
#pragma unroll
    for (int nt = 0; nt < kIQ / 8; ++nt) {
      c[nt][0] = c[nt][2] = -wsum[8 * nt + 2 * tig];
      c[nt][1] = c[nt][3] = -wsum[8 * nt + 2 * tig + 1];
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
          const uint2 bh = bop[word * 4 + grp][nt][lane], bl = bop[8 + word * 4 + grp][nt][lane];
          mma16816(c[nt], af, bl.x, bl.y);
          mma16816(c[nt], af, bh.x, bh.y);
        }
      }
    }
    {
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
          const uint2 bw = bop[16 + s][nt][lane];
          mma16816(c[nt], af, bw.x, bw.y);
        }
      }
    }
    // ---- candidates: approximate score above the query's running threshold ------------------------------
    const int rel = first_rel + it * kStep;
#pragma unroll
    for (int nt = 0; nt < kIQ / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int q = 8 * nt + 2 * tig + (e & 1), r = rel + gid + 8 * (e >> 1);
        const float sc = c[nt][e] * kn[e >> 1];
        if (r < n_valid && sc >= thr[q]) {
          const int pos = atomicAdd(&cnt[q], 1);
          if (pos < kICap) { buf_s[q][pos] = sc; buf_i[q][pos] = r; }
        }
      }
    }
    // ---- prune the buffers that could overflow on the next pass --------------------------------------------
    __syncthreads();                               // every warp's pushes of this pass are in
    const bool need = __syncthreads_or(threadIdx.x < kIQ && cnt[threadIdx.x] > kICap - kStep);
    if (need) {
      for (int q = warp; q < kIQ; q += kIWarps) {
        int n = cnt[q] < kICap ? cnt[q] : kICap;
        if (n <= kICap - kStep) continue;
        // k-th best approximate score (k selections), then keep everything within the slack of it
        float kth = -INFINITY;
        const int kk = n < a.k ? n : a.k;
        float prev_s = INFINITY; int prev_i = -1;
        for (int sel = 0; sel < kk; ++sel) {
          float bs = -INFINITY; int bi = 0x7fffffff;
          for (int p = lane; p < n; p += 32) {
            const float s = buf_s[q][p]; const int id = buf_i[q][p];
            if ((sel == 0 || better(prev_s, prev_i, s, id)) && better(s, id, bs, bi)) { bs = s; bi = id; }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const float s2 = __shfl_xor_sync(QKV_FULL_MASK, bs, o);
            const int i2 = __shfl_xor_sync(QKV_FULL_MASK, bi, o);
            if (better(s2, i2, bs, bi)) { bs = s2; bi = i2; }
          }
          prev_s = bs; prev_i = bi; kth = bs;
        }
        const float cut = (n >= a.k) ? kth - (kRelSlack * fabsf(kth) + kAbsSlack) : -INFINITY;
        int kept = 0;
        for (int p0 = 0; p0 < n; p0 += 32) {          // stable compaction
          const int p = p0 + lane;
          const float s = p < n ? buf_s[q][p] : -INFINITY;
          const int id = p < n ? buf_i[q][p] : -1;
          const bool keep = p < n && s >= cut;
          const unsigned m = __ballot_sync(QKV_FULL_MASK, keep);
          __syncwarp();
          if (keep) {
            const int dst = kept + __popc(m & ((1u << lane) - 1u));
            if (dst < kICap - kStep) { buf_s[q][dst] = s; buf_i[q][dst] = id; }
          }
          kept += __popc(m);
          __syncwarp();
        }
        if (lane == 0) {
          cnt[q] = kept < kICap - kStep ? kept : kICap - kStep;
          thr[q] = cut;
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // ---- per (query, slice): the k + kIExtra best approximate candidates ---------------------------------------
  const int out_k = a.k + kIExtra;
  for (int q = warp; q < kIQ; q += kIWarps) {
    if (q0 + q >= a.M) continue;
    const int n = cnt[q] < kICap ? cnt[q] : kICap;
    const int64_t o = (static_cast<int64_t>(q0 + q) * a.n_slices + slice) * out_k;
    float prev_s = INFINITY; int prev_i = -1;
    for (int sel = 0; sel < out_k; ++sel) {
      float bs = -INFINITY; int bi = 0x7fffffff;
      for (int p = lane; p < n; p += 32) {
        const float s = buf_s[q][p]; const int id = buf_i[q][p];
        if ((sel == 0 || better(prev_s, prev_i, s, id)) && better(s, id, bs, bi)) { bs = s; bi = id; }
      }
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) {
        const float s2 = __shfl_xor_sync(QKV_FULL_MASK, bs, o2);
        const int i2 = __shfl_xor_sync(QKV_FULL_MASK, bi, o2);
        if (better(s2, i2, bs, bi)) { bs = s2; bi = i2; }
      }
      const bool have = bi != 0x7fffffff;
      if (lane == 0) {
        a.list_scores[o + sel] = have ? bs : -INFINITY;
        a.list_ids[o + sel] = have ? n_begin + bi : -1;       // row index inside the index (id_base added later)
      }
      prev_s = bs; prev_i = bi;
      if (!have) {
        for (int s2 = sel + 1 + lane; s2 < out_k; s2 += 32) { a.list_scores[o + s2] = -INFINITY; a.list_ids[o + s2] = -1; }
        break;
      }
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

constexpr size_t kScanMmaSmem = kIWarps * kIStages * kIStageBytes + 24 * (kIQ / 8) * 32 * 8 + 2 * kIQ * kICap * 4;

struct ScanMmaPlan { int n_slices; int64_t slice_len; int n_qtiles; size_t hdr_bytes, qk_bytes, ls_bytes, li_bytes; };

static ScanMmaPlan make_mma_plan(int64_t N, int M, int k) {
  ScanMmaPlan p;
  p.n_qtiles = (M + kIQ - 1) / kIQ;
  int64_t want = (3 * kNumSMs * 2 + p.n_qtiles - 1) / p.n_qtiles;      // ~2 waves of 3 CTAs per SM
  const int64_t chunk = 256;
  const int64_t max_by_len = (N + 8 * chunk - 1) / (8 * chunk);
  if (want > max_by_len) want = max_by_len;
  if (want < 1) want = 1;
  int64_t len = (N + want - 1) / want;
  len = (len + chunk - 1) / chunk * chunk;
  p.slice_len = len;
  p.n_slices = static_cast<int>((N + len - 1) / len);
  const size_t per = static_cast<size_t>(M) * p.n_slices * (k + kIExtra);
  p.hdr_bytes = 256;
  p.qk_bytes = (static_cast<size_t>(M) * 256 * sizeof(float) + 255) / 256 * 256;
  p.ls_bytes = (per * sizeof(float) + 255) / 256 * 256;
  p.li_bytes = per * sizeof(int64_t);
  return p;
}

bool index_mma_ok(int d, int bits, int64_t N, int k, const void* codes, const void* signs, const void* norms) {
  const uintptr_t al = reinterpret_cast<uintptr_t>(codes) | reinterpret_cast<uintptr_t>(signs) |
                       reinterpret_cast<uintptr_t>(norms);
  return d == 128 && bits == 3 && N >= 4096 && k + kIExtra <= kICap - kIWarps * 16 && (al & 15u) == 0;
}

size_t index_mma_workspace_bytes(int64_t N, int M, int k) {
  const ScanMmaPlan p = make_mma_plan(N, M, k);
  return p.hdr_bytes + p.qk_bytes + p.ls_bytes + p.li_bytes;
}

// Prepares look-up tables in the workspace header, rotates the queries, scans, re-scores, merges.
int launch_index_scan_mma(const float* queries, int M, const uint8_t* codes, const uint8_t* signs,
                          const float* norms, int64_t N, const float* Pi, const float* cent, const float* S,
                          float qjl_scale, int k, int64_t id_base, float* out_scores, int64_t* out_ids,
                          void* workspace, size_t workspace_bytes, cudaStream_t st) {
  const ScanMmaPlan p = make_mma_plan(N, M, k);
  if (workspace_bytes < p.hdr_bytes + p.qk_bytes + p.ls_bytes + p.li_bytes) return QKV_EWORKSPACE;
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  uint32_t* tables = reinterpret_cast<uint32_t*>(ws);
  float* qk = reinterpret_cast<float*>(ws + p.hdr_bytes);
  int rc = launch_rotate_with_tables(queries, QKV_F32, M, 128, Pi, S, qjl_scale, 1.f, qk, cent, cent, tables, st);
  if (rc) return rc;
  ScanMmaArgs a{};
  a.qk = qk; a.M = M; a.k = k; a.codes = codes; a.signs = signs; a.norms = norms; a.N = N;
  a.slice_len = p.slice_len; a.n_slices = p.n_slices; a.tables = tables; a.id_base = id_base;
  a.list_scores = reinterpret_cast<float*>(ws + p.hdr_bytes + p.qk_bytes);
  a.list_ids = reinterpret_cast<int64_t*>(ws + p.hdr_bytes + p.qk_bytes + p.ls_bytes);
  if (cudaFuncSetAttribute(index_scan_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kScanMmaSmem)) != cudaSuccess)
    return QKV_ELAUNCH;
  index_scan_mma_kernel<<<dim3(p.n_slices, p.n_qtiles), kIWarps * 32, kScanMmaSmem, st>>>(a);
  const int per_query = p.n_slices * (k + kIExtra);
  const int64_t entries = static_cast<int64_t>(M) * per_query;
  index_rescore_kernel<<<static_cast<unsigned>((entries + 255) / 256), 256, 0, st>>>(
      qk, entries, per_query, reinterpret_cast<const uint32_t*>(codes), reinterpret_cast<const uint32_t*>(signs),
      norms, cent, id_base, a.list_scores, a.list_ids);
  if ((rc = check_launch())) return rc;
  return qkv_topk_merge(a.list_scores, a.list_ids, M, per_query, k, out_scores, out_ids, st);
}

}  // namespace qkv
