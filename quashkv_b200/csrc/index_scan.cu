// Packed-code inner-product scan with a fused top-k, and the candidate-list merge.
//
// scan: grid (database slice, query tile of 16).  The tile's rotated queries sit in shared
// memory; each thread owns one database row per pass (256 rows per CTA pass), decodes every
// coordinate once and feeds 16 query accumulators.  A score above the query's running
// threshold is appended to that query's candidate buffer in shared memory; when a buffer
// could overflow on the next pass a warp prunes it to the best k and raises the threshold.
// Each (slice, query) ends with a sorted list of k candidates in the workspace, and the
// merge kernel reduces the lists of all slices to the final k.
//
// Order everywhere: higher score first, equal scores by lower id.
#include <math.h>
#include <stdlib.h>

#include "common.cuh"

namespace qkv {

constexpr int kMQ = 16;              // queries per CTA
constexpr int kScanThreads = 256;
constexpr int kCap = kScanThreads + QKV_INDEX_MAX_K;   // candidate slots per query

struct ScanArgs {
  const float* qk;       // [M][2][d] rotated queries (scale 1)
  int M, d, k;
  const uint32_t* codes; const uint32_t* signs; const float* norms;
  int64_t N; int64_t slice_len; int n_slices;
  const float* cent;
  int64_t id_base;
  float* list_scores; int64_t* list_ids;    // [M][n_slices*k]
  float* dense;                             // [M][N] when DENSE
  const int* qlist;                         // when set: scan queries qlist[0 .. qlist[M]) only, lists in that order
};

struct ScanPlan { int n_slices; int64_t slice_len; int n_qtiles; size_t qk_bytes, ls_bytes, li_bytes; };

static ScanPlan make_scan_plan(int64_t N, int M, int d, int k) {
  ScanPlan p;
  p.n_qtiles = (M + kMQ - 1) / kMQ;
  int64_t want = (4 * kNumSMs + p.n_qtiles - 1) / p.n_qtiles;
  const int64_t max_by_len = (N + 4 * kScanThreads - 1) / (4 * kScanThreads);
  if (want > max_by_len) want = max_by_len;
  if (want < 1) want = 1;
  int64_t len = (N + want - 1) / want;
  len = (len + kScanThreads - 1) / kScanThreads * kScanThreads;
  p.slice_len = len;
  p.n_slices = static_cast<int>((N + len - 1) / len);
  p.qk_bytes = (static_cast<size_t>(M) * 2 * d * sizeof(float) + 255) / 256 * 256;
  p.ls_bytes = (static_cast<size_t>(M) * p.n_slices * k * sizeof(float) + 255) / 256 * 256;
  p.li_bytes = static_cast<size_t>(M) * p.n_slices * k * sizeof(int64_t);
  return p;
}

__device__ __forceinline__ bool ranks_before(float sa, int64_t ia, float sb, int64_t ib) {
  return sa > sb || (sa == sb && ia < ib);
}

// Warp-wide: keep the best k of cnt candidates at the front of (bs, bi), sorted.
__device__ void prune_warp(float* bs, int* bi, int cnt, int k, float* ts, int* ti, int lane) {
  const int keep = cnt < k ? cnt : k;
  for (int r = 0; r < keep; ++r) {
    float best = -INFINITY; int best_id = 0x7fffffff, best_pos = -1;
    for (int p = lane; p < cnt; p += 32) {
      const float s = bs[p]; const int id = bi[p];
      if (id >= 0 && (best_pos < 0 || ranks_before(s, id, best, best_id))) { best = s; best_id = id; best_pos = p; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float s2 = __shfl_xor_sync(QKV_FULL_MASK, best, o);
      const int i2 = __shfl_xor_sync(QKV_FULL_MASK, best_id, o);
      const int p2 = __shfl_xor_sync(QKV_FULL_MASK, best_pos, o);
      if (p2 >= 0 && (best_pos < 0 || ranks_before(s2, i2, best, best_id))) { best = s2; best_id = i2; best_pos = p2; }
    }
    if (lane == 0) { ts[r] = best; ti[r] = best_id; bi[best_pos] = -1; }
    __syncwarp();
  }
  for (int r = lane; r < keep; r += 32) { bs[r] = ts[r]; bi[r] = ti[r]; }
  __syncwarp();
}

template <int WK, bool DENSE>
__global__ void __launch_bounds__(kScanThreads) index_scan_kernel(ScanArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int d = a.d;
  float4* qa = reinterpret_cast<float4*>(smem_raw);            // [d][4]
  float4* wa = qa + d * 4;                                       // [d][4]
  float* buf_s = reinterpret_cast<float*>(wa + d * 4);          // [kMQ][kCap]
  int* buf_i = reinterpret_cast<int*>(buf_s + kMQ * kCap);      // [kMQ][kCap]
  float* tmp_s = reinterpret_cast<float*>(buf_i + kMQ * kCap);  // [8][MAX_K]
  int* tmp_i = reinterpret_cast<int*>(tmp_s + 8 * QKV_INDEX_MAX_K);
  __shared__ float kc_s[16];
  __shared__ int cnt[kMQ];
  __shared__ float thr[kMQ];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slice = blockIdx.x, q0 = blockIdx.y * kMQ;
  const int n_q = a.qlist ? a.qlist[a.M] : a.M;      // queries to scan (a compacted list, or all of them)
  if (q0 >= n_q) return;                             // CTA-uniform

  for (int idx = threadIdx.x; idx < d * kMQ; idx += blockDim.x) {
    const int j = idx / kMQ, q = idx % kMQ;
    const bool ok = q0 + q < n_q;
    const int64_t qi = ok ? (a.qlist ? a.qlist[q0 + q] : q0 + q) : 0;
    reinterpret_cast<float*>(qa)[idx] = ok ? a.qk[qi * 2 * d + j] : 0.f;
    reinterpret_cast<float*>(wa)[idx] = ok ? a.qk[qi * 2 * d + d + j] : 0.f;
  }
  if (threadIdx.x < 16) kc_s[threadIdx.x] = threadIdx.x < (1 << WK) ? a.cent[threadIdx.x] : 0.f;
  if (threadIdx.x < kMQ) { cnt[threadIdx.x] = 0; thr[threadIdx.x] = -INFINITY; }
  __syncthreads();

  const int groups = d >> 5;
  const int words_k = groups * WK;
  const int64_t n_begin = slice * a.slice_len;
  int64_t n_end = n_begin + a.slice_len;
  if (n_end > a.N) n_end = a.N;

  for (int64_t base = n_begin; base < n_end; base += kScanThreads) {
    const int64_t n = base + threadIdx.x;
    const bool live = n < n_end;
    float acc[kMQ];
#pragma unroll
    for (int q = 0; q < kMQ; ++q) acc[q] = 0.f;
    if (live) {
      for (int g = 0; g < groups; ++g) {
        uint32_t kw[WK];
#pragma unroll
        for (int i = 0; i < WK; ++i) kw[i] = __ldg(a.codes + n * words_k + g * WK + i);
        const uint32_t sw = __ldg(a.signs + n * groups + g);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int bit = c * WK, wi = bit >> 5, sh = bit & 31;
          uint32_t code = kw[wi] >> sh;
          if (sh + WK > 32) code |= kw[(wi + 1 < WK) ? wi + 1 : wi] << (32 - sh);
          code &= (1u << WK) - 1u;
          const float kc = kc_s[code];
          const float sg = ((sw >> c) & 1u) ? 1.f : -1.f;
          const int j = g * 32 + c;
#pragma unroll
          for (int q4 = 0; q4 < kMQ / 4; ++q4) {
            const float4 qv = qa[j * 4 + q4];
            const float4 wv = wa[j * 4 + q4];
            acc[4 * q4 + 0] = fmaf(sg, wv.x, fmaf(qv.x, kc, acc[4 * q4 + 0]));
            acc[4 * q4 + 1] = fmaf(sg, wv.y, fmaf(qv.y, kc, acc[4 * q4 + 1]));
            acc[4 * q4 + 2] = fmaf(sg, wv.z, fmaf(qv.z, kc, acc[4 * q4 + 2]));
            acc[4 * q4 + 3] = fmaf(sg, wv.w, fmaf(qv.w, kc, acc[4 * q4 + 3]));
          }
        }
      }
      const float nrm = __ldg(a.norms + n);
#pragma unroll
      for (int q = 0; q < kMQ; ++q) acc[q] *= nrm;
    }
    if (DENSE) {
      if (live) {
#pragma unroll
        for (int q = 0; q < kMQ; ++q)
          if (q0 + q < a.M) a.dense[static_cast<int64_t>(q0 + q) * a.N + n] = acc[q];
      }
      continue;
    }
    if (live) {
      const int local = static_cast<int>(n - n_begin);
#pragma unroll
      for (int q = 0; q < kMQ; ++q) {
        if (acc[q] > thr[q]) {
          const int pos = atomicAdd(&cnt[q], 1);
          buf_s[q * kCap + pos] = acc[q];
          buf_i[q * kCap + pos] = local;
        }
      }
    }
    __syncthreads();
    for (int q = warp; q < kMQ; q += kScanThreads / 32) {
      const int c = cnt[q];
      if (c > kCap - kScanThreads) {
        prune_warp(buf_s + q * kCap, buf_i + q * kCap, c, a.k, tmp_s + warp * QKV_INDEX_MAX_K,
                   tmp_i + warp * QKV_INDEX_MAX_K, lane);
        if (lane == 0) {
          const int keep = c < a.k ? c : a.k;
          cnt[q] = keep;
          thr[q] = keep >= a.k ? buf_s[q * kCap + a.k - 1] : -INFINITY;
        }
      }
    }
    __syncthreads();
  }
  if (DENSE) return;

  for (int q = warp; q < kMQ; q += kScanThreads / 32) {
    if (q0 + q >= n_q) continue;
    const int c = cnt[q];
    prune_warp(buf_s + q * kCap, buf_i + q * kCap, c, a.k, tmp_s + warp * QKV_INDEX_MAX_K,
               tmp_i + warp * QKV_INDEX_MAX_K, lane);
    const int keep = c < a.k ? c : a.k;
    const int64_t o = (static_cast<int64_t>(q0 + q) * a.n_slices + slice) * a.k;
    for (int r = lane; r < a.k; r += 32) {
      a.list_scores[o + r] = r < keep ? buf_s[q * kCap + r] : -INFINITY;
      a.list_ids[o + r] = r < keep ? a.id_base + n_begin + buf_i[q * kCap + r] : -1;
    }
  }
}

// Warp-wide: the k best of n candidates, in rank order, to (os, oi); the r-th output is the best candidate
// that ranks after output r-1.  Missing results are (-inf, -1).
__device__ void warp_topk(const float* s, const int64_t* ids, int64_t n, int k, float* os, int64_t* oi, int lane) {
  float prev_s = INFINITY; int64_t prev_i = -1; bool have_prev = false;
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY; int64_t best_i = -1; bool have = false;
    for (int64_t p = lane; p < n; p += 32) {
      const float v = s[p]; const int64_t id = ids[p];
      if (id < 0) continue;
      if (have_prev && !ranks_before(prev_s, prev_i, v, id)) continue;
      if (!have || ranks_before(v, id, best, best_i)) { best = v; best_i = id; have = true; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float v2 = __shfl_xor_sync(QKV_FULL_MASK, best, o);
      const int64_t i2 = __shfl_xor_sync(QKV_FULL_MASK, best_i, o);
      const int h2 = __shfl_xor_sync(QKV_FULL_MASK, static_cast<int>(have), o);
      if (h2 && (!have || ranks_before(v2, i2, best, best_i))) { best = v2; best_i = i2; have = true; }
    }
    if (lane == 0) { os[r] = have ? best : -INFINITY; oi[r] = have ? best_i : -1; }
    if (!have) {
      for (int r2 = r + 1 + lane; r2 < k; r2 += 32) { os[r2] = -INFINITY; oi[r2] = -1; }
      break;
    }
    prev_s = best; prev_i = best_i; have_prev = true;
  }
}

// One warp per query.
__global__ void topk_merge_kernel(const float* __restrict__ in_s, const int64_t* __restrict__ in_i, int M,
                                  int64_t n_cand, int k_out, float* __restrict__ out_s,
                                  int64_t* __restrict__ out_i, const int* __restrict__ qlist) {
  const int lane = threadIdx.x & 31;
  const int mc = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);      // position in the input lists
  if (mc >= (qlist ? qlist[M] : M)) return;
  const int m = qlist ? qlist[mc] : mc;                                     // query whose result this is
  warp_topk(in_s + static_cast<int64_t>(mc) * n_cand, in_i + static_cast<int64_t>(mc) * n_cand, n_cand, k_out,
            out_s + static_cast<int64_t>(m) * k_out, out_i + static_cast<int64_t>(m) * k_out, lane);
}

// Long candidate lists (few queries, many slices): one CTA of eight warps per query.  Every warp reduces an
// eighth of the list to its k best in shared memory, then the first warp merges those 8 k.
constexpr int kWideWarps = 8;
__global__ void __launch_bounds__(kWideWarps * 32)
topk_merge_wide_kernel(const float* __restrict__ in_s, const int64_t* __restrict__ in_i, int M, int64_t n_cand,
                       int k_out, float* __restrict__ out_s, int64_t* __restrict__ out_i,
                       const int* __restrict__ qlist) {
  __shared__ float part_s[kWideWarps * QKV_INDEX_MAX_K];
  __shared__ int64_t part_i[kWideWarps * QKV_INDEX_MAX_K];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int mc = blockIdx.x;
  if (mc >= (qlist ? qlist[M] : M)) return;                                 // CTA-uniform
  const int m = qlist ? qlist[mc] : mc;
  const int64_t chunk = (n_cand + kWideWarps - 1) / kWideWarps;
  const int64_t lo = warp * chunk, hi = lo + chunk < n_cand ? lo + chunk : n_cand;
  warp_topk(in_s + static_cast<int64_t>(mc) * n_cand + lo, in_i + static_cast<int64_t>(mc) * n_cand + lo,
            hi > lo ? hi - lo : 0, k_out, part_s + warp * k_out, part_i + warp * k_out, lane);
  __syncthreads();
  if (warp == 0)
    warp_topk(part_s, part_i, kWideWarps * k_out, k_out, out_s + static_cast<int64_t>(m) * k_out,
              out_i + static_cast<int64_t>(m) * k_out, lane);
}

static void launch_topk_merge(const float* in_s, const int64_t* in_i, int M, int64_t n_cand, int k_out,
                              float* out_s, int64_t* out_i, const int* qlist, cudaStream_t st) {
  if (n_cand >= 2048 && k_out <= QKV_INDEX_MAX_K) {
    topk_merge_wide_kernel<<<M, kWideWarps * 32, 0, st>>>(in_s, in_i, M, n_cand, k_out, out_s, out_i, qlist);
  } else {
    const int warps = 4;
    topk_merge_kernel<<<(M + warps - 1) / warps, warps * 32, 0, st>>>(in_s, in_i, M, n_cand, k_out, out_s, out_i,
                                                                       qlist);
  }
}

static size_t scan_smem_bytes(int d) {
  return static_cast<size_t>(d) * 4 * 16 * 2 + static_cast<size_t>(kMQ) * kCap * 8 +
         8 * QKV_INDEX_MAX_K * 8;
}

template <bool DENSE>
static int launch_scan(const ScanArgs& a, int wk, dim3 grid, cudaStream_t st) {
  const size_t smem = scan_smem_bytes(a.d);
#define QKV_SCAN(W)                                                                                      \
  do {                                                                                                   \
    if (cudaFuncSetAttribute(index_scan_kernel<W, DENSE>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                             (int)smem) != cudaSuccess) return QKV_ELAUNCH;                              \
    index_scan_kernel<W, DENSE><<<grid, kScanThreads, smem, st>>>(a);                                    \
  } while (0)
  switch (wk) {
    case 1: QKV_SCAN(1); break;
    case 2: QKV_SCAN(2); break;
    default: QKV_SCAN(3); break;
  }
#undef QKV_SCAN
  return check_launch();
}

static int check_scan(const float* queries, int M, int d, const uint8_t* c, const uint8_t* s, const float* n,
                      int64_t N, int bits, const float* Pi, const float* cent, const float* S, void* ws) {
  if (!queries || !c || !s || !n || !Pi || !cent || !S || !ws) return QKV_ENULL;
  if (d < 32 || d > kMaxD || (d & 31) || M < 1 || N < 1 || N > 0x7fffffff) return QKV_EDIM;
  if (bits < 2 || bits > 4) return QKV_EBITS;
  if ((reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(ws)) & 3u)
    return QKV_EALIGN;
  return QKV_OK;
}

// Flagged queries in ascending order at list[0 ..), their number at list[M] (one CTA, block-wide scan).
__global__ void compact_flags_kernel(const int* __restrict__ flags, int M, int* __restrict__ list) {
  __shared__ int warp_tot[32];
  __shared__ int base_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base_s = 0;
  __syncthreads();
  for (int m0 = 0; m0 < M; m0 += blockDim.x) {
    const int m = m0 + threadIdx.x;
    const bool f = m < M && flags[m] != 0;
    const unsigned bal = __ballot_sync(QKV_FULL_MASK, f);
    if (lane == 0) warp_tot[warp] = __popc(bal);
    __syncthreads();
    int before = base_s;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (f) list[before + __popc(bal & ((1u << lane) - 1u))] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = 0;
      for (int w = 0; w < (blockDim.x >> 5); ++w) t += warp_tot[w];
      base_s += t;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) list[M] = base_s;
}

static size_t flagged_qlist_bytes(int M) { return (static_cast<size_t>(M + 1) * sizeof(int) + 255) / 256 * 256; }

size_t index_flagged_list_bytes(int64_t N, int M, int k) {
  const ScanPlan p = make_scan_plan(N, M, 128, k);
  return p.ls_bytes + (p.li_bytes + 255) / 256 * 256 + flagged_qlist_bytes(M);
}

int launch_scan_flagged(const float* qk, int M, int k, const uint8_t* codes, const uint8_t* signs,
                        const float* norms, int64_t N, const float* cent, int64_t id_base, const int* flags,
                        void* lists, float* out_scores, int64_t* out_ids, cudaStream_t st) {
  const ScanPlan p = make_scan_plan(N, M, 128, k);
  ScanArgs a{};
  a.qk = qk; a.M = M; a.d = 128; a.k = k;
  a.codes = reinterpret_cast<const uint32_t*>(codes); a.signs = reinterpret_cast<const uint32_t*>(signs);
  a.norms = norms; a.N = N; a.slice_len = p.slice_len; a.n_slices = p.n_slices; a.cent = cent;
  a.id_base = id_base;
  unsigned char* lp = reinterpret_cast<unsigned char*>(lists);
  a.list_scores = reinterpret_cast<float*>(lp);
  a.list_ids = reinterpret_cast<int64_t*>(lp + p.ls_bytes);
  int* qlist = reinterpret_cast<int*>(lp + p.ls_bytes + (p.li_bytes + 255) / 256 * 256);
  a.qlist = qlist;
  // The flagged queries are gathered into a dense list first, so that F of them cost ceil(F / 16) query tiles
  // of the scan instead of up to F; the grid covers the worst case and CTAs beyond the list return at once.
  compact_flags_kernel<<<1, 1024, 0, st>>>(flags, M, qlist);
  const int rc = launch_scan<false>(a, 2, dim3(p.n_slices, p.n_qtiles), st);
  if (rc) return rc;
  launch_topk_merge(a.list_scores, a.list_ids, M, static_cast<int64_t>(p.n_slices) * k, k, out_scores, out_ids, qlist,
                    st);
  return check_launch();
}

}  // namespace qkv

using namespace qkv;

extern "C" size_t qkv_index_workspace_bytes(int64_t N, int M, int d, int k) {
  if (N < 1 || M < 1 || d < 32 || k < 1) return 0;
  const ScanPlan p = make_scan_plan(N, M, d, k);
  const size_t generic = p.qk_bytes + p.ls_bytes + p.li_bytes;
  const size_t mma = (d == 128 && k <= QKV_INDEX_MAX_K) ? index_mma_workspace_bytes(N, M, k) : 0;
  return generic > mma ? generic : mma;      // either path may be taken, depending on bits and alignment
}

extern "C" int qkv_index_scan_topk(const float* queries, int M, int d,
                                   const uint8_t* db_codes, const uint8_t* db_signs, const float* db_norms,
                                   int64_t N, int bits,
                                   const float* Pi, const float* centroids, const float* S, float qjl_scale,
                                   int k, int64_t id_base, float* out_scores, int64_t* out_ids,
                                   void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_scan(queries, M, d, db_codes, db_signs, db_norms, N, bits, Pi, centroids, S, workspace);
  if (rc) return rc;
  if (!out_scores || !out_ids) return QKV_ENULL;
  if (k < 1 || k > QKV_INDEX_MAX_K || k > N) return QKV_EARG;
  {   // QUASHKV_B200_CUDA_CORE_SCAN=1 keeps the fp32 CUDA-core scan (for A/B checks)
    const char* env = getenv("QUASHKV_B200_CUDA_CORE_SCAN");
    if (!(env && env[0] == '1') && index_mma_ok(d, bits, N, k, db_codes, db_signs, db_norms))
      return launch_index_scan_mma(queries, M, db_codes, db_signs, db_norms, N, Pi, centroids, S, qjl_scale, k,
                                   id_base, out_scores, out_ids, workspace, workspace_bytes,
                                   static_cast<cudaStream_t>(stream));
  }
  const ScanPlan p = make_scan_plan(N, M, d, k);
  if (workspace_bytes < p.qk_bytes + p.ls_bytes + p.li_bytes) return QKV_EWORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  float* qk = reinterpret_cast<float*>(ws);
  if ((rc = launch_rotate_queries(queries, QKV_F32, M, d, Pi, S, qjl_scale, 1.f, qk, st))) return rc;
  ScanArgs a{};
  a.qk = qk; a.M = M; a.d = d; a.k = k;
  a.codes = reinterpret_cast<const uint32_t*>(db_codes); a.signs = reinterpret_cast<const uint32_t*>(db_signs);
  a.norms = db_norms; a.N = N; a.slice_len = p.slice_len; a.n_slices = p.n_slices; a.cent = centroids;
  a.id_base = id_base;
  a.list_scores = reinterpret_cast<float*>(ws + p.qk_bytes);
  a.list_ids = reinterpret_cast<int64_t*>(ws + p.qk_bytes + p.ls_bytes);
  if ((rc = launch_scan<false>(a, bits - 1, dim3(p.n_slices, p.n_qtiles), st))) return rc;
  return qkv_topk_merge(a.list_scores, a.list_ids, M, static_cast<int64_t>(p.n_slices) * k, k, out_scores,
                        out_ids, stream);
}

extern "C" int qkv_index_scores(const float* queries, int M, int d,
                                const uint8_t* db_codes, const uint8_t* db_signs, const float* db_norms,
                                int64_t N, int bits,
                                const float* Pi, const float* centroids, const float* S, float qjl_scale,
                                float* out_scores, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_scan(queries, M, d, db_codes, db_signs, db_norms, N, bits, Pi, centroids, S, workspace);
  if (rc) return rc;
  if (!out_scores) return QKV_ENULL;
  const ScanPlan p = make_scan_plan(N, M, d, 1);
  if (workspace_bytes < p.qk_bytes) return QKV_EWORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* qk = reinterpret_cast<float*>(workspace);
  if ((rc = launch_rotate_queries(queries, QKV_F32, M, d, Pi, S, qjl_scale, 1.f, qk, st))) return rc;
  ScanArgs a{};
  a.qk = qk; a.M = M; a.d = d; a.k = 1;
  a.codes = reinterpret_cast<const uint32_t*>(db_codes); a.signs = reinterpret_cast<const uint32_t*>(db_signs);
  a.norms = db_norms; a.N = N; a.slice_len = p.slice_len; a.n_slices = p.n_slices; a.cent = centroids;
  a.dense = out_scores;
  return launch_scan<true>(a, bits - 1, dim3(p.n_slices, p.n_qtiles), st);
}

extern "C" int qkv_topk_merge(const float* in_scores, const int64_t* in_ids, int M, int64_t n_cand,
                              int k_out, float* out_scores, int64_t* out_ids, void* stream) {
  if (!in_scores || !in_ids || !out_scores || !out_ids) return QKV_ENULL;
  if (M < 1 || n_cand < 1 || k_out < 1) return QKV_EDIM;
  launch_topk_merge(in_scores, in_ids, M, n_cand, k_out, out_scores, out_ids, nullptr,
                    static_cast<cudaStream_t>(stream));
  return check_launch();
}
