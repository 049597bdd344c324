// Candidate bookkeeping shared by the tensor-core index scans (mma.sync and tcgen05): the argument
// block, the error bound of the approximate scores, and the warp-wide selection inside a candidate
// buffer.
#pragma once

#include <math.h>

#include "attention_common.cuh"
#include "mma_decode.cuh"

namespace qkv {

constexpr int kIQ = 32;                 // queries per CTA
constexpr int kIWarps = 4;
constexpr int kIStages = 3;
constexpr int kIStageBytes = 512 + 256 + 64;     // 16 rows: codes, signs, norms
constexpr int kIExtra = 16;             // list slots beyond k per (query, slice)
constexpr int kIRoom = 16;              // free slots a warp buffer must have before a tile (16 rows)
constexpr float kEps = 4e-4f;           // bound of |approximate - fp32 score| / norm for a unit query
constexpr int64_t kIMaxSlice = 65536;   // rows per slice: candidates are stored as 16-bit offsets

struct ScanMmaArgs {
  const float* qk;       // [M][2][128] rotated queries (scale 1)
  int M, k;
  const uint8_t* codes; const uint8_t* signs; const float* norms;
  int64_t N; int64_t slice_len; int n_slices;
  const uint32_t* tables;              // key table (fp16 pairs) and 1/scale
  float* list_scores; int64_t* list_ids;   // [M][n_slices][k + kIExtra]
  int* flags;                          // [M] set to 1 for queries the CUDA-core scan must redo
  float* gthr;                         // [M] lower bound of the k-th best pessimistic score over the WHOLE index
};

// Every CTA's bound for its slice is also a bound for the whole index (the global top-k can only be
// better), so the CTAs of a query share one rising bound through global memory: a slice that starts late,
// or holds no good rows, then drops almost everything at the first comparison.
__device__ __forceinline__ void publish_bound(float* g, float v) {       // atomic max of a float of either sign
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(g), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(g), __float_as_uint(v));
}

__device__ __forceinline__ bool better(float sa, int ia, float sb, int ib) {
  return sa > sb || (sa == sb && ia < ib);
}

static __global__ void index_init_kernel(int* flags, float* gthr, int M) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < M) { flags[i] = 0; gthr[i] = -INFINITY; }
}

// Raises the shared threshold to at least t (bounded retries: the threshold is only a filter).
__device__ __forceinline__ void raise_threshold(float* thr, float t) {
  int* p = reinterpret_cast<int*>(thr);
  int old = *reinterpret_cast<volatile int*>(p);
  for (int tries = 0; tries < 8 && __int_as_float(old) < t; ++tries) {
    const int seen = atomicCAS(p, old, __float_as_int(t));
    if (seen == old) break;
    old = seen;
  }
}

// Warp-wide selection inside one candidate buffer of n <= CAPW entries (optimistic score, row).
// Ranks every entry (higher score first, equal scores by slot), takes T = (k-th best) - slack
// (-inf while n < k), and rewrites the buffer as the entries with score >= T in rank order.
// Returns how many there are; only the first `limit` of them are stored.  `floor` raises T (rows below a
// bound that is already known need not be kept); T4 = (k4-th best) - slack, from before the raise.
template <int CAPW>
__device__ __forceinline__ int select_sorted(float* bu, uint16_t* br, int n, int k, float slack, int limit,
                                             float floor, int k4, float& T, float& T4, int lane) {
  constexpr int ENT = (CAPW + 31) / 32;
  float u[ENT]; int r[ENT], rank[ENT];
#pragma unroll
  for (int e = 0; e < ENT; ++e) {
    const int slot = lane + 32 * e;
    u[e] = slot < n ? bu[slot] : -INFINITY;
    r[e] = slot < n ? br[slot] : 0;
    rank[e] = 0;
  }
  for (int j = 0; j < n; ++j) {
    const float uj = bu[j];
#pragma unroll
    for (int e = 0; e < ENT; ++e) rank[e] += better(uj, j, u[e], lane + 32 * e) ? 1 : 0;
  }
  float kth = -INFINITY, k4th = -INFINITY;
#pragma unroll
  for (int e = 0; e < ENT; ++e) {
    const bool in = lane + 32 * e < n;
    const unsigned m = __ballot_sync(QKV_FULL_MASK, in && rank[e] == k - 1);
    const unsigned m4 = __ballot_sync(QKV_FULL_MASK, in && rank[e] == k4 - 1);
    const float v = __shfl_sync(QKV_FULL_MASK, u[e], m ? __ffs(m) - 1 : 0);
    const float v4 = __shfl_sync(QKV_FULL_MASK, u[e], m4 ? __ffs(m4) - 1 : 0);
    if (m) kth = v;
    if (m4) k4th = v4;
  }
  T = fmaxf(n >= k ? kth - slack : -INFINITY, floor);
  T4 = n >= k4 ? k4th - slack : -INFINITY;
  int kept = 0;
  bool keep[ENT];
#pragma unroll
  for (int e = 0; e < ENT; ++e) {
    keep[e] = lane + 32 * e < n && u[e] >= T;
    kept += __popc(__ballot_sync(QKV_FULL_MASK, keep[e]));
  }
  __syncwarp();
#pragma unroll
  for (int e = 0; e < ENT; ++e)
    if (keep[e] && rank[e] < limit) { bu[rank[e]] = u[e]; br[rank[e]] = static_cast<uint16_t>(r[e]); }
  __syncwarp();
  return kept;
}

// tcgen05 scan (index_scan_umma.cu): 64 queries per CTA, k <= 12.
bool index_umma_ok(int k);
int index_umma_qtiles(int M);
int launch_index_scan_umma(const ScanMmaArgs& a, int n_qtiles, cudaStream_t st);
unsigned int index_umma_timeouts();

}  // namespace qkv
