// Declarations shared by the generic and the tensor-core attention kernels.
#pragma once

#include "common.cuh"

namespace qkv {

constexpr int kQT = 4;          // query rows per CTA
constexpr int kAttnWarps = 4;
constexpr int kMaxSplits = 64;

struct AttnArgs {
  qkv_cache_t cache;
  int B, Hq, Hkv, G, q_len, d, causal;
  int64_t kv_len;
  const float* qk;      // [rows][2][d]
  const float* kcent; const float* vcent;
  float* part;          // [rows][n_splits][d+2]
  const uint32_t* tables;   // tensor-core path: fp16 look-up tables and their scales (8 words)
  int n_splits; int64_t split_len;
};

constexpr size_t kAttnHeaderBytes = 256;   // workspace header: look-up tables of the tensor-core path

struct AttnPlan { int n_splits; int64_t split_len; int n_qtiles; int64_t rows; size_t qk_bytes, part_bytes; };

inline AttnPlan make_plan(int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d) {
  AttnPlan p;
  const int G = Hq / (Hkv > 0 ? Hkv : 1);
  const int nq = G * q_len;
  p.n_qtiles = (nq + kQT - 1) / kQT;
  p.rows = static_cast<int64_t>(B) * Hq * q_len;
  (void)d;
  const int64_t chunk = 128;   // a multiple of every kernel's tokens per CTA pass (32..128)
  const int64_t ctas = static_cast<int64_t>(B) * Hkv * p.n_qtiles;
  int64_t want = (8 * kNumSMs + ctas - 1) / (ctas > 0 ? ctas : 1);
  const int64_t max_by_len = (kv_len + 4 * chunk - 1) / (4 * chunk);
  if (want > max_by_len) want = max_by_len;
  if (want > kMaxSplits) want = kMaxSplits;
  if (want < 1) want = 1;
  int64_t len = (kv_len + want - 1) / want;
  len = (len + chunk - 1) / chunk * chunk;
  if (len < chunk) len = chunk;
  p.split_len = len;
  p.n_splits = static_cast<int>((kv_len + len - 1) / len);
  if (p.n_splits < 1) p.n_splits = 1;
  p.qk_bytes = static_cast<size_t>(p.rows) * 2 * d * sizeof(float);
  p.qk_bytes = (p.qk_bytes + 255) / 256 * 256;
  p.part_bytes = static_cast<size_t>(p.rows) * p.n_splits * (d + 2) * sizeof(float);
  return p;
}


// Tensor-core decode path (attention_mma.cu): usable when mma_path_ok() holds.
bool mma_path_ok(int d, int key_bits, int val_bits, int group, int q_len);
int launch_attend_mma(const AttnArgs& a, cudaStream_t st);
// Fills the 8-word table block: centroids scaled by a factor in [1,2) chosen so that all of them
// round to fp16 with the smallest relative error, split into low / high byte tables for PRMT.
int launch_prepare_tables(const float* kcent, const float* vcent, uint32_t* tables, cudaStream_t st);

}  // namespace qkv
