// Shared device/host helpers for the quashkv_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/quashkv_b200.h"

#define QKV_FULL_MASK 0xffffffffu

namespace qkv {

constexpr int kMaxD = 128;       // largest head / vector dimension of the rotation kernels
constexpr int kNumSMs = 148;     // B200

// Bytes of one packed row: whole groups of 8 fields for 3-bit codes (3 bytes per group, as
// the reference's pack_bits pads), ceil(d*w/8) otherwise.
__host__ __device__ inline int packed_row_bytes(int d, int w) {
  return w == 3 ? 3 * ((d + 7) >> 3) : (d * w + 7) >> 3;
}

__host__ __device__ inline int64_t map_row(const qkv_rows_t& r, int64_t n) {
  return (n / r.seg_len) * r.seg_stride + r.seg_off + (n % r.seg_len);
}

__device__ __forceinline__ float load_float(const void* base, int dtype, int64_t idx) {
  if (dtype == QKV_F32) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == QKV_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

__device__ __forceinline__ void store_float(void* base, int dtype, int64_t idx, float v) {
  if (dtype == QKV_F32) reinterpret_cast<float*>(base)[idx] = v;
  else if (dtype == QKV_BF16) reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
}

// One w-bit field at stream bit position `bitpos` of a packed row.
__device__ __forceinline__ uint32_t read_field(const uint8_t* row, int bitpos, int w, int row_bytes) {
  const int byte = bitpos >> 3, sh = bitpos & 7;
  uint32_t v = row[byte];
  if (sh + w > 8 && byte + 1 < row_bytes) v |= static_cast<uint32_t>(row[byte + 1]) << 8;
  return (v >> sh) & ((1u << w) - 1u);
}

// Pack 32 codes (one per lane) of width W into W little-endian words: stream bit p of the
// group is bit (p % W) of the code held by lane p / W.  Returns word `lane` on lanes < W.
template <int W>
__device__ __forceinline__ uint32_t pack32_fixed(uint32_t code, int lane) {
  uint32_t mine = 0;
#pragma unroll
  for (int k = 0; k < W; ++k) {
    const int p = 32 * k + lane;
    const uint32_t c = __shfl_sync(QKV_FULL_MASK, code, p / W);
    const uint32_t word = __ballot_sync(QKV_FULL_MASK, (c >> (p % W)) & 1u);
    if (lane == k) mine = word;
  }
  return mine;
}

__device__ __forceinline__ uint32_t pack32(uint32_t code, int w, int lane) {
  switch (w) {
    case 1: return pack32_fixed<1>(code, lane);
    case 2: return pack32_fixed<2>(code, lane);
    case 3: return pack32_fixed<3>(code, lane);
    default: return pack32_fixed<4>(code, lane);
  }
}

// Store the words produced by pack32 at row + byte_off, never touching bytes >= byte_end.
__device__ __forceinline__ void store_packed_words(uint32_t mine, int w, uint8_t* row, int byte_off,
                                                   int byte_end, int lane) {
  if (lane >= w) return;
  const int off = byte_off + 4 * lane;
  uint8_t* p = row + off;
  if (off + 4 <= byte_end && (reinterpret_cast<uintptr_t>(p) & 3u) == 0) {
    *reinterpret_cast<uint32_t*>(p) = mine;
  } else {
#pragma unroll
    for (int b = 0; b < 4; ++b)
      if (off + b < byte_end) p[b] = static_cast<uint8_t>(mine >> (8 * b));
  }
}

// q_rot = q @ Pi^T per row; writes [row][0][d] = q_rot*scale and
// [row][1][d] = qjl_scale*scale*|q_rot|*S.  Defined in attention.cu.
int launch_rotate_queries(const void* q, int q_dtype, int64_t rows, int d, const float* Pi, const float* S,
                          float qjl_scale, float scale, float* qk, cudaStream_t st);

// Same, with one extra CTA that builds the fp16 look-up tables of the tensor-core kernels (8 words
// at `tables`, see prepare_tables_cta) from the key / value centroids.  Defined in attention.cu.
int launch_rotate_with_tables(const void* q, int q_dtype, int64_t rows, int d, const float* Pi, const float* S,
                              float qjl_scale, float scale, float* qk, const float* kcent, const float* vcent,
                              uint32_t* tables, cudaStream_t st);

// Tensor-core index scan (index_scan_mma.cu).
bool index_mma_ok(int d, int bits, int64_t N, int k, const void* codes, const void* signs, const void* norms);
size_t index_mma_workspace_bytes(int64_t N, int M, int k);
int launch_index_scan_mma(const float* queries, int M, const uint8_t* codes, const uint8_t* signs,
                          const float* norms, int64_t N, const float* Pi, const float* cent, const float* S,
                          float qjl_scale, int k, int64_t id_base, float* out_scores, int64_t* out_ids,
                          void* workspace, size_t workspace_bytes, cudaStream_t st);

// CUDA-core scan + merge of exactly the queries whose flag is set (index_scan.cu); `lists` needs
// index_flagged_list_bytes().  Results of the other queries in out_scores / out_ids stay as they are.
size_t index_flagged_list_bytes(int64_t N, int M, int k);
int launch_scan_flagged(const float* qk, int M, int k, const uint8_t* codes, const uint8_t* signs,
                        const float* norms, int64_t N, const float* cent, int64_t id_base, const int* flags,
                        void* lists, float* out_scores, int64_t* out_ids, cudaStream_t st);

inline int check_launch() { return cudaGetLastError() == cudaSuccess ? QKV_OK : QKV_ELAUNCH; }

}  // namespace qkv
