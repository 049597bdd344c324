// Pieces shared by the tensor-core rotation kernels (mma.sync and tcgen05): the exact three-way
// bf16 split, the bucket-table classification of a rotated coordinate, and the fp32 FMA chain that
// re-derives the few coordinates lying within kRecheckEps of a decision boundary.
#pragma once

#include <cuda_bf16.h>

#include "rotate_common.cuh"

namespace qkv {

constexpr int kRD = 128;                    // dimension handled by the tensor-core rotation
constexpr float kRecheckEps = 1e-5f;
constexpr int kLutSize = 16384;
constexpr int kQueueCap = 128;

// x = h + m + l exactly, each term a bf16 (round-to-nearest at every step).
__device__ __forceinline__ void split3(float x, __nv_bfloat16& h, __nv_bfloat16& m, __nv_bfloat16& l) {
  h = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(h);
  m = __float2bfloat16_rn(r1);
  l = __float2bfloat16_rn(r1 - __bfloat162float(m));
}

__device__ __forceinline__ uint32_t pack_bf16(__nv_bfloat16 lo, __nv_bfloat16 hi) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(lo)) | (static_cast<uint32_t>(__bfloat16_as_ushort(hi)) << 16);
}

__device__ __forceinline__ int bucket_of(float y) {
  return __float_as_int(fmaf(y, 4096.f, 4096.f + 8388608.f)) & (kLutSize - 1);
}

template <int BITS>
__device__ __forceinline__ uint32_t count_bounds(const float* bnd, float y) {
  uint32_t c = 0;
#pragma unroll
  for (int b = 0; b < (1 << BITS) - 1; ++b) c += y > bnd[b] ? 1u : 0u;
  return c;
}

// Bucket table: entry k covers y in [(k - 4096.5) / 4096, (k - 4095.5) / 4096); value = code of the
// bucket's centre, | 0x80 when a boundary (or, for the sign bit, a centroid) could lie inside.
template <int BITS, bool IP>
__device__ __forceinline__ void build_bucket_lut(uint8_t* lut, const float* bnd, const float* cent) {
  constexpr int NB = (1 << BITS) - 1;
  for (int k = threadIdx.x; k < kLutSize; k += blockDim.x) {
    uint8_t v = 0x80;
    if (k <= 8192) {
      const float lo = (static_cast<float>(k) - 4096.5f) * (1.f / 4096.f);
      const float hi = (static_cast<float>(k) - 4095.5f) * (1.f / 4096.f);
      const float margin = kRecheckEps + 2e-6f;
      bool amb = false;
      for (int b = 0; b < NB; ++b) amb |= (bnd[b] >= lo - margin && bnd[b] <= hi + margin);
      if (IP)
        for (int c = 0; c <= NB; ++c) amb |= (cent[c] >= lo - margin && cent[c] <= hi + margin);
      const float mid = (static_cast<float>(k) - 4096.f) * (1.f / 4096.f);
      v = static_cast<uint8_t>(count_bounds<BITS>(bnd, mid) | (amb ? 0x80u : 0u));
    }
    lut[k] = v;
  }
}

// Rare path of the classification, kept out of line so that the inlined call sites stay small (an
// unrolled epilogue otherwise outgrows the instruction cache).  Returns code | sign << 8 | near << 16.
static __device__ __noinline__ uint32_t classify_slow(const float* bnd, const float* cent, float s_col, float y,
                                                      int nb, int ip) {
  uint32_t code = 0;
  bool near = !(fabsf(y) <= 1.5f);
  for (int b = 0; b < nb; ++b) {
    code += y > bnd[b] ? 1u : 0u;
    near |= fabsf(y - bnd[b]) < kRecheckEps;
  }
  uint32_t sign = 0;
  if (ip) {
    const float resid = y - cent[code];
    sign = (resid * s_col >= 0.f) ? 1u : 0u;
    near |= fabsf(resid) < kRecheckEps;
  }
  return code | (sign << 8) | (near ? 1u << 16 : 0u);
}

// x_unit . Pi[col] with the CUDA-core kernel's arithmetic: x/norm, fp32 FMA over ascending coordinate.
static __device__ __noinline__ float exact_chain(const CompressArgs& a, int64_t n, int col, float norm) {
  const float* prow = a.Pi + col * kRD;
  float z = 0.f;
#pragma unroll 8
  for (int j = 0; j < kRD; ++j) z = fmaf(load_float(a.x, a.x_dtype, n * a.x_pitch + j) / norm, __ldg(prow + j), z);
  return z;
}

// Same chain from scalars (a kernel that passes its argument block by reference forces the whole block
// into local memory).  The arithmetic is that of exact_chain, coordinate by coordinate in ascending order; only
// the loads differ: a 16-byte aligned bf16 or fp32 row and the row of Pi are fetched in four parts of 32
// coordinates with 16-byte loads that are in flight together.  With one load per coordinate the chain was a
// sequence of sixteen round trips to memory, and a warp that re-derives a few coordinates this way holds up its
// whole CTA at the next barrier.
static __device__ __noinline__ float exact_chain_s(const void* x, int x_dtype, int64_t x_pitch, const float* Pi,
                                                   int64_t n, int col, float norm) {
  const float* prow = Pi + col * kRD;
  float z = 0.f;
  const bool pi16 = (reinterpret_cast<uintptr_t>(Pi) & 15u) == 0;      // rows of Pi are 512 bytes apart
  if (pi16 && x_dtype == QKV_BF16 && ((reinterpret_cast<uintptr_t>(x) | (static_cast<uint64_t>(x_pitch) * 2)) & 15u) == 0) {
    const uint4* xr = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + n * x_pitch);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint4 xv[4];
      float4 pv[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) xv[k] = __ldg(xr + 4 * c + k);
#pragma unroll
      for (int k = 0; k < 8; ++k) pv[k] = __ldg(reinterpret_cast<const float4*>(prow) + 8 * c + k);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t w[4] = {xv[k].x, xv[k].y, xv[k].z, xv[k].w};
        const float4 p0 = pv[2 * k], p1 = pv[2 * k + 1];
        const float pe[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          z = fmaf(__uint_as_float(w[e] << 16) / norm, pe[2 * e], z);
          z = fmaf(__uint_as_float(w[e] & 0xFFFF0000u) / norm, pe[2 * e + 1], z);
        }
      }
    }
    return z;
  }
  if (pi16 && x_dtype == QKV_F32 && ((reinterpret_cast<uintptr_t>(x) | (static_cast<uint64_t>(x_pitch) * 4)) & 15u) == 0) {
    const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + n * x_pitch);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      float4 xv[8], pv[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        xv[k] = __ldg(xr + 8 * c + k);
        pv[k] = __ldg(reinterpret_cast<const float4*>(prow) + 8 * c + k);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        z = fmaf(xv[k].x / norm, pv[k].x, z);
        z = fmaf(xv[k].y / norm, pv[k].y, z);
        z = fmaf(xv[k].z / norm, pv[k].z, z);
        z = fmaf(xv[k].w / norm, pv[k].w, z);
      }
    }
    return z;
  }
#pragma unroll 8
  for (int j = 0; j < kRD; ++j) z = fmaf(load_float(x, x_dtype, n * x_pitch + j) / norm, __ldg(prow + j), z);
  return z;
}

}  // namespace qkv
