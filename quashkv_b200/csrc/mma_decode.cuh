// Register-level building blocks shared by the tensor-core decode attention and the tensor-core
// index scan: the fp16 m16n8k16 MMA, PRMT table look-ups, the shift-free sign-bit operands and
// the cp.async primitives.
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"

namespace qkv {

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int src_bytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }


// Sign bits become MMA operands without a per-pair shift: a masked single bit at position p of a
// 16-bit half IS an fp16 number (0 when clear, v1(p) when set: 2, 2^-7, 2^-11, 2^-13, 2^-14 and
// the subnormals 2^-15, 2^-16 for p = 14..8), so `word & mask` is the operand and the weight
// carries 2 / v1(p); the constant -sum(w) goes into the accumulator's initial value.  Bit 15 (the
// fp16 sign) cannot be used, so four copies of the word (as is, <<7, >>1, <<13) bring all 16
// bit pairs (j, j+16) to positions 8..14.  Pair t of a 32-coordinate slice:
//   t 0..6 : word,      p = 8+t,  coordinates (8+t, 24+t)      t 14: word>>1,  p = 14, (15, 31)
//   t 7..13: word<<7,   p = 1+t,  coordinates (t-6, t+10)      t 15: word<<13, p = 13, (0, 16)
__host__ __device__ constexpr int sign_pos(int t) { return t < 7 ? 8 + t : (t < 14 ? 1 + t : (t == 14 ? 14 : 13)); }
__host__ __device__ constexpr int sign_coord(int t) { return t < 7 ? 8 + t : (t < 14 ? t - 6 : (t == 14 ? 15 : 0)); }
__host__ __device__ constexpr float sign_v1(int p) {
  return p == 14 ? 2.f : (p == 13 ? 0.0078125f : (p == 12 ? 4.8828125e-4f : 1.f / static_cast<float>(1 << (24 - p))));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}


}  // namespace qkv
