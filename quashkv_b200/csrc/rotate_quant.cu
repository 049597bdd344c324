// Compress (normalise -> rotate -> bucketise -> sign bit -> pack) and decompress
// (unpack -> centroid gather -> un-rotate -> rescale) kernels, fp32 CUDA-core rotation.
//
// One CTA keeps the (transposed or plain) rotation matrix in shared memory and loops over
// tiles of 64 vectors; each warp rotates 8 vectors at once with every lane owning the
// output coordinates lane, lane+32, ... so that the matrix row reads are conflict free and
// every matrix element fetched from shared memory feeds 8 FMAs.  The dot products
// accumulate in fp32 with FMA in ascending input-coordinate order.
#include <stdlib.h>

#include "rotate_common.cuh"

namespace qkv {

constexpr int kWarps = 8;       // warps per CTA
constexpr int kVPW = 8;         // vectors rotated together by one warp
constexpr int kThreads = kWarps * 32;

// Shared-memory carve-up common to both kernels.
//   mat   [d][DP]            fp32   (DP = 32*NT)
//   stage [kWarps][d*kVPW]   fp32   per-warp: vector values, later permuted codes
//   tab   [2][16]            fp32   boundaries or centroids of table 0 / 1
//   cent  [2][16], sgn [128] fp32   centroids of table 0 / 1 (sign stage)
//   slot  [128] int16, outl [128] uint8
struct Smem {
  float* mat; float* stage; float* tab; float* cent; float* sgn; int16_t* slot; uint8_t* outl;
};

__device__ __forceinline__ Smem carve(unsigned char* raw, int d, int DP) {
  Smem s;
  s.mat = reinterpret_cast<float*>(raw);
  s.stage = s.mat + static_cast<size_t>(d) * DP;
  s.tab = s.stage + static_cast<size_t>(kWarps) * d * kVPW;
  s.cent = s.tab + 32;
  s.sgn = s.cent + 32;
  s.slot = reinterpret_cast<int16_t*>(s.sgn + kMaxD);
  s.outl = reinterpret_cast<uint8_t*>(s.slot + kMaxD);
  return s;
}

static size_t smem_bytes(int d, int NT) {
  const size_t DP = 32 * NT;
  return (static_cast<size_t>(d) * DP + static_cast<size_t>(kWarps) * d * kVPW + 32 + 32 + kMaxD) * 4 +
         kMaxD * 2 + kMaxD;
}

// Position of every channel in the mixed packed row: outlier channels first (in channel
// order), then the regular ones.  slot[i] = rank; returns the number of outlier channels.
__device__ __forceinline__ void build_slots(const Smem& s, const uint8_t* is_outlier, int d) {
  for (int i = threadIdx.x; i < d; i += blockDim.x) s.outl[i] = is_outlier ? (is_outlier[i] != 0) : 0;
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    int n_out_total = 0, rank = 0;
    for (int j = 0; j < d; ++j) {
      n_out_total += s.outl[j];
      if (j < i && s.outl[j] == s.outl[i]) ++rank;
    }
    s.slot[i] = static_cast<int16_t>(s.outl[i] ? rank : n_out_total + rank);
  }
}

__device__ __forceinline__ int count_outliers(const Smem& s, int d) {
  int n = 0;
  for (int j = 0; j < d; ++j) n += s.outl[j];
  return n;
}

// acc[v][t] += sum_j stage[j][v] * mat[j][lane + 32 t]
template <int NT>
__device__ __forceinline__ void rotate8(const float* __restrict__ mat, const float* __restrict__ stage,
                                        int d, int DP, int lane, float (&acc)[kVPW][NT]) {
#pragma unroll
  for (int v = 0; v < kVPW; ++v)
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[v][t] = 0.f;
  const float4* st4 = reinterpret_cast<const float4*>(stage);
#pragma unroll 4
  for (int j = 0; j < d; ++j) {
    const float4 a = st4[2 * j], b = st4[2 * j + 1];
    const float xv[kVPW] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float m[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) m[t] = mat[j * DP + lane + 32 * t];
#pragma unroll
    for (int v = 0; v < kVPW; ++v)
#pragma unroll
      for (int t = 0; t < NT; ++t) acc[v][t] = fmaf(xv[v], m[t], acc[v][t]);
  }
}

template <int NT>
__global__ void __launch_bounds__(kThreads, 2) compress_kernel(CompressArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int d = a.d, DP = 32 * NT;
  const Smem s = carve(smem_raw, d, DP);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // mat[j][i] = Pi[i][j]  (x_rot_i = sum_j x_j Pi[i][j])
  for (int idx = threadIdx.x; idx < d * DP; idx += blockDim.x) {
    const int j = idx / DP, i = idx % DP;
    s.mat[idx] = (i < d) ? a.Pi[i * d + j] : 0.f;
  }
  const int nb0 = (1 << a.bits0) - 1, nb1 = (a.mode == MODE_MIXED) ? (1 << a.bits1) - 1 : 0;
  // sign stage: the two-stage key quantiser, or the mixed mode when a sign plane is asked for
  const bool with_signs = a.mode == MODE_IP || (a.mode == MODE_MIXED && a.signs != nullptr);
  if (threadIdx.x < 16) {
    s.tab[threadIdx.x] = (threadIdx.x < nb0) ? a.bounds0[threadIdx.x] : 0.f;
    s.tab[16 + threadIdx.x] = (threadIdx.x < nb1) ? a.bounds1[threadIdx.x] : 0.f;
    s.cent[threadIdx.x] = (with_signs && threadIdx.x < (1 << a.bits0)) ? a.centroids[threadIdx.x] : 0.f;
    s.cent[16 + threadIdx.x] =
        (with_signs && a.mode == MODE_MIXED && threadIdx.x < (1 << a.bits1)) ? a.centroids1[threadIdx.x] : 0.f;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) s.sgn[i] = with_signs ? a.S[i] : 0.f;
  build_slots(s, a.mode == MODE_MIXED ? a.is_outlier : nullptr, d);
  __syncthreads();
  const int n_out = (a.mode == MODE_MIXED) ? count_outliers(s, d) : 0;
  if (a.skip_block_aligned && (n_out & 31) == 0) return;      // uniform over the grid: the tcgen05 kernel did it

  float* stage = s.stage + static_cast<size_t>(warp) * d * kVPW;
  uint8_t* cstage = reinterpret_cast<uint8_t*>(stage);   // reused for permuted codes (mixed, packed)

  // Per-lane channel constants.
  int tab_of[NT], nb_of[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int i = lane + 32 * t;
    const bool reg = (a.mode == MODE_MIXED) && (i < d) && !s.outl[i];
    tab_of[t] = reg ? 16 : 0;
    nb_of[t] = reg ? nb1 : nb0;
  }
  const int row_bytes_uniform = packed_row_bytes(d, a.bits0);
  const int seg0_bytes = packed_row_bytes(n_out, a.bits0);
  const int row_bytes_mixed = seg0_bytes + packed_row_bytes(d - n_out, a.bits1);
  const int sign_bytes = (d + 7) >> 3;

  const int64_t n_tiles = (a.n_vec + kWarps * kVPW - 1) / (kWarps * kVPW);
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t v0 = tile * (kWarps * kVPW) + warp * kVPW;
    float nrm[kVPW];
    // ---- load, norm (sum of squares in fp64, rounded once), scale, stage ----------------
#pragma unroll
    for (int v = 0; v < kVPW; ++v) {
      const int64_t n = v0 + v;
      float xv[NT];
      double ss = 0.0;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int i = lane + 32 * t;
        xv[t] = (n < a.n_vec && i < d) ? load_float(a.x, a.x_dtype, n * a.x_pitch + i) : 0.f;
        ss += static_cast<double>(xv[t]) * static_cast<double>(xv[t]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(QKV_FULL_MASK, ss, o);
      const float norm = fmaxf(static_cast<float>(sqrt(ss)), 1e-8f);
      nrm[v] = norm;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int i = lane + 32 * t;
        if (i < d) stage[i * kVPW + v] = xv[t] / norm;
      }
    }
    __syncwarp();
    float acc[kVPW][NT];
    rotate8<NT>(s.mat, stage, d, DP, lane, acc);
    __syncwarp();

    // ---- bucketise, sign bit, store ---------------------------------------------------------
#pragma unroll
    for (int v = 0; v < kVPW; ++v) {
      const int64_t n = v0 + v;
      if (n >= a.n_vec) break;            // warp-uniform
      const int64_t row = map_row(a.rows, n);
      uint32_t code[NT], sbit[NT];
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int i = lane + 32 * t;
        const float y = acc[v][t];
        uint32_t c = 0;
        for (int b = 0; b < nb_of[t]; ++b) c += (y > s.tab[tab_of[t] + b]) ? 1u : 0u;
        code[t] = (i < d) ? c : 0u;
        sbit[t] = 0;
        if (with_signs && i < d) sbit[t] = ((y - s.cent[tab_of[t] + c]) * s.sgn[i] >= 0.f) ? 1u : 0u;
      }
      if (lane == 0) a.norms[row] = nrm[v];
      if (!a.packed) {
        uint8_t* crow = a.codes + row * d;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const int i = lane + 32 * t;
          if (i < d) {
            crow[i] = static_cast<uint8_t>(code[t]);
            if (with_signs) a.signs[row * d + i] = static_cast<uint8_t>(sbit[t]);
          }
        }
      } else if (a.mode != MODE_MIXED) {
        uint8_t* crow = a.codes + row * row_bytes_uniform;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          if (32 * t < d) {
            const uint32_t w = pack32(code[t], a.bits0, lane);
            store_packed_words(w, a.bits0, crow, 4 * t * a.bits0, row_bytes_uniform, lane);
          }
        }
        if (a.mode == MODE_IP) {
          uint8_t* srow = a.signs + row * sign_bytes;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            if (32 * t < d) {
              const uint32_t w = __ballot_sync(QKV_FULL_MASK, sbit[t]);
              store_packed_words(w, 1, srow, 4 * t, sign_bytes, lane);
            }
          }
        }
      } else {
        // mixed, packed: permute codes into slot order through shared memory, then pack the
        // outlier segment at bits0 and the regular segment at bits1.
        __syncwarp();
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const int i = lane + 32 * t;
          if (i < d) cstage[s.slot[i]] = static_cast<uint8_t>(code[t]);
        }
        __syncwarp();
        uint8_t* crow = a.codes + row * row_bytes_mixed;
        for (int g = 0; 32 * g < n_out; ++g) {
          const int k = 32 * g + lane;
          const uint32_t c = (k < n_out) ? cstage[k] : 0u;
          const uint32_t w = pack32(c, a.bits0, lane);
          store_packed_words(w, a.bits0, crow, 4 * g * a.bits0, seg0_bytes, lane);
        }
        for (int g = 0; 32 * g < d - n_out; ++g) {
          const int k = 32 * g + lane;
          const uint32_t c = (k < d - n_out) ? cstage[n_out + k] : 0u;
          const uint32_t w = pack32(c, a.bits1, lane);
          store_packed_words(w, a.bits1, crow, seg0_bytes + 4 * g * a.bits1, row_bytes_mixed, lane);
        }
        if (with_signs) {             // one bit per channel, in channel order
          uint8_t* srow = a.signs + row * sign_bytes;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            if (32 * t < d) {
              const uint32_t w = __ballot_sync(QKV_FULL_MASK, sbit[t]);
              store_packed_words(w, 1, srow, 4 * t, sign_bytes, lane);
            }
          }
        }
      }
    }
    __syncwarp();
  }
}

template <int NT>
__global__ void __launch_bounds__(kThreads, 2) decompress_kernel(DecompressArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int d = a.d, DP = 32 * NT;
  const Smem s = carve(smem_raw, d, DP);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // mat[j][i] = Pi[j][i]  (x_i = sum_j y_j Pi[j][i])
  for (int idx = threadIdx.x; idx < d * DP; idx += blockDim.x) {
    const int j = idx / DP, i = idx % DP;
    s.mat[idx] = (i < d) ? a.Pi[j * d + i] : 0.f;
  }
  const bool mixed = a.mode == MODE_MIXED;
  if (threadIdx.x < 16) {
    s.tab[threadIdx.x] = (threadIdx.x < (1 << a.bits0)) ? a.cents0[threadIdx.x] : 0.f;
    s.tab[16 + threadIdx.x] = (mixed && threadIdx.x < (1 << a.bits1)) ? a.cents1[threadIdx.x] : 0.f;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) s.sgn[i] = a.signs ? a.S[i] : 0.f;
  build_slots(s, mixed ? a.is_outlier : nullptr, d);
  __syncthreads();
  const int n_out = mixed ? count_outliers(s, d) : 0;
  if (a.skip_block_aligned && (n_out & 31) == 0) return;      // uniform over the grid: the tcgen05 kernel did it

  float* stage = s.stage + static_cast<size_t>(warp) * d * kVPW;
  const int row_bytes_uniform = packed_row_bytes(d, a.bits0);
  const int seg0_bytes = packed_row_bytes(n_out, a.bits0);
  const int row_bytes_mixed = seg0_bytes + packed_row_bytes(d - n_out, a.bits1);
  const int sign_bytes = (d + 7) >> 3;

  const int64_t n_tiles = (a.n_vec + kWarps * kVPW - 1) / (kWarps * kVPW);
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t v0 = tile * (kWarps * kVPW) + warp * kVPW;
    float nrm[kVPW];
#pragma unroll
    for (int v = 0; v < kVPW; ++v) {
      const int64_t n = v0 + v;
      const bool live = n < a.n_vec;
      const int64_t row = live ? map_row(a.rows, n) : 0;
      nrm[v] = live ? a.norms[row] : 0.f;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int j = lane + 32 * t;
        if (j >= d) continue;
        float y = 0.f;
        if (live) {
          uint32_t c;
          const bool reg = mixed && !s.outl[j];
          const int w = reg ? a.bits1 : a.bits0;
          if (!a.packed) {
            c = a.codes[row * d + j];
          } else if (!mixed) {
            c = read_field(a.codes + row * row_bytes_uniform, j * w, w, row_bytes_uniform);
          } else {
            const int k = s.slot[j];
            const int bitpos = reg ? seg0_bytes * 8 + (k - n_out) * w : k * w;
            c = read_field(a.codes + row * row_bytes_mixed, bitpos, w, row_bytes_mixed);
          }
          y = s.tab[(reg ? 16 : 0) + c];
          if (a.signs) {
            const uint32_t sb = a.packed ? ((a.signs[row * sign_bytes + (j >> 3)] >> (j & 7)) & 1u)
                                         : a.signs[row * d + j];
            y += a.qjl_scale * (s.sgn[j] * (sb ? 1.f : -1.f));
          }
        }
        stage[j * kVPW + v] = y;
      }
    }
    __syncwarp();
    float acc[kVPW][NT];
    rotate8<NT>(s.mat, stage, d, DP, lane, acc);
    __syncwarp();
#pragma unroll
    for (int v = 0; v < kVPW; ++v) {
      const int64_t n = v0 + v;
      if (n >= a.n_vec) break;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int i = lane + 32 * t;
        if (i < d) store_float(a.out, a.out_dtype, n * a.out_pitch + i, acc[v][t] * nrm[v]);
      }
    }
  }
}

template <typename Args, typename K1, typename K2, typename K3, typename K4>
static int launch_by_nt(const Args& a, int d, int64_t n_vec, cudaStream_t st, K1 k1, K2 k2, K3 k3, K4 k4) {
  const int NT = (d + 31) / 32;
  const size_t smem = smem_bytes(d, NT);
  const int64_t tiles = (n_vec + kWarps * kVPW - 1) / (kWarps * kVPW);
  const int per_sm = smem > 100 * 1024 ? 1 : 2;
  const int grid = static_cast<int>(tiles < kNumSMs * per_sm ? tiles : kNumSMs * per_sm);
#define QKV_LAUNCH(K)                                                                              \
  do {                                                                                             \
    if (cudaFuncSetAttribute(K, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return QKV_ELAUNCH;                                                                          \
    K<<<grid, kThreads, smem, st>>>(a);                                                            \
  } while (0)
  switch (NT) {
    case 1: QKV_LAUNCH(k1); break;
    case 2: QKV_LAUNCH(k2); break;
    case 3: QKV_LAUNCH(k3); break;
    default: QKV_LAUNCH(k4); break;
  }
#undef QKV_LAUNCH
  return check_launch();
}

static int check_common(const void* x, int dtype, int64_t n_vec, int d, const float* Pi) {
  if ((!x && n_vec != 0) || !Pi) return QKV_ENULL;
  if (dtype != QKV_F32 && dtype != QKV_BF16 && dtype != QKV_F16) return QKV_EDTYPE;
  if (d < 1 || d > kMaxD || n_vec < 0) return QKV_EDIM;
  return QKV_OK;
}

static int check_rows(const qkv_rows_t& r) {
  return (r.seg_len >= 1 && r.seg_stride >= 0 && r.seg_off >= 0) ? QKV_OK : QKV_EARG;
}

// QUASHKV_B200_CUDA_CORE_ROTATION=1 keeps every call on the fp32 CUDA-core kernels (for A/B checks).
static bool cuda_core_only() {
  const char* e = getenv("QUASHKV_B200_CUDA_CORE_ROTATION");
  return e && e[0] == '1';
}

// QUASHKV_B200_NO_TCGEN05=1 keeps the tensor-core rotation on the mma.sync kernels (for A/B checks).
static bool no_tcgen05() {
  const char* e = getenv("QUASHKV_B200_NO_TCGEN05");
  return e && e[0] == '1';
}

static int run_compress(const CompressArgs& a, cudaStream_t st) {
  if (a.n_vec == 0) return QKV_OK;
  if (a.mode == MODE_MIXED && a.signs)       // the sign stage of the mixed mode exists in the CUDA-core kernel only
    return launch_by_nt(a, a.d, a.n_vec, st, compress_kernel<1>, compress_kernel<2>, compress_kernel<3>,
                        compress_kernel<4>);
  if (compress_umma_ok(a) && !cuda_core_only() && !no_tcgen05()) {
    const int rc = launch_compress_umma(a, st);
    if (rc || a.mode != MODE_MIXED) return rc;
    // Mixed precision: the tcgen05 kernel works only when the outlier count (known on the device) is a
    // multiple of 32 and returns at once otherwise; the CUDA-core kernel behind it makes the opposite choice.
    CompressArgs b = a;
    b.skip_block_aligned = 1;
    return launch_by_nt(b, b.d, b.n_vec, st, compress_kernel<1>, compress_kernel<2>, compress_kernel<3>,
                        compress_kernel<4>);
  }
  if (compress_mma_ok(a) && !cuda_core_only()) return launch_compress_mma(a, st);
  return launch_by_nt(a, a.d, a.n_vec, st, compress_kernel<1>, compress_kernel<2>, compress_kernel<3>,
                      compress_kernel<4>);
}

}  // namespace qkv

using namespace qkv;

extern "C" int qkv_compress_mse(const void* x, int x_dtype, int64_t x_pitch, int64_t n_vec, int d,
                                const float* Pi, const float* boundaries, int bits,
                                uint8_t* codes_out, int packed, float* norms_out,
                                qkv_rows_t rows, void* stream) {
  int rc = check_common(x, x_dtype, n_vec, d, Pi);
  if (rc) return rc;
  if (!boundaries || ((!codes_out || !norms_out) && n_vec != 0)) return QKV_ENULL;
  if (bits < 1 || bits > 4) return QKV_EBITS;
  if ((rc = check_rows(rows))) return rc;
  CompressArgs a{};
  a.x = x; a.x_dtype = x_dtype; a.x_pitch = x_pitch; a.n_vec = n_vec; a.d = d; a.Pi = Pi;
  a.mode = MODE_MSE; a.bounds0 = boundaries; a.bits0 = bits; a.bits1 = 1;
  a.codes = codes_out; a.packed = packed; a.norms = norms_out; a.rows = rows;
  return run_compress(a, static_cast<cudaStream_t>(stream));
}

extern "C" int qkv_compress_ip(const void* x, int x_dtype, int64_t x_pitch, int64_t n_vec, int d,
                               const float* Pi, const float* boundaries, const float* centroids,
                               int mse_bits, const float* S,
                               uint8_t* codes_out, uint8_t* signs_out, int packed, float* norms_out,
                               qkv_rows_t rows, void* stream) {
  int rc = check_common(x, x_dtype, n_vec, d, Pi);
  if (rc) return rc;
  if (!boundaries || !centroids || !S || ((!codes_out || !signs_out || !norms_out) && n_vec != 0)) return QKV_ENULL;
  if (mse_bits < 1 || mse_bits > 4) return QKV_EBITS;
  if ((rc = check_rows(rows))) return rc;
  CompressArgs a{};
  a.x = x; a.x_dtype = x_dtype; a.x_pitch = x_pitch; a.n_vec = n_vec; a.d = d; a.Pi = Pi;
  a.mode = MODE_IP; a.bounds0 = boundaries; a.bits0 = mse_bits; a.bits1 = 1;
  a.centroids = centroids; a.S = S;
  a.codes = codes_out; a.signs = signs_out; a.packed = packed; a.norms = norms_out; a.rows = rows;
  return run_compress(a, static_cast<cudaStream_t>(stream));
}

extern "C" int qkv_compress_mixed(const void* x, int x_dtype, int64_t x_pitch, int64_t n_vec, int d,
                                  const float* Pi, const uint8_t* is_outlier,
                                  const float* bounds_out, int bits_out,
                                  const float* bounds_reg, int bits_reg,
                                  uint8_t* codes_out, int packed, float* norms_out,
                                  qkv_rows_t rows, void* stream) {
  int rc = check_common(x, x_dtype, n_vec, d, Pi);
  if (rc) return rc;
  if (!is_outlier || !bounds_out || !bounds_reg || ((!codes_out || !norms_out) && n_vec != 0)) return QKV_ENULL;
  if (bits_out < 1 || bits_out > 4 || bits_reg < 1 || bits_reg > 4) return QKV_EBITS;
  if ((rc = check_rows(rows))) return rc;
  CompressArgs a{};
  a.x = x; a.x_dtype = x_dtype; a.x_pitch = x_pitch; a.n_vec = n_vec; a.d = d; a.Pi = Pi;
  a.mode = MODE_MIXED; a.bounds0 = bounds_out; a.bits0 = bits_out; a.bounds1 = bounds_reg; a.bits1 = bits_reg;
  a.is_outlier = is_outlier;
  a.codes = codes_out; a.packed = packed; a.norms = norms_out; a.rows = rows;
  return run_compress(a, static_cast<cudaStream_t>(stream));
}

extern "C" int qkv_compress_mixed_ip(const void* x, int x_dtype, int64_t x_pitch, int64_t n_vec, int d,
                                     const float* Pi, const uint8_t* is_outlier,
                                     const float* bounds_out, const float* cents_out, int bits_out,
                                     const float* bounds_reg, const float* cents_reg, int bits_reg,
                                     const float* S,
                                     uint8_t* codes_out, uint8_t* signs_out, int packed, float* norms_out,
                                     qkv_rows_t rows, void* stream) {
  int rc = check_common(x, x_dtype, n_vec, d, Pi);
  if (rc) return rc;
  if (!is_outlier || !bounds_out || !bounds_reg || !cents_out || !cents_reg || !S ||
      ((!codes_out || !signs_out || !norms_out) && n_vec != 0))
    return QKV_ENULL;
  if (bits_out < 1 || bits_out > 4 || bits_reg < 1 || bits_reg > 4) return QKV_EBITS;
  if ((rc = check_rows(rows))) return rc;
  CompressArgs a{};
  a.x = x; a.x_dtype = x_dtype; a.x_pitch = x_pitch; a.n_vec = n_vec; a.d = d; a.Pi = Pi;
  a.mode = MODE_MIXED; a.bounds0 = bounds_out; a.bits0 = bits_out; a.bounds1 = bounds_reg; a.bits1 = bits_reg;
  a.centroids = cents_out; a.centroids1 = cents_reg; a.S = S;
  a.is_outlier = is_outlier;
  a.codes = codes_out; a.signs = signs_out; a.packed = packed; a.norms = norms_out; a.rows = rows;
  return run_compress(a, static_cast<cudaStream_t>(stream));
}

extern "C" int64_t qkv_mixed_row_bytes(int d, int n_out, int bits_out, int bits_reg) {
  if (d < 1 || n_out < 0 || n_out > d) return QKV_EDIM;
  return packed_row_bytes(n_out, bits_out) + packed_row_bytes(d - n_out, bits_reg);
}

extern "C" int qkv_decompress(const uint8_t* codes, const uint8_t* signs, int packed, const float* norms,
                              qkv_rows_t rows, int64_t n_vec, int d,
                              const float* Pi, const float* centroids, int bits,
                              const float* S, float qjl_scale,
                              void* out, int out_dtype, int64_t out_pitch, void* stream) {
  int rc = check_common(codes, out_dtype, n_vec, d, Pi);
  if (rc) return rc;
  if (!centroids || ((!norms || !out) && n_vec != 0) || (signs && !S)) return QKV_ENULL;
  if (bits < 1 || bits > 4) return QKV_EBITS;
  if ((rc = check_rows(rows))) return rc;
  if (n_vec == 0) return QKV_OK;
  DecompressArgs a{};
  a.codes = codes; a.signs = signs; a.packed = packed; a.norms = norms; a.rows = rows;
  a.n_vec = n_vec; a.d = d; a.Pi = Pi; a.mode = MODE_MSE; a.cents0 = centroids; a.bits0 = bits; a.bits1 = 1;
  a.S = S; a.qjl_scale = qjl_scale; a.out = out; a.out_dtype = out_dtype; a.out_pitch = out_pitch;
  if (decompress_umma_ok(a) && !cuda_core_only() && !no_tcgen05())
    return launch_decompress_umma(a, static_cast<cudaStream_t>(stream));
  if (decompress_mma_ok(a) && !cuda_core_only()) return launch_decompress_mma(a, static_cast<cudaStream_t>(stream));
  return launch_by_nt(a, d, n_vec, static_cast<cudaStream_t>(stream), decompress_kernel<1>,
                      decompress_kernel<2>, decompress_kernel<3>, decompress_kernel<4>);
}

extern "C" int qkv_decompress_mixed(const uint8_t* codes, int packed, const float* norms,
                                    qkv_rows_t rows, int64_t n_vec, int d,
                                    const float* Pi, const uint8_t* is_outlier,
                                    const float* cents_out, int bits_out,
                                    const float* cents_reg, int bits_reg,
                                    void* out, int out_dtype, int64_t out_pitch, void* stream) {
  int rc = check_common(codes, out_dtype, n_vec, d, Pi);
  if (rc) return rc;
  if (!is_outlier || !cents_out || !cents_reg || ((!norms || !out) && n_vec != 0)) return QKV_ENULL;
  if (bits_out < 1 || bits_out > 4 || bits_reg < 1 || bits_reg > 4) return QKV_EBITS;
  if ((rc = check_rows(rows))) return rc;
  if (n_vec == 0) return QKV_OK;
  DecompressArgs a{};
  a.codes = codes; a.packed = packed; a.norms = norms; a.rows = rows;
  a.n_vec = n_vec; a.d = d; a.Pi = Pi; a.mode = MODE_MIXED;
  a.cents0 = cents_out; a.bits0 = bits_out; a.cents1 = cents_reg; a.bits1 = bits_reg;
  a.is_outlier = is_outlier; a.out = out; a.out_dtype = out_dtype; a.out_pitch = out_pitch;
  if (decompress_umma_ok(a) && !cuda_core_only() && !no_tcgen05()) {
    // the tcgen05 kernel takes outlier counts that are multiples of 32 (a device-side test), the CUDA-core
    // kernel behind it the others
    if ((rc = launch_decompress_umma(a, static_cast<cudaStream_t>(stream)))) return rc;
    a.skip_block_aligned = 1;
  }
  return launch_by_nt(a, d, n_vec, static_cast<cudaStream_t>(stream), decompress_kernel<1>,
                      decompress_kernel<2>, decompress_kernel<3>, decompress_kernel<4>);
}

namespace qkv { unsigned int index_umma_timeouts(); unsigned int bulk_copy_timeouts(); }

extern "C" int64_t qkv_tensor_core_timeouts(void) {
  return static_cast<int64_t>(umma_timeouts()) + static_cast<int64_t>(index_umma_timeouts()) +
         static_cast<int64_t>(bulk_copy_timeouts());
}
