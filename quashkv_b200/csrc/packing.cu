// Stand-alone bit packing / unpacking of code planes, and the library's diagnostics.
// Layout: per row an LSB-first stream of w-bit fields; byte k holds stream bits [8k, 8k+8).
#include "common.cuh"

namespace qkv {

// One thread per packed byte: gather the (up to 8) fields that overlap it.
__global__ void pack_kernel(const uint8_t* __restrict__ codes, uint8_t* __restrict__ packed,
                            int64_t n_rows, int d, int w, int row_bytes) {
  const int64_t total = n_rows * row_bytes;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / row_bytes;
    const int k = static_cast<int>(idx % row_bytes);
    const uint8_t* src = codes + r * d;
    const int first = (8 * k) / w, last = (8 * k + 7) / w;
    uint32_t acc = 0;
    for (int f = first; f <= last; ++f) {
      const uint32_t c = (f < d) ? (src[f] & ((1u << w) - 1u)) : 0u;
      const int rel = f * w - 8 * k;        // field start relative to this byte, may be negative
      acc |= rel >= 0 ? (c << rel) : (c >> (-rel));
    }
    packed[idx] = static_cast<uint8_t>(acc);
  }
}

__global__ void unpack_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ codes,
                              int64_t n_rows, int d, int w, int row_bytes) {
  const int64_t total = n_rows * d;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / d;
    const int i = static_cast<int>(idx % d);
    codes[idx] = static_cast<uint8_t>(read_field(packed + r * row_bytes, i * w, w, row_bytes));
  }
}

// Row i of `src` goes to row slots[i] of `dst`, rows of `words` 32-bit words; a negative slot drops the row.
__global__ void scatter_rows_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst,
                                    const int64_t* __restrict__ slots, int64_t n_rows, int words) {
  const int64_t total = n_rows * words;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / words;
    const int w = static_cast<int>(i - r * words);
    const int64_t slot = __ldg(slots + r);
    if (slot >= 0) dst[slot * words + w] = src[i];
  }
}

static int grid_for(int64_t total) {
  const int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
  return static_cast<int>(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

}  // namespace qkv

using namespace qkv;

extern "C" int qkv_abi_version(void) { return QKV_ABI_VERSION; }

extern "C" const char* qkv_strerror(int code) {
  switch (code) {
    case QKV_OK: return "ok";
    case QKV_ENULL: return "a required pointer is NULL";
    case QKV_EDIM: return "unsupported dimension or size";
    case QKV_EBITS: return "unsupported bit width";
    case QKV_EDTYPE: return "unknown dtype";
    case QKV_EALIGN: return "pointer or pitch not aligned as required";
    case QKV_EWORKSPACE: return "workspace size not acceptable";
    case QKV_ELAUNCH: return "CUDA launch failed";
    case QKV_EARG: return "inconsistent arguments";
    default: return "unknown error code";
  }
}

extern "C" int qkv_pack(const uint8_t* codes, uint8_t* packed, int64_t n_rows, int d, int bits, void* stream) {
  if (bits < 1 || bits > 4) return QKV_EBITS;
  if (d < 1 || n_rows < 0) return QKV_EDIM;
  if (n_rows == 0) return QKV_OK;          // nothing to do; empty tensors have no storage
  if (!codes || !packed) return QKV_ENULL;
  const int row_bytes = packed_row_bytes(d, bits);
  pack_kernel<<<grid_for(n_rows * row_bytes), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      codes, packed, n_rows, d, bits, row_bytes);
  return check_launch();
}

extern "C" int qkv_unpack(const uint8_t* packed, uint8_t* codes, int64_t n_rows, int d, int bits, void* stream) {
  if (bits < 1 || bits > 4) return QKV_EBITS;
  if (d < 1 || n_rows < 0) return QKV_EDIM;
  if (n_rows == 0) return QKV_OK;          // nothing to do; empty tensors have no storage
  if (!codes || !packed) return QKV_ENULL;
  const int row_bytes = packed_row_bytes(d, bits);
  unpack_kernel<<<grid_for(n_rows * d), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      packed, codes, n_rows, d, bits, row_bytes);
  return check_launch();
}

extern "C" int qkv_scatter_rows(const void* src, void* dst, const int64_t* slots, int64_t n_rows, int row_bytes,
                                void* stream) {
  if (n_rows < 0 || row_bytes < 4 || (row_bytes & 3)) return QKV_EDIM;
  if (n_rows == 0) return QKV_OK;
  if (!src || !dst || !slots) return QKV_ENULL;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 3u) return QKV_EALIGN;
  const int words = row_bytes / 4;
  scatter_rows_kernel<<<grid_for(n_rows * words), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), slots, n_rows, words);
  return check_launch();
}
