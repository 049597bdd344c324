// Row-major packed planes <-> tile records (tile_format.cuh): exact integer re-arrangements.
//
// qkv_tile_rows stands where the reference appends a block to its list (engine.py:145-172): the
// compress kernels write the reference's packed rows (packing.py:22-94) into a staging area and this
// kernel files every token into the record that the decode kernel streams.  qkv_untile_rows is the
// inverse and yields byte-identical packed rows, which is how block views, whole-cache
// decompression and the byte-level parity checks read a tiled cache.
//
// Eight threads per token: thread j moves 4 bytes of the key-code row, (j < 4) 4 bytes of the sign
// row, (j = 4, 5) a norm, and files the 16 value coordinates 16 j .. 16 j + 15 (6 bytes of the
// 3-bit row) into the token's half of sixteen 6-bit fields.  Those fields are shared with the other
// token of the pair, so the token's bits are cleared and set with atomic AND / OR on the three words.
#include "common.cuh"
#include "tile_format.cuh"

namespace qkv {
namespace {

struct RowPlanes {
  uint8_t* k_codes; uint8_t* k_signs; float* k_norms; uint8_t* v_codes; float* v_norms;
};

__device__ __forceinline__ int64_t token_slot(const qkv_rows_t& map, const int64_t* slots, int64_t i) {
  return slots ? slots[i] : map_row(map, i);
}

__global__ void __launch_bounds__(256) tile_rows_kernel(RowPlanes src, int64_t n_rows, uint8_t* __restrict__ records,
                                                        qkv_rows_t map, const int64_t* __restrict__ slots) {
  const int64_t gt = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t i = gt >> 3;
  const int j = static_cast<int>(gt & 7);
  if (i >= n_rows) return;
  const int64_t slot = token_slot(map, slots, i);
  if (slot < 0) return;                                   // a negative slot drops the row
  uint8_t* rec = records + (slot >> 4) * tile::kBytes;
  const int k = static_cast<int>(slot & 15);
  // key codes, sign bits, norms: whole pieces, unchanged
  *reinterpret_cast<uint32_t*>(rec + tile::key_code_offset(k, j)) =
      *reinterpret_cast<const uint32_t*>(src.k_codes + i * tile::kKeyRowBytes + 4 * j);
  if (j < 4)
    *reinterpret_cast<uint32_t*>(rec + tile::key_sign_offset(k, j)) =
        *reinterpret_cast<const uint32_t*>(src.k_signs + i * tile::kSignRowBytes + 4 * j);
  if (j == 4) *reinterpret_cast<float*>(rec + tile::key_norm_offset(k)) = src.k_norms[i];
  if (j == 5) *reinterpret_cast<float*>(rec + tile::val_norm_offset(k)) = src.v_norms[i];
  // value codes of coordinates 16 j .. 16 j + 15: bytes 6 j .. 6 j + 5 of the 48-byte row
  const uint16_t* vrow = reinterpret_cast<const uint16_t*>(src.v_codes + i * tile::kValRowBytes + 6 * j);
  const uint64_t codes48 = static_cast<uint64_t>(vrow[0]) | (static_cast<uint64_t>(vrow[1]) << 16) |
                           (static_cast<uint64_t>(vrow[2]) << 32);
  uint32_t bits[3], mask[3];
  tile::spread_codes16(codes48, tile::val_half_shift(k), bits, mask);
  const int lane = tile::val_lane(k, j), grp = tile::val_group(k);
#pragma unroll
  for (int w = 0; w < 3; ++w) {
    uint32_t* word = reinterpret_cast<uint32_t*>(rec + tile::val_word_offset(lane, 3 * grp + w));
    atomicAnd(word, ~mask[w]);
    atomicOr(word, bits[w]);
  }
}

__global__ void __launch_bounds__(256) untile_rows_kernel(const uint8_t* __restrict__ records, qkv_rows_t map,
                                                          const int64_t* __restrict__ slots, int64_t n_rows,
                                                          RowPlanes dst) {
  const int64_t gt = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t i = gt >> 3;
  const int j = static_cast<int>(gt & 7);
  if (i >= n_rows) return;
  const int64_t slot = token_slot(map, slots, i);
  if (slot < 0) return;
  const uint8_t* rec = records + (slot >> 4) * tile::kBytes;
  const int k = static_cast<int>(slot & 15);
  *reinterpret_cast<uint32_t*>(dst.k_codes + i * tile::kKeyRowBytes + 4 * j) =
      *reinterpret_cast<const uint32_t*>(rec + tile::key_code_offset(k, j));
  if (j < 4)
    *reinterpret_cast<uint32_t*>(dst.k_signs + i * tile::kSignRowBytes + 4 * j) =
        *reinterpret_cast<const uint32_t*>(rec + tile::key_sign_offset(k, j));
  if (j == 4) dst.k_norms[i] = *reinterpret_cast<const float*>(rec + tile::key_norm_offset(k));
  if (j == 5) dst.v_norms[i] = *reinterpret_cast<const float*>(rec + tile::val_norm_offset(k));
  uint32_t w[3];
  const int lane = tile::val_lane(k, j), grp = tile::val_group(k);
#pragma unroll
  for (int q = 0; q < 3; ++q) w[q] = *reinterpret_cast<const uint32_t*>(rec + tile::val_word_offset(lane, 3 * grp + q));
  const uint64_t codes48 = tile::gather_codes16(w, tile::val_half_shift(k));
  uint16_t* vrow = reinterpret_cast<uint16_t*>(dst.v_codes + i * tile::kValRowBytes + 6 * j);
  vrow[0] = static_cast<uint16_t>(codes48);
  vrow[1] = static_cast<uint16_t>(codes48 >> 16);
  vrow[2] = static_cast<uint16_t>(codes48 >> 32);
}

int check_args(const void* a, const void* b, const void* c, const void* d, const void* e, const void* records,
               int64_t n_rows, const qkv_rows_t& map, const int64_t* slots) {
  if (n_rows < 0) return QKV_EDIM;
  if (n_rows == 0) return QKV_OK;
  if (!a || !b || !c || !d || !e || !records) return QKV_ENULL;
  if (!slots && (map.seg_len < 1 || map.seg_stride < 0 || map.seg_off < 0)) return QKV_EARG;
  const uintptr_t al = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
                       reinterpret_cast<uintptr_t>(e);
  if ((al & 3u) || (reinterpret_cast<uintptr_t>(d) & 1u) || (reinterpret_cast<uintptr_t>(records) & 15u))
    return QKV_EALIGN;
  return 1;   // go
}

}  // namespace
}  // namespace qkv

using namespace qkv;

extern "C" int qkv_tile_rows(const uint8_t* k_codes, const uint8_t* k_signs, const float* k_norms,
                             const uint8_t* v_codes, const float* v_norms, int64_t n_rows,
                             uint8_t* records, qkv_rows_t map, const int64_t* slots, void* stream) {
  const int rc = check_args(k_codes, k_signs, k_norms, v_codes, v_norms, records, n_rows, map, slots);
  if (rc <= 0) return rc;
  const RowPlanes src{const_cast<uint8_t*>(k_codes), const_cast<uint8_t*>(k_signs), const_cast<float*>(k_norms),
                      const_cast<uint8_t*>(v_codes), const_cast<float*>(v_norms)};
  const int64_t threads = n_rows * 8;
  tile_rows_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, n_rows, records, map, slots);
  return check_launch();
}

extern "C" int qkv_untile_rows(const uint8_t* records, qkv_rows_t map, const int64_t* slots, int64_t n_rows,
                               uint8_t* k_codes, uint8_t* k_signs, float* k_norms, uint8_t* v_codes,
                               float* v_norms, void* stream) {
  const int rc = check_args(k_codes, k_signs, k_norms, v_codes, v_norms, records, n_rows, map, slots);
  if (rc <= 0) return rc;
  const RowPlanes dst{k_codes, k_signs, k_norms, v_codes, v_norms};
  const int64_t threads = n_rows * 8;
  untile_rows_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      records, map, slots, n_rows, dst);
  return check_launch();
}
