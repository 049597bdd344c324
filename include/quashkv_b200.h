/*
 * quashkv_b200 — C ABI of the B200 (sm_100a) compressed-KV hot path.
 *
 * Every entry point takes raw DEVICE pointers, explicit sizes and a CUDA stream
 * (passed as void*; NULL = the legacy default stream).  A call validates its
 * arguments on the host, enqueues kernels on the stream and returns:
 * QKV_OK (0) or a negative QKV_E* code when nothing was launched.  Unless a
 * comment says otherwise no entry point allocates, frees or synchronises, and
 * the library keeps no state between calls: the caller owns inputs, outputs and
 * workspaces (sizes from the *_workspace_bytes functions).
 *
 * "Reference" citations are file:line inside the QuashKV project
 * (package directory quashkv/).
 *
 * Conventions
 *   dtype        QKV_F32 / QKV_BF16 / QKV_F16 — storage type of a float tensor;
 *                arithmetic is always fp32 (bf16/f16 inputs are upcast exactly,
 *                as the reference's callers do with .float()).
 *   codes        one uint8 per coordinate ("unpacked"), or "packed": an
 *                LSB-first stream of w-bit fields per row, ceil(d*w/8) bytes
 *                (reference packing.py:22-94).
 *   rows         vector n of a call lives at row  (n / seg_len) * seg_stride +
 *                seg_off + (n % seg_len)  of the code/norm planes.  With
 *                seg_len = n_vec, seg_stride = 0, seg_off = 0 the planes are
 *                dense.  This lets a caller append to, or read from, a
 *                [segments, capacity, bytes] cache in place.
 *   Pi           (d,d) row-major fp32 rotation; rotate = x @ Pi^T, un-rotate = y @ Pi.
 *   d            1..128 for compress/decompress; a multiple of 32 up to 128 for
 *                attention and the index scan.
 */
#ifndef QUASHKV_B200_H
#define QUASHKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QKV_ABI_VERSION 1

enum { QKV_F32 = 0, QKV_BF16 = 1, QKV_F16 = 2 };

enum {
  QKV_OK = 0,
  QKV_ENULL = -1,      /* a required pointer is NULL */
  QKV_EDIM = -2,       /* unsupported d / sizes */
  QKV_EBITS = -3,      /* unsupported bit width */
  QKV_EDTYPE = -4,     /* unknown dtype enum */
  QKV_EALIGN = -5,     /* pointer or row pitch not aligned as documented */
  QKV_EWORKSPACE = -6, /* workspace too small / too large for the static scratch */
  QKV_ELAUNCH = -7,    /* cudaGetLastError() after launch was not cudaSuccess */
  QKV_EARG = -8        /* inconsistent arguments */
};

typedef struct {
  int64_t seg_len;    /* vectors per segment (>=1) */
  int64_t seg_stride; /* rows between segment starts */
  int64_t seg_off;    /* first row inside each segment */
} qkv_rows_t;

/* ---- diagnostics --------------------------------------------------------------------- */
int qkv_abi_version(void);
const char* qkv_strerror(int code);

/* ---- bit packing (reference packing.py:22-94 pack_bits, :97-159 unpack_bits) ------------ */
/* codes (n_rows,d) uint8 -> packed (n_rows, ceil(d*bits/8)).  bits in 1..4. */
int qkv_pack(const uint8_t* codes, uint8_t* packed, int64_t n_rows, int d, int bits, void* stream);
int qkv_unpack(const uint8_t* packed, uint8_t* codes, int64_t n_rows, int d, int bits, void* stream);

/* ---- compress ------------------------------------------------------------------------------
 * normalise -> rotate by Pi -> count boundaries below each rotated coordinate.
 * Replaces MSEQuantizer.compress (reference quantizer.py:113-131) and
 * fused_compress_mse (triton_kernels/compress.py:210-249).
 *   x          (n_vec, d) rows of pitch x_pitch ELEMENTS, dtype x_dtype
 *   boundaries (n_bounds) ascending fp32, n_bounds = 2^bits - 1
 *   codes_out  packed != 0: rows of ceil(d*bits/8) bytes; else rows of d bytes
 *   norms_out  fp32, one per row (norm clamped below at 1e-8 like the reference)
 */
int qkv_compress_mse(const void* x, int x_dtype, int64_t x_pitch, int64_t n_vec, int d,
                     const float* Pi, const float* boundaries, int bits,
                     uint8_t* codes_out, int packed, float* norms_out,
                     qkv_rows_t rows, void* stream);

/* Two-stage key quantiser: codes at `mse_bits`, then the sign bit of
 * (x_rot - centroid) * S with ">= 0" -> 1.  Replaces InnerProductQuantizer.compress
 * (reference quantizer.py:211-242) and fused_compress_ip (compress.py:252-303).
 * signs_out: packed != 0 -> ceil(d/8) bytes per row, else d bytes of 0/1. */
int qkv_compress_ip(const void* x, int x_dtype, int64_t x_pitch, int64_t n_vec, int d,
                    const float* Pi, const float* boundaries, const float* centroids, int mse_bits,
                    const float* S,
                    uint8_t* codes_out, uint8_t* signs_out, int packed, float* norms_out,
                    qkv_rows_t rows, void* stream);

/* Per-channel bit allocation.  Replaces MixedPrecisionMSEQuantizer.compress
 * (reference mixed_precision.py:130-158).  is_outlier (d) uint8 selects, per
 * rotated channel, the outlier table (bits_out) or the regular table (bits_reg).
 * Unpacked output: d bytes per row, as the reference returns.  Packed output (a
 * layout the reference does not define): the outlier channels' codes in channel
 * order as a bits_out stream, ceil(n_out*bits_out/8) bytes, followed by the
 * regular channels' codes as a bits_reg stream. */
int qkv_compress_mixed(const void* x, int x_dtype, int64_t x_pitch, int64_t n_vec, int d,
                       const float* Pi, const uint8_t* is_outlier,
                       const float* bounds_out, int bits_out,
                       const float* bounds_reg, int bits_reg,
                       uint8_t* codes_out, int packed, float* norms_out,
                       qkv_rows_t rows, void* stream);
/* Mixed-precision codes plus the sign bit of the rotated residual on every channel: the two-stage
 * quantiser with per-channel bit allocation.  Replaces MixedPrecisionIPQuantizer.compress (reference
 * mixed_precision.py:270-322).  Codes as qkv_compress_mixed (tables at the callers' bits - 1); the
 * residual is taken against the centroid of the channel's own table (cents_out / cents_reg) and the
 * sign is (residual * S >= 0).  signs_out: unpacked d bytes of 0/1 per row, or packed ceil(d/8) bytes
 * per row in channel order. */
int qkv_compress_mixed_ip(const void* x, int x_dtype, int64_t x_pitch, int64_t n_vec, int d,
                          const float* Pi, const uint8_t* is_outlier,
                          const float* bounds_out, const float* cents_out, int bits_out,
                          const float* bounds_reg, const float* cents_reg, int bits_reg,
                          const float* S,
                          uint8_t* codes_out, uint8_t* signs_out, int packed, float* norms_out,
                          qkv_rows_t rows, void* stream);
/* Bytes per packed mixed row for n_out outlier channels among d. */
int64_t qkv_mixed_row_bytes(int d, int n_out, int bits_out, int bits_reg);

/* ---- decompress ----------------------------------------------------------------------------
 * centroid gather -> un-rotate -> rescale.  Replaces MSEQuantizer.decompress
 * (reference quantizer.py:133-147), fused_decompress_mse (decompress.py:194-232)
 * and, with signs == NULL on key codes, the key path of
 * QuashKVCache._decompress_engine (integrations/hf_cache.py:96-121).
 * With signs != NULL it adds qjl_scale * S * (2*sign-1) before the rotation:
 * fused_decompress_ip (decompress.py:235-285).
 *   out (n_vec, d) rows of pitch out_pitch elements, dtype out_dtype (dense, row n). */
int qkv_decompress(const uint8_t* codes, const uint8_t* signs, int packed, const float* norms,
                   qkv_rows_t rows, int64_t n_vec, int d,
                   const float* Pi, const float* centroids, int bits,
                   const float* S, float qjl_scale,
                   void* out, int out_dtype, int64_t out_pitch, void* stream);

/* Mixed-precision decompress (reference mixed_precision.py:160-187). */
int qkv_decompress_mixed(const uint8_t* codes, int packed, const float* norms,
                         qkv_rows_t rows, int64_t n_vec, int d,
                         const float* Pi, const uint8_t* is_outlier,
                         const float* cents_out, int bits_out,
                         const float* cents_reg, int bits_reg,
                         void* out, int out_dtype, int64_t out_pitch, void* stream);

/* ---- attention over the packed cache ---------------------------------------------------------
 * Replaces QuashKVEngine.attention (reference engine.py:204-299) and
 * fused_quantized_attention (triton_kernels/attention.py:307-394), reading
 * PACKED planes and never materialising keys or values.
 *
 * Cache planes, one segment per (batch, kv head), `capacity` rows per segment:
 *   k_codes  [B*Hkv, capacity, d*(key_bits-1)/8]   k_signs [B*Hkv, capacity, d/8]
 *   k_norms  [B*Hkv, capacity] fp32
 *   v_codes  [B*Hkv, capacity, d*val_bits/8]        v_norms [B*Hkv, capacity] fp32
 * Rows 0..kv_len-1 of each segment are attended.  All plane base pointers must be
 * 16-byte aligned.
 *   q        (B, Hq, q_len, d) contiguous, dtype q_dtype;  query head h reads kv
 *            head h / (Hq/Hkv)  (Hq/Hkv = 1 is the reference's case)
 *   causal   query row i sits at position kv_len - q_len + i and sees rows <= it
 *            (reference engine.py:273-279)
 *   out      (B, Hq, q_len, d) fp32 contiguous
 *   workspace  qkv_attention_workspace_bytes(...) bytes, 16-byte aligned; holds the
 *            rotated queries and the per-split partial (max, sum, accumulator).
 */
typedef struct {
  const uint8_t* k_codes;
  const uint8_t* k_signs;
  const float* k_norms;
  const uint8_t* v_codes;
  const float* v_norms;
  int64_t capacity;
} qkv_cache_t;

size_t qkv_attention_workspace_bytes(int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d);
int qkv_attention(const void* q, int q_dtype, qkv_cache_t cache,
                  int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d,
                  int key_bits, int val_bits,
                  const float* Pi, const float* key_centroids, const float* val_centroids,
                  const float* S, float qjl_scale, float scale, int causal,
                  float* out, void* workspace, size_t workspace_bytes, void* stream);

/* Same computation as qkv_attention for callers that cannot hand over a workspace because they
 * are not allowed to allocate device memory when the call is made: a serving loop that has
 * given all of HBM to a fixed memory plan, a plugin invoked under a framework that forbids
 * cudaMalloc on its streams, code that runs between "begin capture" and "end capture" of a
 * stream.  This entry point has no counterpart in the reference.  The rotated queries and the
 * per-split partial results live in a fixed array inside the library image
 * (QKV_ATTENTION_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the process
 * exits); the call allocates nothing, on the host or the device, and returns QKV_EWORKSPACE
 * when qkv_attention_workspace_bytes(...) for the given shape exceeds that size.
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress) and remembers it; make that first call outside any stream capture.
 * All calls on a device share the one array: two calls whose kernels can overlap on the GPU
 * (different streams, no dependency) race on it and must be ordered by the caller.  Nothing in
 * the array needs clearing between calls; every word that is read is written first by the
 * same call. */
#define QKV_ATTENTION_STATIC_SCRATCH_BYTES (8u << 20)
int qkv_attention_static_scratch(const void* q, int q_dtype, qkv_cache_t cache,
                                 int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d,
                                 int key_bits, int val_bits,
                                 const float* Pi, const float* key_centroids, const float* val_centroids,
                                 const float* S, float qjl_scale, float scale, int causal,
                                 float* out, void* stream);

/* ---- attention over a paged (block-table) cache -------------------------------------------------
 * The storage shape a serving engine's block allocator hands out: the reference keeps one page of
 * `block_size` tokens per entry (integrations/vllm_backend.py:73-79, QuashKVPageConfig.block_size
 * = 16; :82-195 QuashKVPageManager) but attends over its engine's contiguous blocks; here the
 * pages are the storage and every batch entry has its own length.
 *
 * Pool planes, `block_size` rows per (block, kv head):
 *   k_codes [num_blocks, Hkv, block_size, d*(key_bits-1)/8]   k_signs [.., d/8]   k_norms [..] fp32
 *   v_codes [num_blocks, Hkv, block_size, d*val_bits/8]       v_norms [..] fp32
 *   block_table (B, max_blocks) int32: token t of batch entry b is row t % block_size of block
 *               block_table[b][t / block_size]; entries past an entry's length are not read
 *   seq_lens    (B) int32: tokens of each entry (0 gives a zero output row); values above
 *               max_kv_len are clamped to it
 * max_kv_len sizes the split plan and the workspace (qkv_attention_workspace_bytes with kv_len =
 * max_kv_len); with `causal`, query row i of entry b sits at position seq_lens[b] - q_len + i.
 * Everything else as qkv_attention.  block_size a multiple of 16 keeps d = 128, 3/3-bit caches on
 * the tensor-core kernel. */
typedef struct {
  const uint8_t* k_codes;
  const uint8_t* k_signs;
  const float* k_norms;
  const uint8_t* v_codes;
  const float* v_norms;
  const int32_t* block_table;
  const int32_t* seq_lens;
  int max_blocks;
  int block_size;
} qkv_paged_cache_t;

int qkv_attention_paged(const void* q, int q_dtype, qkv_paged_cache_t pool,
                        int B, int Hq, int Hkv, int q_len, int64_t max_kv_len, int d,
                        int key_bits, int val_bits,
                        const float* Pi, const float* key_centroids, const float* val_centroids,
                        const float* S, float qjl_scale, float scale, int causal,
                        float* out, void* workspace, size_t workspace_bytes, void* stream);

/* Row scatter for appends into a paged pool: row i of src (n_rows rows of row_bytes bytes, a
 * multiple of 4) is written to row slots[i] of dst; a negative slot drops the row.  Stands where the
 * reference appends a block to its list (engine.py:145-172). */
int qkv_scatter_rows(const void* src, void* dst, const int64_t* slots, int64_t n_rows, int row_bytes,
                     void* stream);

/* ---- tile records: the cache layout of the fast decode path -----------------------------------------
 * For head_dim 128 with 3-bit keys (2-bit codes + sign bit) and 3-bit values the cache can be kept as
 * RECORDS of 16 consecutive tokens of one (batch, kv head): QKV_TILE_BYTES = 16 * 104 bytes, the same
 * bytes per token as the five planes of qkv_cache_t, arranged in the order in which the tensor-core
 * kernel consumes them (key codes and sign bits as the reference packs them, reference
 * packing.py:22-94, regrouped by lane; value codes as 6-bit fields that hold the two tokens of a
 * multiply-accumulate pair, each as a sign bit and a 2-bit magnitude index, so that a field is the
 * index of a table of ready operand pairs; norms last).  One record is one bulk copy for the
 * kernel.  The re-arrangement is an exact integer permutation: qkv_untile_rows returns the reference's
 * packed rows byte for byte.  The value half of the format presumes a value table with
 * centroid[7 - i] = -centroid[i] (Lloyd-Max tables of a symmetric density).
 *
 * qkv_tile_rows files n_rows tokens, given as dense row-major planes (what qkv_compress_ip /
 * qkv_compress_mse write with packed = 1: k_codes 32 B, k_signs 16 B, v_codes 48 B per row), into
 * records.  Token i goes to token slot  slots[i]  when slots != NULL (negative = drop), else to slot
 * (i / map.seg_len) * map.seg_stride + map.seg_off + i % map.seg_len; slot s is token s % 16 of record
 * s / 16.  For a contiguous cache of `capacity` tokens per segment: seg_len = new tokens per segment,
 * seg_stride = capacity, seg_off = tokens already stored.  Stands where the reference appends a block to
 * its list (engine.py:145-172).  A token's bits are written with plain stores where it owns whole bytes
 * and with atomic AND / OR where it shares a word with its neighbour, so any set of distinct slots may
 * be written by one call or by concurrent calls.  records must be 16-byte aligned. */
#define QKV_TILE_TOKENS 16
#define QKV_TILE_BYTES 1664
int qkv_tile_rows(const uint8_t* k_codes, const uint8_t* k_signs, const float* k_norms,
                  const uint8_t* v_codes, const float* v_norms, int64_t n_rows,
                  uint8_t* records, qkv_rows_t map, const int64_t* slots, void* stream);
/* Inverse: token slots -> dense row-major planes (n_rows rows each). */
int qkv_untile_rows(const uint8_t* records, qkv_rows_t map, const int64_t* slots, int64_t n_rows,
                    uint8_t* k_codes, uint8_t* k_signs, float* k_norms, uint8_t* v_codes, float* v_norms,
                    void* stream);

/* qkv_attention / qkv_attention_paged over a cache of tile records (d = 128, key_bits = val_bits = 3).
 *   contiguous (block_table == NULL): records [B*Hkv, capacity / 16, QKV_TILE_BYTES], capacity a
 *     multiple of 16, tokens 0..kv_len-1 of each segment attended;
 *   paged (block_table != NULL): records [num_blocks, Hkv, block_size / 16, QKV_TILE_BYTES], block_size a
 *     multiple of 16, block_table / seq_lens / max_blocks as in qkv_paged_cache_t, kv_len the host-known
 *     upper bound of seq_lens.
 * Tokens of the last record beyond the length are ignored whatever they hold.  Workspace as
 * qkv_attention_workspace_bytes.  Replaces QuashKVEngine.attention (reference engine.py:204-299).
 * The records and their kernel presume what the reference's Lloyd-Max tables satisfy: a symmetric value table
 * (c[7 - i] == -c[i]) and, with up to four query rows per KV head, a key table that is affine in the two bits
 * of its code (c[0] + c[3] == c[1] + c[2]).  A call with other tables writes NaN to `out`; keep such caches as
 * row-major planes and use qkv_attention. */
typedef struct {
  const uint8_t* records;
  int64_t capacity;
  const int32_t* block_table;
  const int32_t* seq_lens;
  int max_blocks;
  int block_size;
} qkv_tiled_cache_t;

int qkv_attention_tiled(const void* q, int q_dtype, qkv_tiled_cache_t cache,
                        int B, int Hq, int Hkv, int q_len, int64_t kv_len, int d,
                        int key_bits, int val_bits,
                        const float* Pi, const float* key_centroids, const float* val_centroids,
                        const float* S, float qjl_scale, float scale, int causal,
                        float* out, void* workspace, size_t workspace_bytes, void* stream);

/* ---- index scan ------------------------------------------------------------------------------
 * Replaces QuashIndex.search (reference nn_search/index.py:121-163):
 * score[m,n] = norm_n * (q_rot_m . c[code_n] + qjl_scale * sum(|q_rot_m| * S * (2*sign_n-1))),
 * then the k largest per query, descending; equal scores are ordered by lower id.
 *   db_codes [N, d*(bits-1)/8], db_signs [N, d/8] packed, db_norms [N] fp32
 *   queries  (M, d) fp32 contiguous
 *   id_base  added to every returned id (a shard's first global row)
 *   out_scores (M,k) fp32, out_ids (M,k) int64;  k <= QKV_INDEX_MAX_K and k <= N
 * qkv_index_scores writes the dense (M,N) score matrix instead (for k above the limit). */
#define QKV_INDEX_MAX_K 128
size_t qkv_index_workspace_bytes(int64_t N, int M, int d, int k);
int qkv_index_scan_topk(const float* queries, int M, int d,
                        const uint8_t* db_codes, const uint8_t* db_signs, const float* db_norms,
                        int64_t N, int bits,
                        const float* Pi, const float* centroids, const float* S, float qjl_scale,
                        int k, int64_t id_base, float* out_scores, int64_t* out_ids,
                        void* workspace, size_t workspace_bytes, void* stream);
int qkv_index_scores(const float* queries, int M, int d,
                     const uint8_t* db_codes, const uint8_t* db_signs, const float* db_norms,
                     int64_t N, int bits,
                     const float* Pi, const float* centroids, const float* S, float qjl_scale,
                     float* out_scores, void* workspace, size_t workspace_bytes, void* stream);

/* Merge per-shard candidate lists: in (M, n_lists*k_in) -> out (M, k_out), higher score
 * first, then lower id.  The reference has no sharded search; this is the step after an
 * all-gather of every shard's qkv_index_scan_topk result. */
int qkv_topk_merge(const float* in_scores, const int64_t* in_ids, int M, int64_t n_cand,
                   int k_out, float* out_scores, int64_t* out_ids, void* stream);

/* Diagnostics, no reference counterpart: how many bounded waits ran out on the current device since the
 * library was loaded: waits on the tcgen05 tensor core (a CTA that meets one finishes its work with the
 * fp32 CUDA-core arithmetic, so results stay correct) and waits on a record copy of
 * qkv_attention_tiled (that call's output is then not valid).  0 in a healthy run.  Synchronises the
 * device. */
int64_t qkv_tensor_core_timeouts(void);

#ifdef __cplusplus
}
#endif
#endif /* QUASHKV_B200_H */
