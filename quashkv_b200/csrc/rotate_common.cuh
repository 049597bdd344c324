// Argument blocks shared by the CUDA-core and the tensor-core rotation kernels.
#pragma once

#include "common.cuh"

namespace qkv {

enum { MODE_MSE = 0, MODE_IP = 1, MODE_MIXED = 2 };

struct CompressArgs {
  const void* x; int x_dtype; int64_t x_pitch; int64_t n_vec; int d;
  const float* Pi;
  int mode;
  const float* bounds0; int bits0;     // uniform / outlier table
  const float* bounds1; int bits1;     // regular table (mixed)
  const float* centroids;              // sign stage: centroids of table 0
  const float* centroids1;             // sign stage of the mixed mode: centroids of table 1
  const float* S;                      // sign stage (IP mode, or mixed mode with signs != nullptr)
  const uint8_t* is_outlier;           // mixed
  uint8_t* codes; uint8_t* signs; int packed; float* norms;
  qkv_rows_t rows;
  int skip_block_aligned;              // mixed, CUDA-core kernel: return if the outlier count is a multiple of 32
                                       // (the tcgen05 kernel launched before it took that case)
  int test_drop_mma;                   // test hook of the tcgen05 kernel: CTA 0 issues nothing for its second
                                       // tile, so the bounded wait on that accumulator runs out (nothing is left
                                       // in flight) and the CTA finishes with the fp32 chain
};

struct DecompressArgs {
  const uint8_t* codes; const uint8_t* signs; int packed; const float* norms;
  qkv_rows_t rows; int64_t n_vec; int d;
  const float* Pi;
  int mode;                            // MODE_MSE (signs may be set) or MODE_MIXED
  const float* cents0; int bits0;
  const float* cents1; int bits1;
  const uint8_t* is_outlier;
  const float* S; float qjl_scale;
  void* out; int out_dtype; int64_t out_pitch;
  int skip_block_aligned;              // mixed, CUDA-core kernel: return if the outlier count is a multiple of 32
  int test_drop_mma;                   // test hook of the tcgen05 kernel: CTA 0 issues nothing for its second tile, so
                                       // the bounded wait on that accumulator runs out (nothing is left in flight)
                                       // and the CTA finishes with the fp32 chain
};


// Tensor-core rotation (rotate_mma.cu): d == 128, uniform bit width.  Returns QKV_OK after launching.
bool compress_mma_ok(const CompressArgs& a);
int launch_compress_mma(const CompressArgs& a, cudaStream_t st);
bool decompress_mma_ok(const DecompressArgs& a);
// tcgen05 rotation (rotate_umma.cu, decompress_umma.cu): d == 128, packed rows.
bool compress_umma_ok(const CompressArgs& a);
int launch_compress_umma(const CompressArgs& a, cudaStream_t st);
bool decompress_umma_ok(const DecompressArgs& a);
int launch_decompress_umma(const DecompressArgs& a, cudaStream_t st);
unsigned int umma_timeouts();             // bounded waits on the tensor core that ran out (device-wide counter)
int launch_decompress_mma(const DecompressArgs& a, cudaStream_t st);

}  // namespace qkv
