// BSR SpMM, fp16 blocks and dense operand, fp32 accumulation and output:
//   C[i*blk+bi, f] = sum_{p in block-row i} sum_bj A[p,bi,bj] * B[indices[p]*blk+bj, f]
// Semantics: tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:192-249 of the
// reference; generated kernel being replaced: examples/blocksparse/bsr_spmm.py:359-425 (wmma,
// fp16 accumulate).  Block-rows without blocks are written as zeros (T.init of the reference).
//
// This file holds the CUDA-core kernel that works for every block size; bsrmm_tc.cu holds the
// tensor-core kernel for the block sizes it supports and is tried first.
#include <cuda_fp16.h>

#include "common.h"

namespace sptir {

// defined in bsrmm_tc.cu; returns 1 when the shape is not supported by the tensor-core path
int bsrmm_tc_launch(const __half* a, const __half* b, float* c, const int32_t* indptr,
                    const int32_t* indices, int nb, int mb, int nnzb, int blk, int feat,
                    cudaStream_t stream);

namespace {

constexpr int kThreads = 128;
constexpr int kBi = 8;  // output rows of the block handled per thread block pass

// One thread block per (block-row, tile of 128 features, group of kBi rows inside the block).
// Thread t owns feature f = tile*128 + t and kBi accumulators; the A sub-block is staged in
// shared memory, B rows are read coalesced.
__global__ void __launch_bounds__(kThreads)
bsrmm_simt_kernel(const __half* __restrict__ a, const __half* __restrict__ b,
                  float* __restrict__ c, const int32_t* __restrict__ indptr,
                  const int32_t* __restrict__ indices, int blk, int feat) {
  extern __shared__ float a_s[];  // [kBi][blk]
  const int i = blockIdx.x;
  const int f = blockIdx.y * kThreads + threadIdx.x;
  const int bi0 = blockIdx.z * kBi;
  const int nbi = min(kBi, blk - bi0);
  float acc[kBi];
#pragma unroll
  for (int r = 0; r < kBi; ++r) acc[r] = 0.f;
  const int p0 = __ldg(indptr + i), p1 = __ldg(indptr + i + 1);
  for (int p = p0; p < p1; ++p) {
    __syncthreads();
    for (int t = threadIdx.x; t < nbi * blk; t += kThreads) {
      int r = t / blk, bj = t % blk;
      a_s[r * blk + bj] = __half2float(a[(static_cast<size_t>(p) * blk + bi0 + r) * blk + bj]);
    }
    __syncthreads();
    if (f < feat) {
      const __half* brow = b + static_cast<size_t>(__ldg(indices + p)) * blk * feat + f;
      for (int bj = 0; bj < blk; ++bj) {
        float bv = __half2float(brow[static_cast<size_t>(bj) * feat]);
#pragma unroll
        for (int r = 0; r < kBi; ++r)
          if (r < nbi) acc[r] = fmaf(a_s[r * blk + bj], bv, acc[r]);
      }
    }
  }
  if (f < feat) {
#pragma unroll
    for (int r = 0; r < kBi; ++r)
      if (r < nbi) c[(static_cast<size_t>(i) * blk + bi0 + r) * feat + f] = acc[r];
  }
}

}  // namespace
}  // namespace sptir

extern "C" int sparsetir_bsrmm_raw(const void* a_f16, const void* b_f16, float* c,
                                   const int32_t* indptr, const int32_t* indices, int nb, int mb,
                                   int nnzb, int blk, int feat, int device_id, void* stream) {
  using namespace sptir;
  if (nb < 0 || mb < 0 || nnzb < 0 || blk < 1 || feat < 0)
    return fail("sparsetir_bsrmm: invalid size");
  if (nb == 0 || feat == 0) return 0;
  if (!c || !indptr || (nnzb > 0 && (!a_f16 || !b_f16 || !indices)))
    return fail("sparsetir_bsrmm: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (validate_enabled() && validate_csr("sparsetir_bsrmm", indptr, nb, indices, nnzb, mb, st) != 0) return -1;
  const __half* a = static_cast<const __half*>(a_f16);
  const __half* b = static_cast<const __half*>(b_f16);
  int rc = bsrmm_tc_launch(a, b, c, indptr, indices, nb, mb, nnzb, blk, feat, st);
  if (rc <= 0) return rc;
  dim3 grid(nb, ceil_div(feat, kThreads), ceil_div(blk, kBi));
  if (grid.y > 65535 || grid.z > 65535) return fail("sparsetir_bsrmm: shape exceeds the grid limits");
  size_t smem = static_cast<size_t>(kBi) * blk * sizeof(float);
  if (smem > 48 * 1024) return fail("sparsetir_bsrmm: block size %d is too large", blk);
  bsrmm_simt_kernel<<<grid, kThreads, smem, st>>>(a, b, c, indptr, indices, blk, feat);
  SPTIR_LAUNCH_OK("bsrmm_simt_kernel");
  return 0;
}
