// The small operators either side of SpMM / SDDMM in the reference's script collection, fp32:
//   csr_reduce / segment_reduce  B[i] = sum_j A[i,j]                  (sparse_tir_scripts.py:74-110)
//   sparse_softmax               B[i,j] = exp(A[i,j]) / sum_j exp(A[i,j] - max_j A[i,j])   (:503-528)
//   csr2bsr                      scatter of CSR entries into the blocks of a BSR matrix      (:532-557)
//   ellmm                        block-ELL SpMM C[i,bi,f] = sum_j sum_bj A[i,j,bi,bj] B[ind[i,j],bj,f] (:150-181)
// All four stream their operands once: a sub-warp per row (4 lanes for short rows, a warp for
// long ones) for the row-wise ones, a thread per entry for the scatter, a block per block row
// and 128 features for the block-ELL product.
#include <cfloat>

#include "common.h"
#include "vec.cuh"

namespace sptir {
namespace {

constexpr int kThreads = 256;

template <int LPR>
__device__ __forceinline__ float group_sum(float v, unsigned mask) {
#pragma unroll
  for (int o = LPR / 2; o >= 1; o >>= 1) v += __shfl_xor_sync(mask, v, o, LPR);
  return v;
}
template <int LPR>
__device__ __forceinline__ float group_max(float v, unsigned mask) {
#pragma unroll
  for (int o = LPR / 2; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(mask, v, o, LPR));
  return v;
}

template <int LPR>
__global__ void __launch_bounds__(kThreads)
csr_reduce_kernel(const float* __restrict__ a, float* __restrict__ b, const int32_t* __restrict__ indptr,
                  int n) {
  const int lane = threadIdx.x % LPR;
  const unsigned mask = group_mask<LPR>();
  const long long row = static_cast<long long>(blockIdx.x) * (kThreads / LPR) + threadIdx.x / LPR;
  if (row >= n) return;
  const int p0 = __ldg(indptr + row), p1 = __ldg(indptr + row + 1);
  float s = 0.f;
  for (int p = p0 + lane; p < p1; p += LPR) s += __ldg(a + p);
  s = group_sum<LPR>(s, mask);
  if (lane == 0) b[row] = s;
}

// Each lane keeps the first CACHE of its entries of the row in registers (LPR * CACHE entries
// per row: the whole row in the common case), so the row is read from memory once instead of
// three times; exp(a) = exp(a - max) * exp(max) saves the second exponential per entry.
template <int LPR, int CACHE>
__global__ void __launch_bounds__(kThreads)
sparse_softmax_kernel(const float* __restrict__ a, float* __restrict__ b,
                      const int32_t* __restrict__ indptr, int n) {
  const int lane = threadIdx.x % LPR;
  const unsigned mask = group_mask<LPR>();
  const long long row = static_cast<long long>(blockIdx.x) * (kThreads / LPR) + threadIdx.x / LPR;
  if (row >= n) return;
  const int p0 = __ldg(indptr + row), p1 = __ldg(indptr + row + 1);
  float v[CACHE];
  float mx = -FLT_MAX;
#pragma unroll
  for (int k = 0; k < CACHE; ++k) {
    const int p = p0 + lane + k * LPR;
    v[k] = p < p1 ? __ldg(a + p) : -FLT_MAX;
    mx = fmaxf(mx, v[k]);
  }
  for (int p = p0 + lane + CACHE * LPR; p < p1; p += LPR) mx = fmaxf(mx, __ldg(a + p));
  mx = group_max<LPR>(mx, mask);
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < CACHE; ++k) {
    v[k] = (p0 + lane + k * LPR < p1) ? __expf(v[k] - mx) : 0.f;
    s += v[k];
  }
  for (int p = p0 + lane + CACHE * LPR; p < p1; p += LPR) s += expf(__ldg(a + p) - mx);
  s = group_sum<LPR>(s, mask);
  // the reference divides exp(A) — not exp(A - max) — by the shifted sum
  const float scale = expf(mx) / s;
#pragma unroll
  for (int k = 0; k < CACHE; ++k) {
    const int p = p0 + lane + k * LPR;
    if (p < p1) b[p] = v[k] * scale;
  }
  for (int p = p0 + lane + CACHE * LPR; p < p1; p += LPR) b[p] = expf(__ldg(a + p) - mx) * scale;
}

// row of entry p by the search of the lowered code; position of the block by lower bound
__global__ void __launch_bounds__(kThreads)
csr2bsr_kernel(const float* __restrict__ a, float* __restrict__ b, const int32_t* __restrict__ indptr_in,
               const int32_t* __restrict__ indices_in, const int32_t* __restrict__ indptr_out,
               const int32_t* __restrict__ indices_out, int m_in, int nnz_in, int blk) {
  const long long p = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  if (p >= nnz_in) return;
  int lo = 0, hi = m_in + 1;  // row(p) = upper_bound(indptr_in, p) - 1
  while (lo < hi) {
    const int mid = lo + (hi - lo) / 2;
    if (__ldg(indptr_in + mid) > p) hi = mid; else lo = mid + 1;
  }
  const int i = lo - 1;
  const int j = __ldg(indices_in + p);
  const int bo = __ldg(indptr_out + i / blk);
  int low = 0, high = __ldg(indptr_out + i / blk + 1) - bo;
  const int key = j / blk;
  while (low < high) {
    const int mid = low + (high - low) / 2;
    if (__ldg(indices_out + mid + bo) < key) low = mid + 1; else high = mid;
  }
  b[(static_cast<size_t>(low + bo) * blk + i % blk) * blk + j % blk] = __ldg(a + p);
}

// block (block row i, 128 features): the row's A blocks go through shared memory one at a time;
// a thread owns feature f of 128 and walks the block's rows
constexpr int kTileF = 128;
__global__ void __launch_bounds__(kTileF)
ellmm_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
             const int32_t* __restrict__ indices, int col, int blk, int feat) {
  extern __shared__ float s_a[];  // blk x blk
  const int i = blockIdx.x;
  const int f = blockIdx.y * kTileF + threadIdx.x;
  const bool live = f < feat;
  for (int bi0 = 0; bi0 < blk; bi0 += 8) {  // 8 output rows per pass keep the accumulators in registers
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
    for (int j = 0; j < col; ++j) {
      const float* ab = a + (static_cast<size_t>(i) * col + j) * blk * blk;
      __syncthreads();
      for (int e = threadIdx.x; e < blk * blk; e += kTileF) s_a[e] = __ldg(ab + e);
      __syncthreads();
      const float* bb = b + static_cast<size_t>(__ldg(indices + static_cast<size_t>(i) * col + j)) * blk * feat;
      if (live) {
        for (int bj = 0; bj < blk; ++bj) {
          const float x = __ldg(bb + static_cast<size_t>(bj) * feat + f);
#pragma unroll
          for (int r = 0; r < 8; ++r)
            if (bi0 + r < blk) acc[r] = fmaf(s_a[(bi0 + r) * blk + bj], x, acc[r]);
        }
      }
    }
    if (live) {
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (bi0 + r < blk) c[(static_cast<size_t>(i) * blk + bi0 + r) * feat + f] = acc[r];
    }
  }
}

}  // namespace
}  // namespace sptir

extern "C" int sparsetir_csr_reduce_raw(const float* a, float* b, const int32_t* indptr, int n, int nnz,
                                        int device_id, void* stream) {
  using namespace sptir;
  if (n < 0 || nnz < 0) return fail("sparsetir_csr_reduce: negative size");
  if (n == 0) return 0;
  if (!b || !indptr || (nnz > 0 && !a)) return fail("sparsetir_csr_reduce: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (validate_enabled() && validate_indptr("sparsetir_csr_reduce", "indptr", indptr, n, nnz, st) != 0) return -1;
  if (static_cast<double>(nnz) / n >= 24.0) {
    csr_reduce_kernel<32><<<ceil_div(n, kThreads / 32), kThreads, 0, st>>>(a, b, indptr, n);
  } else {
    csr_reduce_kernel<4><<<ceil_div(n, kThreads / 4), kThreads, 0, st>>>(a, b, indptr, n);
  }
  SPTIR_LAUNCH_OK("csr_reduce_kernel");
  return 0;
}

extern "C" int sparsetir_sparse_softmax_raw(const float* a, float* b, const int32_t* indptr, int n,
                                            int nnz, int device_id, void* stream) {
  using namespace sptir;
  if (n < 0 || nnz < 0) return fail("sparsetir_sparse_softmax: negative size");
  if (n == 0 || nnz == 0) return 0;
  if (!a || !b || !indptr) return fail("sparsetir_sparse_softmax: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (validate_enabled() && validate_indptr("sparsetir_sparse_softmax", "indptr", indptr, n, nnz, st) != 0) return -1;
  if (static_cast<double>(nnz) / n >= 24.0) {
    sparse_softmax_kernel<32, 16><<<ceil_div(n, kThreads / 32), kThreads, 0, st>>>(a, b, indptr, n);
  } else {
    sparse_softmax_kernel<4, 4><<<ceil_div(n, kThreads / 4), kThreads, 0, st>>>(a, b, indptr, n);
  }
  SPTIR_LAUNCH_OK("sparse_softmax_kernel");
  return 0;
}

extern "C" int sparsetir_csr2bsr_raw(const float* a, float* b, const int32_t* indptr_in,
                                     const int32_t* indices_in, const int32_t* indptr_out,
                                     const int32_t* indices_out, int m_in, int nnz_in, int blk,
                                     int device_id, void* stream) {
  using namespace sptir;
  if (m_in < 0 || nnz_in < 0 || blk < 1) return fail("sparsetir_csr2bsr: invalid size");
  if (nnz_in == 0) return 0;
  if (!a || !b || !indptr_in || !indices_in || !indptr_out || !indices_out)
    return fail("sparsetir_csr2bsr: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  csr2bsr_kernel<<<ceil_div(nnz_in, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      a, b, indptr_in, indices_in, indptr_out, indices_out, m_in, nnz_in, blk);
  SPTIR_LAUNCH_OK("csr2bsr_kernel");
  return 0;
}

extern "C" int sparsetir_ellmm_raw(const float* a, const float* b, float* c, const int32_t* indices,
                                   int nb, int mb, int feat, int col, int blk, int device_id,
                                   void* stream) {
  using namespace sptir;
  (void)mb;
  if (nb < 0 || feat < 0 || col < 0 || blk < 1) return fail("sparsetir_ellmm: invalid size");
  if (nb == 0 || feat == 0) return 0;
  if (!c || (col > 0 && (!a || !b || !indices))) return fail("sparsetir_ellmm: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  const size_t smem = static_cast<size_t>(blk) * blk * sizeof(float);
  if (smem > 48 * 1024) return fail("sparsetir_ellmm: block size %d is too large", blk);
  if (ceil_div(feat, kTileF) > 65535) return fail("sparsetir_ellmm: feat_size %d is too large", feat);
  dim3 grid(nb, ceil_div(feat, kTileF));
  ellmm_kernel<<<grid, kTileF, smem, static_cast<cudaStream_t>(stream)>>>(a, b, c, indices, col, blk, feat);
  SPTIR_LAUNCH_OK("ellmm_kernel");
  return 0;
}
