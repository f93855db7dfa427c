// Sparse attention over the stored positions of a CSR pattern, fp32, in one pass:
//   score[i,j] = <Q[i,:], K[j,:]>,  P[i,j] = exp(score[i,j]) / sum_j exp(score[i,j] - max_j score[i,j]),
//   O[i,:] = sum_j P[i,j] V[j,:]
// Semantics: `fusedmm` of examples/flash_graph_attention/fusedmm.py:37-96 of the reference (an
// SDDMM, the reference's sparse softmax — whose numerator is not shifted by the row maximum —
// and an SpMM written as one function; the reference has no schedule for it yet).
//
// One sub-warp owns a row and walks its neighbours once: the K rows of a few neighbours are
// gathered together, the dot products with the row's Q (kept in registers) are reduced over the
// sub-warp, and the running maximum / running sum / output accumulator are updated the way
// FlashAttention does (rescaling by exp(old max - new max)), while the V rows of the same
// neighbours are already on their way.  No per-position intermediate is written: the scores and
// probabilities of config-sized graphs (1.2e8 positions) would be 0.9 GB of traffic each way.
// At the end O = acc * exp(max) / sum, which is the reference's unshifted numerator.
#include <cmath>

#include "common.h"
#include "vec.cuh"

namespace sptir {
namespace {

constexpr int kThreads = 256;

template <int LPR, int VPL>  // a lane owns VPL 16-byte pieces of a feature row: feat = 4 * LPR * VPL
__global__ void __launch_bounds__(kThreads)
fusedmm_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
               float* __restrict__ o, const int32_t* __restrict__ indptr,
               const int32_t* __restrict__ indices, int m) {
  constexpr int U = VPL >= 4 ? 1 : (VPL == 2 ? 2 : 4);  // neighbours in flight (K and V rows)
  constexpr int ROW_VECS = LPR * VPL;
  const int lane = threadIdx.x % LPR;
  const unsigned mask = group_mask<LPR>();
  const long long row = static_cast<long long>(blockIdx.x) * (kThreads / LPR) + threadIdx.x / LPR;
  if (row >= m) return;
  const int p0 = __ldg(indptr + row), p1 = __ldg(indptr + row + 1);
  const float4* qv = reinterpret_cast<const float4*>(q) + static_cast<size_t>(row) * ROW_VECS;
  const float4* kv = reinterpret_cast<const float4*>(k);
  const float4* vv = reinterpret_cast<const float4*>(v);
  float4 qr[VPL], acc[VPL];
#pragma unroll
  for (int t = 0; t < VPL; ++t) {
    qr[t] = __ldg(qv + t * LPR + lane);
    acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float mrun = -INFINITY, lsum = 0.f;

  int cid = (p0 + lane < p1) ? __ldg(indices + p0 + lane) : 0;
  for (int s0 = p0; s0 < p1; s0 += LPR) {
    int cidn = 0;
    if (s0 + LPR + lane < p1) cidn = __ldg(indices + s0 + LPR + lane);  // ids of the next batch
    const int cnt = min(LPR, p1 - s0);
    for (int k0 = 0; k0 < cnt; k0 += U) {
      float4 kx[U][VPL], vx[U][VPL];
      float part[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {  // positions past the end ask for row 0: never used
        const size_t src = static_cast<size_t>(__shfl_sync(mask, cid, min(k0 + u, LPR - 1), LPR)) * ROW_VECS;
#pragma unroll
        for (int t = 0; t < VPL; ++t) kx[u][t] = __ldg(kv + src + t * LPR + lane);
#pragma unroll
        for (int t = 0; t < VPL; ++t) vx[u][t] = __ldg(vv + src + t * LPR + lane);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float s = 0.f;
#pragma unroll
        for (int t = 0; t < VPL; ++t) s = Vec<4>::dot(qr[t], kx[u][t], s);
        part[u] = s;
      }
#pragma unroll
      for (int off = LPR / 2; off >= 1; off >>= 1) {
#pragma unroll
        for (int u = 0; u < U; ++u) part[u] += __shfl_xor_sync(mask, part[u], off, LPR);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k0 + u < cnt) {  // uniform inside the sub-warp
          const float mnew = fmaxf(mrun, part[u]);
          const float scale = expf(mrun - mnew);  // 0 on the first position (mrun = -inf)
          const float p = expf(part[u] - mnew);
          lsum = lsum * scale + p;
#pragma unroll
          for (int t = 0; t < VPL; ++t) {
            acc[t].x = fmaf(acc[t].x, scale, p * vx[u][t].x);
            acc[t].y = fmaf(acc[t].y, scale, p * vx[u][t].y);
            acc[t].z = fmaf(acc[t].z, scale, p * vx[u][t].z);
            acc[t].w = fmaf(acc[t].w, scale, p * vx[u][t].w);
          }
          mrun = mnew;
        }
      }
    }
    cid = cidn;
  }
  // rows without stored positions: zeros
  const float f = p1 > p0 ? expf(mrun) / lsum : 0.f;
  float4* ov = reinterpret_cast<float4*>(o) + static_cast<size_t>(row) * ROW_VECS;
#pragma unroll
  for (int t = 0; t < VPL; ++t)
    ov[t * LPR + lane] = make_float4(acc[t].x * f, acc[t].y * f, acc[t].z * f, acc[t].w * f);
}

template <int LPR, int VPL>
int launch(const float* q, const float* k, const float* v, float* o, const int32_t* indptr,
           const int32_t* indices, int m, cudaStream_t st) {
  fusedmm_kernel<LPR, VPL><<<ceil_div(m, kThreads / LPR), kThreads, 0, st>>>(q, k, v, o, indptr, indices, m);
  SPTIR_LAUNCH_OK("fusedmm_kernel");
  return 0;
}

}  // namespace
}  // namespace sptir

extern "C" int sparsetir_sddmm_raw(const float* a, const float* b, float* c, const int32_t* indptr,
                                   const int32_t* indices, const float* scale, int m, int n, int feat,
                                   int nnz, int device_id, void* stream);
extern "C" int sparsetir_sparse_softmax_raw(const float* a, float* b, const int32_t* indptr, int n, int nnz,
                                            int device_id, void* stream);
extern "C" int sparsetir_csrmm_raw(const float* a, const float* b, float* c, const int32_t* indptr,
                                   const int32_t* indices, int m, int n, int feat, int nnz, int device_id,
                                   void* stream);

extern "C" int sparsetir_fusedmm_raw(const float* q, const float* k, const float* v, float* o,
                                     const int32_t* indptr, const int32_t* indices, int m, int n, int nnz,
                                     int feat, int device_id, void* stream) {
  using namespace sptir;
  if (m < 0 || n < 0 || nnz < 0 || feat < 0) return fail("sparsetir_fusedmm: negative size");
  if (m == 0 || feat == 0) return 0;
  if (!q || !o || !indptr || (nnz > 0 && (!k || !v || !indices)))
    return fail("sparsetir_fusedmm: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o);
  if (vec) {
    switch (feat) {
      case 16: return launch<4, 1>(q, k, v, o, indptr, indices, m, st);
      case 32: return launch<8, 1>(q, k, v, o, indptr, indices, m, st);
      case 64: return launch<16, 1>(q, k, v, o, indptr, indices, m, st);
      case 128: return launch<32, 1>(q, k, v, o, indptr, indices, m, st);
      case 256: return launch<32, 2>(q, k, v, o, indptr, indices, m, st);
      case 512: return launch<32, 4>(q, k, v, o, indptr, indices, m, st);
      default: break;
    }
  }
  // other feature sizes: the three operators one after the other, the per-position scores and
  // probabilities in the per-stream workspace (scores first: the SpMM's own use of the workspace
  // for its hub-row list falls into that half, which is dead by then)
  if (nnz == 0) {
    SPTIR_CUDA_OK(cudaMemsetAsync(o, 0, static_cast<size_t>(m) * feat * sizeof(float), st));
    return 0;
  }
  float* ws = static_cast<float*>(workspace(device_id, st, 2 * static_cast<size_t>(nnz) * sizeof(float)));
  if (!ws) return -1;
  if (sparsetir_sddmm_raw(q, k, ws, indptr, indices, nullptr, m, n, feat, nnz, device_id, stream) != 0) return -1;
  if (sparsetir_sparse_softmax_raw(ws, ws + nnz, indptr, m, nnz, device_id, stream) != 0) return -1;
  return sparsetir_csrmm_raw(ws + nnz, v, o, indptr, indices, m, n, feat, nnz, device_id, stream);
}
