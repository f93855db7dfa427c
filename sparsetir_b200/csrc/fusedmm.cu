// Sparse attention over the stored positions of a CSR pattern, fp32, in one pass:
//   score[i,j] = <Q[i,:], K[j,:]>,  P[i,j] = exp(score[i,j]) / sum_j exp(score[i,j] - max_j score[i,j]),
//   O[i,:] = sum_j P[i,j] V[j,:]
// Semantics: `fusedmm` of examples/flash_graph_attention/fusedmm.py:37-96 of the reference (an
// SDDMM, the reference's sparse softmax — whose numerator is not shifted by the row maximum —
// and an SpMM written as one function; the reference has no schedule for it yet).
//
// One sub-warp owns a row and walks its neighbours once, a batch at a time: scores of the batch
// against the row's Q (kept in registers), then the running maximum / running sum / output
// accumulator updated the way FlashAttention does (one rescaling by exp(old max - new max) per
// batch), then the batch's V rows weighted and added.  No per-position intermediate is written: the scores and
// probabilities of config-sized graphs (1.2e8 positions) would be 0.9 GB of traffic each way.
// At the end O = acc * exp(max) / sum, which is the reference's unshifted numerator.
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "common.h"
#include "vec.cuh"

namespace sptir {
namespace {

constexpr int kThreads = 256;

template <int LPR>
__device__ __forceinline__ float sub_max(float v, unsigned mask) {
#pragma unroll
  for (int o = LPR / 2; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(mask, v, o, LPR));
  return v;
}
template <int LPR>
__device__ __forceinline__ float sub_sum(float v, unsigned mask) {
#pragma unroll
  for (int o = LPR / 2; o >= 1; o >>= 1) v += __shfl_xor_sync(mask, v, o, LPR);
  return v;
}

// A batch is LPR neighbours.  (1) their scores: K rows gathered U at a time, LPR partial dot
// products per lane, one transposing butterfly that leaves lane l with the score of neighbour l
// (as in the SDDMM kernel); (2) the softmax bookkeeping once per batch and lane-parallel: batch
// maximum, ONE rescaling of the running sum and accumulator, one exponential per lane = per
// neighbour; (3) V rows gathered U at a time and added with the neighbour's probability
// broadcast by shuffle.
template <int LPR, int VPL>  // a lane owns VPL 16-byte pieces of a feature row: feat = 4 * LPR * VPL
__global__ void __launch_bounds__(kThreads)
fusedmm_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
               float* __restrict__ o, const int32_t* __restrict__ indptr,
               const int32_t* __restrict__ indices, int m) {
  constexpr int U = (VPL >= 4 ? 1 : (VPL == 2 ? 2 : 4)) < LPR ? (VPL >= 4 ? 1 : (VPL == 2 ? 2 : 4)) : LPR;
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
    // (1) scores; positions past the end ask for row 0 and are masked below
    float part[LPR];
#pragma unroll
    for (int k0 = 0; k0 < LPR; k0 += U) {
      if (k0 < cnt) {
        float4 kx[U][VPL];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t src = static_cast<size_t>(__shfl_sync(mask, cid, k0 + u, LPR)) * ROW_VECS;
#pragma unroll
          for (int t = 0; t < VPL; ++t) kx[u][t] = __ldg(kv + src + t * LPR + lane);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float s = 0.f;
#pragma unroll
          for (int t = 0; t < VPL; ++t) s = Vec<4>::dot(qr[t], kx[u][t], s);
          part[k0 + u] = s;
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) part[k0 + u] = 0.f;
      }
    }
#pragma unroll
    for (int offl = LPR / 2, nn = LPR; offl >= 1; offl >>= 1, nn >>= 1) {
      const bool upper = (lane & offl) != 0;
#pragma unroll
      for (int i = 0; i < nn / 2; ++i) {
        const float send = upper ? part[i] : part[i + nn / 2];
        const float keep = upper ? part[i + nn / 2] : part[i];
        part[i] = keep + __shfl_xor_sync(mask, send, offl, LPR);
      }
    }
    // (2) lane l now holds the score of neighbour l
    const bool live = lane < cnt;
    const float sc = live ? part[0] : -INFINITY;
    const float mnew = fmaxf(mrun, sub_max<LPR>(sc, mask));
    const float scale = expf(mrun - mnew);  // 0 on the first batch (mrun = -inf)
    const float prob = live ? expf(sc - mnew) : 0.f;
    lsum = lsum * scale + sub_sum<LPR>(prob, mask);
    mrun = mnew;
#pragma unroll
    for (int t = 0; t < VPL; ++t) {
      acc[t].x *= scale; acc[t].y *= scale; acc[t].z *= scale; acc[t].w *= scale;
    }
    // (3) acc += P V
#pragma unroll
    for (int k0 = 0; k0 < LPR; k0 += U) {
      if (k0 < cnt) {
        float4 vx[U][VPL];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t src = static_cast<size_t>(__shfl_sync(mask, cid, k0 + u, LPR)) * ROW_VECS;
#pragma unroll
          for (int t = 0; t < VPL; ++t) vx[u][t] = __ldg(vv + src + t * LPR + lane);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float pj = __shfl_sync(mask, prob, k0 + u, LPR);  // 0 past the end
#pragma unroll
          for (int t = 0; t < VPL; ++t) Vec<4>::fma(acc[t], pj, vx[u][t]);
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
  // Default: the three operators one after the other.  Their kernels split long rows over many
  // warps and walk the features tile by tile, and measured 1.6-3 x faster than the one-pass
  // kernel (0.39 against 0.63 ms on 7.4 M positions at F = 64 with K and V in L2; 4.2 against
  // 15.5 ms on 117 M positions, where K and V no longer fit).  SPARSETIR_FUSEDMM_PATH=fused
  // selects the one-pass kernel, which needs no per-position scratch memory.
  static const bool one_pass = [] {
    const char* e = std::getenv("SPARSETIR_FUSEDMM_PATH");
    return e && std::strcmp(e, "fused") == 0;
  }();
  if (vec && one_pass) {
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
