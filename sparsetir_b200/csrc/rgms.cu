// RGMS (relational gather-matmul-scatter), fp32:
//   Y[I[i], fo] += sum_{p in CSF row i of relation r} A[p] * sum_fi W[r,fo,fi] * X[J[p],fi]
// Semantics: tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:902-995
// (rgcn_hetero_forward) with Y zero-filled by the caller and accumulated over relations, as the
// runnable reference kernels do (examples/rgms/rgcn/bench_rgcn_non_composable.py:85-108,
// bench_rgcn_composable.py:176-222, bench_rgcn_tensorcore.py:651-858).
//
// Formulation.  The reference multiplies every gathered X row by W_r and then aggregates
// (2*E*F*F flops).  Matrix multiplication distributes over the aggregation, so this kernel
// aggregates first and transforms once per (relation, destination row):
//   Z[i,:] = sum_p A[p] * X[J[p],:]          (gather, memory bound)
//   Y[I[i],:] += Z[i,:] * W_r^T               (dense [TM x F] x [F x F] tile product)
// which needs 2*E*F + 2*nnz_i*F*F flops.  Results differ from the reference order only by
// fp32 re-association.
//
// One thread block owns a tile of up to TM consecutive CSF rows of ONE relation:
//   phase 1  sub-warps gather-aggregate the tile's rows into shared memory (spmm_core.cuh);
//   phase 2  the tile product with W_r staged (transposed) in shared memory;
//   phase 3  the result goes back through shared memory so that every destination row is
//            scattered with 16-byte vector atomics over contiguous addresses.
// Tiles are numbered relation by relation; a block finds its (relation, tile) with a block-wide
// prefix scan over the relation sizes, so no tile table has to be built or stored anywhere.
#include <cstdlib>

#include <cstring>

#include "common.h"
#include "rgms_common.cuh"
#include "spmm_core.cuh"

namespace sptir {

// defined in csrmm.cu: the CSR SpMM launcher with 32-byte lanes, never the hub-row launches
int csrmm_short_rows_impl(const float* a, const float* b, float* c, const int32_t* indptr,
                          const int32_t* indices, int m, int n, int feat, int nnz, int device_id,
                          void* stream);
int rgms_fused_launch(const float* a, const float* w, const float* x, float* y, const int32_t* indptr_i,
                      const int32_t* indices_i, const int32_t* indptr_j, const int32_t* indices_j,
                      int num_rels, int feat, int nnz_i, int nnz_j, int n, int m, cudaStream_t stream);
int rgms_tc_launch(const float* a, const float* w, const float* x, float* y,
                   const int32_t* indptr_i, const int32_t* indices_i, const int32_t* indptr_j,
                   const int32_t* indices_j, int num_rels, int feat, int nnz_i,
                   const float* z, cudaStream_t stream);

namespace {

constexpr int kThreads = kRgmsThreads;
constexpr int kTM = 128;

template <int F>
__global__ void __launch_bounds__(kThreads)
rgms_tile_kernel(const float* __restrict__ a, const float* __restrict__ w,
                 const float* __restrict__ x, float* __restrict__ y,
                 const int32_t* __restrict__ indptr_i, const int32_t* __restrict__ indices_i,
                 const int32_t* __restrict__ indptr_j, const int32_t* __restrict__ indices_j,
                 int num_rels) {
  constexpr int LPR = F / 4;       // lanes that cover one feature row with 16-byte pieces
  constexpr int SUBS = kThreads / LPR;
  constexpr int ZS = F + 1;        // padded row stride of the Z tile: conflict-free column reads
  constexpr int FO = F / 2;        // outputs per thread in phase 2 (two threads per tile row)
  extern __shared__ float smem[];
  float* zt = smem;                // [kTM][ZS]
  float* wt = smem + kTM * ZS;     // [F fi][F fo]  (W_r transposed)

  int rel, row0, row1;
  if (!locate_tile(indptr_i, num_rels, kTM, blockIdx.x, &rel, &row0, &row1)) return;
  const int nrows = row1 - row0;

  // stage W_r^T: wt[fi][fo] = W[rel, fo, fi]
  const float* wr = w + static_cast<size_t>(rel) * F * F;
  for (int t = threadIdx.x; t < F * F; t += kThreads) {
    int fo = t / F, fi = t % F;
    wt[fi * F + fo] = __ldg(wr + t);
  }

  // phase 1: gather-aggregate
  {
    const int lane = threadIdx.x % LPR;
    gather_tile_rows<F, kTM>(a, x, indptr_j, indices_j, row0, nrows, [&](int t, float4 v) {
      float* dst = zt + t * ZS + lane * 4;
      dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    });
  }
  __syncthreads();

  // phase 2: Y_tile[t, fo] = sum_fi Z[t, fi] * W[rel, fo, fi]
  const int t = threadIdx.x % kTM;
  const int fo0 = (threadIdx.x / kTM) * FO;
  float acc[FO];
#pragma unroll
  for (int k = 0; k < FO; ++k) acc[k] = 0.f;
  for (int fi = 0; fi < F; ++fi) {
    const float z = zt[t * ZS + fi];
    const float4* wrow = reinterpret_cast<const float4*>(wt + fi * F + fo0);
#pragma unroll
    for (int k = 0; k < FO / 4; ++k) {
      float4 wv = wrow[k];
      acc[4 * k + 0] = fmaf(z, wv.x, acc[4 * k + 0]);
      acc[4 * k + 1] = fmaf(z, wv.y, acc[4 * k + 1]);
      acc[4 * k + 2] = fmaf(z, wv.z, acc[4 * k + 2]);
      acc[4 * k + 3] = fmaf(z, wv.w, acc[4 * k + 3]);
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < FO; ++k) zt[t * ZS + fo0 + k] = acc[k];
  __syncthreads();

  // phase 3: scatter rows with vector atomics
  {
    const int lane = threadIdx.x % LPR;
    for (int r = threadIdx.x / LPR; r < nrows; r += SUBS) {
      const float* src = zt + r * ZS + lane * 4;
      float4 v = make_float4(src[0], src[1], src[2], src[3]);
      float4* dst = reinterpret_cast<float4*>(y + static_cast<size_t>(__ldg(indices_i + row0 + r)) * F);
      atomicAdd(dst + lane, v);
    }
  }
}

// Any feature size: one warp per CSF row, scalar accumulation through shared memory.
__global__ void __launch_bounds__(kThreads)
rgms_generic_kernel(const float* __restrict__ a, const float* __restrict__ w,
                    const float* __restrict__ x, float* __restrict__ y,
                    const int32_t* __restrict__ indptr_i, const int32_t* __restrict__ indices_i,
                    const int32_t* __restrict__ indptr_j, const int32_t* __restrict__ indices_j,
                    int num_rels, int feat, int nnz_i) {
  extern __shared__ float zs[];  // [warps][feat]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long i = static_cast<long long>(blockIdx.x) * (kThreads / 32) + warp;
  if (i >= nnz_i) return;
  // relation of CSF row i: last r with indptr_i[r] <= i
  int lo = 0, hi = num_rels + 1;
  while (lo < hi) {
    int mid = lo + (hi - lo) / 2;
    if (__ldg(indptr_i + mid) > i) hi = mid; else lo = mid + 1;
  }
  const int rel = lo - 1;
  float* z = zs + warp * feat;
  for (int f = lane; f < feat; f += 32) z[f] = 0.f;
  const int p0 = __ldg(indptr_j + i), p1 = __ldg(indptr_j + i + 1);
  for (int p = p0; p < p1; ++p) {
    const float av = __ldg(a + p);
    const float* xr = x + static_cast<size_t>(__ldg(indices_j + p)) * feat;
    for (int f = lane; f < feat; f += 32) z[f] = fmaf(av, __ldg(xr + f), z[f]);
  }
  __syncwarp();
  const float* wr = w + static_cast<size_t>(rel) * feat * feat;
  float* yr = y + static_cast<size_t>(__ldg(indices_i + i)) * feat;
  for (int fo = lane; fo < feat; fo += 32) {
    const float* wrow = wr + static_cast<size_t>(fo) * feat;
    float s = 0.f;
    for (int fi = 0; fi < feat; ++fi) s = fmaf(__ldg(wrow + fi), z[fi], s);
    atomicAdd(yr + fo, s);
  }
}

template <int F>
int launch_tile(const float* a, const float* w, const float* x, float* y, const int32_t* indptr_i,
                const int32_t* indices_i, const int32_t* indptr_j, const int32_t* indices_j,
                int num_rels, int nnz_i, cudaStream_t st) {
  const size_t smem = (static_cast<size_t>(kTM) * (F + 1) + static_cast<size_t>(F) * F) * sizeof(float);
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(rgms_tile_kernel<F>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured_device = dev;
  }
  // upper bound on the number of tiles: every relation can add one partly filled tile
  const long long blocks = static_cast<long long>(nnz_i) / kTM + num_rels;
  rgms_tile_kernel<F><<<static_cast<unsigned>(blocks), kThreads, smem, st>>>(
      a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels);
  SPTIR_LAUNCH_OK("rgms_tile_kernel");
  return 0;
}

}  // namespace
}  // namespace sptir

extern "C" int sparsetir_rgms_workspace(int feat, int nnz_i, size_t* scratch_bytes) {
  if (!scratch_bytes || feat < 0 || nnz_i < 0) return sptir::fail("sparsetir_rgms_workspace: bad argument");
  // the two-launch form keeps one aggregated feature row per (relation, destination) pair
  *scratch_bytes = feat == 64 ? static_cast<size_t>(nnz_i) * 64 * sizeof(float) : 0;
  return 0;
}

extern "C" int sparsetir_rgms_raw(const float* a, const float* w, const float* x, float* y,
                                  const int32_t* indptr_i, const int32_t* indices_i,
                                  const int32_t* indptr_j, const int32_t* indices_j, int m, int n,
                                  int num_rels, int feat, int nnz_i, int nnz_j, int device_id,
                                  void* stream) {
  using namespace sptir;
  if (num_rels < 0 || feat < 0 || nnz_i < 0 || nnz_j < 0) return fail("sparsetir_rgms: negative size");
  if (nnz_i == 0 || feat == 0 || num_rels == 0) return 0;
  if (!w || !x || !y || !indptr_i || !indices_i || !indptr_j || (nnz_j > 0 && (!a || !indices_j)))
    return fail("sparsetir_rgms: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (validate_enabled() &&
      (validate_indptr("sparsetir_rgms", "indptr_i", indptr_i, num_rels, nnz_i, st) != 0 ||
       validate_range("sparsetir_rgms", "indices_i", indices_i, nnz_i, m, st) != 0 ||
       validate_indptr("sparsetir_rgms", "indptr_j", indptr_j, nnz_i, nnz_j, st) != 0 ||
       validate_range("sparsetir_rgms", "indices_j", indices_j, nnz_j, n, st) != 0))
    return -1;
  const bool al = aligned16(x) && aligned16(y) && aligned16(w);
  if (al) {
    if (feat == 64) {
      // Two launches: (1) Z = A_csf * X, one row per (relation, destination) pair, with the CSR
      // SpMM kernel — thousands of independent short rows in flight instead of one latency chain
      // per tile; (2) the tensor-core tile product and scatter, reading Z tiles with coalesced
      // loads.  Z (nnz_i x 64 floats) lives in the library's per-stream scratch buffer.
      // SPARSETIR_RGMS_FUSED=1 selects the single fused kernel instead (no scratch).
      static const bool fused = [] {
        const char* e = std::getenv("SPARSETIR_RGMS_FUSED");
        return e != nullptr && e[0] == '1';
      }();
      // SPARSETIR_RGMS_PATH=fused selects the one-launch form of rgms_fused.cu instead: it gathers,
      // multiplies and scatters tile by tile and needs no scratch memory, but its sixteen gather
      // warps per SM keep fewer loads in flight than a whole launch of the SpMM kernel does
      // (measured at 100 k nodes / 1.5 M edges: 183 us against 139 us for the two launches).
      static const bool one_launch = [] {
        const char* e = std::getenv("SPARSETIR_RGMS_PATH");
        return e != nullptr && std::strcmp(e, "fused") == 0;
      }();
      if (one_launch && !fused) {
        const int rc1 = rgms_fused_launch(a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, feat,
                                          nnz_i, nnz_j, n, m, st);
        if (rc1 <= 0) return rc1;
      }
      float* z = nullptr;
      if (!fused)
        z = static_cast<float*>(workspace(device_id, st, static_cast<size_t>(nnz_i) * 64 * sizeof(float)));
      if (z != nullptr) {
        if (csrmm_short_rows_impl(a, x, z, indptr_j, indices_j, nnz_i, n, 64, nnz_j, device_id, stream) != 0)
          return -1;
      }
      int rc = rgms_tc_launch(a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, feat,
                              nnz_i, z, st);
      if (rc <= 0) return rc;
    }
    if (feat == 32)
      return launch_tile<32>(a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, nnz_i, st);
    if (feat == 64)
      return launch_tile<64>(a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, nnz_i, st);
    if (feat == 128)
      return launch_tile<128>(a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, nnz_i, st);
  }
  const size_t smem = static_cast<size_t>(kThreads / 32) * feat * sizeof(float);
  if (smem > 48 * 1024) return fail("sparsetir_rgms: feat_size %d is too large", feat);
  rgms_generic_kernel<<<ceil_div(nnz_i, kThreads / 32), kThreads, smem, st>>>(
      a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, feat, nnz_i);
  SPTIR_LAUNCH_OK("rgms_generic_kernel");
  return 0;
}
