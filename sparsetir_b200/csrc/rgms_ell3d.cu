// RGMS over the decomposed ELL3D format, fp32:
//   for every bucket b, group g (relation mid_b[g]), row slot ii, column slot j
//     Y[rows_b[g,ii], fo] += A_b[g,ii,j] * sum_fi W[mid_b[g], fo, fi] * X[cols_b[g,ii,j], fi]
// Replaces the horizontally fused kernel the reference generates from rgcn_hetero_forward after
// format_decompose with the ell3d rule (examples/rgms/rgcn/bench_rgcn_composable.py:140-216;
// buffer definition examples/rgms/rgcn/utils.py:90-108; buckets from CSFToELL3D,
// src/sparse/format.cc:180-343).  Argument list as there: W, X, Y, then per bucket the values
// (the mask cast to float in the example), row ids and column ids, then per bucket the relation id
// of every group.
//
// Like the CSF form (rgms.cu) it aggregates first and transforms once per ELL row:
//   (1) Z[q, :] = sum_j A[q,j] X[cols[q,j], :]   — the hyb SpMM kernel, ELL row q of bucket b
//       writing row base_b + q of one Z array that holds all buckets (the widths are the
//       compile-time-friendly 1/2/4/8...);
//   (2) Y[rows[q], :] += Z[q, :] W_{mid[q / rows_per_group]}^T.
// For feat 64 this is three launches whatever the number of buckets: one SpMM launch over all
// buckets, one small kernel that turns the `mid` arrays into the Z-row range of every (bucket,
// relation) pair and copies the row ids next to each other, one launch of the TMA-fed tcgen05
// kernel of rgms_tc.cu over those ranges.  Other feature sizes go bucket by bucket through a
// CUDA-core tile kernel.  Padding rows (A = 0) contribute zeros.  Z, the ranges and the row ids
// live in the per-(device, stream) workspace.
#include <algorithm>
#include <vector>

#include "common.h"

namespace sptir {

int rgms_tc_launch(const float* a, const float* w, const float* x, float* y,
                   const int32_t* indptr_i, const int32_t* indices_i, const int32_t* indptr_j,
                   const int32_t* indices_j, int num_rels, int feat, int nnz_i, const float* z,
                   cudaStream_t stream);

int rgms_tma_launch_ranges(const float* w, float* y, const int32_t* indptr_i, const int32_t* indices_i,
                           int num_ranges, int rel_mod, int nnz_i, const float* z, cudaStream_t stream);
int hyb_spmm_impl(const float* b, float* c, const SparsetirEllBucket* buckets, const int32_t* row_bases,
                  int num_buckets, int m, int n, int feat, int flags, int device_id, void* stream);

namespace {

constexpr int kThreads = 256;
constexpr int kMaxBuckets = SPARSETIR_HYB_MAX_BUCKETS;

// what the preparation kernel needs to know about the buckets (passed by value)
struct Ell3dTable {
  const int32_t* mid[kMaxBuckets];
  const int32_t* rows[kMaxBuckets];
  int32_t num_groups[kMaxBuckets];
  int32_t rows_per_group[kMaxBuckets];
  int32_t z_base[kMaxBuckets + 1];  // first Z row of every bucket; [nb] = total rows
  int32_t nb;
};

// ranges[b * R + r] = first Z row of relation r inside bucket b (ranges[nb * R] = total rows), and
// all_rows = the buckets' row ids one after the other.  Blocks 0.. cover the row ids; the last
// block computes the ranges.
__global__ void __launch_bounds__(kThreads)
ell3d_prepare_kernel(const __grid_constant__ Ell3dTable tb, int num_rels, int32_t* __restrict__ ranges,
                     int32_t* __restrict__ all_rows) {
  if (blockIdx.x == gridDim.x - 1) {
    for (int e = threadIdx.x; e <= tb.nb * num_rels; e += kThreads) {
      if (e == tb.nb * num_rels) {
        ranges[e] = tb.z_base[tb.nb];
        continue;
      }
      const int b = e / num_rels, r = e % num_rels;
      int lo = 0, hi = tb.num_groups[b];  // first group of the bucket with mid >= r
      while (lo < hi) {
        const int m = lo + (hi - lo) / 2;
        if (__ldg(tb.mid[b] + m) < r) lo = m + 1; else hi = m;
      }
      ranges[e] = tb.z_base[b] + lo * tb.rows_per_group[b];
    }
    return;
  }
  const int total = tb.z_base[tb.nb];
  for (int q = blockIdx.x * kThreads + threadIdx.x; q < total; q += (gridDim.x - 1) * kThreads) {
    int b = 0;
    while (b + 1 < tb.nb && q >= tb.z_base[b + 1]) ++b;
    all_rows[q] = __ldg(tb.rows[b] + (q - tb.z_base[b]));
  }
}

// indptr[r] = rows_per_group * (number of groups whose relation is < r), r = 0..num_rels:
// the Z-row range of every relation, from the ascending per-group relation ids
__global__ void __launch_bounds__(kThreads)
relation_ranges_kernel(const int32_t* __restrict__ mid, int num_groups, int num_rels,
                       int rows_per_group, int32_t* __restrict__ indptr) {
  const int r = blockIdx.x * kThreads + threadIdx.x;
  if (r > num_rels) return;
  int lo = 0, hi = num_groups;  // first group with mid >= r
  while (lo < hi) {
    const int m = lo + (hi - lo) / 2;
    if (__ldg(mid + m) < r) lo = m + 1; else hi = m;
  }
  indptr[r] = lo * rows_per_group;
}

// CUDA-core form of step (2) for feature sizes the tensor-core kernel does not take: a block
// owns 32 consecutive Z rows (staged in shared memory); a thread computes outputs (row, fo) and
// adds them to Y.
constexpr int kTileRows = 32;
__global__ void __launch_bounds__(kThreads)
transform_scatter_kernel(const float* __restrict__ z, const float* __restrict__ w,
                         float* __restrict__ y, const int32_t* __restrict__ rows,
                         const int32_t* __restrict__ mid, int nrows, int rows_per_group, int feat) {
  extern __shared__ float s_z[];  // kTileRows x feat
  const int q0 = blockIdx.x * kTileRows;
  const int nq = min(kTileRows, nrows - q0);
  for (int i = threadIdx.x; i < nq * feat; i += kThreads) s_z[i] = __ldg(z + static_cast<size_t>(q0) * feat + i);
  __syncthreads();
  for (int i = threadIdx.x; i < nq * feat; i += kThreads) {
    const int t = i / feat, fo = i % feat;
    const int q = q0 + t;
    const float* wr = w + (static_cast<size_t>(__ldg(mid + q / rows_per_group)) * feat + fo) * feat;
    const float* zr = s_z + t * feat;
    float acc = 0.f;
    for (int fi = 0; fi < feat; ++fi) acc = fmaf(zr[fi], __ldg(wr + fi), acc);
    atomicAdd(y + static_cast<size_t>(__ldg(rows + q)) * feat + fo, acc);
  }
}

}  // namespace
}  // namespace sptir

extern "C" int sparsetir_rgms_ell3d_raw(const float* w, const float* x, float* y,
                                        const SparsetirEll3dBucket* buckets, int num_buckets, int m,
                                        int n, int num_rels, int feat, int device_id, void* stream) {
  using namespace sptir;
  if (num_buckets < 0 || m < 0 || n < 0 || num_rels < 0 || feat < 0)
    return fail("sparsetir_rgms_ell3d: negative size");
  if (num_buckets > 0 && !buckets) return fail("sparsetir_rgms_ell3d: null bucket list");
  long long max_rows = 0;
  for (int b = 0; b < num_buckets; ++b) {
    const SparsetirEll3dBucket& bk = buckets[b];
    if (bk.num_groups < 0 || bk.rows_per_group < 0 || bk.cols_per_row < 0)
      return fail("sparsetir_rgms_ell3d: bucket %d has a negative size", b);
    const long long nrows = static_cast<long long>(bk.num_groups) * bk.rows_per_group;
    if (nrows == 0) continue;
    if (bk.cols_per_row == 0) return fail("sparsetir_rgms_ell3d: bucket %d has rows but no columns", b);
    if (!bk.a || !bk.rows || !bk.cols || !bk.mid)
      return fail("sparsetir_rgms_ell3d: bucket %d has a null array", b);
    if (nrows > INT32_MAX || nrows * bk.cols_per_row > INT32_MAX)
      return fail("sparsetir_rgms_ell3d: bucket %d is too large for 32-bit indices", b);
    max_rows = std::max(max_rows, nrows);
  }
  if (max_rows == 0 || feat == 0 || m == 0) return 0;
  if (!w || !x || !y) return fail("sparsetir_rgms_ell3d: null pointer argument");
  if (num_rels == 0) return fail("sparsetir_rgms_ell3d: rows but no relations");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if (feat == 64 && num_buckets <= kMaxBuckets) {
    // ---- three launches for all buckets
    Ell3dTable tb{};
    std::vector<SparsetirEllBucket> ell;
    std::vector<int32_t> bases;
    long long total = 0;
    int flags = 0;
    for (int b = 0; b < num_buckets; ++b) {
      const SparsetirEll3dBucket& bk = buckets[b];
      const int nrows = bk.num_groups * bk.rows_per_group;
      if (nrows == 0) continue;
      const int k = tb.nb++;
      tb.mid[k] = bk.mid; tb.rows[k] = bk.rows;
      tb.num_groups[k] = bk.num_groups; tb.rows_per_group[k] = bk.rows_per_group;
      tb.z_base[k] = static_cast<int32_t>(total);
      ell.push_back(SparsetirEllBucket{bk.a, nullptr, bk.cols, nrows, bk.cols_per_row});
      bases.push_back(static_cast<int32_t>(total));
      if (bk.cols_per_row > 32) flags = SPARSETIR_HYB_ZERO_C;  // rows cut into pieces accumulate
      total += nrows;
    }
    const long long num_ranges = static_cast<long long>(tb.nb) * num_rels;
    if (total <= INT32_MAX && num_ranges < INT32_MAX) {
      tb.z_base[tb.nb] = static_cast<int32_t>(total);
      const size_t zb = (static_cast<size_t>(total) * feat * sizeof(float) + 255) & ~static_cast<size_t>(255);
      const size_t rb = (static_cast<size_t>(num_ranges + 1) * sizeof(int32_t) + 255) & ~static_cast<size_t>(255);
      char* wsp = static_cast<char*>(workspace(device_id, st, zb + rb + static_cast<size_t>(total) * sizeof(int32_t)));
      if (!wsp) return -1;
      float* zall = reinterpret_cast<float*>(wsp);
      int32_t* rng = reinterpret_cast<int32_t*>(wsp + zb);
      int32_t* all_rows = reinterpret_cast<int32_t*>(wsp + zb + rb);
      if (hyb_spmm_impl(x, zall, ell.data(), bases.data(), tb.nb, static_cast<int>(total), n, feat, flags,
                        device_id, stream) != 0)
        return -1;
      const int copy_blocks = static_cast<int>(std::min<long long>(ceil_div(static_cast<int>(total), kThreads), 4 * kNumSMs));
      ell3d_prepare_kernel<<<copy_blocks + 1, kThreads, 0, st>>>(tb, num_rels, rng, all_rows);
      SPTIR_LAUNCH_OK("ell3d_prepare_kernel");
      const int rc = rgms_tma_launch_ranges(w, y, rng, all_rows, static_cast<int>(num_ranges), num_rels,
                                            static_cast<int>(total), zall, st);
      if (rc <= 0) return rc;
      // not taken by the tensor-core path: fall through to the per-bucket form (Z is recomputed)
    }
  }

  // workspace: Z of the largest bucket, then the relation ranges
  const size_t z_bytes = (static_cast<size_t>(max_rows) * feat * sizeof(float) + 255) & ~static_cast<size_t>(255);
  const size_t ptr_bytes = static_cast<size_t>(num_rels + 1) * sizeof(int32_t);
  char* ws = static_cast<char*>(workspace(device_id, st, z_bytes + ptr_bytes));
  if (!ws) return -1;
  float* z = reinterpret_cast<float*>(ws);
  int32_t* ranges = reinterpret_cast<int32_t*>(ws + z_bytes);

  for (int b = 0; b < num_buckets; ++b) {
    const SparsetirEll3dBucket& bk = buckets[b];
    const int nrows = bk.num_groups * bk.rows_per_group;
    if (nrows == 0) continue;
    // (1) aggregate: ELL row q -> Z row q.  Rows of up to 32 slots are never cut into pieces, so
    // every Z row has one writer; wider rows are accumulated atomically into a cleared Z.
    SparsetirEllBucket ell{bk.a, nullptr, bk.cols, nrows, bk.cols_per_row};
    const int flags = bk.cols_per_row > 32 ? SPARSETIR_HYB_ZERO_C : 0;
    if (sparsetir_hyb_spmm_raw(x, z, &ell, 1, nrows, n, feat, flags, device_id, stream) != 0) return -1;
    // (2) transform and scatter
    int rc = 1;
    if (feat == 64) {
      relation_ranges_kernel<<<ceil_div(num_rels + 1, kThreads), kThreads, 0, st>>>(
          bk.mid, bk.num_groups, num_rels, bk.rows_per_group, ranges);
      SPTIR_LAUNCH_OK("relation_ranges_kernel");
      rc = rgms_tc_launch(nullptr, w, x, y, ranges, bk.rows, nullptr, nullptr, num_rels, feat, nrows, z, st);
      if (rc < 0) return -1;
    }
    if (rc == 1) {
      const size_t smem = static_cast<size_t>(kTileRows) * feat * sizeof(float);
      if (smem > 48 * 1024) return fail("sparsetir_rgms_ell3d: feat_size %d is too large", feat);
      transform_scatter_kernel<<<ceil_div(nrows, kTileRows), kThreads, smem, st>>>(
          z, w, y, bk.rows, bk.mid, nrows, bk.rows_per_group, feat);
      SPTIR_LAUNCH_OK("transform_scatter_kernel");
    }
  }
  return 0;
}
