// Shared by the RGMS kernels: mapping of a thread block to its (relation, row tile).
#ifndef SPARSETIR_B200_RGMS_COMMON_CUH_
#define SPARSETIR_B200_RGMS_COMMON_CUH_

#include <cuda_runtime.h>
#include <cstdint>

#include "spmm_core.cuh"

namespace sptir {

constexpr int kRgmsThreads = 256;

// Tiles are numbered relation by relation: relation r owns ceil(rows_r / tile_rows) tiles.
// Block-wide lookup: which relation and which row range does tile `tile_id` cover?
// Returns false when tile_id is past the last tile.  All threads must call it.
__device__ inline bool locate_tile(const int32_t* __restrict__ indptr_i, int num_rels, int tile_rows,
                            int tile_id, int* rel, int* row_begin, int* row_end) {
  __shared__ int s_warp_sum[kRgmsThreads / 32];
  __shared__ int s_found[3];
  const int per = (num_rels + kRgmsThreads - 1) / kRgmsThreads;
  const int r_lo = min(num_rels, static_cast<int>(threadIdx.x) * per);
  const int r_hi = min(num_rels, r_lo + per);
  int local = 0;
  for (int r = r_lo; r < r_hi; ++r)
    local += (__ldg(indptr_i + r + 1) - __ldg(indptr_i + r) + tile_rows - 1) / tile_rows;
  // inclusive scan inside the warp, then across warps
  int incl = local;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (threadIdx.x == 0) s_found[0] = -1;
  if (lane == 31) s_warp_sum[warp] = incl;
  __syncthreads();
  int base = incl - local;
  for (int w = 0; w < warp; ++w) base += s_warp_sum[w];
  if (tile_id >= base && tile_id < base + local) {
    int t = base;
    for (int r = r_lo; r < r_hi; ++r) {
      int s = __ldg(indptr_i + r), e = __ldg(indptr_i + r + 1);
      int nt = (e - s + tile_rows - 1) / tile_rows;
      if (tile_id < t + nt) {
        s_found[0] = r;
        s_found[1] = s + (tile_id - t) * tile_rows;
        s_found[2] = min(e, s + (tile_id - t + 1) * tile_rows);
        break;
      }
      t += nt;
    }
  }
  __syncthreads();
  *rel = s_found[0];
  *row_begin = s_found[1];
  *row_end = s_found[2];
  return s_found[0] >= 0;
}

// Phase 1 of both RGMS kernels: Z[t,:] = sum_{p in CSF row row0+t} A[p] * X[J[p],:] for the
// TILE_ROWS rows of a tile (rows >= nrows give zeros).
// The stored entries of a tile are contiguous, so every sub-warp of LPR = F/4 lanes takes
// TILE_ROWS / SUBS consecutive rows and walks their entries as ONE stream (ids prefetched,
// gathers double-buffered across row boundaries, see spmm_core.cuh) instead of paying the
// pointer -> id -> row latency chain once per row; row ends come from the tile's row pointers,
// staged in shared memory.  write_row(t, acc) receives every finished row exactly once.
// Must be called by all threads of the block (it synchronises).
template <int F, int TILE_ROWS, class WriteRow>
__device__ __forceinline__ void gather_tile_rows(const float* __restrict__ a,
                                                 const float* __restrict__ x,
                                                 const int32_t* __restrict__ indptr_j,
                                                 const int32_t* __restrict__ indices_j, int row0,
                                                 int nrows, WriteRow&& write_row) {
  constexpr int LPR = F / 4;
  constexpr int SUBS = kRgmsThreads / LPR;
  constexpr int RPS = TILE_ROWS / SUBS;  // rows per sub-warp
  static_assert(TILE_ROWS % SUBS == 0, "tile rows must divide evenly over the sub-warps");
  __shared__ int32_t s_ptr[TILE_ROWS + 1];
  for (int t = threadIdx.x; t <= nrows; t += kRgmsThreads) s_ptr[t] = __ldg(indptr_j + row0 + t);
  __syncthreads();
  const int lane = threadIdx.x % LPR;
  const unsigned mask = group_mask<LPR>();
  const FeatLane<LPR, 1, 4> fl(F, 0, lane);
  const int r_lo = (threadIdx.x / LPR) * RPS;
  const int r_hi = min(nrows, r_lo + RPS);
  float4 acc[1] = {make_float4(0.f, 0.f, 0.f, 0.f)};
  if (r_lo < r_hi) {
    const int p_begin = s_ptr[r_lo], p_end = s_ptr[r_hi];
    int cur = r_lo, p = p_begin, row_end = s_ptr[r_lo + 1];
    auto flush = [&]() {
      while (cur < r_hi && p >= row_end) {
        write_row(cur, acc[0]);
        acc[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        ++cur;
        if (cur < r_hi) row_end = s_ptr[cur + 1];
      }
    };
    flush();  // rows without entries at the front
    stream_slots<LPR, 1, 4, true, true>(indices_j + p_begin, a + p_begin, p_end - p_begin,
                                        reinterpret_cast<const float4*>(x), fl, lane, mask, acc,
                                        [&](float4(&)[1], int n) {
                                          p += n;
                                          flush();
                                        });
  }
  for (int t = max(r_lo, nrows); t < r_lo + RPS; ++t) write_row(t, make_float4(0.f, 0.f, 0.f, 0.f));
}

// ---- warp-level tile lookup and walk for the kernels whose tiles are 128 rows
constexpr int kTileRows128 = 128;

// Which relation and row range tile `tile_id` covers; called by the 32 lanes of one warp.
__device__ inline bool locate_tile_warp(const int32_t* __restrict__ indptr_i, int num_rels,
                                        int tile_id, int lane, int* rel, int* row0, int* row1) {
  int base = 0;
  for (int r0 = 0; r0 < num_rels; r0 += 32) {
    const int r = r0 + lane;
    int s = 0, e = 0, nt = 0;
    if (r < num_rels) {
      s = __ldg(indptr_i + r);
      e = __ldg(indptr_i + r + 1);
      nt = (e - s + kTileRows128 - 1) / kTileRows128;
    }
    int incl = nt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const int excl = base + incl - nt;
    const bool mine = tile_id >= excl && tile_id < excl + nt;
    const unsigned hit = __ballot_sync(0xffffffffu, mine);
    if (hit != 0) {
      const int src = __ffs(hit) - 1;
      *rel = __shfl_sync(0xffffffffu, r, src);
      *row0 = __shfl_sync(0xffffffffu, s + (tile_id - excl) * kTileRows128, src);
      *row1 = __shfl_sync(0xffffffffu, min(e, s + (tile_id - excl + 1) * kTileRows128), src);
      return true;
    }
    base += __shfl_sync(0xffffffffu, incl, 31);
  }
  return false;
}

struct TileWalk {
  int rel, row0, row1, rel_end;  // rel_end: first row past the relation (cached indptr_i[rel + 1])
  // steps to the tile after this one; false when there is none.  Inside a relation this costs no
  // memory access; the row pointer is read again only when the relation changes.
  __device__ __forceinline__ bool next(const int32_t* __restrict__ indptr_i, int num_rels) {
    const int nrow0 = row1;
    while (nrow0 >= rel_end) {
      if (++rel >= num_rels) return false;
      rel_end = __ldg(indptr_i + rel + 1);
    }
    row0 = nrow0;
    row1 = min(rel_end, nrow0 + kTileRows128);
    return true;
  }
};

}  // namespace sptir
#endif  // SPARSETIR_B200_RGMS_COMMON_CUH_
