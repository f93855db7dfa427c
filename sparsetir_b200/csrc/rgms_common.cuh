// Shared by the RGMS kernels: mapping of a thread block to its (relation, row tile).
#ifndef SPARSETIR_B200_RGMS_COMMON_CUH_
#define SPARSETIR_B200_RGMS_COMMON_CUH_

#include <cuda_runtime.h>
#include <cstdint>

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

}  // namespace sptir
#endif  // SPARSETIR_B200_RGMS_COMMON_CUH_
