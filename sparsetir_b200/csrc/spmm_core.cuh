// The gather-accumulate loop shared by the CSR and the ELL/hyb SpMM kernels.
//
// A group of LPR lanes ("sub-warp") walks a contiguous stream of stored slots
// (column id, weight).  The lanes first read LPR slots with one coalesced load each for ids
// and weights, then broadcast them one by one with shuffles; for every slot each lane loads
// its VPL feature vectors of the dense row B[col] and multiplies-accumulates.  Loads are
// issued U slots ahead of the arithmetic so that U*VPL 16-byte requests per lane are in
// flight — the kernels are bound by HBM/L2 latency x bandwidth, not by arithmetic.
// After every slot the caller's functor decides whether a row of the output is complete.
#ifndef SPARSETIR_B200_SPMM_CORE_CUH_
#define SPARSETIR_B200_SPMM_CORE_CUH_

#include "vec.cuh"

namespace sptir {

template <int LPR, int VPL, int VEC>
struct FeatLane {
  using V = typename Vec<VEC>::type;
  int off[VPL];     // offset of this lane's v-th vector inside a dense row, in vectors
  bool valid[VPL];  // false past the end of the feature dimension
  int row_vecs;     // vectors per dense row
  __device__ __forceinline__ FeatLane(int feat, int tile, int lane) {
    row_vecs = feat / VEC;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      off[v] = tile * (LPR * VPL) + v * LPR + lane;
      valid[v] = off[v] < row_vecs;
    }
  }
};

// cols/wts point at the first slot of the stream, nslots is its length.
// on_slot(acc) is called once per consumed slot, in order.
template <int LPR, int VPL, int VEC, class OnSlot>
__device__ __forceinline__ void stream_slots(const int32_t* __restrict__ cols,
                                             const float* __restrict__ wts, int nslots,
                                             const typename Vec<VEC>::type* __restrict__ B,
                                             const FeatLane<LPR, VPL, VEC>& fl, int lane,
                                             unsigned mask, typename Vec<VEC>::type (&acc)[VPL],
                                             OnSlot&& on_slot) {
  using V = typename Vec<VEC>::type;
  constexpr int U = (8 / VPL) < LPR ? (8 / VPL) : LPR;  // slots loaded ahead
  for (int s0 = 0; s0 < nslots; s0 += LPR) {
    int my = s0 + lane;
    int c = 0;
    float a = 0.f;
    if (my < nslots) {
      c = __ldg(cols + my);
      a = __ldg(wts + my);
    }
    int cnt = min(LPR, nslots - s0);
    for (int k0 = 0; k0 < cnt; k0 += U) {
      V x[U][VPL];
      float ak[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        // slots past cnt carry column 0 / weight 0: the load is harmless and never consumed
        int ck = __shfl_sync(mask, c, k0 + u, LPR);
        ak[u] = __shfl_sync(mask, a, k0 + u, LPR);
        const V* src = B + static_cast<size_t>(ck) * fl.row_vecs;
#pragma unroll
        for (int v = 0; v < VPL; ++v) x[u][v] = fl.valid[v] ? __ldg(src + fl.off[v]) : Vec<VEC>::zero();
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k0 + u < cnt) {
#pragma unroll
          for (int v = 0; v < VPL; ++v) Vec<VEC>::fma(acc[v], ak[u], x[u][v]);
          on_slot(acc);
        }
      }
    }
  }
}

}  // namespace sptir
#endif  // SPARSETIR_B200_SPMM_CORE_CUH_
