// The gather-accumulate loop shared by the CSR and the ELL/hyb SpMM kernels and by the RGMS
// aggregation phase.
//
// A group of LPR lanes ("sub-warp") walks a contiguous stream of stored slots
// (column id, weight).  The lanes read LPR slots at a time with one coalesced load each for ids
// and weights — the ids of the NEXT batch are requested before the current batch is consumed,
// so the id latency is off the critical path — then broadcast them one by one with shuffles;
// for every slot each lane loads its VPL feature vectors of the dense row B[col] and
// multiplies-accumulates.  Loads are issued U slots ahead of the arithmetic so that U*VPL
// 16-byte requests per lane are in flight: the kernels are bound by memory latency x
// bandwidth, not by arithmetic.  After every slot the caller's functor decides whether a row
// of the output is complete; it must not wait on global memory (row ids come from shared
// memory or registers), or the wait would serialise with the next batch of loads.
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
  int c_next = 0;
  float a_next = 0.f;
  if (lane < nslots) {
    c_next = __ldg(cols + lane);
    a_next = __ldg(wts + lane);
  }
  for (int s0 = 0; s0 < nslots; s0 += LPR) {
    const int c = c_next;
    const float a = a_next;
    c_next = 0;
    a_next = 0.f;
    if (s0 + LPR + lane < nslots) {  // request the next batch's ids now
      c_next = __ldg(cols + s0 + LPR + lane);
      a_next = __ldg(wts + s0 + LPR + lane);
    }
    const int cnt = min(LPR, nslots - s0);
    for (int k0 = 0; k0 < cnt; k0 += U) {
      V x[U][VPL];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        // slots past cnt carry column 0 / weight 0: the load is harmless and never consumed
        const int ck = __shfl_sync(mask, c, k0 + u, LPR);
        const V* src = B + static_cast<size_t>(ck) * fl.row_vecs;
#pragma unroll
        for (int v = 0; v < VPL; ++v) x[u][v] = fl.valid[v] ? __ldg(src + fl.off[v]) : Vec<VEC>::zero();
      }
      if (k0 + U <= cnt) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float ak = __shfl_sync(mask, a, k0 + u, LPR);
#pragma unroll
          for (int v = 0; v < VPL; ++v) Vec<VEC>::fma(acc[v], ak, x[u][v]);
          on_slot(acc);
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float ak = __shfl_sync(mask, a, k0 + u, LPR);
          if (k0 + u < cnt) {
#pragma unroll
            for (int v = 0; v < VPL; ++v) Vec<VEC>::fma(acc[v], ak, x[u][v]);
            on_slot(acc);
          }
        }
      }
    }
  }
}

}  // namespace sptir
#endif  // SPARSETIR_B200_SPMM_CORE_CUH_
