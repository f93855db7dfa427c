// The gather-accumulate loop shared by the CSR and the ELL/hyb SpMM kernels and by the RGMS
// aggregation phase.
//
// A group of LPR lanes ("sub-warp") walks a contiguous stream of stored slots
// (column id, weight).  The lanes read LPR slots at a time ("batch") with one coalesced load
// each for ids and weights, then broadcast them slot by slot with shuffles; for every slot each
// lane loads its VPL feature vectors of the dense row B[col] and multiplies-accumulates.
//
// The loop is software-pipelined so that a lane always has memory requests in flight — the
// kernels are bound by memory latency x bandwidth, not by arithmetic:
//  - the ids of batch i+1 are requested at the start of batch i;
//  - slots are handled in chunks of U; the B rows of chunk j+1 are requested before chunk j is
//    consumed (two register buffers), across batch boundaries too.
// After the slots of a chunk the caller's functor is told how many slots were consumed and
// decides whether an output row is complete.  It must not wait on global memory (row ids come
// from shared memory or registers), or that wait would serialise with the loads in flight.
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

// Slots per chunk: 4 vectors per lane and buffer.
template <int LPR, int VPL>
struct ChunkOf {
  static constexpr int kRaw = VPL >= 4 ? 1 : 4 / VPL;
  static constexpr int value = kRaw < LPR ? kRaw : LPR;
};

// cols/wts point at the first slot of the stream, nslots is its length.
// PER_SLOT = true : on_done(acc) is called after every slot.
// PER_SLOT = false: on_done(acc, n) is called after every chunk with the n <= U slots it
//                   consumed; the caller guarantees that no output row ends inside a chunk.
// FULL = true promises that every lane's vectors lie inside the feature dimension.
template <int LPR, int VPL, int VEC, bool PER_SLOT, bool FULL, class OnDone>
__device__ __forceinline__ void stream_slots(const int32_t* __restrict__ cols,
                                             const float* __restrict__ wts, int nslots,
                                             const typename Vec<VEC>::type* __restrict__ B,
                                             const FeatLane<LPR, VPL, VEC>& fl, int lane,
                                             unsigned mask, typename Vec<VEC>::type (&acc)[VPL],
                                             OnDone&& on_done) {
  using V = typename Vec<VEC>::type;
  constexpr int U = ChunkOf<LPR, VPL>::value;
  constexpr int CH = LPR / U;  // chunks per batch (a power of two)
  if (nslots <= 0) return;

  const V* bl[VPL];  // this lane's column of B
#pragma unroll
  for (int v = 0; v < VPL; ++v) bl[v] = B + fl.off[v];
  const size_t stride = static_cast<size_t>(fl.row_vecs);

  auto request = [&](V(&dst)[U][VPL], int ids, int first) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      // slots past the end carry column 0: the load is harmless and never consumed
      const int ck = __shfl_sync(mask, ids, first + u, LPR);
#pragma unroll
      for (int v = 0; v < VPL; ++v)
        dst[u][v] = (FULL || fl.valid[v]) ? __ldg(bl[v] + ck * stride) : Vec<VEC>::zero();
    }
  };
  auto consume = [&](V(&src)[U][VPL], float w, int first, int live) {
    // live = slots of this chunk that exist (>= U for a full chunk)
    if (PER_SLOT) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float ak = __shfl_sync(mask, w, first + u, LPR);
        if (u < live) {
#pragma unroll
          for (int v = 0; v < VPL; ++v) Vec<VEC>::fma(acc[v], ak, src[u][v]);
          on_done(acc, 1);
        }
      }
    } else if (live >= U) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float ak = __shfl_sync(mask, w, first + u, LPR);
#pragma unroll
        for (int v = 0; v < VPL; ++v) Vec<VEC>::fma(acc[v], ak, src[u][v]);
      }
      on_done(acc, U);
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float ak = __shfl_sync(mask, w, first + u, LPR);
        if (u < live) {
#pragma unroll
          for (int v = 0; v < VPL; ++v) Vec<VEC>::fma(acc[v], ak, src[u][v]);
        }
      }
      on_done(acc, live);
    }
  };

  int c = 0, c_next = 0;
  float a = 0.f, a_next = 0.f;
  if (lane < nslots) {
    c = __ldg(cols + lane);
    a = __ldg(wts + lane);
  }
  V buf0[U][VPL], buf1[U][VPL];
  request(buf0, c, 0);
  for (int s0 = 0; s0 < nslots; s0 += LPR) {
    const bool more = s0 + LPR < nslots;
    c_next = 0;
    a_next = 0.f;
    if (s0 + LPR + lane < nslots) {  // ids of the next batch
      c_next = __ldg(cols + s0 + LPR + lane);
      a_next = __ldg(wts + s0 + LPR + lane);
    }
    const int cnt = min(LPR, nslots - s0);
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) {
      const int first = ch * U;
      // request the chunk after this one, then consume this one
      if (ch + 1 < CH) {
        if (first + U < cnt) {
          if (ch % 2 == 0) request(buf1, c, first + U); else request(buf0, c, first + U);
        }
      } else if (more) {
        if (ch % 2 == 0) request(buf1, c_next, 0); else request(buf0, c_next, 0);
      }
      if (first < cnt) {
        if (ch % 2 == 0) consume(buf0, a, first, cnt - first); else consume(buf1, a, first, cnt - first);
      }
    }
    c = c_next;
    a = a_next;
  }
}

// The same walk with the B rows staged through shared memory by asynchronous copies
// (16-byte feature vectors, one per lane and slot, VPL = 1).
//
// Every lane owns a private ring of R 16-byte entries in shared memory: entry e of lane l is
// ring[e * LPR + l].  A lane only ever reads back what it copied itself, so the only
// synchronisation is cp.async.wait_group — the ring is an extension of the register file that
// asynchronous loads can target.  Up to R slots (R * 16 bytes per lane) are in flight, which
// is what hides HBM latency here; a register-resident pipeline of that depth would not fit.
//
// s_cols / s_wts: ids and weights of the stream, already in shared memory.
// bl: this lane's column of B (B + lane offset, in float4 units); stride = vectors per row.
// copy = false makes the lane skip its copies (its features lie past the end of the row).
template <int LPR, int R, bool PER_SLOT, class OnDone>
__device__ __forceinline__ void stream_slots_async(const int32_t* s_cols, const float* s_wts,
                                                   int nslots, const float4* __restrict__ bl,
                                                   size_t stride, bool copy, float4* ring,
                                                   float4& acc, OnDone&& on_done) {
  constexpr int U = 4;        // slots per commit group
  constexpr int NCH = R / U;  // groups the ring holds
  static_assert(R % U == 0 && NCH >= 2, "ring must hold at least two groups");
  const int nchunks = (nslots + U - 1) / U;

  auto issue = [&](int chunk, int ring_chunk) {
    const int s0 = chunk * U;
    if (copy) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (s0 + u < nslots)
          cp_async16(ring + (ring_chunk * U + u) * LPR, bl + s_cols[s0 + u] * stride);
    }
    cp_async_commit();  // committed even when empty: keeps the group count uniform
  };

#pragma unroll
  for (int i = 0; i < NCH; ++i) issue(i, i);
  int rc = 0;  // ring position of the chunk being consumed
  for (int i = 0; i < nchunks; ++i) {
    cp_async_wait<NCH - 1>();
    const int s0 = i * U;
    const int live = min(U, nslots - s0);
    if (PER_SLOT) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (u < live) {
          const float4 x = copy ? ring[(rc * U + u) * LPR] : make_float4(0.f, 0.f, 0.f, 0.f);
          Vec<4>::fma(acc, s_wts[s0 + u], x);
          on_done(acc, 1);
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (u < live) {
          const float4 x = copy ? ring[(rc * U + u) * LPR] : make_float4(0.f, 0.f, 0.f, 0.f);
          Vec<4>::fma(acc, s_wts[s0 + u], x);
        }
      }
      on_done(acc, live);
    }
    issue(i + NCH, rc);
    rc = (rc + 1 == NCH) ? 0 : rc + 1;
  }
  cp_async_wait<0>();  // nothing of this stream may still land in the ring after we return
}

}  // namespace sptir
#endif  // SPARSETIR_B200_SPMM_CORE_CUH_
