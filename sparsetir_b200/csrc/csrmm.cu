// CSR SpMM, fp32:  C[i,:] = sum_{p in row i} A[p] * B[indices[p],:]
// Semantics: tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:22-68 of the reference;
// like the reference's scheduled GPU kernel (examples/spmm/bench_spmm_naive.py:102-119) rows
// without entries are written as zeros.
//
// Mapping: a group of LPR lanes owns 1, 2 or 4 consecutive rows and streams their stored
// entries as one contiguous slot stream (see spmm_core.cuh); each lane keeps VPL 16-byte
// pieces of the output row in registers and stores them when the row's last entry has been
// consumed.  One writer per output row: no atomics, deterministic summation in CSR order.
#include "common.h"
#include "spmm_core.cuh"

namespace sptir {
namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------------------------
// Lean kernel: fast path for 16-byte aligned operands and whole feature tiles.
// A sub-warp of LPR lanes owns `rpi` consecutive rows (rpi < LPR).  Short rows are the hard
// case for CSR: row pointer -> ids -> dense rows is a chain of three dependent memory round
// trips, and a row of two or three entries gives nothing to overlap them with.  So the chain is
// paid once per ITEM, not per row: the rpi+1 row pointers are read with one coalesced load and
// kept in registers (lane j holds indptr[r0+j], fetched by shuffle at row ends), the item's
// entries are one contiguous slot stream whose ids/values are read a batch of LPR ahead, and the
// dense rows are gathered 8 at a time.  One writer per output row, CSR summation order, rows
// without entries written as zeros.
template <int LPR, int W>  // W floats per lane: 4 (16-byte vectors) or 8 (32-byte vectors)
__global__ void __launch_bounds__(kThreads, 4)
csrmm_lean_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                  const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices, int m,
                  int feat, int rpi) {
  using LV = LaneVec<W>;
  using V = typename LV::type;
  constexpr int SUBS = kThreads / LPR;
  constexpr int U = (32 / W) < LPR ? (32 / W) : LPR;  // gathered rows in flight: 32 registers
  const int lane = threadIdx.x % LPR;
  const unsigned mask = group_mask<LPR>();
  const long long item = static_cast<long long>(blockIdx.x) * SUBS + threadIdx.x / LPR;
  const long long r0l = item * rpi;
  if (r0l >= m) return;
  const int r0 = static_cast<int>(r0l);
  const int nr = min(rpi, m - r0);
  const int ptr = __ldg(indptr + r0 + min(lane, nr));  // lane j: start of row r0+j (j <= nr)
  const int p0 = __shfl_sync(mask, ptr, 0, LPR);
  const int nslots = __shfl_sync(mask, ptr, nr, LPR) - p0;
  const unsigned row_bytes = static_cast<unsigned>(feat) * 4u;
  const unsigned off = (blockIdx.y * LPR + lane) * (W * 4u);
  const char* bl = reinterpret_cast<const char*>(b) + off;
  char* cl = reinterpret_cast<char*>(c) + off +
             static_cast<unsigned long long>(static_cast<unsigned>(r0)) * row_bytes;
  const int32_t* cols = indices + p0;
  const float* wts = a + p0;

  V acc = LV::zero();
  int j = 0;                                        // row of the item being accumulated
  int row_end = __shfl_sync(mask, ptr, 1, LPR) - p0;  // its end, as a slot number
  int s = 0;                                        // slots consumed so far
  auto finish_rows = [&]() {  // store every row whose last entry has been consumed
    while (j < nr && s >= row_end) {
      LV::stcs(cl, acc);  // written once: keep B rows in L2
      acc = LV::zero();
      cl += row_bytes;
      ++j;
      row_end = __shfl_sync(mask, ptr, min(j + 1, nr), LPR) - p0;
    }
  };
  finish_rows();  // rows without entries at the front

  int cid = 0, cidn = 0;
  float av = 0.f, avn = 0.f;
  if (lane < nslots) {
    cid = __ldg(cols + lane);
    av = __ldg(wts + lane);
  }
  for (int s0 = 0; s0 < nslots; s0 += LPR) {
    cidn = 0;
    avn = 0.f;
    if (s0 + LPR + lane < nslots) {  // ids and values of the next batch
      cidn = __ldg(cols + s0 + LPR + lane);
      avn = __ldg(wts + s0 + LPR + lane);
    }
    const int cnt = min(LPR, nslots - s0);
#pragma unroll
    for (int k0 = 0; k0 < LPR; k0 += U) {
      if (k0 < cnt) {
        V x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {  // slots past the end ask for column 0: never consumed
          const unsigned col = static_cast<unsigned>(__shfl_sync(mask, cid, k0 + u, LPR));
          x[u] = LV::ldg(bl + static_cast<unsigned long long>(col) * row_bytes);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float ak = __shfl_sync(mask, av, k0 + u, LPR);
          if (k0 + u < cnt) {
            LV::fma(acc, ak, x[u]);
            ++s;
            if (s >= row_end) finish_rows();
          }
        }
      }
    }
    cid = cidn;
    av = avn;
  }
}

template <int LPR, int VPL, int VEC>
__global__ void __launch_bounds__(kThreads)
csrmm_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
             const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices, int m,
             int feat, int rows_per_item) {
  using V = typename Vec<VEC>::type;
  constexpr int SUBS = kThreads / LPR;
  const int lane = threadIdx.x % LPR;
  const unsigned mask = group_mask<LPR>();
  const long long item = static_cast<long long>(blockIdx.x) * SUBS + threadIdx.x / LPR;
  const long long r0l = item * rows_per_item;
  if (r0l >= m) return;
  const int r0 = static_cast<int>(r0l);
  const int r1 = min(m, r0 + rows_per_item);
  const FeatLane<LPR, VPL, VEC> fl(feat, blockIdx.y, lane);
  V* cv = reinterpret_cast<V*>(c);

  int row = r0;
  int row_end = __ldg(indptr + r0 + 1);
  const int p0 = __ldg(indptr + r0);
  const int p1 = __ldg(indptr + r1);
  int p = p0;  // next slot to be consumed

  V acc[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) acc[v] = Vec<VEC>::zero();

  auto flush_finished_rows = [&]() {
    // store every row whose last entry has been consumed (also rows without entries)
    while (row < r1 && p >= row_end) {
      V* dst = cv + static_cast<size_t>(row) * fl.row_vecs;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        if (fl.valid[v]) __stcs(dst + fl.off[v], acc[v]);  // written once: keep B rows in L2
        acc[v] = Vec<VEC>::zero();
      }
      ++row;
      if (row < r1) row_end = __ldg(indptr + row + 1);
    }
  };

  flush_finished_rows();  // leading empty rows
  auto on_done = [&](V(&)[VPL], int n) {
    p += n;
    flush_finished_rows();
  };
  const V* bv = reinterpret_cast<const V*>(b);
  if (feat % (LPR * VPL * VEC) == 0)
    stream_slots<LPR, VPL, VEC, true, true>(indices + p0, a + p0, p1 - p0, bv, fl, lane, mask, acc, on_done);
  else
    stream_slots<LPR, VPL, VEC, true, false>(indices + p0, a + p0, p1 - p0, bv, fl, lane, mask, acc, on_done);
}

template <int LPR, int VPL, int VEC>
int launch(const float* a, const float* b, float* c, const int32_t* indptr, const int32_t* indices,
           int m, int feat, cudaStream_t stream) {
  constexpr int SUBS = kThreads / LPR;
  const int tile_feat = LPR * VPL * VEC;
  // Several consecutive rows per sub-warp amortise the pipeline start-up, but only once there
  // are enough rows to fill the machine a few times over; small matrices get one row each.
  const long long resident_subs = static_cast<long long>(kNumSMs) * 8 * SUBS;
  const int rows_per_item = m >= 4 * resident_subs ? 4 : (m >= 2 * resident_subs ? 2 : 1);
  dim3 grid(ceil_div(ceil_div(m, rows_per_item), SUBS), ceil_div(feat, tile_feat));
  csrmm_kernel<LPR, VPL, VEC><<<grid, kThreads, 0, stream>>>(a, b, c, indptr, indices, m, feat,
                                                              rows_per_item);
  SPTIR_LAUNCH_OK("csrmm_kernel");
  return 0;
}

}  // namespace
}  // namespace sptir

extern "C" int sparsetir_csrmm_raw(const float* a, const float* b, float* c, const int32_t* indptr,
                                   const int32_t* indices, int m, int n, int feat, int nnz,
                                   int device_id, void* stream) {
  using namespace sptir;
  if (m < 0 || feat < 0 || nnz < 0) return fail("sparsetir_csrmm: negative size");
  if (m == 0 || feat == 0) return 0;
  if (!b || !c || !indptr || (nnz > 0 && (!a || !indices)))
    return fail("sparsetir_csrmm: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec4 = (feat % 4 == 0) && aligned16(b) && aligned16(c);
  if (vec4 && static_cast<long long>(feat) * 4 < (1ll << 32) &&
      static_cast<long long>(m) * feat * 4 < (1ll << 32) * 1024) {
    // lanes per row: one per 32-byte vector when the operands allow it, else one per 16-byte
    // vector; narrowed until the n x tile slice of B that a pass over the rows gathers from fits
    // the resident part of L2 (see hyb_spmm.cu)
    const int w = (feat % 32 == 0 && aligned32(b) && aligned32(c)) ? max_lane_floats() : 4;
    const int nv = feat / w;
    int lanes = nv <= 4 ? 4 : (nv <= 8 ? 8 : (nv <= 16 ? 16 : 32));
    if (w == 4 && lanes < 8) lanes = 8;
    const size_t l2_budget = 48u << 20;
    const int min_lanes = w == 8 ? 4 : 8;
    while (lanes > min_lanes && static_cast<size_t>(n) * lanes * w * 4 > l2_budget) lanes /= 2;
    if (feat % (w * lanes) == 0) {
      const int subs = kThreads / lanes;
      // about four id batches per item, but never so few items that SMs sit idle
      const double avg = m > 0 ? static_cast<double>(nnz) / m : 0.0;
      int rpi = static_cast<int>(4.0 * lanes / (avg > 1.0 ? avg : 1.0));
      rpi = rpi < 1 ? 1 : (rpi > lanes - 1 ? lanes - 1 : rpi);
      const long long want_items = 4ll * kNumSMs * 4 * subs;
      while (rpi > 1 && (m + rpi - 1) / rpi < want_items) rpi /= 2;
      dim3 grid(ceil_div(ceil_div(m, rpi), subs), feat / (w * lanes));
#define SPTIR_CSR_LEAN(L, WW) \
  csrmm_lean_kernel<L, WW><<<grid, kThreads, 0, st>>>(a, b, c, indptr, indices, m, feat, rpi)
      if (w == 8) {
        if (lanes == 4) SPTIR_CSR_LEAN(4, 8);
        else if (lanes == 8) SPTIR_CSR_LEAN(8, 8);
        else if (lanes == 16) SPTIR_CSR_LEAN(16, 8);
        else SPTIR_CSR_LEAN(32, 8);
      } else {
        if (lanes == 8) SPTIR_CSR_LEAN(8, 4);
        else if (lanes == 16) SPTIR_CSR_LEAN(16, 4);
        else SPTIR_CSR_LEAN(32, 4);
      }
#undef SPTIR_CSR_LEAN
      SPTIR_LAUNCH_OK("csrmm_lean_kernel");
      return 0;
    }
  }
  if (vec4) {
    const int nv = feat / 4;
    if (nv <= 8) return launch<8, 1, 4>(a, b, c, indptr, indices, m, feat, st);
    if (nv <= 16) return launch<16, 1, 4>(a, b, c, indptr, indices, m, feat, st);
    if (nv <= 32) return launch<32, 1, 4>(a, b, c, indptr, indices, m, feat, st);
    // Wider rows go feature tile by feature tile (blockIdx.y, the slowest grid dimension), the
    // tile chosen so that the n x tile slice of B a pass gathers from stays resident in L2.
    const size_t l2_budget = 56u << 20;  // what stays resident of data that every SM reads
    const size_t slice_128 = static_cast<size_t>(n) * 128 * sizeof(float);
    if (nv > 64 && 4 * slice_128 <= l2_budget)
      return launch<32, 4, 4>(a, b, c, indptr, indices, m, feat, st);
    if (2 * slice_128 <= l2_budget) return launch<32, 2, 4>(a, b, c, indptr, indices, m, feat, st);
    return launch<32, 1, 4>(a, b, c, indptr, indices, m, feat, st);
  }
  if (feat <= 8) return launch<8, 1, 1>(a, b, c, indptr, indices, m, feat, st);
  if (feat <= 16) return launch<16, 1, 1>(a, b, c, indptr, indices, m, feat, st);
  if (feat <= 32) return launch<32, 1, 1>(a, b, c, indptr, indices, m, feat, st);
  return launch<32, 4, 1>(a, b, c, indptr, indices, m, feat, st);  // tiles of 128 features
}
