// CSR SpMM, fp32:  C[i,:] = sum_{p in row i} A[p] * B[indices[p],:]
// Semantics: tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:22-68 of the reference;
// like the reference's scheduled GPU kernel (examples/spmm/bench_spmm_naive.py:102-119) rows
// without entries are written as zeros.
//
// Mapping: a group of LPR lanes owns 1, 2 or 4 consecutive rows and streams their stored
// entries as one contiguous slot stream (see spmm_core.cuh); each lane keeps VPL 16-byte
// pieces of the output row in registers and stores them when the row's last entry has been
// consumed.  One writer per output row: no atomics, deterministic summation in CSR order.
#include <cstdlib>

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
                  int feat, int rpi, int long_row) {
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

  // Rows longer than long_row (hub rows) belong to the long-row launch that follows (it was
  // given their list, and their output rows cleared, by the planning kernel).  An item that
  // contains such rows streams the runs of ordinary rows between them, one run at a time; an
  // item without them (the usual case) is one run.
  unsigned long_rows_mask = 0;
  if (long_row > 0) {
    const int len = __shfl_down_sync(mask, ptr, 1, LPR) - ptr;
    const int shift = (threadIdx.x & 31) / LPR * LPR;
    long_rows_mask = __ballot_sync(mask, lane < nr && len > long_row) >> shift;
  }
  int jb = 0;
  while (jb < nr) {
    int je = nr;
    if (long_rows_mask != 0) {
      const unsigned ordinary = ~long_rows_mask & ((nr < 32 ? (1u << nr) : 0u) - 1u) & (~0u << jb);
      if (ordinary == 0) break;
      jb = __ffs(ordinary) - 1;
      const unsigned longer = long_rows_mask & (~0u << jb);
      je = longer != 0 ? __ffs(longer) - 1 : nr;
    }
    // ---- rows [jb, je) of the item: one contiguous slot stream
    const int p0s = __shfl_sync(mask, ptr, jb, LPR);
    const int nslots_s = __shfl_sync(mask, ptr, je, LPR) - p0s;
    char* cls = cl + static_cast<unsigned>(jb) * row_bytes;
    const int32_t* cols_s = indices + p0s;
    const float* wts_s = a + p0s;
    V acc = LV::zero();
    int j = jb;                                             // row being accumulated
    int row_end = __shfl_sync(mask, ptr, jb + 1, LPR) - p0s;  // its end, as a slot number
    int s = 0;                                              // slots consumed so far
    auto finish_rows = [&]() {  // store every row whose last entry has been consumed
      while (j < je && s >= row_end) {
        LV::stcs(cls, acc);  // written once: keep B rows in L2
        acc = LV::zero();
        cls += row_bytes;
        ++j;
        row_end = __shfl_sync(mask, ptr, min(j + 1, je), LPR) - p0s;
      }
    };
    finish_rows();  // rows without entries at the front

    int cid = 0, cidn = 0;
    float av = 0.f, avn = 0.f;
    if (lane < nslots_s) {
      cid = __ldg(cols_s + lane);
      av = __ldg(wts_s + lane);
    }
    for (int s0 = 0; s0 < nslots_s; s0 += LPR) {
      cidn = 0;
      avn = 0.f;
      if (s0 + LPR + lane < nslots_s) {  // ids and values of the next batch
        cidn = __ldg(cols_s + s0 + LPR + lane);
        avn = __ldg(wts_s + s0 + LPR + lane);
      }
      const int cnt = min(LPR, nslots_s - s0);
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
    jb = je;
  }
}

// ---------------------------------------------------------------------------------------------
// Hub rows.  A row of thousands of entries walked by one sub-warp would set the launch time
// (1.5 ms for the 13,000-entry row of a 170 k-row power-law graph against 60 us for everything
// else), and an item of a dozen 200-entry rows is a smaller tail of the same kind.  So rows of
// more than 32 entries (measured best of 32..256 on that graph: 78 / 113 / 362 us at F = 32 / 128 /
// 512 against 111 / 155 / 436 us at 256) are cut into chunks of kLongChunk (128) entries: a
// planning kernel lists the chunks and clears those output rows, the main kernel leaves the rows
// alone, and a third launch (one sub-warp per listed chunk, upper-bound grid, blocks past the
// list end at once) adds the partial sums atomically.  Rows of up to 128 entries still have one
// writer and CSR summation order; the order in which the chunks of a longer row are added is
// not fixed.  Matrices below 8192 rows and 65536 entries keep the single launch.
constexpr int kLongChunk = 128;

__global__ void __launch_bounds__(kThreads)
csr_plan_long_rows_kernel(const int32_t* __restrict__ indptr, int m, int feat, float* __restrict__ c,
                          int* __restrict__ count, int2* __restrict__ list, int max_entries,
                          int long_row) {
  const int row = blockIdx.x * kThreads + threadIdx.x;
  int len = 0;
  if (row < m) len = __ldg(indptr + row + 1) - __ldg(indptr + row);
  const bool is_long = len > long_row;
  if (is_long) {
    const int nch = (len + kLongChunk - 1) / kLongChunk;
    const int base = atomicAdd(count, nch);
    for (int k = 0; k < nch; ++k)
      if (base + k < max_entries) list[base + k] = make_int2(row, k);
  }
  unsigned todo = __ballot_sync(0xffffffffu, is_long);
  const int lane = threadIdx.x & 31;
  while (todo != 0) {
    const int src = __ffs(todo) - 1;
    todo &= todo - 1;
    const int r = __shfl_sync(0xffffffffu, row, src);
    float* dst = c + static_cast<size_t>(r) * feat;
    for (int f = lane; f < feat; f += 32) dst[f] = 0.f;
  }
}

template <int LPR>  // 16-byte lanes; blockIdx.y = feature tile of 4 * LPR floats
__global__ void __launch_bounds__(kThreads, 4)
csr_long_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                     const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices, int feat,
                     const int* __restrict__ count, const int2* __restrict__ list, int max_entries) {
  constexpr int SUBS = kThreads / LPR;
  constexpr int U = 8;
  const int lane = threadIdx.x % LPR;
  const unsigned mask = group_mask<LPR>();
  const long long e = static_cast<long long>(blockIdx.x) * SUBS + threadIdx.x / LPR;
  if (e >= min(__ldg(count), max_entries)) return;
  const int2 work = list[e];
  const int row_begin = __ldg(indptr + work.x);
  const int p0 = row_begin + work.y * kLongChunk;
  const int nslots = min(kLongChunk, __ldg(indptr + work.x + 1) - p0);
  const unsigned row_bytes = static_cast<unsigned>(feat) * 4u;
  const unsigned off = (blockIdx.y * LPR + lane) * 16u;
  const char* bl = reinterpret_cast<const char*>(b) + off;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < nslots; s0 += LPR) {
    int cid = 0;
    float av = 0.f;
    if (s0 + lane < nslots) {
      cid = __ldg(indices + p0 + s0 + lane);
      av = __ldg(a + p0 + s0 + lane);
    }
    const int cnt = min(LPR, nslots - s0);
#pragma unroll
    for (int k0 = 0; k0 < LPR; k0 += U) {
      if (k0 < cnt) {
        float4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const unsigned col = static_cast<unsigned>(__shfl_sync(mask, cid, k0 + u, LPR));
          x[u] = __ldg(reinterpret_cast<const float4*>(bl + static_cast<unsigned long long>(col) * row_bytes));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float ak = __shfl_sync(mask, av, k0 + u, LPR);  // slots past the end carry 0
          if (k0 + u < cnt) Vec<4>::fma(acc, ak, x[u]);
        }
      }
    }
  }
  atomicAdd(reinterpret_cast<float4*>(reinterpret_cast<char*>(c) + static_cast<size_t>(work.x) * row_bytes + off), acc);
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

namespace sptir {
// The launcher behind sparsetir_csrmm_raw.  hub_rows = false: never uses the hub-row launches
// (and so never touches the per-stream workspace) — for callers that know their rows are short
// or that hold the workspace themselves.
// lane_floats: 0 = the library's default lane width, 8 = 32-byte lanes where the operands allow.
int csrmm_run(const float* a, const float* b, float* c, const int32_t* indptr, const int32_t* indices,
              int m, int n, int feat, int nnz, int device_id, void* stream, bool hub_rows, int lane_floats) {
  if (m < 0 || feat < 0 || nnz < 0) return fail("sparsetir_csrmm: negative size");
  if (m == 0 || feat == 0) return 0;
  if (!b || !c || !indptr || (nnz > 0 && (!a || !indices)))
    return fail("sparsetir_csrmm: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (validate_enabled() && validate_csr("sparsetir_csrmm", indptr, m, indices, nnz, n, st) != 0) return -1;
  const bool vec4 = (feat % 4 == 0) && aligned16(b) && aligned16(c);
  if (vec4 && static_cast<long long>(feat) * 4 < (1ll << 32) &&
      static_cast<long long>(m) * feat * 4 < (1ll << 32) * 1024) {
    // lanes per row: one per 32-byte vector when the operands allow it, else one per 16-byte
    // vector; narrowed until the n x tile slice of B that a pass over the rows gathers from fits
    // the resident part of L2 (see hyb_spmm.cu)
    const int w = (feat % 32 == 0 && aligned32(b) && aligned32(c)) ? (lane_floats == 8 ? 8 : max_lane_floats()) : 4;
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
      // hub rows get their own launches once the matrix is large enough for one of them to
      // matter next to the cost of two more (small) launches
      // rows longer than this go to the hub-row launches (SPARSETIR_CSR_LONG_ROW overrides)
      static const int long_row_len = [] {
        const char* e = std::getenv("SPARSETIR_CSR_LONG_ROW");
        const int v = e ? std::atoi(e) : 0;
        return v >= 32 ? v : 32;
      }();
      const bool long_rows = hub_rows && w == 4 && nnz > long_row_len && (m >= 8192 || nnz >= 65536);
      int* count = nullptr;
      int2* list = nullptr;
      int max_entries = 0;
      if (long_rows) {
        max_entries = nnz / kLongChunk + nnz / long_row_len + 1;
        char* ws = static_cast<char*>(workspace(device_id, st, 16 + static_cast<size_t>(max_entries) * sizeof(int2)));
        if (!ws) return -1;
        count = reinterpret_cast<int*>(ws);
        list = reinterpret_cast<int2*>(ws + 16);
        SPTIR_CUDA_OK(cudaMemsetAsync(count, 0, sizeof(int), st));
        csr_plan_long_rows_kernel<<<ceil_div(m, kThreads), kThreads, 0, st>>>(indptr, m, feat, c, count, list,
                                                                             max_entries, long_row_len);
        SPTIR_LAUNCH_OK("csr_plan_long_rows_kernel");
      }
      const int long_row = long_rows ? long_row_len : 0;
#define SPTIR_CSR_LEAN(L, WW) \
  csrmm_lean_kernel<L, WW><<<grid, kThreads, 0, st>>>(a, b, c, indptr, indices, m, feat, rpi, long_row)
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
      if (long_rows) {
        dim3 lgrid(ceil_div(max_entries, subs), feat / (4 * lanes));
        if (lanes == 8)
          csr_long_rows_kernel<8><<<lgrid, kThreads, 0, st>>>(a, b, c, indptr, indices, feat, count, list, max_entries);
        else if (lanes == 16)
          csr_long_rows_kernel<16><<<lgrid, kThreads, 0, st>>>(a, b, c, indptr, indices, feat, count, list, max_entries);
        else
          csr_long_rows_kernel<32><<<lgrid, kThreads, 0, st>>>(a, b, c, indptr, indices, feat, count, list, max_entries);
        SPTIR_LAUNCH_OK("csr_long_rows_kernel");
      }
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

int csrmm_impl(const float* a, const float* b, float* c, const int32_t* indptr, const int32_t* indices,
               int m, int n, int feat, int nnz, int device_id, void* stream, bool hub_rows) {
  return csrmm_run(a, b, c, indptr, indices, m, n, feat, nnz, device_id, stream, hub_rows, 0);
}

// For matrices of very short rows (the aggregation launch of RGMS: 2.2 entries per row), where the
// kernel is bound by instruction issue: 32-byte lanes halve the instructions per gathered byte
// (60 -> 56.5 us at 690,812 rows x 64 features), although they lose on long rows and on launches
// too small to fill the SMs with the halved number of lanes (a quarter of those rows: 64 against
// 58 us for the whole operator), so they are taken from half a million rows up.
int csrmm_short_rows_impl(const float* a, const float* b, float* c, const int32_t* indptr,
                          const int32_t* indices, int m, int n, int feat, int nnz, int device_id,
                          void* stream) {
  return csrmm_run(a, b, c, indptr, indices, m, n, feat, nnz, device_id, stream, false, m >= (1 << 19) ? 8 : 0);
}
}  // namespace sptir

extern "C" int sparsetir_csrmm_raw(const float* a, const float* b, float* c, const int32_t* indptr,
                                   const int32_t* indices, int m, int n, int feat, int nnz,
                                   int device_id, void* stream) {
  return sptir::csrmm_impl(a, b, c, indptr, indices, m, n, feat, nnz, device_id, stream, true);
}
