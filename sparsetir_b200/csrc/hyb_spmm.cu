// Decomposed hyb SpMM, fp32: for every (partition, bucket) array q, ELL row r, slot s
//     C[rows_q[r], :] (+)= W_q[r,s] * B[cols_q[r,s], :]
// Replaces the horizontally fused kernel the reference generates in
// examples/spmm/bench_spmm.py:116-199 (argument list :207-222).  As there, ONE launch covers
// all buckets: the blockIdx.x range is the concatenation of the buckets' block ranges
// (the idea of src/tir/transforms/horizontal_fusion.cc:80-171), described by a small table
// passed by value in the kernel parameters — no device-side scratch, no host->device copy.
//
// Differences from the reference schedule, all invisible in the results:
//  - a work item (one sub-warp) covers about item_slots() stored slots whatever the bucket:
//    several ELL rows of a narrow bucket, or one item_slots()-slot piece of an ELL row of a wide
//    bucket.  Equal-sized items keep every SM busy until the end of the launch; the reference
//    equalises per block instead (8 * maxBucket slots per block, bench_spmm.py:187-189).
//    Wide buckets are scheduled first.
//  - the reference marks whole buckets atomic (bench_spmm.py:170,174-177).  Here the main (lean)
//    kernel gives every output row one writer: the pieces of a wide ELL row meet in shared memory,
//    the ELL rows of a row that the format split (src/sparse/format.cc:110-116: consecutive ELL
//    rows of the widest bucket repeating the row id) meet in a scratch buffer and are added in
//    order by the last one to finish — no atomics on the output, the same bits on every run.
//    The fallback kernels for odd shapes decide from the data instead: pieces of a chunked wide
//    ELL row and ELL rows whose id equals a neighbour's are added with vector atomics.
//    With several column partitions the same output row appears in several arrays, which the
//    kernels cannot see; the caller says so with SPARSETIR_HYB_ALL_ATOMIC.
#include <algorithm>
#include <cstdlib>
#include <vector>

#include "common.h"
#include "spmm_core.cuh"

namespace sptir {
namespace {

#ifndef SPTIR_HYB_MIN_BLOCKS
#define SPTIR_HYB_MIN_BLOCKS 3  // resident blocks per SM the register budget is sized for
#endif
constexpr int kThreads = 128;
constexpr int kMaxB = SPARSETIR_HYB_MAX_BUCKETS;

// Stored slots covered by one work item (one sub-warp of `lpr` lanes): four id batches, so that
// the per-item set-up is amortised and the id prefetch of spmm_core.cuh has something to hide.
constexpr int item_slots(int lpr) { return 4 * lpr; }
// lean kernel: lpr lanes of w floats each, `tiles` feature tiles (blockIdx.y), `slots` stored
// slots in all buckets.  Batches of ids per item, measured on the 169,343-node power-law graph
// (945,629 slots): with four feature tiles or more, 8 batches of 16-byte lanes (step over
// F = 32..512 0.385 ms; 4 batches 0.394, 12 batches 0.425, 16 batches 0.448; F = 128 59 against
// 64 us, F = 512 183 against 188 us) — longer items hide more of the id loads; with fewer tiles 4
// batches (F = 32: 26.0 against 27.3 us).  Row shards of that graph (half or a quarter of the
// slots) lose 5-9 % with 8 batches (F = 512 on half: 115 against 109 us): a pass over one feature
// tile then has too few blocks, so the longer items are for launches of 3/4 M slots or more.
// 32-byte lanes: 8 batches (the row ids of an item's rows of 8 slots or more travel in one
// register per lane, which caps an item at lpr such rows).
inline int lean_item_slots(int lpr, int w, int tiles, long long slots) {
  return lpr * w * ((w == 4 && tiles >= 4 && slots >= 3 * (1ll << 18)) ? 2 : 1);
}

struct HybTable {
  const float* w[kMaxB];
  const int32_t* rows[kMaxB];
  const int32_t* cols[kMaxB];
  int32_t nrows[kMaxB];
  int32_t width[kMaxB];
  int32_t rows_per_item[kMaxB];    // >= 1; 1 for chunked buckets
  int32_t chunks_per_row[kMaxB];   // 1 unless width > item_slots (lean kernel: sub-warps per ELL row)
  int32_t block_start[kMaxB + 1];
  int32_t row_base[kMaxB];         // buckets without a row-id array: ELL row r -> output row base + r
  int32_t part_base[kMaxB];        // lean kernel: scratch row of ELL row 0, or -1 (bucket has no split rows)
  int32_t nb;
};

__device__ __forceinline__ int find_bucket(const HybTable& tb, int block) {
  int q = 0;
  while (q + 1 < tb.nb && block >= tb.block_start[q + 1]) ++q;
  return q;
}

// A bucket without a row-id array (`rows == nullptr`) writes ELL row r to output row base + r.
__device__ __forceinline__ int row_id(const int32_t* __restrict__ rows, int r, int base) {
  return rows != nullptr ? __ldg(rows + r) : base + r;
}

__device__ __forceinline__ bool is_split_row(const int32_t* __restrict__ rows, int r, int nrows,
                                             int row) {
  if (rows == nullptr) return false;
  return (r > 0 && __ldg(rows + r - 1) == row) || (r + 1 < nrows && __ldg(rows + r + 1) == row);
}

template <int LPR, int VPL, int VEC>
__global__ void __launch_bounds__(kThreads, SPTIR_HYB_MIN_BLOCKS)
hyb_spmm_kernel(const __grid_constant__ HybTable tb, const float* __restrict__ b,
                float* __restrict__ c, int feat, int all_atomic) {
  using V = typename Vec<VEC>::type;
  constexpr int SUBS = kThreads / LPR;
  constexpr int ITEM = item_slots(LPR);
  // row ids of the item's ELL rows and of the two neighbouring ELL rows (-1 outside the
  // bucket): read at every row end, so they must not cost a trip to global memory there
  __shared__ int32_t s_rows[SUBS][ITEM + 2];
  const int lane = threadIdx.x % LPR;
  const int sub = threadIdx.x / LPR;
  const unsigned mask = group_mask<LPR>();
  const int q = find_bucket(tb, blockIdx.x);
  const int width = tb.width[q], nrows = tb.nrows[q];
  const int rpi = tb.rows_per_item[q], cpr = tb.chunks_per_row[q];
  const long long item = static_cast<long long>(blockIdx.x - tb.block_start[q]) * SUBS + sub;
  // slot range [first, first + nslots) of the bucket's flat slot array; `per_row` slots
  // complete one output contribution
  long long r0l;
  int nslots, per_row, nr;
  size_t first;
  if (cpr == 1) {
    r0l = item * rpi;
    if (r0l >= nrows) return;
    nr = static_cast<int>(min(static_cast<long long>(nrows), r0l + rpi) - r0l);
    nslots = nr * width;
    per_row = width;
    first = static_cast<size_t>(r0l) * width;
  } else {
    r0l = item / cpr;
    if (r0l >= nrows) return;
    const int s0 = static_cast<int>(item % cpr) * ITEM;
    nr = 1;
    nslots = min(ITEM, width - s0);
    per_row = nslots;
    first = static_cast<size_t>(r0l) * width + s0;
  }
  const int r0 = static_cast<int>(r0l);
  const int32_t* __restrict__ rows = tb.rows[q];
  for (int j = lane; j < nr + 2; j += LPR) {
    const int idx = r0 - 1 + j;
    s_rows[sub][j] = (idx >= 0 && idx < nrows) ? row_id(rows, idx, tb.row_base[q]) : -1;
  }
  __syncwarp(mask);
  const FeatLane<LPR, VPL, VEC> fl(feat, blockIdx.y, lane);
  V* cv = reinterpret_cast<V*>(c);
  const bool always_atomic = all_atomic || cpr > 1;

  V acc[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) acc[v] = Vec<VEC>::zero();
  int j = 1, left = per_row;  // s_rows[sub][j] is the id of the ELL row being accumulated
  auto on_done = [&](V(&)[VPL], int n) {
    left -= n;
    if (left != 0) return;
    const int row = s_rows[sub][j];
    const bool atomic = always_atomic || s_rows[sub][j - 1] == row || s_rows[sub][j + 1] == row;
    V* dst = cv + static_cast<size_t>(row) * fl.row_vecs;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (fl.valid[v]) {
        if (atomic) Vec<VEC>::atomic_add(dst + fl.off[v], acc[v]);
        else __stcs(dst + fl.off[v], acc[v]);  // written once: do not displace B rows in L2
      }
      acc[v] = Vec<VEC>::zero();
    }
    ++j;
    left = per_row;
  };
  const int32_t* cols = tb.cols[q] + first;
  const float* wts = tb.w[q] + first;
  const V* bv = reinterpret_cast<const V*>(b);
  // Row ends fall on chunk boundaries when the row length is a multiple of the chunk: then the
  // row-end test runs once per chunk instead of once per slot.
  const bool per_slot = per_row % ChunkOf<LPR, VPL>::value != 0;
  const bool full = feat % (LPR * VPL * VEC) == 0;
  if (per_slot) {
    if (full) stream_slots<LPR, VPL, VEC, true, true>(cols, wts, nslots, bv, fl, lane, mask, acc, on_done);
    else stream_slots<LPR, VPL, VEC, true, false>(cols, wts, nslots, bv, fl, lane, mask, acc, on_done);
  } else {
    if (full) stream_slots<LPR, VPL, VEC, false, true>(cols, wts, nslots, bv, fl, lane, mask, acc, on_done);
    else stream_slots<LPR, VPL, VEC, false, false>(cols, wts, nslots, bv, fl, lane, mask, acc, on_done);
  }
}

// ---------------------------------------------------------------------------------------------
// Lean kernel: the fast path for 16-byte aligned operands, whole feature tiles and ELL widths
// of 1, 2, 4 or a multiple of 8 (every power-of-two bucket list).  Written for instruction
// economy — the gathers come from L2 at well over 10 TB/s if, and only if, the warp spends its
// issue slots on loads: per stored slot the loop executes one shuffle + one address + one
// 16-byte load, then one shuffle + four FMAs; row ends sit at compile-time positions of the
// unrolled batch (narrow rows) or are tested once per 8 slots (wide rows); row ids travel in
// registers with two flag bits, so a row end costs one shuffle and a store.
//
// Every output row has ONE writer, so results are bit-identical from run to run and nothing has
// to be cleared between calls:
//  - an ELL row wider than a work item is cut into equal spans, one per sub-warp of the SAME
//    block; the partial sums meet in shared memory and are added in span order;
//  - a row that the format split into several ELL rows (consecutive ELL rows of the widest
//    bucket repeating the row id, src/sparse/format.cc:110-116) is reduced across blocks: each
//    piece stores its partial sum in a scratch row of its own and counts itself in; the piece that
//    counts in last adds all of them in ELL-row order and writes the output row.  The counter is
//    back at zero when the launch ends.
// With SPARSETIR_HYB_ALL_ATOMIC (several column partitions: the same row in several arrays, which
// the kernel cannot see) every contribution is added atomically into the zero-filled output.
// W = floats per lane: 4 (16-byte vectors) or 8 (32-byte vectors, two-wide FMAs)
constexpr int kFlagAtomic = static_cast<int>(0x80000000u);  // add atomically instead of storing

// row_flag(g): flag word of ELL row g (called by the lane that will hold it)
// row_end(acc, flag word): all lanes of the sub-warp, after the last slot of an ELL row
template <int LPR, int WM, int W, class RowFlag, class RowEnd>  // WM = 1, 2, 4: the ELL width itself; 8: a multiple of 8
__device__ __forceinline__ void lean_item(const int32_t* __restrict__ cols,
                                          const float* __restrict__ wts, int r0, int nr, int nslots,
                                          int per_row, const char* __restrict__ bl,
                                          unsigned row_bytes, int lane, unsigned mask,
                                          RowFlag&& row_flag, RowEnd&& row_end) {
  using LV = LaneVec<W>;
  using V = typename LV::type;
  constexpr int U = (32 / W) < LPR ? (32 / W) : LPR;  // gathered rows in flight: 32 registers
  // address of this lane's vector in dense row `col`: one 32x32->64 multiply-add
  auto vec_of = [&](const char* base, int col) -> const char* {
    return base + static_cast<unsigned long long>(static_cast<unsigned>(col)) * row_bytes;
  };
  static_assert(LPR % U == 0, "a batch is a whole number of chunks");
  constexpr int RPB = WM < 8 ? LPR / WM : 0;  // ELL rows that end inside one batch (narrow rows)

  V acc = LV::zero();
  int c = 0, rf = 0;
  float a = 0.f;
  if (lane < nslots) {
    c = __ldg(cols + lane);
    a = __ldg(wts + lane);
  }
  if (WM < 8) {
    if (lane < RPB && lane < nr) rf = row_flag(r0 + lane);   // rows ending in batch 0
  } else {
    if (lane < nr) rf = row_flag(r0 + lane);                  // all rows of the item (nr <= LPR)
  }
  int left = per_row, jrow = 0;  // wide rows only

  for (int s0 = 0; s0 < nslots; s0 += LPR) {
    int cn = 0, rfn = 0;
    float an = 0.f;
    if (s0 + LPR + lane < nslots) {  // ids, weights (and row ids) of the next batch
      cn = __ldg(cols + s0 + LPR + lane);
      an = __ldg(wts + s0 + LPR + lane);
    }
    if (WM < 8 && lane < RPB && (s0 + LPR) / WM + lane < nr) rfn = row_flag(r0 + (s0 + LPR) / WM + lane);
    const int cnt = nslots - s0;  // live slots of this batch if < LPR
    if (cnt >= LPR) {
#pragma unroll
      for (int k0 = 0; k0 < LPR; k0 += U) {
        V x[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          x[u] = LV::ldg(vec_of(bl, __shfl_sync(mask, c, k0 + u, LPR)));
#pragma unroll
        for (int u = 0; u < U; ++u) {
          LV::fma(acc, __shfl_sync(mask, a, k0 + u, LPR), x[u]);
          if (WM < 8 && (k0 + u + 1) % WM == 0)
            row_end(acc, __shfl_sync(mask, rf, (k0 + u) / WM, LPR));
        }
        if (WM == 8) {
          left -= U;
          if (left == 0) {
            row_end(acc, __shfl_sync(mask, rf, jrow, LPR));
            ++jrow;
            left = per_row;
          }
        }
      }
    } else {  // last, partly filled batch: slots past the end are neither added nor stored
#pragma unroll
      for (int k0 = 0; k0 < LPR; k0 += U) {
        if (k0 < cnt) {
          V x[U];
#pragma unroll
          for (int u = 0; u < U; ++u)
            x[u] = LV::ldg(vec_of(bl, __shfl_sync(mask, c, k0 + u, LPR)));  // dead slots: column 0
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const float ak = __shfl_sync(mask, a, k0 + u, LPR);
            const int rfe = (WM < 8) ? __shfl_sync(mask, rf, (k0 + u) / WM, LPR) : 0;
            if (k0 + u < cnt) {
              LV::fma(acc, ak, x[u]);
              if (WM < 8 && (k0 + u + 1) % WM == 0) row_end(acc, rfe);
            }
          }
          if (WM == 8) {  // wide rows: nslots is a multiple of 8, so the chunk was whole
            left -= U;
            if (left == 0) {
              row_end(acc, __shfl_sync(mask, rf, jrow, LPR));
              ++jrow;
              left = per_row;
            }
          }
        }
      }
    }
    c = cn;
    a = an;
    if (WM < 8) rf = rfn;
  }
}

// What the lean kernel needs besides the bucket table.
struct LeanArgs {
  const float* b;
  float* c;
  float* part;          // scratch rows for the pieces of split rows (same row stride as c)
  unsigned* counters;   // [scratch rows][feature tiles], zero before and after every launch
  int feat;
  int all_atomic;
  PeerOut peers;
};

// The one store of a finished piece of an output row: into this GPU's C and, when the call has
// peers, into every peer's copy (plain stores over NVLink; nothing waits on them).
template <int W>
__device__ __forceinline__ void store_out(char* p, const typename LaneVec<W>::type& v, const PeerOut* po) {
  LaneVec<W>::stcs(p, v);
  if (po != nullptr)
    for (int k = 0; k < po->n; ++k) LaneVec<W>::stcg(p + po->delta[k], v);
}

// Bits of `pred` over the LPR lanes of this thread's sub-warp, lane 0 of the sub-warp in bit 0.
template <int LPR>
__device__ __forceinline__ unsigned sub_ballot(unsigned mask, bool pred) {
  const unsigned all = __ballot_sync(mask, pred);
  if constexpr (LPR == 32) {
    return all;
  } else {
    return (all >> ((threadIdx.x & 31) / LPR * LPR)) & ((1u << LPR) - 1u);
  }
}

// The last ELL row `g` of a piece of a split row has been accumulated into `acc` by this
// sub-warp.  A piece is the part of a run of equal row ids that lies inside one work item
// (items hold `rpi` consecutive ELL rows; rpi = 1 for wide buckets).  Pieces are numbered in
// ELL-row order; piece k keeps its partial sum in the scratch row of its first ELL row.
template <int LPR, int W>
__device__ __noinline__ void finish_split_row(typename LaneVec<W>::type acc,
                                              const int32_t* __restrict__ rows, int nrows, int g,
                                              int rpi, int rid, int part_base, char* pl, char* cl,
                                              unsigned* counters, unsigned row_bytes, int lane,
                                              unsigned mask, const PeerOut* po) {
  using LV = LaneVec<W>;
  constexpr unsigned kFull = LPR == 32 ? 0xffffffffu : ((1u << LPR) - 1u);
  int first = g, last = g;
  while (true) {  // LPR ELL rows per step, backwards then forwards
    const int idx = first - 1 - lane;
    const unsigned bits = sub_ballot<LPR>(mask, idx >= 0 && __ldg(rows + idx) == rid);
    const int n = bits == kFull ? LPR : __ffs(~bits) - 1;
    first -= n;
    if (n < LPR) break;
  }
  while (true) {
    const int idx = last + 1 + lane;
    const unsigned bits = sub_ballot<LPR>(mask, idx < nrows && __ldg(rows + idx) == rid);
    const int n = bits == kFull ? LPR : __ffs(~bits) - 1;
    last += n;
    if (n < LPR) break;
  }
  const int item0 = first / rpi;
  const int npieces = last / rpi - item0 + 1;
  char* dst = cl + static_cast<unsigned long long>(static_cast<unsigned>(rid)) * row_bytes;
  if (npieces == 1) {  // the whole run lies inside this item
    store_out<W>(dst, acc, po);
    return;
  }
  const int mine = max(first, g / rpi * rpi);
  auto part_of = [&](int ell_row) -> char* {
    return pl + static_cast<unsigned long long>(static_cast<unsigned>(part_base + ell_row)) * row_bytes;
  };
  LV::stcg(part_of(mine), acc);
  __threadfence();
  __syncwarp(mask);
  unsigned* counter = counters + static_cast<size_t>(part_base + first) * gridDim.y + blockIdx.y;
  unsigned seen = 0;
  if (lane == 0) seen = atomicAdd(counter, 1u);
  seen = __shfl_sync(mask, seen, 0, LPR);
  if (seen + 1 != static_cast<unsigned>(npieces)) return;
  // last piece to arrive: every other piece's partial sum is visible
  if (lane == 0) *counter = 0u;
  __threadfence();
  typename LV::type sum = LV::ldcg(part_of(first));
  for (int k = 1; k < npieces; ++k) LV::add(sum, LV::ldcg(part_of((item0 + k) * rpi)));
  store_out<W>(dst, sum, po);
}

// A narrow item of the widest bucket that holds ELL rows of a split row (rare: only bucket lists
// whose last width is small put split rows into a narrow bucket).  Plain loop, one ELL row at a
// time; consecutive ELL rows of the same output row inside the item are added up first.
template <int LPR, int W>
__device__ __noinline__ void split_item(const int32_t* __restrict__ cols, const float* __restrict__ wts,
                                        const int32_t* __restrict__ rows, int nrows, int r0, int nr,
                                        int width, int rpi, int part_base, const char* __restrict__ bl,
                                        char* pl, char* cl, unsigned* counters, unsigned row_bytes,
                                        int lane, unsigned mask, const PeerOut* po) {
  using LV = LaneVec<W>;
  typename LV::type acc = LV::zero();
  for (int j = 0; j < nr; ++j) {
    const int g = r0 + j;
    for (int s = 0; s < width; ++s) {
      const int col = __ldg(cols + j * width + s);
      const float a = __ldg(wts + j * width + s);
      LV::fma(acc, a, LV::ldg(bl + static_cast<unsigned long long>(static_cast<unsigned>(col)) * row_bytes));
    }
    const int rid = __ldg(rows + g);
    const bool next_same = g + 1 < nrows && __ldg(rows + g + 1) == rid;
    if (next_same && j + 1 < nr) continue;  // the next ELL row of this item continues the row
    if (next_same || (g > 0 && __ldg(rows + g - 1) == rid))
      finish_split_row<LPR, W>(acc, rows, nrows, g, rpi, rid, part_base, pl, cl, counters, row_bytes, lane, mask,
                               po);
    else
      store_out<W>(cl + static_cast<unsigned long long>(static_cast<unsigned>(rid)) * row_bytes, acc, po);
    acc = LV::zero();
  }
}

template <int LPR, int W, bool PEERS>
__global__ void __launch_bounds__(kThreads, 8)
hyb_spmm_lean_kernel(const __grid_constant__ HybTable tb, const __grid_constant__ LeanArgs la) {
  using LV = LaneVec<W>;
  using V = typename LV::type;
  const PeerOut* po = PEERS ? &la.peers : nullptr;
  constexpr int SUBS = kThreads / LPR;
  __shared__ __align__(32) float s_part[SUBS][LPR * W];  // wide rows: partial sums of the spans
  const int lane = threadIdx.x % LPR;
  const int sub = threadIdx.x / LPR;
  const unsigned mask = group_mask<LPR>();
  const int q = find_bucket(tb, blockIdx.x);
  const int width = tb.width[q], nrows = tb.nrows[q];
  const int rpi = tb.rows_per_item[q], spr = tb.chunks_per_row[q];
  const int part_base = tb.part_base[q];
  const unsigned stride = static_cast<unsigned>(la.feat) * 4u;  // bytes per dense row
  const unsigned off = (blockIdx.y * LPR + lane) * (W * 4u);  // this lane's piece of the tile
  const char* bl = reinterpret_cast<const char*>(la.b) + off;
  char* cl = reinterpret_cast<char*>(la.c) + off;
  char* pl = reinterpret_cast<char*>(la.part) + off;
  const int32_t* rows = tb.rows[q];
  if (rows == nullptr) cl += static_cast<size_t>(tb.row_base[q]) * stride;
  const bool all_atomic = la.all_atomic != 0;
  auto y_of = [&](int rid) -> char* {
    return cl + static_cast<unsigned long long>(static_cast<unsigned>(rid)) * stride;
  };

  if (spr == 1) {
    // ---- narrow bucket: a sub-warp owns rpi whole ELL rows
    const long long item = static_cast<long long>(blockIdx.x - tb.block_start[q]) * SUBS + sub;
    const long long r0l = item * rpi;
    if (r0l >= nrows) return;
    const int r0 = static_cast<int>(r0l);
    const int nr = min(nrows, r0 + rpi) - r0;
    const size_t first = static_cast<size_t>(r0) * width;
    if (!all_atomic && part_base >= 0) {
      // the widest bucket: an item that holds an ELL row of a split row takes the careful path
      bool any = false;
      for (int j = lane; j < nr; j += LPR) any = any || is_split_row(rows, r0 + j, nrows, __ldg(rows + r0 + j));
      if (sub_ballot<LPR>(mask, any) != 0u) {
        split_item<LPR, W>(tb.cols[q] + first, tb.w[q] + first, rows, nrows, r0, nr, width, rpi, part_base,
                           bl, pl, cl, la.counters, stride, lane, mask, po);
        return;
      }
    }
    auto row_flag = [&](int g) -> int {
      // a bucket without row ids has its base folded into cl
      return row_id(rows, g, 0) | (all_atomic ? kFlagAtomic : 0);
    };
    auto row_end = [&](V& acc, int rf) {
      if (rf < 0) LV::atomic_add(y_of(rf & 0x7fffffff), acc);
      else store_out<W>(y_of(rf), acc, po);  // written once: do not displace B rows in L2
      acc = LV::zero();
    };
    const int32_t* cols = tb.cols[q] + first;
    const float* wts = tb.w[q] + first;
    const int nslots = nr * width;
    if (width == 1) lean_item<LPR, 1, W>(cols, wts, r0, nr, nslots, width, bl, stride, lane, mask, row_flag, row_end);
    else if (width == 2) lean_item<LPR, 2, W>(cols, wts, r0, nr, nslots, width, bl, stride, lane, mask, row_flag, row_end);
    else if (width == 4) lean_item<LPR, 4, W>(cols, wts, r0, nr, nslots, width, bl, stride, lane, mask, row_flag, row_end);
    else lean_item<LPR, 8, W>(cols, wts, r0, nr, nslots, width, bl, stride, lane, mask, row_flag, row_end);
    return;
  }

  // ---- wide bucket: spr sub-warps of this block share one ELL row, each takes one span of it
  const int rpb = SUBS / spr;  // ELL rows per block
  const int part = sub % spr;
  const long long rl = static_cast<long long>(blockIdx.x - tb.block_start[q]) * rpb + sub / spr;
  const bool live = rl < nrows;
  const int r = live ? static_cast<int>(rl) : 0;
  const int span = ((width + spr - 1) / spr + 7) & ~7;  // slots per span, a multiple of 8
  V total = LV::zero();
  if (live && part * span < width) {
    const int s0 = part * span;
    const int nslots = min(span, width - s0);
    const size_t first = static_cast<size_t>(r) * width + s0;
    auto no_flag = [](int) -> int { return 0; };
    auto keep = [&](V& acc, int) { total = acc; };
    lean_item<LPR, 8, W>(tb.cols[q] + first, tb.w[q] + first, r, 1, nslots, nslots, bl, stride, lane, mask,
                         no_flag, keep);
  }
  if (part != 0) LV::sts(&s_part[sub][lane * W], total);
  __syncthreads();
  if (!live || part != 0) return;
  for (int k = 1; k < spr; ++k) LV::add(total, LV::lds(&s_part[sub + k][lane * W]));
  const int rid = row_id(rows, r, 0);
  if (all_atomic) {
    LV::atomic_add(y_of(rid), total);
  } else if (part_base >= 0 && is_split_row(rows, r, nrows, rid)) {
    finish_split_row<LPR, W>(total, rows, nrows, r, 1, rid, part_base, pl, cl, la.counters, stride, lane, mask,
                             po);
  } else {
    store_out<W>(y_of(rid), total, po);
  }
}

// The main kernel for 16-byte aligned operands: B rows are staged through per-lane rings in
// shared memory by asynchronous copies (see stream_slots_async), ids / weights / row ids of the
// item are read into shared memory once, with coalesced loads, before the pipeline starts.
// One lane covers one 16-byte vector of a 4*LPR-float feature tile; blockIdx.y walks the tiles.
constexpr int kRing = 12;  // slots in flight per lane

template <int LPR>
struct AsyncSmem {
  static constexpr int SUBS = kThreads / LPR;
  static constexpr int ITEM = item_slots(LPR);
  static constexpr size_t ring_bytes = sizeof(float4) * SUBS * kRing * LPR;
  static constexpr size_t bytes = ring_bytes + sizeof(int32_t) * SUBS * (ITEM + ITEM + ITEM + 2);
};

template <int LPR>
__global__ void __launch_bounds__(kThreads, 3)
hyb_spmm_async_kernel(const __grid_constant__ HybTable tb, const float* __restrict__ b,
                      float* __restrict__ c, int feat, int all_atomic) {
  using S = AsyncSmem<LPR>;
  constexpr int SUBS = S::SUBS, ITEM = S::ITEM;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x % LPR;
  const int sub = threadIdx.x / LPR;
  float4* ring = reinterpret_cast<float4*>(smem_raw) + sub * (kRing * LPR) + lane;
  int32_t* s_ids = reinterpret_cast<int32_t*>(smem_raw + S::ring_bytes) + sub * ITEM;
  float* s_wts = reinterpret_cast<float*>(smem_raw + S::ring_bytes) + SUBS * ITEM + sub * ITEM;
  int32_t* s_rows = reinterpret_cast<int32_t*>(smem_raw + S::ring_bytes) + 2 * SUBS * ITEM +
                    sub * (ITEM + 2);
  const unsigned mask = group_mask<LPR>();
  const int q = find_bucket(tb, blockIdx.x);
  const int width = tb.width[q], nrows = tb.nrows[q];
  const int rpi = tb.rows_per_item[q], cpr = tb.chunks_per_row[q];
  const long long item = static_cast<long long>(blockIdx.x - tb.block_start[q]) * SUBS + sub;
  long long r0l;
  int nslots, per_row, nr;
  size_t first;
  if (cpr == 1) {
    r0l = item * rpi;
    if (r0l >= nrows) return;
    nr = static_cast<int>(min(static_cast<long long>(nrows), r0l + rpi) - r0l);
    nslots = nr * width;
    per_row = width;
    first = static_cast<size_t>(r0l) * width;
  } else {
    r0l = item / cpr;
    if (r0l >= nrows) return;
    const int s0 = static_cast<int>(item % cpr) * ITEM;
    nr = 1;
    nslots = min(ITEM, width - s0);
    per_row = nslots;
    first = static_cast<size_t>(r0l) * width + s0;
  }
  const int r0 = static_cast<int>(r0l);
  {
    const int32_t* __restrict__ cols = tb.cols[q] + first;
    const float* __restrict__ wts = tb.w[q] + first;
    const int32_t* __restrict__ rows = tb.rows[q];
    for (int s = lane; s < nslots; s += LPR) {
      s_ids[s] = __ldg(cols + s);
      s_wts[s] = __ldg(wts + s);
    }
    for (int j = lane; j < nr + 2; j += LPR) {
      const int idx = r0 - 1 + j;
      s_rows[j] = (idx >= 0 && idx < nrows) ? row_id(rows, idx, tb.row_base[q]) : -1;
    }
  }
  __syncwarp(mask);
  const int row_vecs = feat / 4;
  const int off = blockIdx.y * LPR + lane;
  const bool valid = off < row_vecs;
  float4* cv = reinterpret_cast<float4*>(c) + off;
  const bool always_atomic = all_atomic || cpr > 1;

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  int j = 1, left = per_row;
  auto on_done = [&](float4&, int n) {
    left -= n;
    if (left != 0) return;
    const int row = s_rows[j];
    const bool atomic = always_atomic || s_rows[j - 1] == row || s_rows[j + 1] == row;
    float4* dst = cv + static_cast<size_t>(row) * row_vecs;
    if (valid) {
      if (atomic) atomicAdd(dst, acc);
      else __stcs(dst, acc);  // written once: do not displace B rows in L2
    }
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    ++j;
    left = per_row;
  };
  const float4* bl = reinterpret_cast<const float4*>(b) + off;
  // Row ends fall on group boundaries when the row length is a multiple of 4: then the row-end
  // test runs once per group instead of once per slot.
  if (per_row % 4 != 0)
    stream_slots_async<LPR, kRing, true>(s_ids, s_wts, nslots, bl, static_cast<size_t>(row_vecs),
                                         valid, ring, acc, on_done);
  else
    stream_slots_async<LPR, kRing, false>(s_ids, s_wts, nslots, bl, static_cast<size_t>(row_vecs),
                                          valid, ring, acc, on_done);
}

// Fallback kernels only: zeroes the output rows that they accumulate into atomically (chunked wide
// rows and split rows), so that repeated calls on the same C stay correct without a full memset.
// One thread inspects one ELL row (coalesced reads of the row ids); the rows that need clearing
// are rare, and each is then cleared by the whole warp.
__global__ void __launch_bounds__(kThreads)
hyb_rearm_kernel(const __grid_constant__ HybTable tb, float* __restrict__ c, int feat) {
  const int q = find_bucket(tb, blockIdx.x);
  const int nrows = tb.nrows[q];
  const int32_t* __restrict__ rows = tb.rows[q];
  const long long r = static_cast<long long>(blockIdx.x - tb.block_start[q]) * kThreads + threadIdx.x;
  int row = -1;
  bool clear = false;
  if (r < nrows) {
    row = row_id(rows, static_cast<int>(r), tb.row_base[q]);
    clear = tb.chunks_per_row[q] > 1 || is_split_row(rows, static_cast<int>(r), nrows, row);
    // of a run of equal ids only the first ELL row clears
    if (clear && r > 0 && rows != nullptr && __ldg(rows + r - 1) == row) clear = false;
  }
  unsigned todo = __ballot_sync(0xffffffffu, clear);
  const int lane = threadIdx.x & 31;
  while (todo != 0) {
    const int src = __ffs(todo) - 1;
    todo &= todo - 1;
    const int rr = __shfl_sync(0xffffffffu, row, src);
    float* dst = c + static_cast<size_t>(rr) * feat;
    for (int f = lane; f < feat; f += 32) dst[f] = 0.f;
  }
}

// Scratch (bytes) the lean kernel may use for the pieces of split rows before it falls back to
// atomic accumulation; SPARSETIR_HYB_SCRATCH_MB overrides the default of 1 GiB.
size_t hyb_scratch_limit() {
  static const size_t v = [] {
    const char* e = std::getenv("SPARSETIR_HYB_SCRATCH_MB");
    const long mb = e ? std::atol(e) : -1;
    return static_cast<size_t>(mb >= 0 ? mb : 1024) << 20;
  }();
  return v;
}

void plan_items(HybTable& tb, int item) {
  for (int q = 0; q < tb.nb; ++q) {
    tb.rows_per_item[q] = std::max(1, item / tb.width[q]);
    tb.chunks_per_row[q] = tb.width[q] > item ? ceil_div(tb.width[q], item) : 1;
  }
}

// Lean kernel: a bucket wider than an item gives each ELL row a power-of-two number of sub-warps of
// one block (all of them from SUBS * item slots on; a sub-warp then walks a longer span).
void plan_items_lean(HybTable& tb, int item, int subs) {
  for (int q = 0; q < tb.nb; ++q) {
    tb.rows_per_item[q] = std::max(1, item / tb.width[q]);
    // rows of 8 slots or more: the row ids of an item travel in one register per lane
    if (tb.width[q] >= 8) tb.rows_per_item[q] = std::min(tb.rows_per_item[q], kThreads / subs);
    int spr = 1;
    while (spr < subs && spr * item < tb.width[q]) spr *= 2;
    tb.chunks_per_row[q] = spr;
    if (spr > 1) tb.rows_per_item[q] = 1;
  }
}

long long plan_blocks_lean(HybTable& tb, int subs) {
  long long blocks = 0;
  for (int q = 0; q < tb.nb; ++q) {
    tb.block_start[q] = static_cast<int32_t>(blocks);
    const int spr = tb.chunks_per_row[q];
    const long long per_block = spr > 1 ? subs / spr : static_cast<long long>(subs) * tb.rows_per_item[q];
    blocks += (tb.nrows[q] + per_block - 1) / per_block;
    if (blocks > INT32_MAX) return -1;
  }
  tb.block_start[tb.nb] = static_cast<int32_t>(blocks);
  return blocks;
}

// Lanes per dense row, the first template argument of the kernel used: one lane per 16-byte
// vector, at most a warp.  Rows wider than the lanes cover are walked feature tile by feature
// tile (blockIdx.y, the slowest grid dimension).  A pass gathers from an n x tile slice of B; the
// tile is narrowed until that slice fits the part of L2 that stays resident for data every SM
// reads (measured: about half of the 126 MB), because re-reading the index arrays once per tile
// costs little next to re-fetching B rows from HBM.
int lanes_per_row_impl(int feat, bool vec4, int n, int lane_w) {
  const int units = vec4 ? feat / lane_w : feat;
  const int min_lanes = lane_w == 8 ? 4 : 8;
  int lanes = units <= min_lanes ? min_lanes : (units <= 8 ? 8 : (units <= 16 ? 16 : 32));
  if (vec4) {
    // SPARSETIR_L2_BUDGET_MB overrides the default for tuning on other parts
    static const size_t l2_budget = [] {
      const char* e = std::getenv("SPARSETIR_L2_BUDGET_MB");
      const long mb = e ? std::atol(e) : 0;
      return static_cast<size_t>(mb > 0 ? mb : 48) << 20;
    }();
    while (lanes > min_lanes && static_cast<size_t>(n) * lanes * lane_w * 4 > l2_budget) lanes /= 2;
    // Up to `narrow_passes` passes over the index arrays the narrowest tile wins even when a
    // wider slice would fit L2: twice the independent sub-warps per block keep more gathers in
    // flight (measured on B200: F = 64 38 vs 41 us, F = 128 60 vs 66 us, F = 256 equal, F = 512
    // 211 vs 197 us, where the 16 passes re-read 120 MB of ids).
    static const int narrow_passes = [] {
      const char* e = std::getenv("SPARSETIR_HYB_NARROW_PASSES");
      const int v = e ? std::atoi(e) : -1;
      return v >= 0 ? v : 4;
    }();
    if (lanes > min_lanes && feat % (min_lanes * lane_w) == 0 && feat / (min_lanes * lane_w) <= narrow_passes)
      lanes = min_lanes;
  }
  return lanes;
}

// Fills block_start for SUBS items per block; returns the number of blocks or -1.
long long plan_blocks(HybTable& tb, int subs) {
  long long blocks = 0;
  for (int q = 0; q < tb.nb; ++q) {
    tb.block_start[q] = static_cast<int32_t>(blocks);
    const long long items = tb.chunks_per_row[q] > 1
                                ? static_cast<long long>(tb.nrows[q]) * tb.chunks_per_row[q]
                                : ceil_div(tb.nrows[q], tb.rows_per_item[q]);
    blocks += (items + subs - 1) / subs;
    if (blocks > INT32_MAX) return -1;
  }
  tb.block_start[tb.nb] = static_cast<int32_t>(blocks);
  return blocks;
}

template <int LPR, int W>
int launch_lean(HybTable& tb, const LeanArgs& la, cudaStream_t stream) {
  long long slots = 0;
  for (int q = 0; q < tb.nb; ++q) slots += static_cast<long long>(tb.nrows[q]) * tb.width[q];
  plan_items_lean(tb, lean_item_slots(LPR, W, la.feat / (W * LPR), slots), kThreads / LPR);
  const long long blocks = plan_blocks_lean(tb, kThreads / LPR);
  if (blocks < 0) return fail("sparsetir_hyb_spmm: too many thread blocks");
  dim3 grid(static_cast<unsigned>(blocks), la.feat / (W * LPR));
  if (la.peers.n > 0) {
    if constexpr (W == 4)
      hyb_spmm_lean_kernel<LPR, W, true><<<grid, kThreads, 0, stream>>>(tb, la);
    else
      return fail("sparsetir_hyb_spmm_peers: no 32-byte-lane form");  // the dispatcher picks 16-byte lanes
  } else {
    hyb_spmm_lean_kernel<LPR, W, false><<<grid, kThreads, 0, stream>>>(tb, la);
  }
  SPTIR_LAUNCH_OK("hyb_spmm_lean_kernel");
  return 0;
}

int dispatch_lean(HybTable& tb, const LeanArgs& la, int lanes, int lane_w, cudaStream_t st) {
  if (lane_w == 8) {
    if (lanes == 4) return launch_lean<4, 8>(tb, la, st);
    if (lanes == 8) return launch_lean<8, 8>(tb, la, st);
    if (lanes == 16) return launch_lean<16, 8>(tb, la, st);
    return launch_lean<32, 8>(tb, la, st);
  }
  if (lanes == 8) return launch_lean<8, 4>(tb, la, st);
  if (lanes == 16) return launch_lean<16, 4>(tb, la, st);
  return launch_lean<32, 4>(tb, la, st);
}

template <int LPR>
int launch_async(HybTable& tb, const float* b, float* c, int feat, int all_atomic,
                 cudaStream_t stream) {
  using S = AsyncSmem<LPR>;
  const long long blocks = plan_blocks(tb, S::SUBS);
  if (blocks < 0) return fail("sparsetir_hyb_spmm: too many thread blocks");
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(hyb_spmm_async_kernel<LPR>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(S::bytes)));
    configured_device = dev;
  }
  dim3 grid(static_cast<unsigned>(blocks), ceil_div(feat / 4, LPR));
  hyb_spmm_async_kernel<LPR><<<grid, kThreads, S::bytes, stream>>>(tb, b, c, feat, all_atomic);
  SPTIR_LAUNCH_OK("hyb_spmm_async_kernel");
  return 0;
}

template <int LPR, int VPL, int VEC>
int launch(HybTable& tb, const float* b, float* c, int feat, int all_atomic, cudaStream_t stream) {
  const long long blocks = plan_blocks(tb, kThreads / LPR);
  if (blocks < 0) return fail("sparsetir_hyb_spmm: too many thread blocks");
  const int tile_feat = LPR * VPL * VEC;
  dim3 grid(static_cast<unsigned>(blocks), ceil_div(feat, tile_feat));
  hyb_spmm_kernel<LPR, VPL, VEC><<<grid, kThreads, 0, stream>>>(tb, b, c, feat, all_atomic);
  SPTIR_LAUNCH_OK("hyb_spmm_kernel");
  return 0;
}

}  // namespace
}  // namespace sptir

namespace sptir {
size_t hyb_scratch_limit_bytes() { return hyb_scratch_limit(); }
int lanes_per_row(int feat, bool vec4, int n, int lane_w) { return lanes_per_row_impl(feat, vec4, n, lane_w); }

// The launcher behind sparsetir_hyb_spmm_raw.  row_bases (may be null): for buckets whose `rows`
// array is null, ELL row r of bucket q is written to output row row_bases[q] + r.
int hyb_spmm_run(const float* b, float* c, const SparsetirEllBucket* buckets, const int32_t* row_bases,
                 int num_buckets, int m, int n, int feat, int flags, int device_id, void* stream,
                 const PeerOut* peers) {
  if (num_buckets < 0 || num_buckets > kMaxB)
    return fail("sparsetir_hyb_spmm: %d buckets exceed the maximum of %d", num_buckets, kMaxB);
  if (m < 0 || feat < 0) return fail("sparsetir_hyb_spmm: negative size");
  if (num_buckets > 0 && !buckets) return fail("sparsetir_hyb_spmm: null bucket table");
  if (feat == 0 || m == 0) return 0;
  if (!b || !c) return fail("sparsetir_hyb_spmm: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int all_atomic = (flags & SPARSETIR_HYB_ALL_ATOMIC) ? 1 : 0;

  // Table in launch order: widest bucket first, empty buckets dropped.
  std::vector<int> order;
  for (int q = 0; q < num_buckets; ++q) {
    const SparsetirEllBucket& bk = buckets[q];
    if (bk.nrows < 0 || bk.width < 0) return fail("sparsetir_hyb_spmm: negative bucket size");
    if (bk.nrows == 0) continue;
    if (bk.width == 0) return fail("sparsetir_hyb_spmm: bucket %d has rows but width 0", q);
    // rows may be null: ELL row r then belongs to output row r
    if (!bk.w || !bk.cols) return fail("sparsetir_hyb_spmm: null bucket array");
    order.push_back(q);
  }
  std::stable_sort(order.begin(), order.end(),
                   [&](int x, int y) { return buckets[x].width > buckets[y].width; });
  HybTable tb{};
  tb.nb = static_cast<int32_t>(order.size());
  for (int k = 0; k < tb.nb; ++k) {
    const SparsetirEllBucket& bk = buckets[order[k]];
    tb.w[k] = bk.w; tb.rows[k] = bk.rows; tb.cols[k] = bk.cols;
    tb.nrows[k] = bk.nrows; tb.width[k] = bk.width;
    tb.row_base[k] = row_bases ? row_bases[order[k]] : 0;
  }
  if (validate_enabled()) {
    for (int k = 0; k < tb.nb; ++k) {
      const long long slots = static_cast<long long>(tb.nrows[k]) * tb.width[k];
      if (validate_range("sparsetir_hyb_spmm", "a bucket's row_indices", tb.rows[k], tb.nrows[k], m, st) != 0 ||
          validate_range("sparsetir_hyb_spmm", "a bucket's col_indices", tb.cols[k], slots, n, st) != 0)
        return -1;
    }
  }
  const bool vec4 = (feat % 4 == 0) && aligned16(b) && aligned16(c);
  // the lean kernel takes whole feature tiles and ELL widths of 1, 2, 4 or a multiple of 8; with
  // 32-byte aligned operands and a multiple of 32 features its lanes own 8 floats, else 4
  bool lean = vec4 && static_cast<long long>(feat) * 4 < (1ll << 32);
  for (int q = 0; q < tb.nb; ++q) {
    const int w = tb.width[q];
    lean = lean && (w == 1 || w == 2 || w == 4 || w % 8 == 0);
  }
  const bool to_peers = peers != nullptr && peers->n > 0;
  // the form that stores to peers exists for 16-byte lanes only (the library's default)
  int lane_w = (lean && !to_peers && feat % 32 == 0 && aligned32(b) && aligned32(c)) ? max_lane_floats() : 4;
  int lanes = lanes_per_row_impl(feat, vec4, n, lane_w);
  if (lane_w == 8 && feat % (lane_w * lanes) != 0) {  // no whole tiles of 8-float lanes
    lane_w = 4;
    lanes = lanes_per_row_impl(feat, vec4, n, lane_w);
  }
  lean = lean && feat % (lane_w * lanes) == 0;
  const size_t c_bytes = static_cast<size_t>(m) * feat * sizeof(float);
  if (to_peers && (!lean || all_atomic || (flags & SPARSETIR_HYB_ZERO_C)))
    return fail("sparsetir_hyb_spmm_peers: needs the one-writer kernel (feat_size a multiple of its tile, "
                "16-byte aligned b and c, bucket widths 1, 2, 4 or multiples of 8, no ALL_ATOMIC or ZERO_C "
                "flag); run sparsetir_hyb_spmm and sparsetir_peer_scatter instead");
  if (tb.nb == 0) {
    if (flags & SPARSETIR_HYB_ZERO_C) SPTIR_CUDA_OK(cudaMemsetAsync(c, 0, c_bytes, st));
    return 0;
  }

  if (lean) {
    // ---- one writer per output row (or everything atomic when the caller asks for it)
    LeanArgs la{b, c, nullptr, nullptr, feat, all_atomic, PeerOut{}};
    if (to_peers) la.peers = *peers;
    bool clear = (flags & SPARSETIR_HYB_ZERO_C) || (all_atomic && (flags & SPARSETIR_HYB_REARM));
    for (int q = 0; q < tb.nb; ++q) tb.part_base[q] = -1;
    if (!all_atomic) {
      // split rows live in the widest bucket(s) that carry row ids: one scratch row per ELL row
      int maxw = 0;
      for (int q = 0; q < tb.nb; ++q)
        if (tb.rows[q] != nullptr) maxw = std::max(maxw, tb.width[q]);
      long long part_rows = 0;
      for (int q = 0; q < tb.nb; ++q)
        if (tb.rows[q] != nullptr && tb.width[q] == maxw) {
          tb.part_base[q] = static_cast<int32_t>(part_rows);
          part_rows += tb.nrows[q];
        }
      const int tiles = feat / (lane_w * lanes);
      const size_t part_bytes = static_cast<size_t>(part_rows) * feat * sizeof(float);
      const size_t counter_bytes = static_cast<size_t>(part_rows) * tiles * sizeof(unsigned);
      if (part_rows > INT32_MAX || part_bytes > hyb_scratch_limit()) {
        // a bucket list whose widest bucket holds most of the matrix: adding atomically into a
        // cleared C costs less memory than a scratch copy of that size
        if (to_peers)
          return fail("sparsetir_hyb_spmm_peers: the split rows need %zu bytes of scratch, beyond the limit; "
                      "run sparsetir_hyb_spmm and sparsetir_peer_scatter instead", part_bytes);
        for (int q = 0; q < tb.nb; ++q) tb.part_base[q] = -1;
        la.all_atomic = 1;
        clear = true;
      } else if (part_rows > 0) {
        la.part = static_cast<float*>(workspace(device_id, st, part_bytes));
        la.counters = static_cast<unsigned*>(zeroed_workspace(device_id, st, counter_bytes));
        if (la.part == nullptr || la.counters == nullptr) return -1;
      }
    }
    if (clear) SPTIR_CUDA_OK(cudaMemsetAsync(c, 0, c_bytes, st));
    return dispatch_lean(tb, la, lanes, lane_w, st);
  }

  // ---- fallback kernels for odd widths, feature counts or alignments
  plan_items(tb, item_slots(lanes));
  if (flags & SPARSETIR_HYB_ZERO_C) {
    SPTIR_CUDA_OK(cudaMemsetAsync(c, 0, c_bytes, st));
  } else if (flags & SPARSETIR_HYB_REARM) {
    if (all_atomic) {
      SPTIR_CUDA_OK(cudaMemsetAsync(c, 0, c_bytes, st));
    } else {
      long long blocks = 0;
      for (int q = 0; q < tb.nb; ++q) {
        tb.block_start[q] = static_cast<int32_t>(blocks);
        blocks += ceil_div(tb.nrows[q], kThreads);
      }
      tb.block_start[tb.nb] = static_cast<int32_t>(blocks);
      if (blocks > INT32_MAX) return fail("sparsetir_hyb_spmm: too many thread blocks");
      hyb_rearm_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, st>>>(tb, c, feat);
      SPTIR_LAUNCH_OK("hyb_rearm_kernel");
    }
  }

  if (vec4) {
    if (lanes == 8) return launch_async<8>(tb, b, c, feat, all_atomic, st);
    if (lanes == 16) return launch_async<16>(tb, b, c, feat, all_atomic, st);
    return launch_async<32>(tb, b, c, feat, all_atomic, st);
  }
  if (feat <= 8) return launch<8, 1, 1>(tb, b, c, feat, all_atomic, st);
  if (feat <= 16) return launch<16, 1, 1>(tb, b, c, feat, all_atomic, st);
  if (feat <= 32) return launch<32, 1, 1>(tb, b, c, feat, all_atomic, st);
  return launch<32, 4, 1>(tb, b, c, feat, all_atomic, st);
}

int hyb_spmm_impl(const float* b, float* c, const SparsetirEllBucket* buckets, const int32_t* row_bases,
                  int num_buckets, int m, int n, int feat, int flags, int device_id, void* stream) {
  return hyb_spmm_run(b, c, buckets, row_bases, num_buckets, m, n, feat, flags, device_id, stream, nullptr);
}
}  // namespace sptir

extern "C" int sparsetir_hyb_spmm_tile(int n, int feat, int* lanes, int* lane_floats) {
  if (!lanes || !lane_floats || feat <= 0 || feat % 4 != 0)
    return sptir::fail("sparsetir_hyb_spmm_tile: feat_size must be a positive multiple of 4");
  int lane_w = feat % 32 == 0 ? sptir::max_lane_floats() : 4;
  int l = sptir::lanes_per_row(feat, true, n, lane_w);
  if (lane_w == 8 && feat % (lane_w * l) != 0) {
    lane_w = 4;
    l = sptir::lanes_per_row(feat, true, n, lane_w);
  }
  *lanes = l;
  *lane_floats = lane_w;
  return 0;
}

extern "C" int sparsetir_hyb_spmm_workspace(const SparsetirEllBucket* buckets, int num_buckets,
                                            int feat, size_t* scratch_bytes,
                                            size_t* counter_bytes) {
  if (num_buckets < 0 || (num_buckets > 0 && !buckets) || feat < 0 || !scratch_bytes || !counter_bytes)
    return sptir::fail("sparsetir_hyb_spmm_workspace: bad argument");
  int maxw = 0;
  for (int q = 0; q < num_buckets; ++q)
    if (buckets[q].nrows > 0 && buckets[q].rows != nullptr) maxw = std::max(maxw, buckets[q].width);
  size_t rows = 0;
  for (int q = 0; q < num_buckets; ++q)
    if (buckets[q].nrows > 0 && buckets[q].rows != nullptr && buckets[q].width == maxw)
      rows += static_cast<size_t>(buckets[q].nrows);
  const size_t part = rows * static_cast<size_t>(feat) * sizeof(float);
  const bool fits = part <= sptir::hyb_scratch_limit_bytes();
  *scratch_bytes = fits ? part : 0;
  // a feature tile is at least 32 floats wide
  *counter_bytes = fits ? rows * static_cast<size_t>((feat + 31) / 32) * sizeof(unsigned) : 0;
  return 0;
}

extern "C" int sparsetir_hyb_spmm_peers_raw(const float* b, float* c, const SparsetirEllBucket* buckets,
                                            int num_buckets, int m, int n, int feat, int flags,
                                            int n_peers, void* const* peer_c, int device_id, void* stream) {
  sptir::PeerOut po{};
  if (sptir::peer_table("sparsetir_hyb_spmm_peers", c, n_peers, peer_c, 32, &po) != 0) return -1;
  return sptir::hyb_spmm_run(b, c, buckets, nullptr, num_buckets, m, n, feat, flags, device_id, stream, &po);
}

extern "C" int sparsetir_hyb_spmm_raw(const float* b, float* c, const SparsetirEllBucket* buckets,
                                      int num_buckets, int m, int n, int feat, int flags,
                                      int device_id, void* stream) {
  return sptir::hyb_spmm_impl(b, c, buckets, nullptr, num_buckets, m, n, feat, flags, device_id, stream);
}
