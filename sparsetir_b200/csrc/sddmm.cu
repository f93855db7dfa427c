// SDDMM, fp32:  C[p] = sum_k A[row(p),k] * B[indices[p],k]   (optionally times scale[p])
// Semantics: tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:458-507 (sddmm) and
// :510-569 (fused_sddmm with the edge->row binary search) of the reference; generated kernel
// being replaced: examples/sddmm/bench_sddmm.py:97-167.
//
// Mapping.  The reference runs a separate preprocess kernel that stores row(p) for every
// stored position and then gives every (ty, group) slot one edge with the dot product split
// over tx lanes and reduced across threads.  Here one kernel does both:
//  - a warp owns a contiguous range of stored positions and walks it 32 positions at a time;
//    lane l reads indices[base+l] (coalesced) and finds row(base+l) by advancing from the
//    warp's current row through indptr (the positions are sorted by row, so this is a short
//    walk, with a binary search as the fallback for long runs of empty rows);
//  - the 32 positions are split over the warp's sub-warps of LPR lanes, LPR positions each;
//    a sub-warp loads the B row of one position at a time (every lane VPL 16-byte pieces,
//    several positions in flight), keeps the A row in registers while the row id stays the
//    same, and accumulates one partial sum per position in its own registers;
//  - the LPR partial sums held by each of the LPR lanes are then reduced with a transposing
//    butterfly: LPR-1 shuffles leave lane l with the finished dot product of position l,
//    instead of log2(LPR) shuffles per position; the warp stores 32 consecutive results with
//    one coalesced store.
#include <cstdint>
#include <cstdlib>

#include <algorithm>

#include "common.h"
#include "vec.cuh"

namespace sptir {
namespace {

constexpr int kThreads = 256;
constexpr int kEdgesPerWarp = 256;

// row(p) = upper_bound(indptr[0..m], p) - 1, the search of
// tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:530-549
__device__ __forceinline__ int edge_row_search(const int32_t* __restrict__ indptr, int lo_row,
                                               int m, int p) {
  int low = lo_row, high = m + 1;
  while (low < high) {
    int mid = low + (high - low) / 2;
    if (__ldg(indptr + mid) > p) high = mid; else low = mid + 1;
  }
  return low - 1;
}

template <int LPR, int VPL, int VEC>
__global__ void __launch_bounds__(kThreads)
sddmm_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
             const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices,
             const float* __restrict__ scale, int m, int feat, int nnz) {
  using V = typename Vec<VEC>::type;
  constexpr int U = (8 / VPL) < LPR ? (8 / VPL) : LPR;  // positions whose B rows are in flight
  const int wlane = threadIdx.x & 31;
  const int lane = wlane % LPR;
  const int sub = wlane / LPR;
  const unsigned mask = group_mask<LPR>();
  const long long warp = static_cast<long long>(blockIdx.x) * (kThreads / 32) + threadIdx.x / 32;
  const long long e_begin = warp * kEdgesPerWarp;
  if (e_begin >= nnz) return;
  const int e_end = static_cast<int>(min(static_cast<long long>(nnz), e_begin + kEdgesPerWarp));
  const int row_vecs = feat / VEC;
  const V* av = reinterpret_cast<const V*>(a);
  const V* bv = reinterpret_cast<const V*>(b);

  int off[VPL];
  bool valid[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    off[v] = v * LPR + lane;
    valid[v] = off[v] < row_vecs;
  }

  int warp_row = max(0, min(m - 1, edge_row_search(indptr, 0, m, static_cast<int>(e_begin))));
  int cur_row = -1;
  V arow[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) arow[v] = Vec<VEC>::zero();

  int warp_end = __ldg(indptr + warp_row + 1);  // first position past the warp's current row
  for (int base = static_cast<int>(e_begin); base < e_end; base += 32) {
    if (base + 32 <= min(warp_end, e_end)) {
      // Fast path: all 32 positions belong to the warp's current row (the common case when rows
      // are longer than a batch) — no row lookup, no per-position row bookkeeping.
      const int col = __ldg(indices + base + wlane);
      if (cur_row != warp_row) {
        cur_row = warp_row;
        const V* src = av + static_cast<size_t>(cur_row) * row_vecs;
#pragma unroll
        for (int v = 0; v < VPL; ++v) arow[v] = valid[v] ? __ldg(src + off[v]) : Vec<VEC>::zero();
      }
      float part[LPR];
#pragma unroll
      for (int k0 = 0; k0 < LPR; k0 += U) {
        V x[U][VPL];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const V* src = bv + static_cast<size_t>(__shfl_sync(mask, col, k0 + u, LPR)) * row_vecs;
#pragma unroll
          for (int v = 0; v < VPL; ++v) x[u][v] = valid[v] ? __ldg(src + off[v]) : Vec<VEC>::zero();
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float s = 0.f;
#pragma unroll
          for (int v = 0; v < VPL; ++v) s = Vec<VEC>::dot(arow[v], x[u][v], s);
          part[k0 + u] = s;
        }
      }
#pragma unroll
      for (int offl = LPR / 2, n = LPR; offl >= 1; offl >>= 1, n >>= 1) {
        const bool upper = (lane & offl) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
          float send = upper ? part[i] : part[i + n / 2];
          float keep = upper ? part[i + n / 2] : part[i];
          part[i] = keep + __shfl_xor_sync(mask, send, offl, LPR);
        }
      }
      float r = part[0];
      if (scale != nullptr) r *= __ldg(scale + base + wlane);
      c[base + wlane] = r;
      continue;
    }
    const int e = base + wlane;
    const bool live = e < e_end;
    int col = 0, row = warp_row;
    if (live) {
      col = __ldg(indices + e);
      int steps = 0;
      // row < m - 1 keeps every read inside indptr even if nnz disagrees with indptr[m]
      while (row < m - 1 && __ldg(indptr + row + 1) <= e) {
        ++row;
        if (++steps == 8) {  // long run of empty rows: finish with a search
          row = min(m - 1, edge_row_search(indptr, row, m, e));
          break;
        }
      }
    }
    // the next batch starts from the row of this batch's last live position
    warp_row = __shfl_sync(0xffffffffu, row, min(31, e_end - 1 - base));
    warp_end = __ldg(indptr + warp_row + 1);

    const int cnt = min(LPR, e_end - (base + sub * LPR));  // live positions of this sub-warp (may be <= 0)
    float part[LPR];
#pragma unroll
    for (int k = 0; k < LPR; ++k) part[k] = 0.f;
#pragma unroll
    for (int k0 = 0; k0 < LPR; k0 += U) {
      if (k0 < cnt) {  // uniform inside the sub-warp
        V x[U][VPL];
        int rk[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          int ck = __shfl_sync(mask, col, k0 + u, LPR);  // dead positions carry column 0
          rk[u] = __shfl_sync(mask, row, k0 + u, LPR);
          const V* src = bv + static_cast<size_t>(ck) * row_vecs;
#pragma unroll
          for (int v = 0; v < VPL; ++v) x[u][v] = valid[v] ? __ldg(src + off[v]) : Vec<VEC>::zero();
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (rk[u] != cur_row) {  // uniform inside the sub-warp
            cur_row = rk[u];
            const V* src = av + static_cast<size_t>(cur_row) * row_vecs;
#pragma unroll
            for (int v = 0; v < VPL; ++v) arow[v] = valid[v] ? __ldg(src + off[v]) : Vec<VEC>::zero();
          }
          float s = 0.f;
#pragma unroll
          for (int v = 0; v < VPL; ++v) s = Vec<VEC>::dot(arow[v], x[u][v], s);
          part[k0 + u] = s;
        }
      }
    }
    // transposing butterfly: afterwards part[0] of lane l is the dot product of position l
#pragma unroll
    for (int offl = LPR / 2, n = LPR; offl >= 1; offl >>= 1, n >>= 1) {
      const bool upper = (lane & offl) != 0;
#pragma unroll
      for (int i = 0; i < n / 2; ++i) {
        float send = upper ? part[i] : part[i + n / 2];
        float keep = upper ? part[i + n / 2] : part[i];
        part[i] = keep + __shfl_xor_sync(mask, send, offl, LPR);
      }
    }
    if (live) {
      float r = part[0];
      if (scale != nullptr) r *= __ldg(scale + e);
      c[e] = r;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Lean variant for feature counts that are multiples of 32 with 32-byte aligned operands.
//
// One launch covers a tile of 8*LPR consecutive features [foff, foff + 8*LPR) of every stored
// position; the host walks the tiles with one launch each, the first storing C and the others
// adding to it, and picks the tile so that the slice of B a launch gathers from stays in L2.
// A lane owns 8 consecutive features: one 256-bit load per gathered row, the dot product as
// packed two-wide fp32 FMAs.  A warp owns `chunk` consecutive positions, finds the row of its
// first position with a 32-ary search done by the whole warp (4 dependent reads instead of 18
// at 2^18 rows), and loads the column ids of the next batch before it gathers for this one.
// first index idx in [0, m+1] with idx == m+1 or indptr[idx] > p, found by the whole warp;
// row(p) is that index minus one (the search of sparse_tir_lowered_buffer_scripts.py:530-549)
__device__ __forceinline__ int warp_row_search(const int32_t* __restrict__ indptr, int m, int p,
                                               int wlane) {
  int lo = 0, hi = m + 1;
  while (hi - lo >= 32) {
    const int step = (hi - lo + 31) / 32;
    const long long probe = static_cast<long long>(lo) + static_cast<long long>(wlane + 1) * step;
    const bool gt = probe >= hi || __ldg(indptr + probe) > p;
    const int first = __ffs(__ballot_sync(0xffffffffu, gt)) - 1;  // lane 31 probes >= hi: always set
    const int q = lo + (first + 1) * step;
    if (first > 0) lo = q - step + 1;
    hi = min(hi, q);
  }
  const int idx = lo + wlane;
  const bool gt = idx >= hi || __ldg(indptr + idx) > p;  // lane hi - lo (< 32) has idx == hi
  return lo + __ffs(__ballot_sync(0xffffffffu, gt)) - 1;
}

// With PEERS the finished value of every position (the last feature tile's pass) is also stored
// into the peers' copies of c: 128 contiguous bytes per warp and peer, over NVLink.
template <int LPR, bool PEERS>
__global__ void __launch_bounds__(kThreads, LPR <= 8 ? 4 : 2)
sddmm_lean_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                  const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                  const float* __restrict__ scale, int m, int nnz, int ld, int foff, int accumulate,
                  int chunk, int last_tile, const __grid_constant__ PeerOut po) {
  constexpr int U = LPR < 4 ? LPR : 4;  // gathered rows in flight per lane (8 registers each)
  const int wlane = threadIdx.x & 31;
  const int lane = wlane % LPR;
  const unsigned mask = group_mask<LPR>();
  const long long warp = static_cast<long long>(blockIdx.x) * (kThreads / 32) + threadIdx.x / 32;
  const long long e_begin = warp * chunk;
  if (e_begin >= nnz) return;
  const int e_end = static_cast<int>(min(static_cast<long long>(nnz), e_begin + chunk));
  const float* a_lane = a + foff + lane * 8;
  const float* b_lane = b + foff + lane * 8;

  int warp_row = max(0, min(m - 1, warp_row_search(indptr, m, static_cast<int>(e_begin), wlane) - 1));
  int warp_end = __ldg(indptr + warp_row + 1);  // first position past the warp's current row
  int cur_row = -1;
  Pack4 arow = pack4_zero();

  int col_next = (static_cast<int>(e_begin) + wlane < e_end) ? __ldg(indices + e_begin + wlane) : 0;
  for (int base = static_cast<int>(e_begin); base < e_end; base += 32) {
    const int e = base + wlane;
    const bool live = e < e_end;
    const int col = col_next;
    if (e + 32 < e_end) col_next = __ldg(indices + e + 32);
    float mul = 1.f, old = 0.f;
    if (live) {
      if (scale != nullptr) mul = __ldg(scale + e);
      if (accumulate) old = c[e];
    }
    float part[LPR];
    if (base + 32 <= min(warp_end, e_end)) {
      // every position of the batch lies in the warp's current row
      if (cur_row != warp_row) {
        cur_row = warp_row;
        arow = ldg256(a_lane + static_cast<size_t>(cur_row) * ld);
      }
#pragma unroll
      for (int k0 = 0; k0 < LPR; k0 += U) {
        Pack4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          x[u] = ldg256(b_lane + static_cast<size_t>(__shfl_sync(mask, col, k0 + u, LPR)) * ld);
#pragma unroll
        for (int u = 0; u < U; ++u) part[k0 + u] = dot8(arow, x[u]);
      }
    } else {
      int row = warp_row;
      if (live) {
        int steps = 0;
        // row < m - 1 keeps every read inside indptr even if nnz disagrees with indptr[m]
        while (row < m - 1 && __ldg(indptr + row + 1) <= e) {
          ++row;
          if (++steps == 8) {  // long run of empty rows: finish with a search
            row = min(m - 1, edge_row_search(indptr, row, m, e));
            break;
          }
        }
      }
      // the next batch starts from the row of this batch's last live position
      warp_row = __shfl_sync(0xffffffffu, row, min(31, e_end - 1 - base));
      warp_end = __ldg(indptr + warp_row + 1);
#pragma unroll
      for (int k0 = 0; k0 < LPR; k0 += U) {
        Pack4 x[U];
        int rk[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {  // dead positions carry column 0 and the warp's row
          rk[u] = __shfl_sync(mask, row, k0 + u, LPR);
          x[u] = ldg256(b_lane + static_cast<size_t>(__shfl_sync(mask, col, k0 + u, LPR)) * ld);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (rk[u] != cur_row) {  // uniform inside the sub-warp
            cur_row = rk[u];
            arow = ldg256(a_lane + static_cast<size_t>(cur_row) * ld);
          }
          part[k0 + u] = dot8(arow, x[u]);
        }
      }
    }
    // transposing butterfly: afterwards part[0] of lane l is the dot product of position l
#pragma unroll
    for (int offl = LPR / 2, n = LPR; offl >= 1; offl >>= 1, n >>= 1) {
      const bool upper = (lane & offl) != 0;
#pragma unroll
      for (int i = 0; i < n / 2; ++i) {
        const float send = upper ? part[i] : part[i + n / 2];
        const float keep = upper ? part[i + n / 2] : part[i];
        part[i] = keep + __shfl_xor_sync(mask, send, offl, LPR);
      }
    }
    if (live) {
      const float v = fmaf(part[0], mul, old);
      c[e] = v;
      if constexpr (PEERS) {
        if (last_tile)
          for (int k = 0; k < po.n; ++k)
            *reinterpret_cast<float*>(reinterpret_cast<char*>(c + e) + po.delta[k]) = v;
      }
    }
  }
}

// Fallback for feature sizes beyond the register-resident variants: a full warp per position,
// looping over the feature dimension.
__global__ void __launch_bounds__(kThreads)
sddmm_generic_kernel(const float* __restrict__ a, const float* __restrict__ b,
                     float* __restrict__ c, const int32_t* __restrict__ indptr,
                     const int32_t* __restrict__ indices, const float* __restrict__ scale, int m,
                     int feat, int nnz) {
  const int lane = threadIdx.x & 31;
  const long long warp = static_cast<long long>(blockIdx.x) * (kThreads / 32) + threadIdx.x / 32;
  const long long e_begin = warp * 32;
  if (e_begin >= nnz) return;
  const int e_end = static_cast<int>(min(static_cast<long long>(nnz), e_begin + 32));
  int row = max(0, min(m - 1, edge_row_search(indptr, 0, m, static_cast<int>(e_begin))));
  for (int e = static_cast<int>(e_begin); e < e_end; ++e) {
    while (row < m - 1 && __ldg(indptr + row + 1) <= e) ++row;
    const float* ar = a + static_cast<size_t>(row) * feat;
    const float* br = b + static_cast<size_t>(__ldg(indices + e)) * feat;
    float s = 0.f;
    for (int k = lane; k < feat; k += 32) s = fmaf(__ldg(ar + k), __ldg(br + k), s);
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) c[e] = scale ? s * __ldg(scale + e) : s;
  }
}

__global__ void __launch_bounds__(kThreads)
edge_to_row_kernel(const int32_t* __restrict__ indptr, int32_t* __restrict__ mid, int m, int nnz) {
  const long long p = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  if (p < nnz) mid[p] = edge_row_search(indptr, 0, m, static_cast<int>(p));
}

template <int LPR, int VPL, int VEC>
int launch(const float* a, const float* b, float* c, const int32_t* indptr, const int32_t* indices,
           const float* scale, int m, int feat, int nnz, cudaStream_t stream) {
  const int warps = ceil_div(nnz, kEdgesPerWarp);
  const int blocks = ceil_div(warps, kThreads / 32);
  sddmm_kernel<LPR, VPL, VEC><<<blocks, kThreads, 0, stream>>>(a, b, c, indptr, indices, scale, m,
                                                              feat, nnz);
  SPTIR_LAUNCH_OK("sddmm_kernel");
  return 0;
}

// Blocks of sddmm_lean_kernel<LPR> that fit one SM at a time (asked of the runtime once per device).
template <int LPR>
int lean_blocks_per_sm() {
  static thread_local int cached_device = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 4;
  if (dev != cached_device) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, sddmm_lean_kernel<LPR, false>, kThreads, 0) != cudaSuccess || n < 1)
      n = 4;
    cached = n;
    cached_device = dev;
  }
  return cached;
}

template <int LPR>
int launch_lean_tile(const float* a, const float* b, float* c, const int32_t* indptr,
                     const int32_t* indices, const float* scale, int m, int feat, int nnz, int foff,
                     int last_tile, const PeerOut& po, cudaStream_t stream) {
  // long chunks amortise the row search; short ones keep small inputs spread over the SMs
  int chunk = nnz >= (1 << 22) ? 1024 : 256;
  const int wpb = kThreads / 32;
  int blocks = ceil_div(ceil_div(nnz, chunk), wpb);
  // A launch of only a few waves of blocks ends with a partly filled wave (3.02 waves cost as
  // much as 4): then the chunk is resized so that the blocks fill a whole number of waves.
  const long long resident = static_cast<long long>(kNumSMs) * lean_blocks_per_sm<LPR>();
  if (nnz >= (1 << 22) && blocks > resident / 2 && blocks < 8 * resident) {
    const long long waves = std::max<long long>(1, (blocks + resident / 2) / resident);
    const long long want_warps = waves * resident * wpb;
    chunk = static_cast<int>((nnz + want_warps - 1) / want_warps);
    chunk = (chunk + 31) & ~31;
    blocks = ceil_div(ceil_div(nnz, chunk), wpb);
  }
  if (po.n > 0)
    sddmm_lean_kernel<LPR, true><<<blocks, kThreads, 0, stream>>>(a, b, c, indptr, indices, scale, m, nnz, feat,
                                                                  foff, foff != 0, chunk, last_tile, po);
  else
    sddmm_lean_kernel<LPR, false><<<blocks, kThreads, 0, stream>>>(a, b, c, indptr, indices, scale, m, nnz, feat,
                                                                   foff, foff != 0, chunk, last_tile, po);
  SPTIR_LAUNCH_OK("sddmm_lean_kernel");
  return 0;
}

// What stays resident in L2 of data that every SM reads (about half of the 126 MB);
// SPARSETIR_L2_BUDGET_MB overrides it for tuning on other parts.
size_t l2_budget_bytes() {
  static const size_t budget = [] {
    const char* e = std::getenv("SPARSETIR_L2_BUDGET_MB");
    const long mb = e ? std::atol(e) : 0;
    return static_cast<size_t>(mb > 0 ? mb : 48) << 20;
  }();
  return budget;
}

// feat is a multiple of 32: the widest tile (32..256 features) that divides feat and whose
// slice of B (n rows) fits the L2 budget; one launch per tile, in stream order.
int launch_lean(const float* a, const float* b, float* c, const int32_t* indptr,
                const int32_t* indices, const float* scale, int m, int n, int feat, int nnz,
                const PeerOut& po, cudaStream_t stream) {
  int tile = 32;
  for (int t = 256; t > 32; t /= 2)
    if (feat % t == 0 && static_cast<size_t>(n) * t * 4 <= l2_budget_bytes()) {
      tile = t;
      break;
    }
  for (int foff = 0; foff < feat; foff += tile) {
    int rc;
    const int last = foff + tile >= feat;
    switch (tile) {
      case 256: rc = launch_lean_tile<32>(a, b, c, indptr, indices, scale, m, feat, nnz, foff, last, po, stream); break;
      case 128: rc = launch_lean_tile<16>(a, b, c, indptr, indices, scale, m, feat, nnz, foff, last, po, stream); break;
      case 64: rc = launch_lean_tile<8>(a, b, c, indptr, indices, scale, m, feat, nnz, foff, last, po, stream); break;
      default: rc = launch_lean_tile<4>(a, b, c, indptr, indices, scale, m, feat, nnz, foff, last, po, stream); break;
    }
    if (rc != 0) return rc;
  }
  return 0;
}

}  // namespace
}  // namespace sptir

namespace sptir {
namespace {
int sddmm_run(const float* a, const float* b, float* c, const int32_t* indptr, const int32_t* indices,
              const float* scale, int m, int n, int feat, int nnz, int device_id, void* stream,
              const PeerOut& po) {
  if (m < 0 || n < 0 || feat < 0 || nnz < 0) return fail("sparsetir_sddmm: negative size");
  if (nnz == 0) return 0;
  if (m < 1) return fail("sparsetir_sddmm: %d stored entries but no rows", nnz);
  if (!c || !indptr || !indices || (feat > 0 && (!a || !b)))
    return fail("sparsetir_sddmm: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (validate_enabled() && validate_csr("sparsetir_sddmm", indptr, m, indices, nnz, n, st) != 0) return -1;
  const bool lean = feat > 0 && feat % 32 == 0 && aligned32(a) && aligned32(b);
  if (po.n > 0 && !lean)
    return fail("sparsetir_sddmm_peers: needs feat_size a positive multiple of 32 and 32-byte aligned a and b; "
                "run sparsetir_sddmm and sparsetir_peer_scatter instead");
  if (feat == 0) {
    SPTIR_CUDA_OK(cudaMemsetAsync(c, 0, static_cast<size_t>(nnz) * sizeof(float), st));
    return 0;
  }
  if (lean) return launch_lean(a, b, c, indptr, indices, scale, m, n, feat, nnz, po, st);
  const bool vec4 = (feat % 4 == 0) && aligned16(a) && aligned16(b);
  if (vec4) {
    const int nv = feat / 4;
    if (nv <= 8) return launch<8, 1, 4>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
    if (nv <= 16) return launch<16, 1, 4>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
    if (nv <= 32) return launch<32, 1, 4>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
    if (nv <= 64) return launch<32, 2, 4>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
    if (nv <= 128) return launch<32, 4, 4>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
  } else {
    if (feat <= 8) return launch<8, 1, 1>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
    if (feat <= 16) return launch<16, 1, 1>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
    if (feat <= 32) return launch<32, 1, 1>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
    if (feat <= 64) return launch<32, 2, 1>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
    if (feat <= 128) return launch<32, 4, 1>(a, b, c, indptr, indices, scale, m, feat, nnz, st);
  }
  const int blocks = ceil_div(ceil_div(nnz, 32), kThreads / 32);
  sddmm_generic_kernel<<<blocks, kThreads, 0, st>>>(a, b, c, indptr, indices, scale, m, feat, nnz);
  SPTIR_LAUNCH_OK("sddmm_generic_kernel");
  return 0;
}
}  // namespace
}  // namespace sptir

extern "C" int sparsetir_sddmm_raw(const float* a, const float* b, float* c, const int32_t* indptr,
                                   const int32_t* indices, const float* scale, int m, int n,
                                   int feat, int nnz, int device_id, void* stream) {
  return sptir::sddmm_run(a, b, c, indptr, indices, scale, m, n, feat, nnz, device_id, stream, sptir::PeerOut{});
}

extern "C" int sparsetir_sddmm_peers_raw(const float* a, const float* b, float* c, const int32_t* indptr,
                                         const int32_t* indices, const float* scale, int m, int n,
                                         int feat, int nnz, int n_peers, void* const* peer_c,
                                         int device_id, void* stream) {
  sptir::PeerOut po{};
  if (sptir::peer_table("sparsetir_sddmm_peers", c, n_peers, peer_c, 4, &po) != 0) return -1;
  return sptir::sddmm_run(a, b, c, indptr, indices, scale, m, n, feat, nnz, device_id, stream, po);
}

extern "C" int sparsetir_sddmm_edge_to_row_raw(const int32_t* indptr, int32_t* mid, int m, int nnz,
                                               int device_id, void* stream) {
  using namespace sptir;
  if (m < 0 || nnz < 0) return fail("sparsetir_sddmm_edge_to_row: negative size");
  if (nnz == 0) return 0;
  if (!indptr || !mid) return fail("sparsetir_sddmm_edge_to_row: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  edge_to_row_kernel<<<ceil_div(nnz, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      indptr, mid, m, nnz);
  SPTIR_LAUNCH_OK("edge_to_row_kernel");
  return 0;
}
