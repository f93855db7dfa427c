// One-launch tensor-core RGMS for feat_size 64, fp32 in and out, CSF operand:
//   Y[I[i], fo] += sum_{p in CSF row i of relation r} A[p] * sum_fi W[r,fo,fi] * X[J[p],fi]
// Semantics and formulation (aggregate first, transform once per (relation, row)) as rgms.cu.
//
// The two-launch form (rgms.cu + rgms_tc.cu) writes the aggregated rows Z (nnz_i x 64 floats)
// to a scratch buffer with one launch and reads them back with the next: 2 x 177 MB of HBM
// traffic at 690 k rows, and two launches of about the same length one after the other.  Here
// the aggregated rows never leave the SM: sixteen gather warps build each 128-row tile straight
// in the swizzled shared-memory layout the tensor core reads, while the tensor core multiplies
// the previous tile and the epilogue warps scatter the one before.
//
// One persistent block per SM walks consecutive tiles (tiles are numbered relation by relation,
// 128 CSF rows each).  800 threads in three roles that hand tiles to each other through mbarriers:
//   warps 9-24   gather: thread = (row slot, 16-byte piece of the feature row); a thread owns the
//                same piece of four rows of the tile.  Row pointers, column ids and values of a tile
//                are contiguous in memory; they are fetched ONE TILE AHEAD into registers with
//                coalesced loads and parked in shared memory, so that the X rows of a tile are
//                requested without any dependent load in front of them, eight per thread at a time.
//                The finished row piece is stored twice: as it is (the tensor core reads the upper
//                19 bits of an fp32 operand: the "high" part) and its remainder z - tf32(z).
//                The same warps stage W_r (raw and remainder) when the relation changes.
//   warp 0       issues the 3xTF32 product of a tile as 16 instructions (W and its remainders
//                stacked into one 128-row operand) into one of two TMEM accumulators;
//                tcgen05.commit frees the stage and publishes the accumulator.
//   warps 1-4, 5-8  epilogue (even / odd tiles): TMEM -> registers -> padded shared-memory row ->
//                read back 8 lanes per row -> 16-byte vector atomics into Y[I[t], :].
// Every mbarrier wait is bounded (tc05.cuh); a wait that runs out is counted and the block leaves.
#include <cstdlib>
#include <cstring>

#include "common.h"
#include "rgms_common.cuh"
#include "tc05.cuh"

namespace sptir {

__device__ unsigned int g_rgms_fused_timeouts = 0;

// Self-checking build (-DSPTIR_RGMS_CHECK): every index the gather and epilogue roles are about to
// use is compared with its limit first; the first violation is recorded (code, value, limit, block,
// thread) and the access is redirected to element 0, so nothing out of bounds is ever touched.
#ifdef SPTIR_RGMS_CHECK
__device__ long long g_rgms_check[6] = {0, 0, 0, 0, 0, 0};
__device__ __forceinline__ long long rgms_checked(int code, long long v, long long limit) {
  if (v < 0 || v >= limit) {
    if (atomicCAS(reinterpret_cast<unsigned long long*>(&g_rgms_check[0]), 0ull,
                  static_cast<unsigned long long>(code)) == 0ull) {
      g_rgms_check[1] = v;
      g_rgms_check[2] = limit;
      g_rgms_check[3] = blockIdx.x;
      g_rgms_check[4] = threadIdx.x;
    }
    return 0;
  }
  return v;
}
#define RGMS_CHK(code, v, limit) rgms_checked(code, v, limit)
#else
#define RGMS_CHK(code, v, limit) (v)
#endif

// Probe build (-DSPTIR_RGMS_PROF): clock cycles the first gather thread of every block spends in
// each step of a tile, summed over all blocks.
#ifdef SPTIR_RGMS_PROF
__device__ unsigned long long g_rgms_prof[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define RGMS_T(var) const long long var = clock64()
#define RGMS_ADD(slot, t0, t1) do { if (gt == 0) atomicAdd(&g_rgms_prof[slot], static_cast<unsigned long long>((t1) - (t0))); } while (0)
#else
#define RGMS_T(var)
#define RGMS_ADD(slot, t0, t1)
#endif

namespace {

constexpr int kF = 64;
constexpr int kTM = 128;
constexpr int kFThreads = 800;
constexpr int kGatherWarp0 = 9;
constexpr int kGatherWarps = 16;
constexpr int kGatherThreads = kGatherWarps * 32;  // 512
constexpr int kRowsPerThread = kTM * 16 / kGatherThreads;  // 4
constexpr int kEdgeCap = 1024;                     // stored entries of a tile held in shared memory at a time

constexpr int kStages = 2;
constexpr int kZBox = kTM * 128;     // one swizzled box: 128 rows x 32 floats
constexpr int kZTile = 2 * kZBox;    // 32 KB
constexpr int kWBox = 2 * kF * 128;  // W_r and its remainders, 128 rows x 32 floats: 16 KB
constexpr int kWAll = 2 * kWBox;     // 32 KB
constexpr int kOutStride = 128 + 16;  // padded half row of the epilogue's transposition buffer
constexpr int kPtrStride = kTM + 8;   // 129 row pointers + up to 3 in front of them, in 16-byte pieces
constexpr int kEdgeBuf = kEdgeCap + 8;  // staged entries + up to 3 in front of them
constexpr int kOffZRaw = 0;
constexpr int kOffZLo = kOffZRaw + kStages * kZTile;
constexpr int kOffW = kOffZLo + kStages * kZTile;
constexpr int kOffOut = kOffW + kWAll;
constexpr int kOffIdx = kOffOut + 2 * kTM * kOutStride;
constexpr int kOffVal = kOffIdx + 2 * kEdgeBuf * 4;
constexpr int kOffPtr = kOffVal + 2 * kEdgeBuf * 4;
constexpr int kOffBnd = kOffPtr + 2 * kPtrStride * 4;
constexpr int kOffTab = kOffBnd + 64;
constexpr int kMaxRelsTab = 512;
constexpr int kFusedSmem = kOffTab + 2 * (kMaxRelsTab + 1) * 4 + 1024;  // + slack to align to 1024 bytes

__device__ __forceinline__ float tf32_hi(float x) {
  return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);  // what the tensor core keeps
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc05::smem_u32(bar)) : "memory");
}
// offset of 16-byte chunk `kc` (0..15) of row `row` in a tile stored as two 128-byte-swizzled boxes
__device__ __forceinline__ int swz_off(int row, int kc, int box_bytes) {
  return (kc >> 3) * box_bytes + (row >> 3) * 1024 + (row & 7) * 128 + (((kc & 7) ^ (row & 7)) << 4);
}
// barrier among the gather warps only
__device__ __forceinline__ void gather_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kGatherThreads) : "memory");
}
// one lane waits, the warp follows; false when the bounded wait ran out
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int lane) {
  bool ok = true;
  if (lane == 0) ok = tc05::mbar_wait(bar, parity);
  return __shfl_sync(0xffffffffu, ok, 0);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

constexpr int kMaxRels = kMaxRelsTab;  // relations whose tile table fits the block's shared memory

// Tiles are numbered relation by relation (relation r owns ceil(rows_r / 128) tiles); the block
// keeps the first tile id and the first CSF row of every relation in shared memory.
struct TileTable {
  const int32_t* tstart;  // [num_rels + 1] first tile id of relation r (shared memory)
  const int32_t* relptr;  // [num_rels + 1] indptr_i (shared memory)
  int num_rels;
  __device__ __forceinline__ void locate(int tile, int* rel, int* row0, int* row1) const {
    int lo = 0, hi = num_rels;  // last r with tstart[r] <= tile
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tstart[mid] <= tile) lo = mid; else hi = mid;
    }
    *rel = lo;
    *row0 = relptr[lo] + (tile - tstart[lo]) * kTM;
    *row1 = min(relptr[lo + 1], *row0 + kTM);
  }
};

__global__ void __launch_bounds__(kFThreads, 1)
rgms_fused_kernel(const float* __restrict__ a, const float* __restrict__ w,
                  const float* __restrict__ x, float* __restrict__ y,
                  const int32_t* __restrict__ indptr_i, const int32_t* __restrict__ indices_i,
                  const int32_t* __restrict__ indptr_j, const int32_t* __restrict__ indices_j,
                  int num_rels, int nnz_i, int nnz_j, int n_x, int m_y) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_conv[kStages];    // tile built in the stage (one arrival per gather warp)
  __shared__ __align__(8) uint64_t bar_empty[kStages];   // tensor core has read the stage
  __shared__ __align__(8) uint64_t bar_acc_full[2];      // accumulator holds a finished tile
  __shared__ __align__(8) uint64_t bar_acc_empty[2];     // epilogue has read it (128 arrivals)
  __shared__ uint32_t s_tmem;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned char* base = smem_raw + ((1024u - (tc05::smem_u32(smem_raw) & 1023u)) & 1023u);
  int32_t* s_tstart = reinterpret_cast<int32_t*>(base + kOffTab);
  int32_t* s_relptr = s_tstart + (kMaxRels + 1);

  if (warp == 0) {
    // tile table: prefix sums of the relations' tile counts, 32 relations per step
    int running = 0;
    for (int r0 = 0; r0 <= num_rels; r0 += 32) {
      const int r = r0 + lane;
      int s = 0, e = 0, nt = 0;
      if (r <= num_rels) s = __ldg(indptr_i + r);
      if (r < num_rels) {
        e = __ldg(indptr_i + r + 1);
        nt = (e - s + kTM - 1) / kTM;
      }
      int incl = nt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      if (r <= num_rels) {
        s_tstart[r] = running + incl - nt;
        s_relptr[r] = s;
      }
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      for (int s = 0; s < kStages; ++s) {
        tc05::mbar_init(&bar_conv[s], kGatherWarps);
        tc05::mbar_init(&bar_empty[s], 1);
      }
      for (int b = 0; b < 2; ++b) {
        tc05::mbar_init(&bar_acc_full[b], 1);
        tc05::mbar_init(&bar_acc_empty[b], 128);
      }
      tc05::fence_mbar_init();
    }
    __syncwarp();
    tc05::tmem_alloc(&s_tmem, 4 * kF);
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = s_tmem;
  const TileTable tab{s_tstart, s_relptr, num_rels};
  const int num_tiles = s_tstart[num_rels];
  // this block's tiles: blockIdx.x, + gridDim.x, ... — heavy and light relations are spread over
  // all blocks (a tile is 128 rows whatever the number of entries behind them)
  const int first = blockIdx.x, step = gridDim.x;
  const int my_tiles = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;
  bool ok = true;

  if (warp == 0) {
    // ---- MMA issuer
    if (lane == 0) {
      // Two instructions per K-step: z * [W; Wlo]^T (N = 128: columns 0..63 receive z*W, columns
      // 64..127 z*Wlo) and zlo * W^T (N = 64, added to columns 0..63); the epilogue adds the halves.
      constexpr uint32_t idesc128 = tc05::instr_desc(tc05::kFmtTF32, kTM, 2 * kF, /*a_mn=*/0, /*b_mn=*/0);
      constexpr uint32_t idesc64 = tc05::instr_desc(tc05::kFmtTF32, kTM, kF, /*a_mn=*/0, /*b_mn=*/0);
      const uint64_t dw0 = tc05::smem_desc_swizzled(tc05::smem_u32(base + kOffW), 0, 1024, tc05::kSwizzle128B);
      const uint64_t dzh0 = tc05::smem_desc_swizzled(tc05::smem_u32(base + kOffZRaw), 0, 1024, tc05::kSwizzle128B);
      const uint64_t dzl0 = tc05::smem_desc_swizzled(tc05::smem_u32(base + kOffZLo), 0, 1024, tc05::kSwizzle128B);
      for (int k = 0; k < my_tiles; ++k) {
        const int s = k % kStages, use = k / kStages, buf = k & 1, buse = k >> 1;
        if (!tc05::mbar_wait(&bar_conv[s], use & 1)) { ok = false; break; }
        if (buse > 0 && !tc05::mbar_wait(&bar_acc_empty[buf], (buse - 1) & 1)) { ok = false; break; }
        tc05::fence_after_sync();
        const uint64_t dzh_s = tc05::desc_advance(dzh0, s * kZTile);
        const uint64_t dzl_s = tc05::desc_advance(dzl0, s * kZTile);
        const uint32_t acc = tmem + buf * 2 * kF;
#pragma unroll
        for (int ks = 0; ks < kF / 8; ++ks) {  // K = 8 floats = 32 bytes inside the swizzled row
          const uint32_t zo = (ks >> 2) * kZBox + (ks & 3) * 32, wo = (ks >> 2) * kWBox + (ks & 3) * 32;
          const uint64_t dw = tc05::desc_advance(dw0, wo);
          tc05::mma_tf32(acc, tc05::desc_advance(dzh_s, zo), dw, idesc128, ks > 0 ? 1u : 0u);
          tc05::mma_tf32(acc, tc05::desc_advance(dzl_s, zo), dw, idesc64, 1u);
        }
        tc05::mma_commit(&bar_empty[s]);
        tc05::mma_commit(&bar_acc_full[buf]);
      }
    }
  } else if (warp >= kGatherWarp0) {
    // ---- gather: build the tile's aggregated rows in the stage
    const int gt = tid - kGatherWarp0 * 32;
    const int piece = gt & 15, slot = gt >> 4;
    const float4* xl = reinterpret_cast<const float4*>(x) + piece;  // this lane's piece of X row r: xl[r * 16]
    int32_t* s_ptr = reinterpret_cast<int32_t*>(base + kOffPtr);
    int32_t* s_idx = reinterpret_cast<int32_t*>(base + kOffIdx);
    float* s_val = reinterpret_cast<float*>(base + kOffVal);

    // Every global address below is clamped into its array, so it is valid for every thread
    // whatever the compiler does with the guard around the access.
    // A tile's row pointers and stored entries are brought into shared memory ONE TILE AHEAD with
    // asynchronous 4-byte copies (no register holds them while the current tile is gathered), its
    // entry bounds TWO tiles ahead (they are the addresses of those copies).
    int32_t* s_bnd = reinterpret_cast<int32_t*>(base + kOffBnd);  // [4][2]: entry bounds of tile k in slot k & 3
    auto tile_rows = [&](int tile_k, int* r0, int* r1) {
      int rel;
      tab.locate(min(first + tile_k * step, max(num_tiles - 1, 0)), &rel, r0, r1);
    };
    auto copy4 = [](void* dst, const void* src) {
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(tc05::smem_u32(dst)), "l"(src) : "memory");
    };
    // 16-byte copy of which only the first `bytes` (1..16) are read from memory, the rest zero-filled
    auto copy16 = [](void* dst, const void* src, int bytes) {
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(tc05::smem_u32(dst)), "l"(src), "r"(bytes)
                   : "memory");
    };
    auto request_bounds = [&](int tile_k) {  // one thread; lands in s_bnd[tile_k & 3]
      int r0, r1;
      tile_rows(tile_k, &r0, &r1);
      copy4(s_bnd + (tile_k & 3) * 2, indptr_j + RGMS_CHK(1, min(max(r0, 0), nnz_i), nnz_i + 1));
      copy4(s_bnd + (tile_k & 3) * 2 + 1, indptr_j + RGMS_CHK(2, min(max(r1, 0), nnz_i), nnz_i + 1));
    };
    // All gather threads; lands in buffer tile_k & 1.  The three arrays are copied in aligned
    // 16-byte pieces (4-byte asynchronous copies are issued one element at a time and took 3,000
    // clocks per tile): a range that starts at element e is copied from element e & ~3 on, and read
    // back at an offset of e & 3.
    auto request_tile = [&](int tile_k, int lo, int hi) {
      int r0, r1;
      tile_rows(tile_k, &r0, &r1);
      const int buf = tile_k & 1;
      const int pa = r0 & ~3;
      const int pidx = pa + 4 * gt;  // row pointers r0 .. r1
      if (pidx <= r1 && pidx <= nnz_i)
        copy16(s_ptr + buf * kPtrStride + 4 * gt, indptr_j + RGMS_CHK(4, max(pidx, 0), nnz_i + 1),
               min(16, (nnz_i + 1 - pidx) * 4));
      const int ea = lo & ~3;
      const int last = lo + min(hi - lo, kEdgeCap);  // one past the last entry staged
      const int eidx = ea + 4 * gt;
      if (eidx < last && eidx < nnz_j) {
        const int bytes = min(16, (nnz_j - eidx) * 4);
        copy16(s_idx + buf * kEdgeBuf + 4 * gt, indices_j + RGMS_CHK(5, max(eidx, 0), nnz_j), bytes);
        copy16(s_val + buf * kEdgeBuf + 4 * gt, a + RGMS_CHK(5, max(eidx, 0), nnz_j), bytes);
      }
    };
    // prologue: bounds of tiles 0 and 1 directly, data of tile 0 and bounds of tile 2 on their way
    int e_lo = 0, e_hi = 0, e_lo1 = 0, e_hi1 = 0;
    if (my_tiles > 0) {
      int r0, r1;
      tile_rows(0, &r0, &r1);
      e_lo = __ldg(indptr_j + min(max(r0, 0), nnz_i));
      e_hi = __ldg(indptr_j + min(max(r1, 0), nnz_i));
      if (my_tiles > 1) {
        tile_rows(1, &r0, &r1);
        e_lo1 = __ldg(indptr_j + min(max(r0, 0), nnz_i));
        e_hi1 = __ldg(indptr_j + min(max(r1, 0), nnz_i));
      }
      request_tile(0, e_lo, e_hi);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    int staged_rel = -1;
    for (int k = 0; k < my_tiles; ++k) {
      const int s = k % kStages, use = k / kStages, eb = k & 1;
      RGMS_T(t_a);
      // (1) this tile's pointers and entries (requested during the previous tile) have landed
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      gather_sync();
      RGMS_T(t_b);
      int rel, row0, row1;
      tab.locate(first + k * step, &rel, &row0, &row1);
      const int nrows = row1 - row0;
      if (k > 0) {  // bounds of tile k + 1 arrived with the copies just waited for
        e_lo = e_lo1;
        e_hi = e_hi1;
        e_lo1 = s_bnd[((k + 1) & 3) * 2];
        e_hi1 = s_bnd[((k + 1) & 3) * 2 + 1];
      }
      const int ne = e_hi - e_lo;
      const int32_t* sp = s_ptr + eb * kPtrStride + (row0 & 3);  // sp[t] = row pointer of tile row t
      int32_t* si = s_idx + eb * kEdgeBuf;
      float* sv = s_val + eb * kEdgeBuf;
      const int she = e_lo & 3;  // entry q of the tile sits at si[she + q] (first staging only)
      // (2) request the next tile's pointers and entries and the bounds of the tile after it
      if (k + 1 < my_tiles) request_tile(k + 1, e_lo1, e_hi1);
      if (gt == 0 && k + 2 < my_tiles) request_bounds(k + 2);
      asm volatile("cp.async.commit_group;" ::: "memory");
      RGMS_T(t_c);
      // (3) this thread's piece of four CONSECUTIVE rows of the tile.  Their entries are one
      // contiguous run of the tile's entries, walked eight at a time whatever row they belong to:
      // the number of rounds (each one memory latency long) follows the entries of the four rows
      // together, not the longest of them.
      float4 acc[kRowsPerThread];
      int bnd[kRowsPerThread + 1];  // entry range of row j of this thread: [bnd[j], bnd[j + 1])
#pragma unroll
      for (int j = 0; j <= kRowsPerThread; ++j) {
        const int t = min(kRowsPerThread * slot + j, nrows);
        bnd[j] = min(max(sp[t] - e_lo, 0), ne);  // inside the tile's range whatever the pointers say
        if (j > 0) bnd[j] = max(bnd[j], bnd[j - 1]);
      }
#pragma unroll
      for (int j = 0; j < kRowsPerThread; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c0 = 0; c0 == 0 || c0 < ne; c0 += kEdgeCap) {  // ne is the same for all gather threads
        int shift = she;
        if (c0 > 0) {  // a tile with more entries than the staging holds: the rest comes in directly
          gather_sync();
          for (int q = c0 + gt; q < min(ne, c0 + kEdgeCap); q += kGatherThreads) {
            const int e = min(max(e_lo + q, 0), nnz_j - 1);
            si[q - c0] = __ldg(indices_j + RGMS_CHK(10, e, nnz_j));
            sv[q - c0] = __ldg(a + RGMS_CHK(10, e, nnz_j));
          }
          gather_sync();
          shift = 0;
        }
        const int c1 = min(ne, c0 + kEdgeCap);
        const int f_end = min(bnd[kRowsPerThread], c1);
        for (int f0 = max(bnd[0], c0); f0 < f_end; f0 += 8) {
          float4 xv[8];
          float av[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const bool live = f0 + u < f_end;
            const int se = live ? shift + f0 + u - c0 : 0;
            const int col = live ? si[RGMS_CHK(11, se, kEdgeBuf)] : 0;  // dead slots read row 0 and add nothing
            av[u] = live ? sv[RGMS_CHK(11, se, kEdgeBuf)] : 0.f;
            xv[u] = __ldg(xl + static_cast<size_t>(RGMS_CHK(12, min(max(col, 0), n_x - 1), n_x)) * 16);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int f = f0 + u;
#pragma unroll
            for (int j = 0; j < kRowsPerThread; ++j) {
              const float wj = (f >= bnd[j] && f < bnd[j + 1]) ? av[u] : 0.f;
              acc[j].x = fmaf(wj, xv[u].x, acc[j].x);
              acc[j].y = fmaf(wj, xv[u].y, acc[j].y);
              acc[j].z = fmaf(wj, xv[u].z, acc[j].z);
              acc[j].w = fmaf(wj, xv[u].w, acc[j].w);
            }
          }
        }
      }
      RGMS_T(t_d);
      // the stage is free when the MMAs of tile k-2 have read it
      if (use > 0 && !warp_wait(&bar_empty[s], (use - 1) & 1, lane)) { ok = false; break; }
      RGMS_T(t_e);
      if (rel != staged_rel) {
        staged_rel = rel;
        const float4* wr = reinterpret_cast<const float4*>(
            w + static_cast<size_t>(RGMS_CHK(6, min(max(rel, 0), num_rels - 1), num_rels)) * kF * kF);
        constexpr int kWPerThread = kF * kF / 4 / kGatherThreads;  // 2
        float4 wv[kWPerThread];
#pragma unroll
        for (int i = 0; i < kWPerThread; ++i) wv[i] = __ldg(wr + gt + i * kGatherThreads);  // on their way during the wait
        // the MMAs of the previous tile are the last readers of the staged W
        if (k > 0 && !warp_wait(&bar_empty[(k - 1) % kStages], ((k - 1) / kStages) & 1, lane)) { ok = false; break; }
#pragma unroll
        for (int i = 0; i < kWPerThread; ++i) {
          const int ch = gt + i * kGatherThreads;
          const int fo = ch >> 4, kc = ch & 15;
          const float4 v = wv[i];
          const float4 l = make_float4(v.x - tf32_hi(v.x), v.y - tf32_hi(v.y), v.z - tf32_hi(v.z), v.w - tf32_hi(v.w));
          *reinterpret_cast<float4*>(base + kOffW + swz_off(fo, kc, kWBox)) = v;
          *reinterpret_cast<float4*>(base + kOffW + swz_off(kF + fo, kc, kWBox)) = l;
        }
      }
      // (4) the row pieces, as they are and their remainders, at the swizzled offsets
      unsigned char* zr = base + kOffZRaw + s * kZTile;
      unsigned char* zl = base + kOffZLo + s * kZTile;
#pragma unroll
      for (int j = 0; j < kRowsPerThread; ++j) {
        const int t = kRowsPerThread * slot + j;
        if (t < nrows) {  // rows past the end of a short tile are never read back
          const float4 v = acc[j];
          const int off = swz_off(t, piece, kZBox);
          *reinterpret_cast<float4*>(zr + off) = v;
          *reinterpret_cast<float4*>(zl + off) =
              make_float4(v.x - tf32_hi(v.x), v.y - tf32_hi(v.y), v.z - tf32_hi(v.z), v.w - tf32_hi(v.w));
        }
      }
      tc05::fence_async_smem();  // these stores -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_conv[s]);
      RGMS_T(t_f);
      RGMS_ADD(0, t_a, t_b); RGMS_ADD(1, t_b, t_c); RGMS_ADD(2, t_c, t_d); RGMS_ADD(3, t_d, t_e); RGMS_ADD(4, t_e, t_f);
      RGMS_ADD(5, 0, 1);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // nothing of this thread's may still be in flight
  } else {
    // ---- epilogue, two groups of four warps: group 0 (warps 1-4) takes the even tiles and
    // accumulator 0, group 1 (warps 5-8) the odd tiles and accumulator 1.  A warp reads the TMEM
    // lanes 32 * (warp % 4) .. + 31: any four consecutive warps cover the 128 rows of a tile.
    // thread = tile row = TMEM lane
    const int grp = warp >= 5 ? 1 : 0;
    const int t = (warp & 3) * 32 + lane;
    unsigned char* gbuf = base + kOffOut + grp * (kTM * kOutStride);
    unsigned char* my_row = gbuf + t * kOutStride;
    const unsigned char* wbase = gbuf + (warp & 3) * 32 * kOutStride;
    int rel, row0 = 0, row1 = 0;
    if (grp < my_tiles) tab.locate(first + grp * step, &rel, &row0, &row1);
    int dst_row = __ldg(indices_i + RGMS_CHK(16, min(max(row0 + t, 0), nnz_i - 1), nnz_i));
    for (int k = grp; k < my_tiles; k += 2) {
      const int buse = k >> 1;
      const int nrows = row1 - row0;
      // destination rows of this group's next tile (two tiles on): requested now, needed later
      int nrow0 = row0, nrow1 = row1;
      if (k + 2 < my_tiles) tab.locate(first + (k + 2) * step, &rel, &nrow0, &nrow1);
      const int dst_next = __ldg(indices_i + RGMS_CHK(17, min(max(nrow0 + t, 0), nnz_i - 1), nnz_i));
      if (!tc05::mbar_wait(&bar_acc_full[grp], buse & 1)) { ok = false; break; }
      tc05::fence_after_sync();
      const uint32_t taddr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + grp * 2 * kF;
#pragma unroll
      for (int half = 0; half < 2; ++half) {  // 32 output columns at a time
        uint32_t r[32];
        tc05::tmem_ld32(taddr + half * 32, r);            // z*W + zlo*W
#pragma unroll
        for (int part = 0; part < 2; ++part) {            // + z*Wlo, 16 columns at a time
          uint32_t r2[16];
          tmem_ld16(taddr + kF + half * 32 + part * 16, r2);
#pragma unroll
          for (int q = 0; q < 16; ++q)
            r[part * 16 + q] = __float_as_uint(__uint_as_float(r[part * 16 + q]) + __uint_as_float(r2[q]));
        }
        if (half == 1) {  // both halves are in registers or on their way to Y: accumulator free
          tc05::fence_before_sync();
          mbar_arrive(&bar_acc_empty[grp]);
        }
        // transpose through shared memory: a thread holds one row, the reductions want a row
        // spread over 8 lanes (four whole 128-byte lines per warp instruction)
        __syncwarp();  // the warp's reads of the previous half are over
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<uint4*>(my_row + q * 16) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        __syncwarp();
#pragma unroll 4
        for (int i = 0; i < 8; ++i) {
          const int lr = 4 * i + (lane >> 3);  // row inside the warp's 32
          const int drow = __shfl_sync(0xffffffffu, dst_row, lr);
          if ((warp & 3) * 32 + lr < nrows) {
            const float4 v = *reinterpret_cast<const float4*>(wbase + lr * kOutStride + (lane & 7) * 16);
            atomicAdd(reinterpret_cast<float4*>(y + static_cast<size_t>(RGMS_CHK(15, min(max(drow, 0), m_y - 1), m_y)) * kF + half * 32) + (lane & 7), v);
          }
        }
      }
      row0 = nrow0;
      row1 = nrow1;
      dst_row = dst_next;
    }
  }

  const bool all_ok = !__syncthreads_or(!ok);
  if (!all_ok && tid == 0) atomicAdd(&g_rgms_fused_timeouts, 1u);
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tmem, 4 * kF);
}

}  // namespace

// 0 when launched, 1 when this path cannot take the call (caller falls back), -1 on error
int rgms_fused_launch(const float* a, const float* w, const float* x, float* y, const int32_t* indptr_i,
                      const int32_t* indices_i, const int32_t* indptr_j, const int32_t* indices_j,
                      int num_rels, int feat, int nnz_i, int nnz_j, int n, int m, cudaStream_t stream) {
  if (feat != kF || nnz_i <= 0 || num_rels <= 0 || num_rels > kMaxRels || nnz_j <= 0 || n <= 0 || m <= 0) return 1;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(y) & 15u) ||
      (reinterpret_cast<uintptr_t>(w) & 15u))
    return 1;
  // the index arrays are staged with 16-byte copies
  if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(indptr_j) & 15u) ||
      (reinterpret_cast<uintptr_t>(indices_j) & 15u))
    return 1;
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(rgms_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFusedSmem));
    configured_device = dev;
  }
  const long long tiles = static_cast<long long>(nnz_i) / kTM + num_rels;  // upper bound
  const long long grid = tiles < kNumSMs ? tiles : kNumSMs;
  rgms_fused_kernel<<<static_cast<unsigned>(grid), kFThreads, kFusedSmem, stream>>>(
      a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, nnz_i, nnz_j, n, m);
  SPTIR_LAUNCH_OK("rgms_fused_kernel");
  return 0;
}

#ifdef SPTIR_RGMS_CHECK
extern "C" __attribute__((visibility("default"))) int sparsetir_rgms_check_words(long long* out) {
  cudaDeviceSynchronize();
  return cudaMemcpyFromSymbol(out, g_rgms_check, sizeof(long long) * 6) == cudaSuccess ? 0 : -1;
}
#endif

#ifdef SPTIR_RGMS_PROF
extern "C" __attribute__((visibility("default"))) int sparsetir_rgms_prof_words(unsigned long long* out) {
  cudaDeviceSynchronize();
  return cudaMemcpyFromSymbol(out, g_rgms_prof, sizeof(unsigned long long) * 8) == cudaSuccess ? 0 : -1;
}
#endif

int rgms_fused_timeouts(unsigned int* count) {
  SPTIR_CUDA_OK(cudaMemcpyFromSymbol(count, g_rgms_fused_timeouts, sizeof(unsigned int)));
  return 0;
}

}  // namespace sptir
