// Tensor-core BSR SpMM for 32 x 32 blocks (fp16 blocks and dense operand, fp32 accumulate/out):
//   C[i*32+bi, f] = sum_{p in block-row i} sum_bj A[p,bi,bj] * B[indices[p]*32+bj, f]
// Semantics as bsrmm.cu; replaces the wmma kernel of examples/blocksparse/bsr_spmm.py:359-425.
//
// A block-row is 32 rows tall but the 5th-generation tensor core multiplies M = 64 or 128 rows,
// so the product is computed transposed: one thread block owns (block-row i, 128 features) and
//   D^T[f, bi] (128 x 32, fp32 in TMEM)  +=  Bt[f, bj] (128 x 32)  *  A_p[bi, bj]^T (32 x 32)
// for every stored block p of the row — M = 128 features, N = 32 block rows, K = 32 block
// columns = two tcgen05.mma.kind::f16 of K = 16.  The feature-contiguous B rows are an MN-major
// operand, the row-major A block a K-major operand; neither needs a transpose in memory.
//
// Pipeline: operands travel global -> registers -> shared memory.  (Asynchronous 16-byte
// copies straight into shared memory were measured at about 16 bytes per clock per SM on this
// part, which capped the kernel at ~5 TB/s of L2 reads; plain 16-byte loads are not so limited.)
// Every thread owns five 16-byte pieces of a block's operands and keeps THREE blocks in registers:
// the loads of block it+3 are issued before the pieces of block it are multiplied, so the wait
// for a load is hidden behind three iterations and behind the other thread blocks of the SM
// (3 stages = 30 KB, all 512 blocks of a 128 x 128-block matrix at 512 features are resident at
// once).  The pieces are stored in the un-swizzled core-matrix layout the tensor core reads
// (tc05.cuh), one elected thread issues the MMAs, tcgen05.commit arrives on the stage's mbarrier
// when the tensor core has finished reading it, and a thread waits on that mbarrier before it
// overwrites the stage three blocks later.  Epilogue: TMEM -> registers (lane = feature,
// 32 columns = 32 block rows) -> 32 coalesced row stores per warp.
// Every mbarrier wait is bounded; a timeout is counted in a device-side status word and the block
// gives up cleanly (TMEM freed), so a protocol error cannot hang the GPU.
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "common.h"
#include "tc05.cuh"
#include "tmap.h"
#include "vec.cuh"

namespace sptir {

__device__ unsigned int g_tc_timeouts = 0;  // bounded waits that ran out, since module load
int rgms_tc_timeouts(unsigned int* count);  // the same counter of rgms_tc.cu
int tcspmm_timeouts(unsigned int* count);   // ... and of tcspmm.cu
int rgms_f16_timeouts(unsigned int* count);  // ... and of rgms_f16.cu
int rgms_fused_timeouts(unsigned int* count);  // ... and of rgms_fused.cu

namespace {

constexpr int kThreads = 128;
constexpr int kBlk = 32;
constexpr int kTileF = 128;
constexpr int kStages = 3;
constexpr int kSets = 3;  // blocks a thread holds in registers (loaded, not yet stored to shared memory)
constexpr int kBBytes = kBlk * kTileF * 2;  // B tile of one block: 32 x 128 fp16 = 8 KB
constexpr int kABytes = kBlk * kBlk * 2;    // A block: 2 KB
constexpr int kStageBytes = kBBytes + kABytes;
constexpr uint32_t kTmemCols = 32;
constexpr int kColCache = 256;

// B tile stage layout (MN-major operand): core matrix (kc = bj/8, fc = f/8) at (kc*16+fc)*128,
// inside it K-step bj%8 at 16-byte stride, 8 features contiguous.
constexpr uint32_t kB_SBO = 128;        // next 8 features
constexpr uint32_t kB_LBO = 16 * 128;   // next 8 block columns
// A block stage layout (K-major operand): core matrix (kc = bj/8, ng = bi/8) at (kc*4+ng)*128,
// inside it row bi%8 at 16-byte stride, 8 block columns contiguous.
constexpr uint32_t kA_SBO = 128;        // next 8 block rows
constexpr uint32_t kA_LBO = 4 * 128;    // next 8 block columns

__global__ void __launch_bounds__(kThreads)
bsrmm_tc_kernel(const __half* __restrict__ a, const __half* __restrict__ b, float* __restrict__ c,
                const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices, int feat) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_free[kStages];  // stage may be overwritten
  __shared__ __align__(8) uint64_t bar_done;           // all MMAs of the row have finished
  __shared__ uint32_t s_tmem;
  __shared__ int32_t s_cols[kColCache];  // block columns of the row: keeps a dependent global
                                         // load out of every pipeline step
  const int i = blockIdx.x;
  const int f0 = blockIdx.y * kTileF;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int p0 = __ldg(indptr + i), nblk = __ldg(indptr + i + 1) - p0;

  float* crow = c + (static_cast<size_t>(i) * kBlk) * feat + f0 + warp * 32 + lane;
  if (nblk <= 0) {  // empty block-row: zeros, no tensor-core work
#pragma unroll 4
    for (int bi = 0; bi < kBlk; ++bi) crow[static_cast<size_t>(bi) * feat] = 0.f;
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) tc05::mbar_init(&bar_free[s], 1);
    tc05::mbar_init(&bar_done, 1);
    tc05::fence_mbar_init();
  }
  if (warp == 0) tc05::tmem_alloc(&s_tmem, kTmemCols);
  for (int t = tid; t < min(nblk, kColCache); t += kThreads) s_cols[t] = __ldg(indices + p0 + t);
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = s_tmem;

  // this thread's share of a block: 4 pieces of the B tile, 1 piece of the A block (16 bytes each)
  // B tile: 32 rows (block columns bj) x 16 chunks of 8 features.  Loads want whole 128-byte lines
  // (8 consecutive chunks of a row); conflict-free 16-byte stores into the core-matrix layout want
  // the 32 lanes of a warp to cover all 8 values of bj%8 (the 16-byte slot inside a 128-byte core
  // matrix).  A load instruction k covers rows 4k..4k+3 (+16 for warps 2, 3) x 8 chunks, and
  // store instruction j of a lane writes the piece it loaded with instruction j ^ (lane & 1): even
  // and odd chunks of one store come from rows 4 apart, which makes the 8 slots appear 4 times each.
  const int b_fc = (warp & 1) * 8 + (lane & 7);         // feature chunk 0..15
  const int b_row0 = (warp >> 1) * 16 + (lane >> 3);    // row of load instruction 0; +4 per instruction
  const bool b_odd = (lane & 1) != 0;
  const int a_bi = tid >> 2, a_kc = tid & 3;    // A: block row, 8-column chunk
  struct Pieces {
    uint4 b[4];
    uint4 a;
  };
  auto load_block = [&](int it, Pieces& x) {
    const int p = p0 + it;
    const size_t brow0 = static_cast<size_t>(it < kColCache ? s_cols[it] : __ldg(indices + p)) * kBlk;
#pragma unroll
    for (int kc = 0; kc < 4; ++kc)
      x.b[kc] = __ldg(reinterpret_cast<const uint4*>(b + (brow0 + b_row0 + kc * 4) * feat + f0 + b_fc * 8));
    x.a = __ldg(reinterpret_cast<const uint4*>(a + static_cast<size_t>(p) * (kBlk * kBlk) + a_bi * kBlk + a_kc * 8));
  };
  auto store_block = [&](int stage, const Pieces& x) {
    unsigned char* st = smem + stage * kStageBytes;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 v = b_odd ? x.b[j ^ 1] : x.b[j];
      const int row = b_row0 + (b_odd ? (j ^ 1) : j) * 4;  // block column bj of the piece
      *reinterpret_cast<uint4*>(st + ((row >> 3) * 16 + b_fc) * 128 + (row & 7) * 16) = v;
    }
    *reinterpret_cast<uint4*>(st + kBBytes + (a_kc * 4 + (a_bi >> 3)) * 128 + (a_bi & 7) * 16) = x.a;
  };

  constexpr uint32_t idesc = tc05::instr_desc(tc05::kFmtF16, kTileF, kBlk, /*a_mn=*/1, /*b_mn=*/0);
  bool ok = true;

  // one pipeline step: block `it` (already in registers) -> shared memory -> tensor core, and
  // the loads of block it+kSets into the same registers; false when a bounded wait ran out
  auto step = [&](int it, Pieces& x) -> bool {
    const int stage = it % kStages;
    if (it >= kStages) {  // the MMAs of block it-kStages are the previous use of this stage
      if (!tc05::mbar_wait(&bar_free[stage], ((it - kStages) / kStages) & 1)) ok = false;
    }
    if (ok) store_block(stage, x);
    if (it + kSets < nblk) load_block(it + kSets, x);
    tc05::fence_async_smem();
    if (__syncthreads_or(!ok)) return false;
    if (warp == 0 && lane == 0) {
      tc05::fence_after_sync();
      const uint32_t sb = tc05::smem_u32(smem + stage * kStageBytes);
      const uint32_t sa = sb + kBBytes;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {  // K = 32 block columns = 2 x 16
        const uint64_t da = tc05::smem_desc(sb + ks * 2 * kB_LBO, kB_LBO, kB_SBO);
        const uint64_t db = tc05::smem_desc(sa + ks * 2 * kA_LBO, kA_LBO, kA_SBO);
        tc05::mma_f16(tmem, da, db, idesc, (it > 0 || ks > 0) ? 1u : 0u);
      }
      tc05::mma_commit(&bar_free[stage]);
      if (it == nblk - 1) tc05::mma_commit(&bar_done);
    }
    return true;
  };

  Pieces x[kSets];
#pragma unroll
  for (int k = 0; k < kSets; ++k)
    if (k < nblk) load_block(k, x[k]);
  for (int it = 0; it < nblk && ok; it += kSets) {
#pragma unroll
    for (int k = 0; k < kSets; ++k) {
      if (ok && it + k < nblk && !step(it + k, x[k])) ok = false;  // uniform: step ends in a barrier vote
    }
  }

  if (ok && !tc05::mbar_wait(&bar_done, 0)) ok = false;
  ok = !__syncthreads_or(!ok);
  tc05::fence_after_sync();
  if (ok) {
    uint32_t r[32];
    tc05::tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16), r);
#pragma unroll
    for (int bi = 0; bi < kBlk; ++bi) __stcs(crow + static_cast<size_t>(bi) * feat, __uint_as_float(r[bi]));
  } else if (tid == 0) {
    atomicAdd(&g_tc_timeouts, 1u);
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tmem, kTmemCols);
}


// ---------------------------------------------------------------------------------------------
// TMA-fed variant (the default): the same tiles and the same MMAs, but the operands are brought
// in by the tensor memory accelerator.  Warp 0 is the producer: per stored block it waits for the
// stage to be free, arms the stage's "full" mbarrier with the byte count and issues three tile
// loads (two 64-feature x 32-row boxes of B with the 128-byte swizzle, one 32 x 32 box of A with
// the 64-byte swizzle).  Warp 1 issues the MMAs when "full" completes and lets tcgen05.commit
// arrive on the stage's "empty" mbarrier.  No thread touches the operands, there is no block-wide
// barrier inside the loop, and the loads in flight are bounded by the stages (4 x 10 KB), not by
// registers.  All four warps run the epilogue.
constexpr int kTStages = 4;
constexpr int kTmaSmem = kTStages * kStageBytes + 1024;  // + slack to align the tiles to 1024 bytes

__global__ void __launch_bounds__(kThreads)
bsrmm_tma_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 float* __restrict__ c, const int32_t* __restrict__ indptr,
                 const int32_t* __restrict__ indices, int feat) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kTStages];   // operands of the stage have landed
  __shared__ __align__(8) uint64_t bar_empty[kTStages];  // the tensor core has read the stage
  __shared__ __align__(8) uint64_t bar_done;             // all MMAs of the row have finished
  __shared__ uint32_t s_tmem;
  const int i = blockIdx.x;
  const int f0 = blockIdx.y * kTileF;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int p0 = __ldg(indptr + i), nblk = __ldg(indptr + i + 1) - p0;

  float* crow = c + (static_cast<size_t>(i) * kBlk) * feat + f0 + warp * 32 + lane;
  if (nblk <= 0) {  // empty block-row: zeros, no tensor-core work
#pragma unroll 4
    for (int bi = 0; bi < kBlk; ++bi) crow[static_cast<size_t>(bi) * feat] = 0.f;
    return;
  }
  // swizzle atoms repeat every 1024 bytes of shared-memory address
  unsigned char* tiles = smem_raw + ((1024u - (tc05::smem_u32(smem_raw) & 1023u)) & 1023u);

  if (tid == 0) {
    for (int s = 0; s < kTStages; ++s) {
      tc05::mbar_init(&bar_full[s], 1);
      tc05::mbar_init(&bar_empty[s], 1);
    }
    tc05::mbar_init(&bar_done, 1);
    tc05::fence_mbar_init();
    tc05::prefetch_tensormap(&tm_a);
    tc05::prefetch_tensormap(&tm_b);
  }
  if (warp == 0) tc05::tmem_alloc(&s_tmem, kTmemCols);
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = s_tmem;
  constexpr uint32_t idesc = tc05::instr_desc(tc05::kFmtF16, kTileF, kBlk, /*a_mn=*/1, /*b_mn=*/0);
  bool ok = true;
  int armed = 0;  // producer: blocks whose loads have been issued

  if (warp == 0) {
    int cols = 0;
    for (int it = 0; it < nblk; ++it) {
      const int stage = it % kTStages, use = it / kTStages;
      if ((it & 31) == 0) cols = (it + lane < nblk) ? __ldg(indices + p0 + it + lane) : 0;
      const int col = __shfl_sync(0xffffffffu, cols, it & 31);
      if (use > 0) {
        if (lane == 0) ok = tc05::mbar_wait(&bar_empty[stage], (use - 1) & 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      if (lane == 0) {
        unsigned char* st = tiles + stage * kStageBytes;
        tc05::mbar_arrive_expect_tx(&bar_full[stage], kStageBytes);
        tc05::tma_load_2d(st, &tm_b, f0, col * kBlk, &bar_full[stage]);
        tc05::tma_load_2d(st + kBBytes / 2, &tm_b, f0 + 64, col * kBlk, &bar_full[stage]);
        tc05::tma_load_2d(st + kBBytes, &tm_a, 0, (p0 + it) * kBlk, &bar_full[stage]);
      }
      armed = it + 1;
    }
  } else if (warp == 1) {
    // descriptors of stage 0, built once; the loop advances their address fields
    // B tile, MN-major: 16 K rows of 128 bytes per step; the two 64-feature atoms are 4 KB apart
    const uint64_t da0 = tc05::smem_desc_swizzled(tc05::smem_u32(tiles), kBBytes / 2, 1024, tc05::kSwizzle128B);
    // A block, K-major: rows of 64 bytes, 16 columns (32 bytes) per step inside the row
    const uint64_t db0 = tc05::smem_desc_swizzled(tc05::smem_u32(tiles) + kBBytes, 0, 512, tc05::kSwizzle64B);
    for (int it = 0; it < nblk; ++it) {
      const int stage = it % kTStages, use = it / kTStages;
      if (lane == 0) ok = tc05::mbar_wait(&bar_full[stage], use & 1);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane == 0) {
        tc05::fence_after_sync();
        const uint64_t da_s = tc05::desc_advance(da0, stage * kStageBytes);
        const uint64_t db_s = tc05::desc_advance(db0, stage * kStageBytes);
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)  // K = 32 block columns = 2 x 16
          tc05::mma_f16(tmem, tc05::desc_advance(da_s, ks * 16 * 128), tc05::desc_advance(db_s, ks * 32), idesc,
                        (it > 0 || ks > 0) ? 1u : 0u);
        tc05::mma_commit(&bar_empty[stage]);
        if (it == nblk - 1) tc05::mma_commit(&bar_done);
      }
      __syncwarp();
    }
  }

  if (ok && !tc05::mbar_wait(&bar_done, 0)) ok = false;
  ok = !__syncthreads_or(!ok);
  tc05::fence_after_sync();
  if (ok) {
    uint32_t r[32];
    tc05::tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16), r);
#pragma unroll
    for (int bi = 0; bi < kBlk; ++bi) __stcs(crow + static_cast<size_t>(bi) * feat, __uint_as_float(r[bi]));
  } else {
    // gave up: let the copies already issued land (bounded) before the block's memory is released
    if (tid == 0) {
      atomicAdd(&g_tc_timeouts, 1u);
      for (int it = max(0, armed - kTStages); it < armed; ++it)
        tc05::mbar_wait(&bar_full[it % kTStages], (it / kTStages) & 1);
    }
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tmem, kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// Persistent variant (the default when feat is a multiple of 256): at 128 x 128 blocks and 512
// features the kernel above is 512 short-lived thread blocks, and what a call costs is mostly what
// every one of them pays before and after its dozen tile loads: barrier set-up, TMEM allocation,
// the first load's latency with nothing to overlap it, an epilogue nothing overlaps either.  Here
// one block per SM walks work items (block row, 256 features), so that
//   - barriers and TMEM are set up once per SM,
//   - the producer warp runs ahead across item boundaries: while the tensor core finishes one
//     item, the tiles of the next are already landing (8 stages of 18 KB),
//   - two TMEM accumulators alternate, so the epilogue of an item (TMEM -> registers -> 32
//     coalesced row stores per warp) overlaps the loads and MMAs of the next,
//   - the A block of a stored block is loaded once for two feature tiles.
// Roles: warp 0 producer (TMA), warp 1 MMA issuer, warps 2-5 epilogue (a warp reads the TMEM lanes
// 32 * (warp % 4) .. + 31: lane = feature inside the tile, column = row inside the block row).
// Every mbarrier wait is bounded.
constexpr int kPThreads = 192;
constexpr int kPTiles = 2;                              // feature tiles of 128 per work item
constexpr int kPStageBytes = kPTiles * kBBytes + kABytes;  // 18 KB
constexpr int kPStages = 6;
constexpr int kPSmem = kPStages * kPStageBytes + 1024;
constexpr uint32_t kPAccCols = kPTiles * kBlk;          // 64 TMEM columns per accumulator

__global__ void __launch_bounds__(kPThreads, 2)
bsrmm_persist_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     float* __restrict__ c, const int32_t* __restrict__ indptr,
                     const int32_t* __restrict__ indices, int feat, int num_items, int items_per_row) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kPStages];   // operands of the stage have landed
  __shared__ __align__(8) uint64_t bar_empty[kPStages];  // the tensor core has read the stage
  __shared__ __align__(8) uint64_t bar_acc_full[2];      // accumulator holds a finished item
  __shared__ __align__(8) uint64_t bar_acc_empty[2];     // the epilogue has read it (128 arrivals)
  __shared__ uint32_t s_tmem;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned char* tiles = smem_raw + ((1024u - (tc05::smem_u32(smem_raw) & 1023u)) & 1023u);

  if (tid == 0) {
    for (int s = 0; s < kPStages; ++s) {
      tc05::mbar_init(&bar_full[s], 1);
      tc05::mbar_init(&bar_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc05::mbar_init(&bar_acc_full[b], 1);
      tc05::mbar_init(&bar_acc_empty[b], 128);
    }
    tc05::fence_mbar_init();
    tc05::prefetch_tensormap(&tm_a);
    tc05::prefetch_tensormap(&tm_b);
  }
  if (warp == 0) tc05::tmem_alloc(&s_tmem, 2 * kPAccCols);
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = s_tmem;
  bool ok = true;
  int armed = 0;  // producer: stored blocks whose loads have been issued

  if (warp == 0) {
    // ---- producer: one stage per stored block, across item boundaries
    int bk = 0;  // stored blocks issued so far by this thread block
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int i = item / items_per_row, f0 = (item % items_per_row) * (kPTiles * kTileF);
      const int p0 = __ldg(indptr + i), nblk = __ldg(indptr + i + 1) - p0;
      int cols = 0;
      for (int it = 0; it < nblk; ++it, ++bk) {
        const int stage = bk % kPStages, use = bk / kPStages;
        if ((it & 31) == 0) cols = (it + lane < nblk) ? __ldg(indices + p0 + it + lane) : 0;
        const int col = __shfl_sync(0xffffffffu, cols, it & 31);
        if (use > 0) {
          if (lane == 0) ok = tc05::mbar_wait(&bar_empty[stage], (use - 1) & 1);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
        }
        if (lane == 0) {
          unsigned char* st = tiles + stage * kPStageBytes;
          tc05::mbar_arrive_expect_tx(&bar_full[stage], kPStageBytes);
#pragma unroll
          for (int tt = 0; tt < kPTiles; ++tt) {
            tc05::tma_load_2d(st + tt * kBBytes, &tm_b, f0 + tt * kTileF, col * kBlk, &bar_full[stage]);
            tc05::tma_load_2d(st + tt * kBBytes + kBBytes / 2, &tm_b, f0 + tt * kTileF + 64, col * kBlk, &bar_full[stage]);
          }
          tc05::tma_load_2d(st + kPTiles * kBBytes, &tm_a, 0, (p0 + it) * kBlk, &bar_full[stage]);
        }
        armed = bk + 1;
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    constexpr uint32_t idesc = tc05::instr_desc(tc05::kFmtF16, kTileF, kBlk, /*a_mn=*/1, /*b_mn=*/0);
    // B tile, MN-major: 16 K rows of 128 bytes per step; the two 64-feature atoms are 4 KB apart
    const uint64_t da0 = tc05::smem_desc_swizzled(tc05::smem_u32(tiles), kBBytes / 2, 1024, tc05::kSwizzle128B);
    // A block, K-major: rows of 64 bytes, 16 columns (32 bytes) per step inside the row
    const uint64_t db0 = tc05::smem_desc_swizzled(tc05::smem_u32(tiles) + kPTiles * kBBytes, 0, 512, tc05::kSwizzle64B);
    int bk = 0, acc_it = 0;  // stored blocks / non-empty items so far
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int i = item / items_per_row;
      const int nblk = __ldg(indptr + i + 1) - __ldg(indptr + i);
      if (nblk <= 0) continue;
      const int buf = acc_it & 1, buse = acc_it >> 1;
      if (buse > 0) {
        if (lane == 0) ok = tc05::mbar_wait(&bar_acc_empty[buf], (buse - 1) & 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      for (int it = 0; it < nblk; ++it, ++bk) {
        const int stage = bk % kPStages, use = bk / kPStages;
        if (lane == 0) ok = tc05::mbar_wait(&bar_full[stage], use & 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (lane == 0) {
          tc05::fence_after_sync();
          const uint64_t db_s = tc05::desc_advance(db0, stage * kPStageBytes);
#pragma unroll
          for (int tt = 0; tt < kPTiles; ++tt) {
            const uint64_t da_s = tc05::desc_advance(da0, stage * kPStageBytes + tt * kBBytes);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)  // K = 32 block columns = 2 x 16
              tc05::mma_f16(tmem + buf * kPAccCols + tt * kBlk, tc05::desc_advance(da_s, ks * 16 * 128),
                            tc05::desc_advance(db_s, ks * 32), idesc, (it > 0 || ks > 0) ? 1u : 0u);
          }
          tc05::mma_commit(&bar_empty[stage]);
          if (it == nblk - 1) tc05::mma_commit(&bar_acc_full[buf]);
        }
        __syncwarp();
      }
      ++acc_it;
    }
  } else {
    // ---- epilogue: thread = feature inside the 128-feature tile
    const int q = warp & 3;  // TMEM lane quarter of this warp
    int acc_it = 0;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      const int i = item / items_per_row, f0 = (item % items_per_row) * (kPTiles * kTileF);
      const int nblk = __ldg(indptr + i + 1) - __ldg(indptr + i);
      float* crow = c + (static_cast<size_t>(i) * kBlk) * feat + f0 + q * 32 + lane;
      if (nblk <= 0) {  // empty block-row: zeros, no tensor-core work
#pragma unroll
        for (int tt = 0; tt < kPTiles; ++tt)
#pragma unroll 4
          for (int bi = 0; bi < kBlk; ++bi) crow[static_cast<size_t>(bi) * feat + tt * kTileF] = 0.f;
        continue;
      }
      const int buf = acc_it & 1, buse = acc_it >> 1;
      if (!tc05::mbar_wait(&bar_acc_full[buf], buse & 1)) { ok = false; break; }
      tc05::fence_after_sync();
#pragma unroll
      for (int tt = 0; tt < kPTiles; ++tt) {
        uint32_t r[32];
        tc05::tmem_ld32(tmem + (static_cast<uint32_t>(q * 32) << 16) + buf * kPAccCols + tt * kBlk, r);
        if (tt == kPTiles - 1) {  // everything of this accumulator is in registers
          tc05::fence_before_sync();
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc05::smem_u32(&bar_acc_empty[buf])) : "memory");
        }
#pragma unroll
        for (int bi = 0; bi < kBlk; ++bi)
          __stcs(crow + static_cast<size_t>(bi) * feat + tt * kTileF, __uint_as_float(r[bi]));
      }
      ++acc_it;
    }
  }

  const bool all_ok = !__syncthreads_or(!ok);
  if (!all_ok && tid == 0) {
    atomicAdd(&g_tc_timeouts, 1u);
    // gave up: let the copies already issued land (bounded) before the block's memory is released
    for (int bk = max(0, armed - kPStages); bk < armed; ++bk)
      tc05::mbar_wait(&bar_full[bk % kPStages], (bk / kPStages) & 1);
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tmem, 2 * kPAccCols);
}

// 0 when launched, 1 when this path cannot take the call (caller falls back), -1 on error
int bsrmm_persist_launch(const __half* a, const __half* b, float* c, const int32_t* indptr,
                         const int32_t* indices, int nb, int mb, int nnzb, int feat, cudaStream_t stream) {
  if (nnzb <= 0 || mb <= 0 || feat % (kPTiles * kTileF) != 0) return 1;
  CUtensorMap tm_a, tm_b;
  if (make_tmap_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a, kBlk, static_cast<uint64_t>(nnzb) * kBlk,
                   kBlk * 2, kBlk, kBlk, CU_TENSOR_MAP_SWIZZLE_64B) != 0)
    return 1;
  if (make_tmap_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, b, static_cast<uint64_t>(feat),
                   static_cast<uint64_t>(mb) * kBlk, static_cast<uint64_t>(feat) * 2, 64, kBlk,
                   CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return 1;
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(bsrmm_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPSmem));
    configured_device = dev;
  }
  const int items_per_row = feat / (kPTiles * kTileF);
  const long long items = static_cast<long long>(nb) * items_per_row;
  if (items > INT32_MAX) return 1;
  const int grid = static_cast<int>(items < 2 * kNumSMs ? items : 2 * kNumSMs);  // two blocks per SM (shared memory)
  bsrmm_persist_kernel<<<grid, kPThreads, kPSmem, stream>>>(tm_a, tm_b, c, indptr, indices, feat,
                                                            static_cast<int>(items), items_per_row);
  SPTIR_LAUNCH_OK("bsrmm_persist_kernel");
  return 0;
}

// 0 when launched, 1 when this path cannot take the call (caller falls back), -1 on error
int bsrmm_tma_launch(const __half* a, const __half* b, float* c, const int32_t* indptr,
                     const int32_t* indices, int nb, int mb, int nnzb, int feat, cudaStream_t stream) {
  if (nnzb <= 0 || mb <= 0) return 1;
  CUtensorMap tm_a, tm_b;
  if (make_tmap_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a, kBlk, static_cast<uint64_t>(nnzb) * kBlk,
                   kBlk * 2, kBlk, kBlk, CU_TENSOR_MAP_SWIZZLE_64B) != 0)
    return 1;
  if (make_tmap_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, b, static_cast<uint64_t>(feat),
                   static_cast<uint64_t>(mb) * kBlk, static_cast<uint64_t>(feat) * 2, 64, kBlk,
                   CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return 1;
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(bsrmm_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kTmaSmem));
    configured_device = dev;
  }
  dim3 grid(nb, feat / kTileF);
  bsrmm_tma_kernel<<<grid, kThreads, kTmaSmem, stream>>>(tm_a, tm_b, c, indptr, indices, feat);
  SPTIR_LAUNCH_OK("bsrmm_tma_kernel");
  return 0;
}

}  // namespace

// Returns 0 when launched, 1 when the shape is not handled here, -1 on error.
int bsrmm_tc_launch(const __half* a, const __half* b, float* c, const int32_t* indptr,
                    const int32_t* indices, int nb, int mb, int nnzb, int blk, int feat,
                    cudaStream_t stream) {
  (void)mb; (void)nnzb;
  if (blk != kBlk || feat % kTileF != 0) return 1;
  if (!aligned16(a) || !aligned16(b) || !aligned16(c)) return 1;
  if (feat / kTileF > 65535) return 1;
  // SPARSETIR_BSR_PATH=regs keeps the operands on the load/store path (comparison switch)
  static const bool use_tma = [] {
    const char* e = std::getenv("SPARSETIR_BSR_PATH");
    return !(e && std::strcmp(e, "regs") == 0);
  }();
  // SPARSETIR_BSR_PATH=tma keeps one thread block per (block row, 128 features)
  static const bool persistent = [] {
    const char* e = std::getenv("SPARSETIR_BSR_PATH");
    return e == nullptr || e[0] == '\0';
  }();
  if (persistent) {
    const int rc = bsrmm_persist_launch(a, b, c, indptr, indices, nb, mb, nnzb, feat, stream);
    if (rc <= 0) return rc;
  }
  if (use_tma) {
    const int rc = bsrmm_tma_launch(a, b, c, indptr, indices, nb, mb, nnzb, feat, stream);
    if (rc <= 0) return rc;
  }
  const size_t smem = static_cast<size_t>(kStages) * kStageBytes;
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(bsrmm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
    configured_device = dev;
  }
  dim3 grid(nb, feat / kTileF);
  bsrmm_tc_kernel<<<grid, kThreads, smem, stream>>>(a, b, c, indptr, indices, feat);
  SPTIR_LAUNCH_OK("bsrmm_tc_kernel");
  return 0;
}

}  // namespace sptir

// Number of bounded tensor-core waits that ran out on `device_id` since the library was loaded
// (0 in a healthy run).  Synchronises the device.
extern "C" int sparsetir_tc_timeouts(int device_id, unsigned int* count) {
  using namespace sptir;
  if (!count) return fail("sparsetir_tc_timeouts: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  SPTIR_CUDA_OK(cudaDeviceSynchronize());
  unsigned int bsr = 0, rgms = 0;
  SPTIR_CUDA_OK(cudaMemcpyFromSymbol(&bsr, g_tc_timeouts, sizeof(unsigned int)));
  if (rgms_tc_timeouts(&rgms) != 0) return -1;
  unsigned int tcs = 0;
  if (tcspmm_timeouts(&tcs) != 0) return -1;
  unsigned int rh = 0;
  if (rgms_f16_timeouts(&rh) != 0) return -1;
  unsigned int rf = 0;
  if (rgms_fused_timeouts(&rf) != 0) return -1;
  *count = bsr + rgms + tcs + rh + rf;
  return 0;
}
