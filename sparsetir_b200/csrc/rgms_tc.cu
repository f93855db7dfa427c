// Tensor-core RGMS for feat_size 64, fp32 in and out:
//   Y[I[i], fo] += sum_{p in CSF row i of relation r} A[p] * sum_fi W[r,fo,fi] * X[J[p],fi]
// Semantics and formulation (aggregate first, transform once per (relation, row)) as rgms.cu;
// replaces the wmma kernel of examples/rgms/rgcn/bench_rgcn_tensorcore.py:651-858, which
// multiplies fp16 copies of X and W.
//
// One thread block owns a tile of up to 128 CSF rows of one relation:
//   phase 1  sub-warps gather-aggregate Z[t,:] = sum_p A[p] X[J[p],:] in fp32 registers and
//            write it to shared memory directly in the core-matrix layout the tensor core
//            reads (tc05.cuh), split into a TF32-exact high part and a low remainder;
//   phase 2  D[t,fo] (128 x 64 fp32 in TMEM) = Z[t,fi] * W_r[fo,fi]^T with tcgen05.mma.kind::tf32,
//            M = 128 tile rows, N = 64, K = 64 = 8 steps of 8.  Plain TF32 (10-bit mantissa)
//            would miss the fp32 tolerance of this operator (rtol 1e-4), so every step runs the
//            three products Zhi*Whi + Zlo*Whi + Zhi*Wlo ("3xTF32"), which carries ~21 bits;
//   phase 3  TMEM -> registers (lane = tile row, 32 columns per thread) -> 16-byte vector
//            atomics into Y[I[t], :].
// The one mbarrier wait (tensor core done) is bounded; a timeout is counted and the block gives
// up cleanly.
#include "common.h"
#include "rgms_common.cuh"
#include "spmm_core.cuh"
#include <cstdlib>
#include <cstring>

#include "tc05.cuh"
#include "tmap.h"

namespace sptir {

__device__ unsigned int g_rgms_tc_timeouts = 0;

namespace {

constexpr int kF = 64;
constexpr int kTM = 128;
constexpr int kLPR = kF / 4;                   // 16 lanes cover a feature row
constexpr int kZBytes = kTM * kF * 4;          // 32 KB per Z part
constexpr int kWBytes = kF * kF * 4;           // 16 KB per W part
constexpr size_t kSmemBytes = 2 * kZBytes + 2 * kWBytes;
// K-major operands, no swizzle: core matrix (g = row/8, kc = fi/4) at (g*16 + kc)*128, row%8
// at 16-byte stride inside it, 4 floats of K contiguous.  With the 16 K-chunks of a row group
// adjacent, a warp that copies 8 rows x 4 chunks reads 64 contiguous bytes per row from global
// memory and writes 512 contiguous bytes of shared memory: coalesced and bank-conflict free.
constexpr uint32_t kZ_LBO = 128, kZ_SBO = kLPR * 128;  // next K chunk / next 8 rows
constexpr uint32_t kW_LBO = 128, kW_SBO = kLPR * 128;
__device__ __forceinline__ int core_off(int row, int kc) {
  return ((row >> 3) * kLPR + kc) * 128 + (row & 7) * 16;
}
// chunk index -> (row, kc) such that the 32 lanes of a warp cover 8 rows x 4 K-chunks
__device__ __forceinline__ void chunk_of(int ch, int* row, int* kc) {
  const int lane = ch & 31, blk = ch >> 5;       // blk: (row group, quarter of the K chunks)
  *row = (blk >> 2) * 8 + (lane & 7);
  *kc = (blk & 3) * 4 + (lane >> 3);
}

__device__ __forceinline__ float tf32_hi(float x) {
  return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);  // what the tensor core keeps
}

// Persistent form: a block walks `tiles_per_cta` consecutive tiles.  Tiles are numbered relation
// by relation, so consecutive tiles mostly share the relation: W_r is staged once per change of
// relation, the first tile is found with the block-wide scan and the following ones by stepping
// through indptr_i, TMEM and the mbarrier are set up once, and (two-launch form) the next tile's
// Z rows are already on their way into registers while the tensor core works on this one.
__global__ void __launch_bounds__(kRgmsThreads)
rgms_tc_kernel(const float* __restrict__ a, const float* __restrict__ w,
               const float* __restrict__ x, float* __restrict__ y,
               const int32_t* __restrict__ indptr_i, const int32_t* __restrict__ indices_i,
               const int32_t* __restrict__ indptr_j, const int32_t* __restrict__ indices_j,
               int num_rels, const float* __restrict__ z, int tiles_per_cta) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t s_tmem;
  unsigned char* z_hi = smem;
  unsigned char* z_lo = smem + kZBytes;
  unsigned char* w_hi = smem + 2 * kZBytes;
  unsigned char* w_lo = w_hi + kWBytes;
  constexpr int kZPerThread = kTM * kLPR / kRgmsThreads;  // 16-byte chunks of a Z tile per thread

  int rel, row0, row1;
  if (!locate_tile(indptr_i, num_rels, kTM, blockIdx.x * tiles_per_cta, &rel, &row0, &row1)) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane32 = tid & 31;

  if (tid == 0) {
    tc05::mbar_init(&bar_done, 1);
    tc05::fence_mbar_init();
  }
  if (warp == 0) tc05::tmem_alloc(&s_tmem, kF);
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = s_tmem;

  // this thread's chunks of a Z tile, fetched ahead of use (two-launch form)
  float4 zreg[kZPerThread];
  auto fetch_z = [&](int r0, int nr) {
    const float4* zt = reinterpret_cast<const float4*>(z + static_cast<size_t>(r0) * kF);
#pragma unroll
    for (int k = 0; k < kZPerThread; ++k) {
      int t, kc;
      chunk_of(tid + k * kRgmsThreads, &t, &kc);
      zreg[k] = t < nr ? __ldg(zt + t * kLPR + kc) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  if (z != nullptr) fetch_z(row0, row1 - row0);

  int staged_rel = -1;
  uint32_t parity = 0;
  bool ok = true;
  for (int it = 0; it < tiles_per_cta; ++it) {
    const int nrows = row1 - row0;
    // W_r[fo, fi] -> core matrices, split hi/lo, when the relation changed
    if (rel != staged_rel) {
      staged_rel = rel;
      const float4* wr = reinterpret_cast<const float4*>(w + static_cast<size_t>(rel) * kF * kF);
      for (int ch = tid; ch < kF * kF / 4; ch += kRgmsThreads) {
        int fo, kc;
        chunk_of(ch, &fo, &kc);
        const float4 v = __ldg(wr + fo * kLPR + kc);
        const float4 h = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
        const float4 l = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
        const int off = core_off(fo, kc);
        *reinterpret_cast<float4*>(w_hi + off) = h;
        *reinterpret_cast<float4*>(w_lo + off) = l;
      }
    }
    // phase 1: the tile's aggregated rows -> shared memory, split hi/lo
    if (z != nullptr) {
#pragma unroll
      for (int k = 0; k < kZPerThread; ++k) {
        int t, kc;
        chunk_of(tid + k * kRgmsThreads, &t, &kc);
        const float4 v = zreg[k];
        const float4 h = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
        const float4 l = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
        const int off = core_off(t, kc);
        *reinterpret_cast<float4*>(z_hi + off) = h;
        *reinterpret_cast<float4*>(z_lo + off) = l;
      }
    } else {  // fused form: gather-aggregate here; lane = kc
      const int lane = tid % kLPR;
      gather_tile_rows<kF, kTM>(a, x, indptr_j, indices_j, row0, nrows, [&](int t, float4 v) {
        const float4 h = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
        const float4 l = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
        const int off = core_off(t, lane);
        *reinterpret_cast<float4*>(z_hi + off) = h;
        *reinterpret_cast<float4*>(z_lo + off) = l;
      });
    }
    tc05::fence_async_smem();  // shared-memory writes above -> visible to the tensor core
    tc05::fence_before_sync();
    __syncthreads();
    tc05::fence_after_sync();
    // phase 2: one thread issues 8 K-steps x 3 products
    if (tid == 0) {
      constexpr uint32_t idesc = tc05::instr_desc(tc05::kFmtTF32, kTM, kF, /*a_mn=*/0, /*b_mn=*/0);
      const uint32_t zh = tc05::smem_u32(z_hi), zl = tc05::smem_u32(z_lo);
      const uint32_t wh = tc05::smem_u32(w_hi), wl = tc05::smem_u32(w_lo);
#pragma unroll
      for (int ks = 0; ks < kF / 8; ++ks) {  // K = 8 floats = two core matrices per step
        const uint64_t dzh = tc05::smem_desc(zh + ks * 2 * kZ_LBO, kZ_LBO, kZ_SBO);
        const uint64_t dzl = tc05::smem_desc(zl + ks * 2 * kZ_LBO, kZ_LBO, kZ_SBO);
        const uint64_t dwh = tc05::smem_desc(wh + ks * 2 * kW_LBO, kW_LBO, kW_SBO);
        const uint64_t dwl = tc05::smem_desc(wl + ks * 2 * kW_LBO, kW_LBO, kW_SBO);
        tc05::mma_tf32(tmem, dzl, dwh, idesc, ks > 0 ? 1u : 0u);  // small terms first
        tc05::mma_tf32(tmem, dzh, dwl, idesc, 1u);
        tc05::mma_tf32(tmem, dzh, dwh, idesc, 1u);
      }
      tc05::mma_commit(&bar_done);
    }

    // while the tensor core works: find the next tile, start fetching its rows, and read the
    // destination row id this thread will scatter to
    int nrel = rel, nrow0 = row1;
    int rel_end = __ldg(indptr_i + rel + 1);
    while (nrel < num_rels && nrow0 >= rel_end) {
      ++nrel;
      if (nrel < num_rels) rel_end = __ldg(indptr_i + nrel + 1);
    }
    const bool has_next = (it + 1 < tiles_per_cta) && nrel < num_rels;
    const int nrow1 = min(rel_end, nrow0 + kTM);
    if (z != nullptr && has_next) fetch_z(nrow0, nrow1 - nrow0);
    const int t = (warp & 3) * 32 + lane32;  // tile row whose accumulators this thread reads
    const int dst_row = t < nrows ? __ldg(indices_i + row0 + t) : 0;

    if (!tc05::mbar_wait(&bar_done, parity)) ok = false;
    parity ^= 1u;
    ok = !__syncthreads_or(!ok);
    tc05::fence_after_sync();
    if (!ok) break;

    // phase 3: warps w and w+4 share TMEM lanes 32*(w%4)..+31 and take 32 columns each
    {
      const int col0 = (warp >> 2) * 32;
      uint32_t r[32];
      tc05::tmem_ld32(tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + col0, r);
      if (t < nrows) {
        float4* dst = reinterpret_cast<float4*>(y + static_cast<size_t>(dst_row) * kF + col0);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          atomicAdd(dst + k, make_float4(__uint_as_float(r[4 * k]), __uint_as_float(r[4 * k + 1]),
                                         __uint_as_float(r[4 * k + 2]), __uint_as_float(r[4 * k + 3])));
      }
    }
    // every thread has read its accumulators before the next tile's first MMA overwrites them
    tc05::fence_before_sync();
    __syncthreads();
    tc05::fence_after_sync();
    if (!has_next) break;
    rel = nrel;
    row0 = nrow0;
    row1 = nrow1;
  }
  if (!ok && tid == 0) atomicAdd(&g_rgms_tc_timeouts, 1u);
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tmem, kF);
}


// ---------------------------------------------------------------------------------------------
// TMA-fed, warp-specialised form for the two-launch path (rows already aggregated in z).
// One persistent block per SM walks consecutive tiles; its 16 warps are four roles that hand
// tiles to each other through mbarriers, so loading, splitting, multiplying and scattering of
// different tiles overlap:
//   warp 0      producer: two TMA tile loads (128 rows x 128 bytes, 128-byte swizzle) bring the
//               tile's z rows into one of two stages;
//   warps 8-11  converters: the tensor core reads only the upper 19 bits of an fp32 operand, so
//               the raw tile serves as the "high" part as it is; the converters compute the
//               remainder z - tf32(z) element by element into a second buffer at the same
//               (swizzled) offsets, and stage W_r (raw and remainder) when the relation changes;
//   warp 1      issues the 8 K-steps of the 3xTF32 product as two instructions each (W and its
//               remainders stacked into one 128-row operand) into one of two TMEM accumulators
//               of 128 columns, tcgen05.commit frees the stage and publishes the accumulator;
//   warps 4-7, 12-15  epilogue (even / odd tiles): TMEM -> registers -> one padded half row of
//               shared memory per thread -> read back 8 lanes per row -> 16-byte vector atomics
//               into Y[I[t], :], four whole 128-byte lines per warp instruction.  (One bulk reduce-add per row, cp.reduce.async.bulk, was
//               measured first: the block issues a bulk operation only every ~20 clocks, which
//               made the epilogue the slowest role at 3,200 clocks per tile.)
// Every mbarrier wait is bounded.
constexpr int kPThreads = 512;
constexpr int kZStages = 2;
constexpr int kZBox = kTM * 128;     // one swizzled box: 128 rows x 32 floats
constexpr int kZTile = 2 * kZBox;    // 32 KB
// W_r as ONE operand of 128 rows: rows 0..63 = W (its upper 19 bits are what the tensor core
// reads), rows 64..127 = the remainders W - tf32(W); two boxes of 128 rows x 32 floats
constexpr int kWBox = 2 * kF * 128;  // 16 KB
constexpr int kWAll = 2 * kWBox;     // 32 KB
constexpr int kOutStride = 128 + 16;  // padded half row: 16-byte stores of 32 rows spread over all banks
constexpr int kOffZRaw = 0;
constexpr int kOffZLo = kOffZRaw + kZStages * kZTile;
constexpr int kOffW = kOffZLo + kZStages * kZTile;
constexpr int kOffOut = kOffW + kWAll;
constexpr int kPSmemBytes = kOffOut + 2 * kTM * kOutStride + 1024;  // two epilogue groups; + slack to align to 1024 bytes

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc05::smem_u32(bar)) : "memory");
}
// offset of 16-byte chunk `kc` (0..15) of row `row` in a tile stored as two 128-byte-swizzled boxes
__device__ __forceinline__ int swz_off(int row, int kc, int box_bytes) {
  return (kc >> 3) * box_bytes + (row >> 3) * 1024 + (row & 7) * 128 + (((kc & 7) ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(kPThreads, 1)
rgms_tma_kernel(const __grid_constant__ CUtensorMap tm_z, const float* __restrict__ w,
                float* __restrict__ y, const int32_t* __restrict__ indptr_i,
                const int32_t* __restrict__ indices_i, int num_rels, int nnz_i, int tiles_per_cta,
                int rel_mod) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kZStages];   // z rows of the stage have landed
  __shared__ __align__(8) uint64_t bar_conv[kZStages];   // remainders written (128 arrivals)
  __shared__ __align__(8) uint64_t bar_empty[kZStages];  // tensor core has read the stage
  __shared__ __align__(8) uint64_t bar_acc_full[2];      // accumulator holds a finished tile
  __shared__ __align__(8) uint64_t bar_acc_empty[2];     // epilogue has read it (128 arrivals)
  __shared__ uint32_t s_tmem;
  __shared__ int s_tile[4];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned char* base = smem_raw + ((1024u - (tc05::smem_u32(smem_raw) & 1023u)) & 1023u);

  if (warp == 0) {
    int rel, row0, row1;
    const bool found = locate_tile_warp(indptr_i, num_rels, blockIdx.x * tiles_per_cta, lane, &rel, &row0, &row1);
    if (lane == 0) {
      s_tile[0] = found ? 1 : 0; s_tile[1] = rel; s_tile[2] = row0; s_tile[3] = row1;
      for (int s = 0; s < kZStages; ++s) {
        tc05::mbar_init(&bar_full[s], 1);
        tc05::mbar_init(&bar_conv[s], 128);
        tc05::mbar_init(&bar_empty[s], 1);
      }
      for (int b = 0; b < 2; ++b) {
        tc05::mbar_init(&bar_acc_full[b], 1);
        tc05::mbar_init(&bar_acc_empty[b], 128);
      }
      tc05::fence_mbar_init();
      tc05::prefetch_tensormap(&tm_z);
    }
    __syncwarp();
    tc05::tmem_alloc(&s_tmem, 4 * kF);
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  if (s_tile[0] == 0) {  // no tile for this block (uniform)
    if (warp == 0) tc05::tmem_dealloc(s_tmem, 4 * kF);
    return;
  }
  const uint32_t tmem = s_tmem;
  TileWalk tw{s_tile[1], s_tile[2], s_tile[3], __ldg(indptr_i + s_tile[1] + 1)};
  bool ok = true;
  int armed = 0;

  if (warp == 0) {
    // ---- producer
    if (lane == 0) {
      for (int k = 0; k < tiles_per_cta; ++k) {
        const int s = k % kZStages, use = k / kZStages;
        if (use > 0 && !tc05::mbar_wait(&bar_empty[s], (use - 1) & 1)) { ok = false; break; }
        unsigned char* dst = base + kOffZRaw + s * kZTile;
        tc05::mbar_arrive_expect_tx(&bar_full[s], kZTile);
        tc05::tma_load_2d(dst, &tm_z, 0, tw.row0, &bar_full[s]);
        tc05::tma_load_2d(dst + kZBox, &tm_z, 32, tw.row0, &bar_full[s]);
        armed = k + 1;
        if (k + 1 == tiles_per_cta || !tw.next(indptr_i, num_rels)) break;
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      // Two instructions per K-step instead of three: z * [W; Wlo]^T (N = 128: columns 0..63
      // receive z*W, columns 64..127 z*Wlo) and zlo * W^T (N = 64, added to columns 0..63); the
      // epilogue adds the two column halves.  An MMA of this size costs about the same whatever
      // N <= 128, so the instruction count is what the issue warp is bound by.
      constexpr uint32_t idesc128 = tc05::instr_desc(tc05::kFmtTF32, kTM, 2 * kF, /*a_mn=*/0, /*b_mn=*/0);
      constexpr uint32_t idesc64 = tc05::instr_desc(tc05::kFmtTF32, kTM, kF, /*a_mn=*/0, /*b_mn=*/0);
      // descriptors are built once; the loop only advances their address fields (a lone thread
      // issues one dependent instruction every few clocks)
      const uint64_t dw0 = tc05::smem_desc_swizzled(tc05::smem_u32(base + kOffW), 0, 1024, tc05::kSwizzle128B);
      const uint64_t dzh0 = tc05::smem_desc_swizzled(tc05::smem_u32(base + kOffZRaw), 0, 1024, tc05::kSwizzle128B);
      const uint64_t dzl0 = tc05::smem_desc_swizzled(tc05::smem_u32(base + kOffZLo), 0, 1024, tc05::kSwizzle128B);
      for (int k = 0; k < tiles_per_cta; ++k) {
        const int s = k % kZStages, use = k / kZStages, buf = k & 1, buse = k >> 1;
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
        if (k + 1 == tiles_per_cta || !tw.next(indptr_i, num_rels)) break;
      }
    }
  } else if (warp >= 8 && warp < 12) {
    // ---- converters
    const int ct = tid - 256;
    int staged_rel = -1;
    for (int k = 0; k < tiles_per_cta; ++k) {
      const int s = k % kZStages, use = k / kZStages;
      // rel_mod > 0: the row ranges are (bucket, relation) pairs, W is indexed by the relation
      const int wrel = rel_mod > 0 ? tw.rel % rel_mod : tw.rel;
      if (wrel != staged_rel) {
        // the MMAs of the previous tile are the last readers of the staged W
        if (k > 0 && !tc05::mbar_wait(&bar_empty[(k - 1) % kZStages], ((k - 1) / kZStages) & 1)) { ok = false; break; }
        staged_rel = wrel;
        const float4* wr = reinterpret_cast<const float4*>(w + static_cast<size_t>(wrel) * kF * kF);
        for (int ch = ct; ch < kF * kF / 4; ch += 128) {
          const int fo = ch >> 4, kc = ch & 15;
          const float4 v = __ldg(wr + ch);
          const float4 l = make_float4(v.x - tf32_hi(v.x), v.y - tf32_hi(v.y), v.z - tf32_hi(v.z), v.w - tf32_hi(v.w));
          *reinterpret_cast<float4*>(base + kOffW + swz_off(fo, kc, kWBox)) = v;
          *reinterpret_cast<float4*>(base + kOffW + swz_off(kF + fo, kc, kWBox)) = l;
        }
      }
      if (!tc05::mbar_wait(&bar_full[s], use & 1)) { ok = false; break; }
      const unsigned char* zr = base + kOffZRaw + s * kZTile;
      unsigned char* zl = base + kOffZLo + s * kZTile;
#pragma unroll 4
      for (int j = 0; j < kZTile / 16 / 128; ++j) {
        const int off = (j * 128 + ct) * 16;
        const float4 v = *reinterpret_cast<const float4*>(zr + off);
        *reinterpret_cast<float4*>(zl + off) =
            make_float4(v.x - tf32_hi(v.x), v.y - tf32_hi(v.y), v.z - tf32_hi(v.z), v.w - tf32_hi(v.w));
      }
      tc05::fence_async_smem();
      mbar_arrive(&bar_conv[s]);
      if (k + 1 == tiles_per_cta || !tw.next(indptr_i, num_rels)) break;
    }
  } else if (warp >= 4) {
    // ---- epilogue, two groups of four warps: group 0 (warps 4-7) takes the even tiles and
    // accumulator 0, group 1 (warps 12-15) the odd tiles and accumulator 1, so that one group
    // reads TMEM and transposes while the other is busy issuing its atomics.
    // thread = tile row = TMEM lane
    const int grp = warp >= 12 ? 1 : 0;
    const int t = (warp & 3) * 32 + lane;
    unsigned char* gbuf = base + kOffOut + grp * (kTM * kOutStride);
    unsigned char* my_row = gbuf + t * kOutStride;
    const unsigned char* wbase = gbuf + (warp & 3) * 32 * kOutStride;
    bool have = true;
    if (grp == 1) have = tiles_per_cta > 1 && tw.next(indptr_i, num_rels);
    int nrows = tw.row1 - tw.row0;
    int dst_row = __ldg(indices_i + min(tw.row0 + t, nnz_i - 1));
    for (int k = grp; have && k < tiles_per_cta; k += 2) {
      const int buse = k >> 1;
      // destination rows of this group's next tile (two tiles on): requested now, needed later
      bool has_next = (k + 2 < tiles_per_cta) && tw.next(indptr_i, num_rels);
      has_next = has_next && tw.next(indptr_i, num_rels);
      const int dst_next = __ldg(indices_i + min(tw.row0 + t, nnz_i - 1));
      if (!tc05::mbar_wait(&bar_acc_full[grp], buse & 1)) { ok = false; break; }
      tc05::fence_after_sync();
      const uint32_t taddr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + grp * 2 * kF;
#pragma unroll
      for (int half = 0; half < 2; ++half) {  // 32 output columns at a time
        uint32_t r[32], r2[32];
        tc05::tmem_ld32(taddr + half * 32, r);            // z*W + zlo*W
        tc05::tmem_ld32(taddr + kF + half * 32, r2);      // z*Wlo
#pragma unroll
        for (int q = 0; q < 32; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) + __uint_as_float(r2[q]));
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
            atomicAdd(reinterpret_cast<float4*>(y + static_cast<size_t>(drow) * kF + half * 32) + (lane & 7), v);
          }
        }
      }
      if (!has_next) break;
      nrows = tw.row1 - tw.row0;  // tw already describes this group's next tile
      dst_row = dst_next;
    }
  }

  const bool all_ok = !__syncthreads_or(!ok);
  if (!all_ok && tid == 0) {
    atomicAdd(&g_rgms_tc_timeouts, 1u);
    // gave up: let the tile loads already issued land (bounded) before the block's memory is released
    for (int k = max(0, armed - kZStages); k < armed; ++k)
      tc05::mbar_wait(&bar_full[k % kZStages], (k / kZStages) & 1);
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tmem, 4 * kF);
}

// 0 when launched, 1 when this path cannot take the call (caller falls back), -1 on error
int rgms_tma_launch(const float* w, float* y, const int32_t* indptr_i, const int32_t* indices_i,
                    int num_rels, int nnz_i, const float* z, cudaStream_t stream, int rel_mod = 0) {
  if (nnz_i <= 0 || num_rels <= 0) return 1;
  if ((reinterpret_cast<uintptr_t>(z) & 15u) || (reinterpret_cast<uintptr_t>(y) & 15u) ||
      (reinterpret_cast<uintptr_t>(w) & 15u))
    return 1;
  CUtensorMap tm_z;
  if (make_tmap_2d(&tm_z, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, z, kF, static_cast<uint64_t>(nnz_i), kF * 4, 32,
                   kTM, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return 1;
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(rgms_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPSmemBytes));
    configured_device = dev;
  }
  const long long tiles = static_cast<long long>(nnz_i) / kTM + num_rels;  // upper bound
  const long long grid = tiles < kNumSMs ? tiles : kNumSMs;
  const int tiles_per_cta = static_cast<int>((tiles + grid - 1) / grid);
  rgms_tma_kernel<<<static_cast<unsigned>(grid), kPThreads, kPSmemBytes, stream>>>(
      tm_z, w, y, indptr_i, indices_i, num_rels, nnz_i, tiles_per_cta, rel_mod);
  SPTIR_LAUNCH_OK("rgms_tma_kernel");
  return 0;
}

}  // namespace

// The TMA-fed kernel over `num_ranges` row ranges of z (indptr_i) whose W is W[range % rel_mod]:
// several buckets' (bucket, relation) ranges in one launch.  0 when launched, 1 when this path
// cannot take the call, -1 on error.
int rgms_tma_launch_ranges(const float* w, float* y, const int32_t* indptr_i, const int32_t* indices_i,
                           int num_ranges, int rel_mod, int nnz_i, const float* z, cudaStream_t stream) {
  static const bool use_tma = [] {
    const char* e = std::getenv("SPARSETIR_RGMS_PATH");
    return !(e && std::strcmp(e, "regs") == 0);
  }();
  if (!use_tma) return 1;
  return rgms_tma_launch(w, y, indptr_i, indices_i, num_ranges, nnz_i, z, stream, rel_mod);
}

// Returns 0 when launched, 1 when the shape is not handled here, -1 on error.
// z: rows already aggregated by a preceding launch (two-kernel form), or nullptr (fused form).
int rgms_tc_launch(const float* a, const float* w, const float* x, float* y,
                   const int32_t* indptr_i, const int32_t* indices_i, const int32_t* indptr_j,
                   const int32_t* indices_j, int num_rels, int feat, int nnz_i,
                   const float* z, cudaStream_t stream) {
  if (feat != kF) return 1;
  // SPARSETIR_RGMS_PATH=regs keeps the tile on the load/store path (comparison switch)
  static const bool use_tma = [] {
    const char* e = std::getenv("SPARSETIR_RGMS_PATH");
    return !(e && std::strcmp(e, "regs") == 0);
  }();
  if (z != nullptr && use_tma) {
    const int rc = rgms_tma_launch(w, y, indptr_i, indices_i, num_rels, nnz_i, z, stream);
    if (rc <= 0) return rc;
  }
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(rgms_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kSmemBytes)));
    configured_device = dev;
  }
  // upper bound on the number of tiles: every relation can add one partly filled tile
  const long long tiles = static_cast<long long>(nnz_i) / kTM + num_rels;
  // two resident blocks per SM (shared memory), each walking a contiguous run of tiles
  const long long grid = tiles < 2ll * kNumSMs ? tiles : 2ll * kNumSMs;
  const int tiles_per_cta = static_cast<int>((tiles + grid - 1) / grid);
  rgms_tc_kernel<<<static_cast<unsigned>(grid), kRgmsThreads, kSmemBytes, stream>>>(
      a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, z, tiles_per_cta);
  SPTIR_LAUNCH_OK("rgms_tc_kernel");
  return 0;
}

int rgms_tc_timeouts(unsigned int* count) {
  SPTIR_CUDA_OK(cudaMemcpyFromSymbol(count, g_rgms_tc_timeouts, sizeof(unsigned int)));
  return 0;
}

}  // namespace sptir
