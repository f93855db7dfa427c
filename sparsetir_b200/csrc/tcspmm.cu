// Condensed tensor-core SpMM ("tcspmm"), fp16 operands, fp32 accumulation:
//   C[io*t + ii, f] = sum_{jo in [indptr[io], indptr[io+1])} sum_{ji < g} A[jo,ii,ji] * B[indices[jo*g+ji], f]
// Semantics: examples/spmm/bench_tc_spmm.py:537-565 of the reference (operator `tcspmm`; the
// wmma schedule it replaces: :591-640); the condensed operands come from ConDense
// (src/sparse/format.cc:353-429): every t-row tile keeps the sorted distinct columns it touches,
// g at a time; A holds the t x g values (mask) of a group, `indices` its g source rows.
//
// Tensor-core mapping (g = 16, t = 8, 16 or 32, feat a multiple of 128).  A group is a
// (t x 16) x (16 x F) product — far too short for M, so, as in the BSR kernel, it is computed
// transposed: one thread block owns (row tile io, 128 features),
//   D^T[f, ii] (128 x T, fp32 in TMEM)  +=  Bg^T[f, ji] (128 x 16)  *  A_jo[ii, ji]^T (16 x T)
// one tcgen05.mma.kind::f16 (M = 128 features, N = T tile rows, K = 16 slots) per group; T is t
// padded to 16 (the rows 8..15 of the A operand stay zero for t = 8).  The 16 gathered rows of B
// are the MN-major operand (features contiguous), the group's A block the K-major one.
// Operands travel global -> registers -> shared memory in the un-swizzled core-matrix layout
// (whole 128-byte lines per load, conflict-free 16-byte stores: see bsrmm_tc.cu); a thread
// keeps two groups in registers, three shared-memory stages, bounded mbarrier waits.
// Row tiles with many groups (hub rows) are cut into chunks of 32 groups handled by different
// thread blocks: a small planning kernel lists the extra chunks (and clears the output rows of
// those tiles), the main launch has one block per tile plus one per possible extra chunk, and
// the chunks of a cut tile add their partial results atomically.
// Other shapes run on CUDA cores.
#include <cuda_fp16.h>

#include "common.h"
#include "tc05.cuh"
#include "vec.cuh"

namespace sptir {

__device__ unsigned int g_tcspmm_timeouts = 0;

namespace {

constexpr int kThreads = 128;
constexpr int kG = 16;
constexpr int kTileF = 128;
constexpr int kStages = 3;
constexpr int kSets = 2;
constexpr int kBBytes = kG * kTileF * 2;   // gathered rows of one group: 16 x 128 fp16 = 4 KB
constexpr int kAMax = 32 * kG * 2;         // A block, T <= 32 rows: 1 KB
constexpr int kStageBytes = kBBytes + kAMax;
constexpr int kChunk = 32;                 // groups per thread block
constexpr int kIdxCache = kChunk * kG;     // source rows of the block's groups
// B operand (MN-major): core matrix (kc = ji/8, fc = f/8) at (kc*16 + fc)*128, slot ji%8 at
// 16-byte stride inside it, 8 features contiguous
constexpr uint32_t kB_SBO = 128, kB_LBO = 16 * 128;

template <typename OutT> __device__ __forceinline__ OutT to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ void add_out(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void add_out(__half* p, float v) { atomicAdd(p, __float2half_rn(v)); }

// Lists the chunks 1, 2, ... of every row tile with more than kChunk groups as (tile, chunk)
// pairs and clears the output rows of those tiles (their chunks accumulate atomically).
template <typename OutT>
__global__ void __launch_bounds__(256)
tcspmm_plan_kernel(const int32_t* __restrict__ indptr, int mb, int t, int feat, OutT* __restrict__ c,
                   int* __restrict__ count, int2* __restrict__ list, int max_extra) {
  const int io = blockIdx.x * 256 + threadIdx.x;
  int ngrp = 0;
  if (io < mb) ngrp = __ldg(indptr + io + 1) - __ldg(indptr + io);
  const bool heavy = ngrp > kChunk;
  if (heavy) {
    const int extra = (ngrp + kChunk - 1) / kChunk - 1;
    const int base = atomicAdd(count, extra);
    for (int k = 0; k < extra; ++k)
      if (base + k < max_extra) list[base + k] = make_int2(io, k + 1);
  }
  unsigned todo = __ballot_sync(0xffffffffu, heavy);
  const int lane = threadIdx.x & 31;
  while (todo != 0) {
    const int src = __ffs(todo) - 1;
    todo &= todo - 1;
    const int tile = __shfl_sync(0xffffffffu, io, src);
    OutT* dst = c + static_cast<size_t>(tile) * t * feat;
    for (int e = lane; e < t * feat; e += 32) dst[e] = to_out<OutT>(0.f);
  }
}

template <int T, typename OutT>  // T = tile rows padded to a multiple of 16
__global__ void __launch_bounds__(kThreads)
tcspmm_tc_kernel(const __half* __restrict__ a, const __half* __restrict__ b, OutT* __restrict__ c,
                 const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices, int t,
                 int feat, int mb, const int* __restrict__ count, const int2* __restrict__ list,
                 int max_extra) {
  __shared__ __align__(128) unsigned char smem[kStages * kStageBytes];
  __shared__ __align__(8) uint64_t bar_free[kStages];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t s_tmem;
  __shared__ int32_t s_idx[kIdxCache];
  // blocks 0..mb-1: chunk 0 of tile blockIdx.x; the others: an entry of the list of extra chunks
  int io = blockIdx.x, chunk = 0;
  if (io >= mb) {
    const int e = io - mb;
    if (e >= min(__ldg(count), max_extra)) return;
    const int2 w = list[e];
    io = w.x;
    chunk = w.y;
  }
  const int f0 = blockIdx.y * kTileF;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile_g0 = __ldg(indptr + io), tile_ngrp = __ldg(indptr + io + 1) - tile_g0;
  const bool accumulate = tile_ngrp > kChunk;  // the tile is cut: partial results are added
  const int g0 = tile_g0 + chunk * kChunk;
  const int ngrp = min(kChunk, tile_ngrp - chunk * kChunk);

  OutT* crow = c + (static_cast<size_t>(io) * t) * feat + f0 + warp * 32 + lane;
  if (ngrp <= 0) {  // empty tile: zeros, no tensor-core work
    for (int ii = 0; ii < t; ++ii) crow[static_cast<size_t>(ii) * feat] = to_out<OutT>(0.f);
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) tc05::mbar_init(&bar_free[s], 1);
    tc05::mbar_init(&bar_done, 1);
    tc05::fence_mbar_init();
  }
  if (warp == 0) tc05::tmem_alloc(&s_tmem, 32);
  for (int i = tid; i < min(ngrp * kG, kIdxCache); i += kThreads)
    s_idx[i] = __ldg(indices + static_cast<size_t>(g0) * kG + i);
  // rows t..T-1 of the A operand are never loaded: they must read as zero
  if (T != 0) {
    for (int i = tid; i < kStages * kAMax / 16; i += kThreads) {
      const int s = i / (kAMax / 16), r = i % (kAMax / 16);
      *reinterpret_cast<uint4*>(smem + s * kStageBytes + kBBytes + r * 16) = make_uint4(0, 0, 0, 0);
    }
  }
  tc05::fence_async_smem();
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = s_tmem;

  // B: a load instruction k (k = 0, 1) covers rows 4k..4k+3 (+8 for warps 2, 3) x 8 chunks of 16
  // bytes; store j writes the piece loaded by instruction j ^ (lane & 1) (see bsrmm_tc.cu)
  const int b_fc = (warp & 1) * 8 + (lane & 7);
  const int b_row0 = (warp >> 1) * 8 + (lane >> 3);
  const bool b_odd = (lane & 1) != 0;
  // A: piece p < 2t = (row ii = p / 2, 8-slot chunk kc = p % 2), 16 bytes
  const int a_ii = tid >> 1, a_kc = tid & 1;
  const bool a_mine = tid < 2 * t;
  struct Pieces {
    uint4 b[2];
    uint4 a;
  };
  auto load_group = [&](int it, Pieces& x) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int slot = it * kG + b_row0 + k * 4;
      const int src = s_idx[slot];
      x.b[k] = __ldg(reinterpret_cast<const uint4*>(b + static_cast<size_t>(src) * feat + f0 + b_fc * 8));
    }
    if (a_mine)
      x.a = __ldg(reinterpret_cast<const uint4*>(a + (static_cast<size_t>(g0 + it) * t + a_ii) * kG + a_kc * 8));
  };
  auto store_group = [&](int stage, const Pieces& x) {
    unsigned char* st = smem + stage * kStageBytes;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint4 v = b_odd ? x.b[j ^ 1] : x.b[j];
      const int row = b_row0 + (b_odd ? (j ^ 1) : j) * 4;  // slot ji of the piece
      *reinterpret_cast<uint4*>(st + ((row >> 3) * 16 + b_fc) * 128 + (row & 7) * 16) = v;
    }
    // A operand (K-major): core matrix (kc, ng = ii/8) at (kc*(T/8) + ng)*128, row ii%8 at 16 bytes
    if (a_mine)
      *reinterpret_cast<uint4*>(st + kBBytes + (a_kc * (T / 8) + (a_ii >> 3)) * 128 + (a_ii & 7) * 16) = x.a;
  };

  constexpr uint32_t idesc = tc05::instr_desc(tc05::kFmtF16, kTileF, T, /*a_mn=*/1, /*b_mn=*/0);
  const uint64_t da0 = tc05::smem_desc(tc05::smem_u32(smem), kB_LBO, kB_SBO);
  const uint64_t db0 = tc05::smem_desc(tc05::smem_u32(smem) + kBBytes, (T / 8) * 128, 128);
  bool ok = true;
  auto step = [&](int it, Pieces& x) -> bool {
    const int stage = it % kStages;
    if (it >= kStages) {  // the MMA of group it-kStages was the previous reader of this stage
      if (!tc05::mbar_wait(&bar_free[stage], ((it - kStages) / kStages) & 1)) ok = false;
    }
    if (ok) store_group(stage, x);
    if (it + kSets < ngrp) load_group(it + kSets, x);
    tc05::fence_async_smem();
    if (__syncthreads_or(!ok)) return false;
    if (warp == 0 && lane == 0) {
      tc05::fence_after_sync();
      tc05::mma_f16(tmem, tc05::desc_advance(da0, stage * kStageBytes),
                    tc05::desc_advance(db0, stage * kStageBytes), idesc, it > 0 ? 1u : 0u);
      tc05::mma_commit(&bar_free[stage]);
      if (it == ngrp - 1) tc05::mma_commit(&bar_done);
    }
    return true;
  };

  Pieces x[kSets];
#pragma unroll
  for (int k = 0; k < kSets; ++k) {
    x[k].a = make_uint4(0, 0, 0, 0);
    if (k < ngrp) load_group(k, x[k]);
  }
  for (int it = 0; it < ngrp && ok; it += kSets) {
#pragma unroll
    for (int k = 0; k < kSets; ++k)
      if (ok && it + k < ngrp && !step(it + k, x[k])) ok = false;  // uniform: ends in a barrier vote
  }

  if (ok && !tc05::mbar_wait(&bar_done, 0)) ok = false;
  ok = !__syncthreads_or(!ok);
  tc05::fence_after_sync();
  if (ok) {
    uint32_t r[32];
    tc05::tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16), r);  // columns >= T: unused
#pragma unroll
    for (int ii = 0; ii < T; ++ii) {
      if (ii < t) {
        if (accumulate) add_out(crow + static_cast<size_t>(ii) * feat, __uint_as_float(r[ii]));
        else crow[static_cast<size_t>(ii) * feat] = to_out<OutT>(__uint_as_float(r[ii]));
      }
    }
  } else if (tid == 0) {
    atomicAdd(&g_tcspmm_timeouts, 1u);
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tmem, 32);
}

// CUDA-core form for every other shape: a block per row tile; a thread owns output elements
// (ii, f) and walks the groups.
template <typename OutT>
__global__ void __launch_bounds__(256)
tcspmm_simt_kernel(const __half* __restrict__ a, const __half* __restrict__ b, OutT* __restrict__ c,
                   const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices, int t,
                   int g, int feat) {
  const int io = blockIdx.x;
  const int g0 = __ldg(indptr + io), g1 = __ldg(indptr + io + 1);
  for (int e = threadIdx.x; e < t * feat; e += blockDim.x) {
    const int ii = e / feat, f = e % feat;
    float acc = 0.f;
    for (int jo = g0; jo < g1; ++jo) {
      const __half* ar = a + (static_cast<size_t>(jo) * t + ii) * g;
      const int32_t* ix = indices + static_cast<size_t>(jo) * g;
      for (int ji = 0; ji < g; ++ji) {
        const float av = __half2float(__ldg(ar + ji));
        if (av != 0.f) acc = fmaf(av, __half2float(__ldg(b + static_cast<size_t>(__ldg(ix + ji)) * feat + f)), acc);
      }
    }
    c[(static_cast<size_t>(io) * t + ii) * feat + f] = to_out<OutT>(acc);
  }
}

template <typename OutT>
int launch_all(const __half* a, const __half* b, OutT* c, const int32_t* indptr, const int32_t* indices,
               int mb, int nnzb, int t, int g, int feat, int device_id, cudaStream_t st) {
  const bool tc = g == kG && (t == 8 || t == 16 || t == 32) && feat % kTileF == 0 &&
                  feat / kTileF <= 65535 && aligned16(a) && aligned16(b);
  if (tc) {
    // work list of the extra chunks of cut tiles: at most nnzb / kChunk entries
    const int max_extra = nnzb / kChunk + 1;
    char* ws = static_cast<char*>(workspace(device_id, st, 16 + static_cast<size_t>(max_extra) * sizeof(int2)));
    if (!ws) return -1;
    int* count = reinterpret_cast<int*>(ws);
    int2* list = reinterpret_cast<int2*>(ws + 16);
    SPTIR_CUDA_OK(cudaMemsetAsync(count, 0, sizeof(int), st));
    tcspmm_plan_kernel<OutT><<<ceil_div(mb, 256), 256, 0, st>>>(indptr, mb, t, feat, c, count, list, max_extra);
    SPTIR_LAUNCH_OK("tcspmm_plan_kernel");
    if (static_cast<long long>(mb) + max_extra > INT32_MAX) return fail("sparsetir_tcspmm: too many thread blocks");
    dim3 grid(mb + max_extra, feat / kTileF);
    if (t <= 16)
      tcspmm_tc_kernel<16, OutT><<<grid, kThreads, 0, st>>>(a, b, c, indptr, indices, t, feat, mb, count, list, max_extra);
    else
      tcspmm_tc_kernel<32, OutT><<<grid, kThreads, 0, st>>>(a, b, c, indptr, indices, t, feat, mb, count, list, max_extra);
    SPTIR_LAUNCH_OK("tcspmm_tc_kernel");
    return 0;
  }
  tcspmm_simt_kernel<OutT><<<mb, 256, 0, st>>>(a, b, c, indptr, indices, t, g, feat);
  SPTIR_LAUNCH_OK("tcspmm_simt_kernel");
  return 0;
}

}  // namespace

int tcspmm_timeouts(unsigned int* count) {
  SPTIR_CUDA_OK(cudaMemcpyFromSymbol(count, g_tcspmm_timeouts, sizeof(unsigned int)));
  return 0;
}

}  // namespace sptir

extern "C" int sparsetir_tcspmm_raw(const void* a_f16, const void* b_f16, void* c, int c_is_f16,
                                    const int32_t* indptr, const int32_t* indices, int mb, int nb,
                                    int nnzb, int feat, int tile_size, int group_size, int device_id,
                                    void* stream) {
  using namespace sptir;
  (void)nb;
  if (mb < 0 || nnzb < 0 || feat < 0 || tile_size < 1 || group_size < 1)
    return fail("sparsetir_tcspmm: invalid size");
  if (mb == 0 || feat == 0) return 0;
  if (!c || !indptr || (nnzb > 0 && (!a_f16 || !b_f16 || !indices)))
    return fail("sparsetir_tcspmm: null pointer argument");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half* a = static_cast<const __half*>(a_f16);
  const __half* b = static_cast<const __half*>(b_f16);
  if (c_is_f16)
    return launch_all<__half>(a, b, static_cast<__half*>(c), indptr, indices, mb, nnzb, tile_size, group_size, feat,
                              device_id, st);
  return launch_all<float>(a, b, static_cast<float*>(c), indptr, indices, mb, nnzb, tile_size, group_size, feat,
                           device_id, st);
}
