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
#include "tc05.cuh"

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

}  // namespace

// Returns 0 when launched, 1 when the shape is not handled here, -1 on error.
// z: rows already aggregated by a preceding launch (two-kernel form), or nullptr (fused form).
int rgms_tc_launch(const float* a, const float* w, const float* x, float* y,
                   const int32_t* indptr_i, const int32_t* indices_i, const int32_t* indptr_j,
                   const int32_t* indices_j, int num_rels, int feat, int nnz_i,
                   const float* z, cudaStream_t stream) {
  if (feat != kF) return 1;
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
