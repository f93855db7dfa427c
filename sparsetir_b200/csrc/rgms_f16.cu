// RGMS over ELL3D buckets with half-precision operands and rectangular weights:
//   for every bucket b, group g (relation r = mid_b[g]), row slot ii, column slot j
//     Y[rows_b[g,ii], fo] += A_b[g,ii,j] * sum_fi X[cols_b[g,ii,j], fi] * W[r, fi, fo]
// X is n x feat_in, W is num_rels x feat_in x feat_out, both fp16; Y is m x feat_out, fp16 or fp32;
// products are accumulated in fp32.  Replaces the kernel the reference builds from
// rgcn_hetero_forward with its ELL3D decomposition and tensor-core intrinsics
// (examples/rgms/rgcn/bench_rgcn_tensorcore.py:564-609 the computation, :651-858 schedule, buffers
// and argument list W, X, Y, {mask, rows, cols} per bucket, {mid} per bucket), which is also what
// the sparse convolution driver calls with one relation per kernel offset and buckets = [1]
// (examples/rgms/sparse_conv/sparse_conv.py:93-125).
//
// Two launches whatever the number of buckets (one when there is a single bucket with one column
// per row, see rgms_f16_tc_kernel<OutT, true>):
//   (1) Z[q, :] = sum_j A[q,j] X[cols[q,j], :] for every ELL row q of every bucket (fp32 sums,
//       stored as fp16), the buckets' rows one after the other in one Z array; the same launch
//       copies the row ids next to each other and turns the ascending `mid` arrays into the Z-row
//       range of every (bucket, relation) pair;
//   (2) Y[rows[q], :] += Z[q, :] W_r over those ranges: a persistent tcgen05 kernel, one tile =
//       128 Z rows of one range.  A producer warp streams, per 64-wide slice of feat_in, the Z
//       box (128 x 64, K-major, 128-byte swizzle) and the matching 64 x feat_out slice of W_r
//       (N-major boxes of 64 x 64) through a 3-stage ring with TMA; one thread issues 4 MMAs
//       (M = 128, N = feat_out, K = 16) per slice into one of two TMEM accumulators; two groups
//       of four warps take the even / odd tiles out of TMEM and add them to Y.
// A single one-column bucket whose (relation, destination) pairs never repeat and whose values
// are 0 / 1 can also be computed destination-stationary, without reductions (rgms_f16_os_kernel).
// Shapes the tensor-core launch does not take (feat_in or feat_out not a multiple of 64, feat_out
// above 256, unaligned operands) go through a CUDA-core transform with the same Z.
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "common.h"
#include "rgms_common.cuh"
#include "tc05.cuh"
#include "tmap.h"

namespace sptir {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxBuckets = SPARSETIR_HYB_MAX_BUCKETS;

__device__ unsigned int g_rgms_f16_timeouts = 0;

struct BucketTable {
  const __half* a[kMaxBuckets];
  const int32_t* cols[kMaxBuckets];
  const int32_t* rows[kMaxBuckets];
  const int32_t* mid[kMaxBuckets];
  int32_t num_groups[kMaxBuckets];
  int32_t rows_per_group[kMaxBuckets];
  int32_t width[kMaxBuckets];
  int32_t z_base[kMaxBuckets + 1];  // first Z row of every bucket; [nb] = total rows
  int32_t nb;
};

__device__ __forceinline__ int bucket_of(const BucketTable& tb, int q) {
  int b = 0;
  while (b + 1 < tb.nb && q >= tb.z_base[b + 1]) ++b;
  return b;
}

// ---- launch (1).  A thread owns VEC consecutive features of one Z row; consecutive threads own
// consecutive pieces of the same row.  The last block computes the (bucket, relation) ranges:
// ranges[b * R + r] = first Z row of relation r inside bucket b, ranges[nb * R] = total rows.
template <int VEC>
__global__ void __launch_bounds__(kThreads)
gather_rows_f16_kernel(const __grid_constant__ BucketTable tb, const __half* __restrict__ x,
                       __half* __restrict__ z, int32_t* __restrict__ all_rows,
                       int32_t* __restrict__ ranges, int num_rels, int feat_in) {
  if (blockIdx.x == gridDim.x - 1) {
    for (int e = threadIdx.x; e <= tb.nb * num_rels; e += kThreads) {
      if (e == tb.nb * num_rels) {
        ranges[e] = tb.z_base[tb.nb];
        continue;
      }
      const int b = e / num_rels, r = e % num_rels;
      int lo = 0, hi = tb.num_groups[b];  // first group of the bucket with mid >= r
      while (lo < hi) {
        const int m = lo + (hi - lo) / 2;
        if (__ldg(tb.mid[b] + m) < r) lo = m + 1; else hi = m;
      }
      ranges[e] = tb.z_base[b] + lo * tb.rows_per_group[b];
    }
    return;
  }
  // a block walks tiles of kThreads / chunks consecutive rows; 32-bit index arithmetic only
  const int chunks = feat_in / VEC;
  const int rows_per_tile = max(1, kThreads / chunks);
  const int total = tb.z_base[tb.nb];
  const int rl = static_cast<int>(threadIdx.x) / chunks, ch = static_cast<int>(threadIdx.x) % chunks;
  if (rl >= rows_per_tile && chunks <= kThreads) return;
  for (long long row0 = static_cast<long long>(blockIdx.x) * rows_per_tile; row0 < total;
       row0 += static_cast<long long>(gridDim.x - 1) * rows_per_tile) {
   for (int c0 = ch; c0 < chunks; c0 += kThreads) {  // more pieces than threads: rows of > 2048 features
    const int ch = c0;
    if (row0 + rl >= total) continue;
    const int q = static_cast<int>(row0) + rl;
    const int b = bucket_of(tb, q);
    const int e = q - tb.z_base[b], width = tb.width[b];
    const __half* ap = tb.a[b] + static_cast<size_t>(e) * width;
    const int32_t* cp = tb.cols[b] + static_cast<size_t>(e) * width;
    __half* zr = z + static_cast<size_t>(q) * feat_in + ch * VEC;
    if (ch == 0) all_rows[q] = __ldg(tb.rows[b] + e);
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
#pragma unroll 4
    for (int j = 0; j < width; ++j) {
      const float av = __half2float(__ldg(ap + j));
      const __half* xr = x + static_cast<size_t>(__ldg(cp + j)) * feat_in + ch * VEC;
      if (VEC == 8) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xr));
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float2 f = __half22float2(h[v]);
          acc[2 * v] = fmaf(av, f.x, acc[2 * v]);
          acc[2 * v + 1] = fmaf(av, f.y, acc[2 * v + 1]);
        }
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = fmaf(av, __half2float(__ldg(xr + v)), acc[v]);
      }
    }
    if (VEC == 8) {
      uint4 out;
      __half2* h = reinterpret_cast<__half2*>(&out);
#pragma unroll
      for (int v = 0; v < 4; ++v) h[v] = __floats2half2_rn(acc[2 * v], acc[2 * v + 1]);
      *reinterpret_cast<uint4*>(zr) = out;
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) zr[v] = __float2half_rn(acc[v]);
    }
   }
  }
}

// ---- launch (1) when every bucket has one column per row (the sparse-convolution shape): the Z
// row is the X row times one value.  A thread owns one 16-byte piece of R rows that lie
// kThreads / chunks rows apart and keeps the R chains (value, column id -> X row) in flight
// together.  Same outputs as gather_rows_f16_kernel.
constexpr int kCopyR = 4;
__global__ void __launch_bounds__(kThreads)
scale_rows_f16_kernel(const __grid_constant__ BucketTable tb, const __half* __restrict__ x,
                      __half* __restrict__ z, int32_t* __restrict__ all_rows,
                      int32_t* __restrict__ ranges, int num_rels, int feat_in) {
  if (blockIdx.x == gridDim.x - 1) {
    for (int e = threadIdx.x; e <= tb.nb * num_rels; e += kThreads) {
      if (e == tb.nb * num_rels) {
        ranges[e] = tb.z_base[tb.nb];
        continue;
      }
      const int b = e / num_rels, r = e % num_rels;
      int lo = 0, hi = tb.num_groups[b];
      while (lo < hi) {
        const int m = lo + (hi - lo) / 2;
        if (__ldg(tb.mid[b] + m) < r) lo = m + 1; else hi = m;
      }
      ranges[e] = tb.z_base[b] + lo * tb.rows_per_group[b];
    }
    return;
  }
  const int chunks = feat_in / 8;                     // <= kThreads (checked by the caller)
  const int rows_per_pass = kThreads / chunks;
  const int total = tb.z_base[tb.nb];
  const int rl = static_cast<int>(threadIdx.x) / chunks, ch = static_cast<int>(threadIdx.x) % chunks;
  if (rl >= rows_per_pass) return;
  for (long long row0 = static_cast<long long>(blockIdx.x) * rows_per_pass * kCopyR; row0 < total;
       row0 += static_cast<long long>(gridDim.x - 1) * rows_per_pass * kCopyR) {
    float av[kCopyR];
    int col[kCopyR], q[kCopyR];
#pragma unroll
    for (int r = 0; r < kCopyR; ++r) {
      const long long row = row0 + r * rows_per_pass + rl;
      q[r] = row < total ? static_cast<int>(row) : -1;
      av[r] = 0.f;
      col[r] = 0;
      if (q[r] >= 0) {
        const int b = bucket_of(tb, q[r]);
        const int e = q[r] - tb.z_base[b];
        av[r] = __half2float(__ldg(tb.a[b] + e));
        col[r] = __ldg(tb.cols[b] + e);
        if (ch == 0) all_rows[q[r]] = __ldg(tb.rows[b] + e);
      }
    }
    uint4 raw[kCopyR];
#pragma unroll
    for (int r = 0; r < kCopyR; ++r)
      raw[r] = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(col[r]) * feat_in) + ch);
#pragma unroll
    for (int r = 0; r < kCopyR; ++r) {
      if (q[r] < 0) continue;
      if (av[r] != 1.f) {
        __half2* h = reinterpret_cast<__half2*>(&raw[r]);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float2 f = __half22float2(h[v]);
          h[v] = __floats2half2_rn(av[r] * f.x, av[r] * f.y);
        }
      }
      *(reinterpret_cast<uint4*>(z + static_cast<size_t>(q[r]) * feat_in) + ch) = raw[r];
    }
  }
}

// ---- additions to Y
__device__ __forceinline__ void add_out(float* y, float v) { atomicAdd(y, v); }
__device__ __forceinline__ void add_out(__half* y, float v) { atomicAdd(y, __float2half_rn(v)); }
// 4 consecutive outputs of one row (destination aligned to 4 elements)
__device__ __forceinline__ void add_out4(float* y, const float4& v) { atomicAdd(reinterpret_cast<float4*>(y), v); }
// 8 consecutive float16 outputs of one row (16-byte aligned destination): one vector reduction
__device__ __forceinline__ void add_out8(__half* y, const float4& a, const float4& b) {
  const __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w);
  const __half2 h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
  asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(y),
               "r"(*reinterpret_cast<const uint32_t*>(&h0)), "r"(*reinterpret_cast<const uint32_t*>(&h1)),
               "r"(*reinterpret_cast<const uint32_t*>(&h2)), "r"(*reinterpret_cast<const uint32_t*>(&h3))
               : "memory");
}
// the 32 staged columns of the warp's rows go to Y: 8 lanes x 16 bytes per row for a float32 Y,
// 4 lanes x 16 bytes per row for a float16 Y
__device__ __forceinline__ void scatter32(float* y, const unsigned char* wbase, int stride, int dst_row, int row_base,
                                          int nrows, int feat_out, int c0, int lane) {
#pragma unroll 4
  for (int i = 0; i < 8; ++i) {
    const int lr = 4 * i + (lane >> 3);  // row inside the warp's 32
    const int drow = __shfl_sync(0xffffffffu, dst_row, lr);
    if (row_base + lr < nrows) {
      const float4 v = *reinterpret_cast<const float4*>(wbase + lr * stride + (lane & 7) * 16);
      add_out4(y + static_cast<size_t>(drow) * feat_out + c0 + (lane & 7) * 4, v);
    }
  }
}
__device__ __forceinline__ void scatter32(__half* y, const unsigned char* wbase, int stride, int dst_row, int row_base,
                                          int nrows, int feat_out, int c0, int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = 8 * i + (lane >> 2);
    const int drow = __shfl_sync(0xffffffffu, dst_row, lr);
    if (row_base + lr < nrows) {
      const float4 a = *reinterpret_cast<const float4*>(wbase + lr * stride + (lane & 3) * 32);
      const float4 b = *reinterpret_cast<const float4*>(wbase + lr * stride + (lane & 3) * 32 + 16);
      add_out8(y + static_cast<size_t>(drow) * feat_out + c0 + (lane & 3) * 8, a, b);
    }
  }
}

// ---- CUDA-core form of launch (2): a block owns 32 consecutive Z rows (staged in shared memory
// as fp32); a thread computes outputs (row, fo), consecutive threads consecutive fo.
constexpr int kSimtRows = 32;
template <typename OutT>
__global__ void __launch_bounds__(kThreads)
transform_scatter_f16_kernel(const __grid_constant__ BucketTable tb, const __half* __restrict__ z,
                             const __half* __restrict__ w, OutT* __restrict__ y,
                             const int32_t* __restrict__ all_rows, int feat_in, int feat_out) {
  extern __shared__ float s_z[];  // kSimtRows x feat_in
  __shared__ int s_rel[kSimtRows];
  const int total = tb.z_base[tb.nb];
  const int q0 = blockIdx.x * kSimtRows;
  const int nq = min(kSimtRows, total - q0);
  for (int i = threadIdx.x; i < nq * feat_in; i += kThreads)
    s_z[i] = __half2float(__ldg(z + static_cast<size_t>(q0) * feat_in + i));
  if (threadIdx.x < nq) {
    const int q = q0 + threadIdx.x;
    const int b = bucket_of(tb, q);
    s_rel[threadIdx.x] = __ldg(tb.mid[b] + (q - tb.z_base[b]) / tb.rows_per_group[b]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nq * feat_out; i += kThreads) {
    const int t = i / feat_out, fo = i % feat_out;
    const __half* wr = w + static_cast<size_t>(s_rel[t]) * feat_in * feat_out + fo;
    const float* zr = s_z + t * feat_in;
    float acc = 0.f;
    for (int fi = 0; fi < feat_in; ++fi)
      acc = fmaf(zr[fi], __half2float(__ldg(wr + static_cast<size_t>(fi) * feat_out)), acc);
    add_out(y + static_cast<size_t>(__ldg(all_rows + q0 + t)) * feat_out + fo, acc);
  }
}

// ---- tensor-core form of launch (2)
constexpr int kTM = kTileRows128;
constexpr int kKC = 64;                       // slice of feat_in per stage (one 128-byte swizzled row)
constexpr int kZBoxB = kTM * kKC * 2;         // 16 KB
constexpr int kWBoxB = kKC * 64 * 2;          // 8 KB: 64 K rows x 64 outputs
constexpr int kMaxOut = 256;
constexpr int kStageB = kZBoxB + (kMaxOut / 64) * kWBoxB;  // 48 KB
constexpr int kStagesH = 3;
constexpr int kOutStride = 128 + 16;          // padded row of 32 floats: 16-byte stores of 32 rows spread over all banks
constexpr int kOffOut = kStagesH * kStageB;
constexpr int kSmemH = kOffOut + 2 * kTM * kOutStride + 1024;  // two epilogue groups; + slack to align to 1024 bytes
constexpr int kTcThreads = 384;               // warp 0 loads, warp 1 MMAs, warps 4-7 / 8-11 epilogue
constexpr int kTcThreadsG = 512;              // ... and warps 12-15 gather X rows (one-launch form)

__device__ __forceinline__ void mbar_arrive_local(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc05::smem_u32(bar)) : "memory");
}

// GATHER = true is the one-launch form for a single bucket with one column per row (the
// sparse-convolution shape): there is no Z array; four more warps copy the tile's X rows
// (row t of the tile = X[gcols[row0 + t]]) straight into the swizzled stage with 16-byte
// asynchronous copies, 8 lanes per 128-byte row slice, and the row's value gvals[row0 + t]
// multiplies the finished row in the epilogue.
template <typename OutT, bool GATHER>
__global__ void __launch_bounds__(GATHER ? kTcThreadsG : kTcThreads, 1)
rgms_f16_tc_kernel(const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_w,
                   OutT* __restrict__ y, const int32_t* __restrict__ ranges,
                   const int32_t* __restrict__ all_rows, int num_ranges, int num_rels, int total_rows,
                   int tiles_per_cta, int feat_in, int feat_out, int tmem_cols,
                   const __half* __restrict__ x, const int32_t* __restrict__ gcols,
                   const __half* __restrict__ gvals, const int32_t* __restrict__ run_if_set) {
  // run_if_set != nullptr: this launch is the fall-back of the reduction-free form and runs only
  // when that form found the input unsuitable (flag set on the device)
  if (run_if_set != nullptr && __ldg(run_if_set) == -1) return;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStagesH];   // the stage's boxes have landed
  __shared__ __align__(8) uint64_t bar_empty[kStagesH];  // the tensor core has read the stage
  __shared__ __align__(8) uint64_t bar_acc_full[2];      // accumulator holds a finished tile
  __shared__ __align__(8) uint64_t bar_acc_empty[2];     // epilogue has read it (128 arrivals)
  __shared__ uint32_t s_tmem;
  __shared__ int s_tile[4];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned char* base = smem_raw + ((1024u - (tc05::smem_u32(smem_raw) & 1023u)) & 1023u);
  const int nkc = feat_in / kKC, nwb = feat_out / 64;

  if (warp == 0) {
    int rel, row0, row1;
    const bool found = locate_tile_warp(ranges, num_ranges, blockIdx.x * tiles_per_cta, lane, &rel, &row0, &row1);
    if (lane == 0) {
      s_tile[0] = found ? 1 : 0; s_tile[1] = rel; s_tile[2] = row0; s_tile[3] = row1;
      for (int s = 0; s < kStagesH; ++s) {
        tc05::mbar_init(&bar_full[s], GATHER ? 1 + 128 : 1);  // the W boxes (+ the 128 gathering threads)
        tc05::mbar_init(&bar_empty[s], 1);
      }
      for (int b = 0; b < 2; ++b) {
        tc05::mbar_init(&bar_acc_full[b], 1);
        tc05::mbar_init(&bar_acc_empty[b], 128);
      }
      tc05::fence_mbar_init();
      if (!GATHER) tc05::prefetch_tensormap(&tm_z);
      tc05::prefetch_tensormap(&tm_w);
    }
    __syncwarp();
    tc05::tmem_alloc(&s_tmem, tmem_cols);
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  if (s_tile[0] == 0) {  // no tile for this block (uniform)
    if (warp == 0) tc05::tmem_dealloc(s_tmem, tmem_cols);
    return;
  }
  const uint32_t tmem = s_tmem;
  TileWalk tw{s_tile[1], s_tile[2], s_tile[3], __ldg(ranges + s_tile[1] + 1)};
  bool ok = true;
  int armed = 0;  // producer: stages whose loads have been issued

  if (warp == 0) {
    // ---- producer
    if (lane == 0) {
      int it = 0;
      const uint32_t stage_bytes = (GATHER ? 0 : kZBoxB) + nwb * kWBoxB;
      for (int k = 0; k < tiles_per_cta && ok; ++k) {
        const int wrow = (tw.rel % num_rels) * feat_in;
        for (int c = 0; c < nkc; ++c, ++it) {
          const int s = it % kStagesH, use = it / kStagesH;
          if (use > 0 && !tc05::mbar_wait(&bar_empty[s], (use - 1) & 1)) { ok = false; break; }
          unsigned char* st = base + s * kStageB;
          tc05::mbar_arrive_expect_tx(&bar_full[s], stage_bytes);
          if (!GATHER) tc05::tma_load_2d(st, &tm_z, c * kKC, tw.row0, &bar_full[s]);
          for (int j = 0; j < nwb; ++j)
            tc05::tma_load_2d(st + kZBoxB + j * kWBoxB, &tm_w, j * 64, wrow + c * kKC, &bar_full[s]);
          armed = it + 1;
        }
        if (k + 1 == tiles_per_cta || !tw.next(ranges, num_ranges)) break;
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = tc05::instr_desc(tc05::kFmtF16, kTM, feat_out, /*a_mn=*/0, /*b_mn=*/1);
      // Z box, K-major: rows of 128 bytes, groups of 8 rows 1024 bytes apart; 16 columns = 32 bytes per step
      const uint64_t dz0 = tc05::smem_desc_swizzled(tc05::smem_u32(base), 0, 1024, tc05::kSwizzle128B);
      // W boxes, N-major: 64 outputs per 128-byte row, boxes (atoms of 64 outputs) kWBoxB apart,
      // groups of 8 K rows 1024 bytes apart; 16 K rows = 2048 bytes per step
      const uint64_t dw0 = tc05::smem_desc_swizzled(tc05::smem_u32(base) + kZBoxB, kWBoxB, 1024, tc05::kSwizzle128B);
      int it = 0;
      for (int k = 0; k < tiles_per_cta && ok; ++k) {
        const int buf = k & 1, buse = k >> 1;
        if (buse > 0 && !tc05::mbar_wait(&bar_acc_empty[buf], (buse - 1) & 1)) { ok = false; break; }
        const uint32_t acc = tmem + buf * feat_out;
        for (int c = 0; c < nkc; ++c, ++it) {
          const int s = it % kStagesH, use = it / kStagesH;
          if (!tc05::mbar_wait(&bar_full[s], use & 1)) { ok = false; break; }
          tc05::fence_after_sync();
          const uint64_t dz = tc05::desc_advance(dz0, s * kStageB);
          const uint64_t dw = tc05::desc_advance(dw0, s * kStageB);
#pragma unroll
          for (int ks = 0; ks < kKC / 16; ++ks)
            tc05::mma_f16(acc, tc05::desc_advance(dz, ks * 32), tc05::desc_advance(dw, ks * 2048), idesc,
                          (c > 0 || ks > 0) ? 1u : 0u);
          tc05::mma_commit(&bar_empty[s]);
        }
        if (!ok) break;
        tc05::mma_commit(&bar_acc_full[buf]);
        if (k + 1 == tiles_per_cta || !tw.next(ranges, num_ranges)) break;
      }
    }
  } else if (GATHER && warp >= 12) {
    // ---- gather warps: warp gw copies rows gw*32 .. gw*32+31 of the tile.  A stage is announced
    // one step late: after the next stage's copies have been issued, wait for all but those,
    // make the data visible to the tensor core's proxy, arrive.
    const int gw = warp - 12;
    int it = 0, pending = -1;
    for (int k = 0; k < tiles_per_cta && ok; ++k) {
      const int mycol = __ldg(gcols + min(tw.row0 + gw * 32 + lane, total_rows - 1));
      for (int c = 0; c < nkc; ++c, ++it) {
        const int s = it % kStagesH, use = it / kStagesH;
        if (use > 0 && !tc05::mbar_wait(&bar_empty[s], (use - 1) & 1)) { ok = false; break; }
        const uint32_t st = tc05::smem_u32(base + s * kStageB);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int lr = 4 * i + (lane >> 3);  // row inside the warp's 32
          const int col = __shfl_sync(0xffffffffu, mycol, lr);
          const int row = gw * 32 + lr, chunk = lane & 7;
          const __half* src = x + static_cast<size_t>(col) * feat_in + c * kKC + chunk * 8;
          const uint32_t dst = st + (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (pending >= 0) {
          asm volatile("cp.async.wait_group 1;" ::: "memory");
          tc05::fence_async_smem();
          mbar_arrive_local(&bar_full[pending]);
        }
        pending = s;
      }
      if (k + 1 == tiles_per_cta || !tw.next(ranges, num_ranges)) break;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // also when giving up: nothing may land later
    if (ok && pending >= 0) {
      tc05::fence_async_smem();
      mbar_arrive_local(&bar_full[pending]);
    }
  } else if (warp >= 4 && warp < 12) {
    // ---- epilogue: group 0 (warps 4-7) takes the even tiles and accumulator 0, group 1 (warps
    // 8-11) the odd ones; thread = tile row = TMEM lane.  32 columns at a time go through a
    // padded shared-memory buffer so that 8 lanes add one row's 128 bytes (whole lines per
    // request instead of 32 rows x 16 bytes).
    const int grp = warp >= 8 ? 1 : 0;
    const int t = (warp & 3) * 32 + lane;
    unsigned char* gbuf = base + kOffOut + grp * (kTM * kOutStride);
    unsigned char* my_row = gbuf + t * kOutStride;
    const unsigned char* wbase = gbuf + (warp & 3) * 32 * kOutStride;
    bool have = true;
    if (grp == 1) have = tiles_per_cta > 1 && tw.next(ranges, num_ranges);
    for (int k = grp; have && k < tiles_per_cta; k += 2) {
      const int buse = k >> 1;
      const int nrows = tw.row1 - tw.row0;
      const int dst_row = __ldg(all_rows + min(tw.row0 + t, total_rows - 1));
      const float a_t = GATHER ? __half2float(__ldg(gvals + min(tw.row0 + t, total_rows - 1))) : 1.f;
      if (!tc05::mbar_wait(&bar_acc_full[grp], buse & 1)) { ok = false; break; }
      tc05::fence_after_sync();
      const uint32_t taddr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + grp * feat_out;
      for (int c0 = 0; c0 < feat_out; c0 += 32) {
        uint32_t r[32];
        tc05::tmem_ld32(taddr + c0, r);
        if (c0 + 32 >= feat_out) {  // the accumulator is in registers: the next tile may overwrite it
          tc05::fence_before_sync();
          mbar_arrive_local(&bar_acc_empty[grp]);
        }
        if (GATHER) {
#pragma unroll
          for (int q = 0; q < 32; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) * a_t);
        }
        __syncwarp();  // the warp's reads of the previous 32 columns are over
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<uint4*>(my_row + q * 16) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        __syncwarp();
        scatter32(y, wbase, kOutStride, dst_row, (warp & 3) * 32, nrows, feat_out, c0, lane);
      }
      bool has_next = (k + 2 < tiles_per_cta) && tw.next(ranges, num_ranges);
      has_next = has_next && tw.next(ranges, num_ranges);
      if (!has_next) break;
    }
  }

  const bool all_ok = !__syncthreads_or(!ok);
  if (!all_ok && tid == 0) {
    atomicAdd(&g_rgms_f16_timeouts, 1u);
    // gave up: let the loads already issued land (bounded) before the block's memory is released
    for (int it = max(0, armed - kStagesH); it < armed; ++it)
      tc05::mbar_wait(&bar_full[it % kStagesH], (it / kStagesH) & 1);
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tmem, tmem_cols);
}

// ---- reduction-free form for the sparse-convolution shape.  When every (relation, destination)
// pair occurs at most once and every value is 0 or 1, Y can be computed destination-stationary:
// a tile is 128 consecutive destination rows, its accumulator sums over ALL relations in TMEM
// (row t of relation r's operand is X[map[dst, r]] or zeros), and Y is read and written once
// instead of receiving one reduction per pair.  conv_map_kernel builds map[dst * R + r] (both it
// and *flag start as -1, one memset) and sets *flag to 1 when the input does not qualify; the kernel below then returns at once and the launch of
// rgms_f16_tc_kernel<OutT, true> that follows it (run_if_set) does the work instead.
__global__ void __launch_bounds__(kThreads)
conv_map_kernel(const __half* __restrict__ vals, const int32_t* __restrict__ rows,
                const int32_t* __restrict__ cols, const int32_t* __restrict__ mid, int rows_per_group,
                int num_rels, int total, int32_t* __restrict__ map, int32_t* __restrict__ flag) {
  const int q = blockIdx.x * kThreads + threadIdx.x;
  if (q >= total) return;
  const float v = __half2float(__ldg(vals + q));
  if (v == 0.f) return;  // padding row
  if (v != 1.f) {
    *flag = 1;
    return;
  }
  const int rel = __ldg(mid + q / rows_per_group);
  const int32_t old = atomicCAS(map + static_cast<size_t>(__ldg(rows + q)) * num_rels + rel, -1, __ldg(cols + q));
  if (old != -1) *flag = 1;  // a second entry for the same (relation, destination)
}

constexpr int kOsMaxRels = 512;
constexpr int kOsMaxStages = 8;
constexpr int kOsMaxGroups = 4;
constexpr int kOsThreads = 384 + 128 * kOsMaxGroups;  // warps 12.. are the gather groups
constexpr int kOsSmemLimit = 226 * 1024;  // dynamic part: the static barriers count against the 227 KB too

// the 32 staged columns of the warp's rows are added to Y with plain loads and stores; all loads
// of the old values are issued before the first store (stores to Y would otherwise order them)
__device__ __forceinline__ void store32(float* y, const unsigned char* wbase, int stride, int row_base, int nrows,
                                        int feat_out, int c0, int lane) {
  float4 old[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int lr = 4 * i + (lane >> 3);
    old[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (lr < nrows)
      old[i] = __ldcs(reinterpret_cast<const float4*>(y + static_cast<size_t>(row_base + lr) * feat_out + c0) + (lane & 7));
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int lr = 4 * i + (lane >> 3);
    if (lr < nrows) {
      const float4 v = *reinterpret_cast<const float4*>(wbase + lr * stride + (lane & 7) * 16);
      __stcs(reinterpret_cast<float4*>(y + static_cast<size_t>(row_base + lr) * feat_out + c0) + (lane & 7),
             make_float4(old[i].x + v.x, old[i].y + v.y, old[i].z + v.z, old[i].w + v.w));
    }
  }
}
__device__ __forceinline__ void store32(__half* y, const unsigned char* wbase, int stride, int row_base, int nrows,
                                        int feat_out, int c0, int lane) {
  uint4 old[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = 8 * i + (lane >> 2);
    old[i] = make_uint4(0u, 0u, 0u, 0u);
    if (lr < nrows)
      old[i] = __ldcs(reinterpret_cast<const uint4*>(y + static_cast<size_t>(row_base + lr) * feat_out + c0) + (lane & 3));
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = 8 * i + (lane >> 2);
    if (lr < nrows) {
      const float4 a = *reinterpret_cast<const float4*>(wbase + lr * stride + (lane & 3) * 32);
      const float4 b = *reinterpret_cast<const float4*>(wbase + lr * stride + (lane & 3) * 32 + 16);
      uint4 o = old[i];
      __half2* h = reinterpret_cast<__half2*>(&o);
      h[0] = __hadd2(h[0], __floats2half2_rn(a.x, a.y));
      h[1] = __hadd2(h[1], __floats2half2_rn(a.z, a.w));
      h[2] = __hadd2(h[2], __floats2half2_rn(b.x, b.y));
      h[3] = __hadd2(h[3], __floats2half2_rn(b.z, b.w));
      __stcs(reinterpret_cast<uint4*>(y + static_cast<size_t>(row_base + lr) * feat_out + c0) + (lane & 3), o);
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(kOsThreads, 1)
rgms_f16_os_kernel(const __grid_constant__ CUtensorMap tm_w, OutT* __restrict__ y,
                   const __half* __restrict__ x, const int32_t* __restrict__ map,
                   const int32_t* __restrict__ flag, int m, int num_rels, int feat_in, int feat_out,
                   int tmem_cols, int nstages, int groups) {
  if (__ldg(flag) != -1) return;  // the input does not qualify: the next launch does the work
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kOsMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kOsMaxStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t s_tmem;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned char* base = smem_raw + ((1024u - (tc05::smem_u32(smem_raw) & 1023u)) & 1023u);
  const int nkc = feat_in / kKC, nwb = feat_out / 64;
  // a stage is the gathered Z box plus feat_out / 64 W boxes; the transposing buffer of the
  // epilogue follows the nstages stages
  const int stride = kZBoxB + nwb * kWBoxB;
  const int off_out = nstages * stride;
  const int ntiles = (m + kTM - 1) / kTM;
  // tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the grid never exceeds the number of tiles
  const int my_tiles = (ntiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int steps = num_rels * nkc;  // stages per tile

  if (warp == 0) {
    if (lane == 0) {
      for (int s = 0; s < nstages; ++s) {
        tc05::mbar_init(&bar_full[s], 1 + 128);
        tc05::mbar_init(&bar_empty[s], 1);
      }
      for (int b = 0; b < 2; ++b) {
        tc05::mbar_init(&bar_acc_full[b], 1);
        tc05::mbar_init(&bar_acc_empty[b], 128);
      }
      tc05::fence_mbar_init();
      tc05::prefetch_tensormap(&tm_w);
    }
    __syncwarp();
    tc05::tmem_alloc(&s_tmem, tmem_cols);
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = s_tmem;
  bool ok = true;
  int armed = 0;

  if (warp == 0) {
    // ---- W slices by TMA: relation r, slice c of every tile
    if (lane == 0) {
      int it = 0;
      const uint32_t stage_bytes = nwb * kWBoxB;
      for (int k = 0; k < my_tiles && ok; ++k) {
        for (int sidx = 0; sidx < steps; ++sidx, ++it) {
          const int s = it % nstages, use = it / nstages;
          if (use > 0 && !tc05::mbar_wait(&bar_empty[s], (use - 1) & 1)) { ok = false; break; }
          unsigned char* st = base + s * stride;
          tc05::mbar_arrive_expect_tx(&bar_full[s], stage_bytes);
          for (int j = 0; j < nwb; ++j)
            tc05::tma_load_2d(st + kZBoxB + j * kWBoxB, &tm_w, j * 64, sidx * kKC, &bar_full[s]);
          armed = it + 1;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one accumulator per tile, summed over all relations and slices
    if (lane == 0) {
      const uint32_t idesc = tc05::instr_desc(tc05::kFmtF16, kTM, feat_out, /*a_mn=*/0, /*b_mn=*/1);
      const uint64_t dz0 = tc05::smem_desc_swizzled(tc05::smem_u32(base), 0, 1024, tc05::kSwizzle128B);
      const uint64_t dw0 = tc05::smem_desc_swizzled(tc05::smem_u32(base) + kZBoxB, kWBoxB, 1024, tc05::kSwizzle128B);
      int it = 0;
      for (int k = 0; k < my_tiles && ok; ++k) {
        const int buf = k & 1, buse = k >> 1;
        if (buse > 0 && !tc05::mbar_wait(&bar_acc_empty[buf], (buse - 1) & 1)) { ok = false; break; }
        const uint32_t acc = tmem + buf * feat_out;
        for (int sidx = 0; sidx < steps; ++sidx, ++it) {
          const int s = it % nstages, use = it / nstages;
          if (!tc05::mbar_wait(&bar_full[s], use & 1)) { ok = false; break; }
          tc05::fence_after_sync();
          const uint64_t dz = tc05::desc_advance(dz0, s * stride);
          const uint64_t dw = tc05::desc_advance(dw0, s * stride);
#pragma unroll
          for (int ks = 0; ks < kKC / 16; ++ks)
            tc05::mma_f16(acc, tc05::desc_advance(dz, ks * 32), tc05::desc_advance(dw, ks * 2048), idesc,
                          (sidx > 0 || ks > 0) ? 1u : 0u);
          tc05::mma_commit(&bar_empty[s]);
        }
        if (!ok) break;
        tc05::mma_commit(&bar_acc_full[buf]);
      }
    }
  } else if (warp >= 12) {
    // ---- gather groups: group g (four warps) fills the Z box of the steps g, g + G, g + 2G, ...
    // (warp gw of the group rows gw*32 .. gw*32+31): wait for the stage, issue the copies, wait
    // for them to land, make them visible to the tensor core's proxy, arrive.  G groups keep G
    // gathers in flight.  A missing pair (-1 in the map) is a zero-filled copy.
    const int g = (warp - 12) >> 2, gw = (warp - 12) & 3;
    const int total_steps = my_tiles * steps;
    auto map_entry = [&](int n) -> int {  // source row of this lane's tile row at step n
      const int k = n / steps, r = (n - k * steps) / nkc;
      const int row = (static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x)) * kTM + gw * 32 + lane;
      return row < m ? __ldg(map + static_cast<size_t>(row) * num_rels + r) : -1;
    };
    int entry = g < groups && g < total_steps ? map_entry(g) : -1;
    for (int n = g; g < groups && n < total_steps; n += groups) {
      const int c = n % nkc;
      const int entry_next = n + groups < total_steps ? map_entry(n + groups) : -1;
      const int s = n % nstages, use = n / nstages;
      if (use > 0 && !tc05::mbar_wait(&bar_empty[s], (use - 1) & 1)) { ok = false; break; }
      const uint32_t st = tc05::smem_u32(base + s * stride);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int lr = 4 * i + (lane >> 3);  // row inside the warp's 32
        const int src_row = __shfl_sync(0xffffffffu, entry, lr);
        const int row = gw * 32 + lr, chunk = lane & 7;
        const __half* src = x + static_cast<size_t>(max(src_row, 0)) * feat_in + c * kKC + chunk * 8;
        const uint32_t dst = st + (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4);
        const uint32_t bytes = src_row >= 0 ? 16u : 0u;  // 0: the 16 bytes are filled with zeros
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      tc05::fence_async_smem();
      mbar_arrive_local(&bar_full[s]);
      entry = entry_next;
    }
  } else if (warp >= 4) {
    // ---- epilogue: group 0 (warps 4-7) even tiles, group 1 (warps 8-11) odd tiles; thread = row
    const int grp = warp >= 8 ? 1 : 0;
    const int t = (warp & 3) * 32 + lane;
    unsigned char* gbuf = base + off_out + grp * (kTM * kOutStride);
    unsigned char* my_row = gbuf + t * kOutStride;
    const unsigned char* wbase = gbuf + (warp & 3) * 32 * kOutStride;
    for (int k = grp; k < my_tiles; k += 2) {
      const int buse = k >> 1;
      const int row_base = (static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x)) * kTM + (warp & 3) * 32;
      const int nrows = min(32, m - row_base);  // live rows among the warp's 32 (may be <= 0)
      if (!tc05::mbar_wait(&bar_acc_full[grp], buse & 1)) { ok = false; break; }
      tc05::fence_after_sync();
      const uint32_t taddr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + grp * feat_out;
      for (int c0 = 0; c0 < feat_out; c0 += 32) {
        uint32_t r[32];
        tc05::tmem_ld32(taddr + c0, r);
        if (c0 + 32 >= feat_out) {
          tc05::fence_before_sync();
          mbar_arrive_local(&bar_acc_empty[grp]);
        }
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<uint4*>(my_row + q * 16) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        __syncwarp();
        store32(y, wbase, kOutStride, row_base, nrows, feat_out, c0, lane);
      }
    }
  }

  const bool all_ok = !__syncthreads_or(!ok);
  if (!all_ok && tid == 0) {
    atomicAdd(&g_rgms_f16_timeouts, 1u);
    for (int it = max(0, armed - nstages); it < armed; ++it)
      tc05::mbar_wait(&bar_full[it % nstages], (it / nstages) & 1);
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc05::tmem_dealloc(tmem, tmem_cols);
}

}  // namespace

int rgms_f16_timeouts(unsigned int* count) {
  SPTIR_CUDA_OK(cudaMemcpyFromSymbol(count, g_rgms_f16_timeouts, sizeof(unsigned int)));
  return 0;
}

namespace {

// ranges[b * R + r] for every bucket (what the last block of the gather launches computes)
__global__ void __launch_bounds__(kThreads)
bucket_ranges_kernel(const __grid_constant__ BucketTable tb, int num_rels, int32_t* __restrict__ ranges) {
  for (int e = threadIdx.x; e <= tb.nb * num_rels; e += kThreads) {
    if (e == tb.nb * num_rels) {
      ranges[e] = tb.z_base[tb.nb];
      continue;
    }
    const int b = e / num_rels, r = e % num_rels;
    int lo = 0, hi = tb.num_groups[b];
    while (lo < hi) {
      const int m = lo + (hi - lo) / 2;
      if (__ldg(tb.mid[b] + m) < r) lo = m + 1; else hi = m;
    }
    ranges[e] = tb.z_base[b] + lo * tb.rows_per_group[b];
  }
}

// 0 when launched, 1 when this path cannot take the call (caller falls back), -1 on error.
// GATHER: z is unused, (x, gcols, gvals) describe the rows of the single one-column bucket.
template <typename OutT, bool GATHER>
int launch_tc(const __half* z, const __half* w, OutT* y, const int32_t* ranges, const int32_t* all_rows,
              int num_ranges, int num_rels, int total_rows, int feat_in, int feat_out, cudaStream_t st,
              const __half* x = nullptr, const int32_t* gcols = nullptr, const __half* gvals = nullptr,
              const int32_t* run_if_set = nullptr) {
  CUtensorMap tm_z, tm_w;
  if (make_tmap_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, w, static_cast<uint64_t>(feat_out),
                   static_cast<uint64_t>(num_rels) * feat_in, static_cast<uint64_t>(feat_out) * 2, 64, kKC,
                   CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return 1;
  if (GATHER) {
    tm_z = tm_w;  // not used
  } else if (make_tmap_2d(&tm_z, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, z, static_cast<uint64_t>(feat_in),
                          static_cast<uint64_t>(total_rows), static_cast<uint64_t>(feat_in) * 2, kKC, kTM,
                          CU_TENSOR_MAP_SWIZZLE_128B) != 0) {
    return 1;
  }
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(rgms_f16_tc_kernel<OutT, GATHER>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemH));
    configured_device = dev;
  }
  int tmem_cols = 32;
  while (tmem_cols < 2 * feat_out) tmem_cols *= 2;
  const long long tiles = static_cast<long long>(total_rows) / kTM + num_ranges;  // upper bound
  const long long grid = tiles < kNumSMs ? tiles : kNumSMs;
  const int tiles_per_cta = static_cast<int>((tiles + grid - 1) / grid);
  rgms_f16_tc_kernel<OutT, GATHER><<<static_cast<unsigned>(grid), GATHER ? kTcThreadsG : kTcThreads, kSmemH, st>>>(
      tm_z, tm_w, y, ranges, all_rows, num_ranges, num_rels, total_rows, tiles_per_cta, feat_in, feat_out,
      tmem_cols, x, gcols, gvals, run_if_set);
  SPTIR_LAUNCH_OK("rgms_f16_tc_kernel");
  return 0;
}

// 0 when launched, 1 when this form cannot take the call, -1 on error
template <typename OutT>
int launch_os(const __half* w, OutT* y, const __half* x, const int32_t* map, const int32_t* flag, int m,
              int num_rels, int feat_in, int feat_out, cudaStream_t st) {
  CUtensorMap tm_w;
  if (make_tmap_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, w, static_cast<uint64_t>(feat_out),
                   static_cast<uint64_t>(num_rels) * feat_in, static_cast<uint64_t>(feat_out) * 2, 64, kKC,
                   CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return 1;
  static thread_local int configured_device = -1;
  int dev = 0;
  SPTIR_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    SPTIR_CUDA_OK(cudaFuncSetAttribute(rgms_f16_os_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kOsSmemLimit));
    configured_device = dev;
  }
  // as many stages as fit beside the epilogue's buffer and the map slab
  const int stride = kZBoxB + (feat_out / 64) * kWBoxB;
  const int fixed = 2 * kTM * kOutStride + 1024;
  const int nstages = std::min(kOsMaxStages, (kOsSmemLimit - fixed) / stride);
  if (nstages < 3) return 1;
  const int smem = nstages * stride + fixed;
  const int groups = std::min(kOsMaxGroups, nstages - 1);
  int tmem_cols = 32;
  while (tmem_cols < 2 * feat_out) tmem_cols *= 2;
  const int ntiles = ceil_div(m, kTM);
  const int grid = ntiles < kNumSMs ? ntiles : kNumSMs;
  rgms_f16_os_kernel<OutT><<<grid, kOsThreads, smem, st>>>(tm_w, y, x, map, flag, m, num_rels, feat_in,
                                                             feat_out, tmem_cols, nstages, groups);
  SPTIR_LAUNCH_OK("rgms_f16_os_kernel");
  return 0;
}

template <typename OutT>
int run(const BucketTable& tb, const __half* w, const __half* x, OutT* y, int m, int num_rels, int feat_in,
        int feat_out, int device_id, cudaStream_t st) {
  const int total = tb.z_base[tb.nb];
  const long long num_ranges = static_cast<long long>(tb.nb) * num_rels;
  if (num_ranges >= INT32_MAX) return fail("sparsetir_rgms_ell3d_f16: too many (bucket, relation) pairs");
  // SPARSETIR_RGMS_F16_PATH=simt keeps the transform on the CUDA cores, =two keeps the two-launch
  // form where the one-launch form would be taken, =atomic keeps the one-launch form with
  // reductions where the reduction-free form would be tried, =os tries the reduction-free form
  // for every shape it can take (comparison switches)
  static const int path = [] {
    const char* e = std::getenv("SPARSETIR_RGMS_F16_PATH");
    if (e && std::strcmp(e, "simt") == 0) return 2;
    if (e && std::strcmp(e, "two") == 0) return 1;
    if (e && std::strcmp(e, "atomic") == 0) return 3;
    if (e && std::strcmp(e, "os") == 0) return 4;
    return 0;
  }();
  const bool tc_shape = path != 2 && feat_in % kKC == 0 && feat_out % 64 == 0 && feat_out <= kMaxOut &&
                        aligned16(w) && aligned16(y);
  if (tc_shape && (path == 0 || path == 3 || path == 4) && tb.nb == 1 && tb.width[0] == 1 && aligned16(x)) {
    // one bucket, one column per row: no Z array.  Scratch: the relation ranges, a flag, and —
    // for the reduction-free form — the (destination, relation) -> source map.
    // The reduction-free form's time grows with feat_in (steps per tile, bound by the thread that
    // issues the MMAs) and hardly with feat_out; the form with reductions grows with the bytes
    // added to Y.  Measured on 100,000 points x 27 offsets (us, reduction-free / reductions):
    // float32 Y 64->64 122/108, 64->128 138/188, 64->256 171/428, 128->128 211/197,
    // 128->256 266/480, 256->256 476/546, 128->64 199/123; float16 Y 64->64 119/85,
    // 64->128 132/142, 64->256 166/260, 128->256 254/282, 256->256 454/321.  By default it is
    // tried when feat_out >= 2 * feat_in.
    const bool os_pays = path == 4 || feat_out >= 2 * feat_in;
    const bool try_os = (path == 0 || path == 4) && os_pays && num_rels <= kOsMaxRels &&
                        static_cast<long long>(m) * num_rels < (1ll << 30);
    const size_t rb1 = (static_cast<size_t>(num_ranges + 1) * sizeof(int32_t) + 255) & ~static_cast<size_t>(255);
    const size_t map_bytes = try_os ? static_cast<size_t>(m) * num_rels * sizeof(int32_t) : 0;
    char* ws1 = static_cast<char*>(workspace(device_id, st, rb1 + 256 + map_bytes));
    if (!ws1) return -1;
    int32_t* ranges1 = reinterpret_cast<int32_t*>(ws1);
    int32_t* flag = reinterpret_cast<int32_t*>(ws1 + rb1);
    int32_t* map = reinterpret_cast<int32_t*>(ws1 + rb1 + 256);
    bucket_ranges_kernel<<<1, kThreads, 0, st>>>(tb, num_rels, ranges1);
    SPTIR_LAUNCH_OK("bucket_ranges_kernel");
    int rc = 1;
    if (try_os) {
      SPTIR_CUDA_OK(cudaMemsetAsync(flag, 0xFF, 256 + map_bytes, st));  // flag = -1 (eligible), map = -1
      conv_map_kernel<<<ceil_div(total, kThreads), kThreads, 0, st>>>(tb.a[0], tb.rows[0], tb.cols[0], tb.mid[0],
                                                                     tb.rows_per_group[0], num_rels, total, map, flag);
      SPTIR_LAUNCH_OK("conv_map_kernel");
      rc = launch_os<OutT>(w, y, x, map, flag, m, num_rels, feat_in, feat_out, st);
      if (rc < 0) return rc;
    }
    // rc == 0: the reduction-free launch is queued; this one runs only if it found the flag set
    rc = launch_tc<OutT, true>(nullptr, w, y, ranges1, tb.rows[0], static_cast<int>(num_ranges), num_rels, total,
                               feat_in, feat_out, st, x, tb.cols[0], tb.a[0], rc == 0 ? flag : nullptr);
    if (rc <= 0) return rc;
  }
  const size_t zb = (static_cast<size_t>(total) * feat_in * sizeof(__half) + 255) & ~static_cast<size_t>(255);
  const size_t rb = (static_cast<size_t>(num_ranges + 1) * sizeof(int32_t) + 255) & ~static_cast<size_t>(255);
  char* ws = static_cast<char*>(workspace(device_id, st, zb + rb + static_cast<size_t>(total) * sizeof(int32_t)));
  if (!ws) return -1;
  __half* z = reinterpret_cast<__half*>(ws);
  int32_t* ranges = reinterpret_cast<int32_t*>(ws + zb);
  int32_t* all_rows = reinterpret_cast<int32_t*>(ws + zb + rb);

  const bool vec = feat_in % 8 == 0 && aligned16(x);
  const int rows_per_tile = std::max(1, kThreads / (vec ? feat_in / 8 : feat_in));
  const int blocks = static_cast<int>(std::min<long long>(ceil_div(total, rows_per_tile), 64ll * kNumSMs));
  bool one_column = vec && feat_in / 8 <= kThreads;
  for (int b = 0; b < tb.nb; ++b) one_column = one_column && tb.width[b] == 1;
  if (one_column) {
    const int rows_per_block = (kThreads / (feat_in / 8)) * kCopyR;
    const int nblk = static_cast<int>(std::min<long long>(ceil_div(total, rows_per_block), 64ll * kNumSMs));
    scale_rows_f16_kernel<<<nblk + 1, kThreads, 0, st>>>(tb, x, z, all_rows, ranges, num_rels, feat_in);
  } else if (vec)
    gather_rows_f16_kernel<8><<<blocks + 1, kThreads, 0, st>>>(tb, x, z, all_rows, ranges, num_rels, feat_in);
  else
    gather_rows_f16_kernel<1><<<blocks + 1, kThreads, 0, st>>>(tb, x, z, all_rows, ranges, num_rels, feat_in);
  SPTIR_LAUNCH_OK("gather_rows_f16_kernel");

  if (tc_shape) {
    const int rc = launch_tc<OutT, false>(z, w, y, ranges, all_rows, static_cast<int>(num_ranges), num_rels, total,
                                          feat_in, feat_out, st);
    if (rc <= 0) return rc;
  }
  const size_t smem = static_cast<size_t>(kSimtRows) * feat_in * sizeof(float);
  if (smem > 48 * 1024) return fail("sparsetir_rgms_ell3d_f16: feat_in %d is too large", feat_in);
  transform_scatter_f16_kernel<OutT><<<ceil_div(total, kSimtRows), kThreads, smem, st>>>(
      tb, z, w, y, all_rows, feat_in, feat_out);
  SPTIR_LAUNCH_OK("transform_scatter_f16_kernel");
  return 0;
}

}  // namespace
}  // namespace sptir

extern "C" int sparsetir_rgms_ell3d_f16_raw(const void* w, const void* x, void* y, int y_is_f16,
                                            const SparsetirEll3dBucketH* buckets, int num_buckets, int m,
                                            int n, int num_rels, int feat_in, int feat_out, int device_id,
                                            void* stream) {
  using namespace sptir;
  if (num_buckets < 0 || m < 0 || n < 0 || num_rels < 0 || feat_in < 0 || feat_out < 0)
    return fail("sparsetir_rgms_ell3d_f16: negative size");
  if (num_buckets > kMaxBuckets)
    return fail("sparsetir_rgms_ell3d_f16: %d buckets, at most %d are supported", num_buckets, kMaxBuckets);
  if (num_buckets > 0 && !buckets) return fail("sparsetir_rgms_ell3d_f16: null bucket list");
  BucketTable tb{};
  long long total = 0;
  for (int b = 0; b < num_buckets; ++b) {
    const SparsetirEll3dBucketH& bk = buckets[b];
    if (bk.num_groups < 0 || bk.rows_per_group < 0 || bk.cols_per_row < 0)
      return fail("sparsetir_rgms_ell3d_f16: bucket %d has a negative size", b);
    const long long nrows = static_cast<long long>(bk.num_groups) * bk.rows_per_group;
    if (nrows == 0) continue;
    if (bk.cols_per_row == 0) return fail("sparsetir_rgms_ell3d_f16: bucket %d has rows but no columns", b);
    if (!bk.a || !bk.rows || !bk.cols || !bk.mid)
      return fail("sparsetir_rgms_ell3d_f16: bucket %d has a null array", b);
    if (nrows * bk.cols_per_row > INT32_MAX || total + nrows > INT32_MAX)
      return fail("sparsetir_rgms_ell3d_f16: the buckets are too large for 32-bit indices");
    const int k = tb.nb++;
    tb.a[k] = static_cast<const __half*>(bk.a);
    tb.cols[k] = bk.cols; tb.rows[k] = bk.rows; tb.mid[k] = bk.mid;
    tb.num_groups[k] = bk.num_groups; tb.rows_per_group[k] = bk.rows_per_group;
    tb.width[k] = bk.cols_per_row;
    tb.z_base[k] = static_cast<int32_t>(total);
    total += nrows;
  }
  tb.z_base[tb.nb] = static_cast<int32_t>(total);
  if (total == 0 || feat_out == 0 || m == 0) return 0;
  if (!w || !x || !y) return fail("sparsetir_rgms_ell3d_f16: null pointer argument");
  if (num_rels == 0) return fail("sparsetir_rgms_ell3d_f16: rows but no relations");
  if (feat_in == 0) return 0;  // empty sums: Y is left as it is
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (y_is_f16)
    return run<__half>(tb, static_cast<const __half*>(w), static_cast<const __half*>(x), static_cast<__half*>(y),
                       m, num_rels, feat_in, feat_out, device_id, st);
  return run<float>(tb, static_cast<const __half*>(w), static_cast<const __half*>(x), static_cast<float*>(y),
                    m, num_rels, feat_in, feat_out, device_id, st);
}
