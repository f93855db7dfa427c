// Small helpers shared by the SIMT kernels: 1- or 4-wide feature vectors, read-only loads,
// sub-warp shuffles with the sub-warp's own participation mask.
#ifndef SPARSETIR_B200_VEC_CUH_
#define SPARSETIR_B200_VEC_CUH_

#include <cuda_runtime.h>
#include <cstdint>

namespace sptir {

template <int VEC> struct Vec;
template <> struct Vec<1> {
  using type = float;
  static __device__ __forceinline__ float zero() { return 0.f; }
  static __device__ __forceinline__ void fma(float& acc, float a, float x) { acc = fmaf(a, x, acc); }
  static __device__ __forceinline__ float dot(float a, float b, float acc) { return fmaf(a, b, acc); }
  static __device__ __forceinline__ void atomic_add(float* dst, float v) { atomicAdd(dst, v); }
};
template <> struct Vec<4> {
  using type = float4;
  static __device__ __forceinline__ float4 zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ void fma(float4& acc, float a, float4 x) {
    acc.x = fmaf(a, x.x, acc.x); acc.y = fmaf(a, x.y, acc.y);
    acc.z = fmaf(a, x.z, acc.z); acc.w = fmaf(a, x.w, acc.w);
  }
  static __device__ __forceinline__ float dot(float4 a, float4 b, float acc) {
    acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
    return acc;
  }
  // One 16-byte reduction instead of four 4-byte ones (vector atomics exist from sm_90 on).
  static __device__ __forceinline__ void atomic_add(float4* dst, float4 v) { atomicAdd(dst, v); }
};

// Participation mask of the LPR-lane group this thread belongs to.
template <int LPR>
__device__ __forceinline__ unsigned group_mask() {
  if constexpr (LPR == 32) {
    return 0xffffffffu;
  } else {
    return ((1u << LPR) - 1u) << ((threadIdx.x & 31) / LPR * LPR);
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Smallest power of two >= x, clamped to [lo, hi].
inline int pow2_clamp(int x, int lo, int hi) {
  int p = lo;
  while (p < x && p < hi) p <<= 1;
  return p;
}

// Asynchronous 16-byte copy global -> shared (LDGSTS).  The data does not pass through
// registers, so the number of copies a thread keeps in flight is bounded by shared memory, not
// by its register budget.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;\n" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

}  // namespace sptir
#endif  // SPARSETIR_B200_VEC_CUH_
