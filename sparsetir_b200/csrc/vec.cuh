// Small helpers shared by the SIMT kernels: 1- or 4-wide feature vectors, read-only loads,
// sub-warp shuffles with the sub-warp's own participation mask.
#ifndef SPARSETIR_B200_VEC_CUH_
#define SPARSETIR_B200_VEC_CUH_

#include <cuda_runtime.h>
#include <cstdint>
#include <cstdlib>

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

// Eight consecutive floats held as four packed pairs: moved with one 256-bit load or store and
// multiplied with the two-wide fp32 instructions of sm_100 (each half is an ordinary fp32 FMA).
struct Pack4 {
  unsigned long long q[4];
};
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }
// Floats per lane the SpMM dispatchers pick when the operands allow either width.  Measured on
// B200, 16-byte lanes are the faster choice for the SpMM kernels (hyb step 0.42 ms against
// 0.47 ms with 32-byte lanes; twice the lanes per dense row keep more independent gathers going),
// so 4 is the default; SPARSETIR_LANE_FLOATS=8 selects the 32-byte variants.
inline int max_lane_floats() {
  static const int v = [] {
    const char* e = std::getenv("SPARSETIR_LANE_FLOATS");
    return (e && std::atoi(e) == 8) ? 8 : 4;
  }();
  return v;
}

__device__ __forceinline__ Pack4 pack4_zero() {
  Pack4 r;
  r.q[0] = r.q[1] = r.q[2] = r.q[3] = 0ull;
  return r;
}
// read-only 32-byte load; the address must be 32-byte aligned
__device__ __forceinline__ Pack4 ldg256(const void* p) {
  Pack4 r;
  asm volatile("ld.global.nc.v4.b64 {%0,%1,%2,%3}, [%4];"
               : "=l"(r.q[0]), "=l"(r.q[1]), "=l"(r.q[2]), "=l"(r.q[3])
               : "l"(p));
  return r;
}
// streaming 32-byte store (evict-first: the line is written once and not read again)
__device__ __forceinline__ void stcs256(void* p, const Pack4& v) {
  asm volatile("st.global.cs.v4.b64 [%0], {%1,%2,%3,%4};" ::"l"(p), "l"(v.q[0]), "l"(v.q[1]),
               "l"(v.q[2]), "l"(v.q[3])
               : "memory");
}
__device__ __forceinline__ unsigned long long pack_pair(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_pair(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0,%1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// acc[i] += w * x[i] for the 8 floats
__device__ __forceinline__ void fma8(Pack4& acc, float w, const Pack4& x) {
  const unsigned long long ww = pack_pair(w, w);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc.q[i]) : "l"(ww), "l"(x.q[i]));
}
// sum over the 8 floats of x[i] * y[i]
__device__ __forceinline__ float dot8(const Pack4& x, const Pack4& y) {
  unsigned long long acc;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(acc) : "l"(x.q[0]), "l"(y.q[0]));
#pragma unroll
  for (int i = 1; i < 4; ++i)
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(x.q[i]), "l"(y.q[i]));
  float lo, hi;
  unpack_pair(acc, lo, hi);
  return lo + hi;
}

// A lane's piece of a dense row: 4 floats (one 16-byte vector) or 8 floats (one 32-byte vector).
template <int W> struct LaneVec;
template <> struct LaneVec<4> {
  using type = float4;
  static __device__ __forceinline__ float4 zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ float4 ldg(const void* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ void stcs(void* p, const float4& v) { __stcs(reinterpret_cast<float4*>(p), v); }
  static __device__ __forceinline__ void fma(float4& acc, float w, const float4& x) { Vec<4>::fma(acc, w, x); }
  static __device__ __forceinline__ void atomic_add(void* p, const float4& v) { atomicAdd(reinterpret_cast<float4*>(p), v); }
  // L2-coherent accesses for data that another block wrote during this launch
  static __device__ __forceinline__ float4 ldcg(const void* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ void stcg(void* p, const float4& v) { __stcg(reinterpret_cast<float4*>(p), v); }
  static __device__ __forceinline__ void add(float4& acc, const float4& x) {
    acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
  }
  // shared memory (16-byte aligned)
  static __device__ __forceinline__ void sts(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
  static __device__ __forceinline__ float4 lds(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct LaneVec<8> {
  using type = Pack4;
  static __device__ __forceinline__ Pack4 zero() { return pack4_zero(); }
  static __device__ __forceinline__ Pack4 ldg(const void* p) { return ldg256(p); }
  static __device__ __forceinline__ void stcs(void* p, const Pack4& v) { stcs256(p, v); }
  static __device__ __forceinline__ void fma(Pack4& acc, float w, const Pack4& x) { fma8(acc, w, x); }
  static __device__ __forceinline__ void atomic_add(void* p, const Pack4& v) {  // two 16-byte reductions
    float4 lo, hi;
    unpack_pair(v.q[0], lo.x, lo.y); unpack_pair(v.q[1], lo.z, lo.w);
    unpack_pair(v.q[2], hi.x, hi.y); unpack_pair(v.q[3], hi.z, hi.w);
    atomicAdd(reinterpret_cast<float4*>(p), lo);
    atomicAdd(reinterpret_cast<float4*>(p) + 1, hi);
  }
  static __device__ __forceinline__ Pack4 ldcg(const void* p) {
    Pack4 r;
    asm volatile("ld.global.cg.v4.b64 {%0,%1,%2,%3}, [%4];"
                 : "=l"(r.q[0]), "=l"(r.q[1]), "=l"(r.q[2]), "=l"(r.q[3])
                 : "l"(p) : "memory");
    return r;
  }
  static __device__ __forceinline__ void stcg(void* p, const Pack4& v) {
    asm volatile("st.global.cg.v4.b64 [%0], {%1,%2,%3,%4};" ::"l"(p), "l"(v.q[0]), "l"(v.q[1]),
                 "l"(v.q[2]), "l"(v.q[3])
                 : "memory");
  }
  static __device__ __forceinline__ void add(Pack4& acc, const Pack4& x) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      asm("add.rn.f32x2 %0, %0, %1;" : "+l"(acc.q[i]) : "l"(x.q[i]));
  }
  // shared memory (32-byte aligned)
  static __device__ __forceinline__ void sts(float* p, const Pack4& v) {
    ulonglong2* d = reinterpret_cast<ulonglong2*>(p);
    d[0] = make_ulonglong2(v.q[0], v.q[1]);
    d[1] = make_ulonglong2(v.q[2], v.q[3]);
  }
  static __device__ __forceinline__ Pack4 lds(const float* p) {
    const ulonglong2* d = reinterpret_cast<const ulonglong2*>(p);
    Pack4 r;
    r.q[0] = d[0].x; r.q[1] = d[0].y; r.q[2] = d[1].x; r.q[3] = d[1].y;
    return r;
  }
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
