// Thin inline-PTX layer over the sm_100a tensor-core instructions (tcgen05) used by the
// block-dense kernels: shared-memory matrix descriptors, the instruction descriptor, TMEM
// allocation, MMA issue, completion through mbarriers (with BOUNDED waits) and TMEM loads.
//
// Conventions used by the kernels in this library:
//  - operands live in shared memory in the un-swizzled canonical layout: 8 x 16-byte "core
//    matrices" stored as 128 contiguous bytes;
//      K-major  operand: a core matrix is 8 rows (M or N index) x 16 bytes of K;
//      MN-major operand: a core matrix is 8 K-steps x 16 bytes of M (or N);
//    the descriptor gives the byte stride between core matrices adjacent along K (LBO) and
//    along M/N (SBO);
//  - accumulators are fp32 in TMEM: row m of D in TMEM lane m, column n in TMEM column n;
//  - every wait on an mbarrier gives up after kSpinLimit polls and reports it, so a protocol
//    error ends the kernel instead of hanging the GPU.
#ifndef SPARSETIR_B200_TC05_CUH_
#define SPARSETIR_B200_TC05_CUH_

#include <cuda_runtime.h>
#include <cstdint>

namespace sptir {
namespace tc05 {

constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 64-bit shared-memory matrix descriptor, no swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version of this architecture
  return d;         // base offset 0, layout type 0 (no swizzle)
}

// Swizzled operand layouts (what a TMA tile load with the same swizzle mode writes): rows of
// 128 / 64 / 32 bytes whose 16-byte chunks are XORed with the row number inside an 8-row atom.
//   K-major : a row is one M/N index; SBO = byte stride between 8-row groups; LBO unused; a K step
//             inside the swizzled row is taken by advancing the start address.
//   MN-major: a row is one K index holding 64 / 32 / 16 ... contiguous M/N elements; SBO = byte
//             stride between groups of 8 K rows, LBO = byte stride between row-wide M/N atoms.
// Atoms must start on a multiple of 8 rows (1024 / 512 / 256 bytes).
enum : uint64_t { kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6 };
__device__ __forceinline__ uint64_t smem_desc_swizzled(uint32_t addr, uint32_t lbo_bytes,
                                                       uint32_t sbo_bytes, uint64_t swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version of this architecture
  d |= swizzle << 61;
  return d;
}

// Descriptor of the same layout `bytes` further on in shared memory (bytes a multiple of 16; the
// 14-bit address field must not overflow, which holds inside one block's shared memory): one
// 32-bit add, for issue loops that would otherwise rebuild a descriptor per MMA.
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) {
  const uint32_t lo = static_cast<uint32_t>(desc) + (bytes >> 4);
  return (desc & 0xFFFFFFFF00000000ull) | lo;
}

enum : uint32_t { kFmtF16 = 0, kFmtBF16 = 1, kFmtTF32 = 2 };

// 32-bit instruction descriptor: fp32 accumulate, dense, no negation.
// a_mn / b_mn: 1 when the operand is MN-major (contiguous along M / N), 0 when K-major.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, int m, int n, uint32_t a_mn,
                                                  uint32_t b_mn) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn << 15) | (b_mn << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Makes shared-memory writes of the generic proxy (st.shared, cp.async) visible to the
// asynchronous proxy that the tensor core reads through.
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Bounded wait for the phase with the given parity; false when the limit was hit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// Producer side of a TMA pipeline: one arrival plus the number of bytes the copies will deliver.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// 2-D tiled TMA load into this block's shared memory; completes on `bar` with the tile's bytes.
// x (innermost coordinate) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tensor_map, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      :
      : "r"(smem_u32(smem_dst)), "l"(tensor_map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const void* tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}

// TMEM allocation: executed by one whole warp; the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D(tmem) (+)= A(smem) * B(smem)^T, issued by ONE thread.  kind: f16 (also bf16) or tf32.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u),
        "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u),
        "r"(0u), "r"(0u)
      : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Warp w of the block reads TMEM lanes 32w..32w+31 (thread = lane), 32 consecutive columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace tc05
}  // namespace sptir
#endif  // SPARSETIR_B200_TC05_CUH_
