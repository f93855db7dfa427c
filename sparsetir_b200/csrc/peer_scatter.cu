// Block scatter over NVLink: one GPU's output block is read once from its own memory and
// written into the same place of every peer's buffer with plain stores through peer-mapped
// pointers.  This is the sending half of an all-gather of row shards: every rank runs it on its
// own block, and a rank's buffer is complete once every peer's kernel has ended (the caller
// orders that with a host- or stream-level barrier between the ranks).  The kernel waits on
// nothing, so it cannot stall on a peer.
//
// The reference has no multi-GPU path (its operators run on one device); the sharded layer of
// this library gathers the row blocks of Y that the shards of A produce.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>

#include "common.h"

namespace sptir {
namespace {

struct PeerPtrs {
  void* p[SPARSETIR_MAX_PEERS];
  int n;
};

// 16-byte pieces; `head` and `tail` bytes around them go out as 4-byte words (every block of the
// sharded layer is a whole number of 4-byte elements).
template <int U>
__global__ void __launch_bounds__(256)
peer_scatter_kernel(const uint4* __restrict__ src, size_t n16, const __grid_constant__ PeerPtrs dst) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + (U - 1) * stride < n16; i += U * stride) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = __ldcs(src + i + u * stride);
    for (int k = 0; k < dst.n; ++k) {
      uint4* d = static_cast<uint4*>(dst.p[k]);
#pragma unroll
      for (int u = 0; u < U; ++u) d[i + u * stride] = v[u];
    }
  }
  for (; i < n16; i += stride) {
    const uint4 v = __ldcs(src + i);
    for (int k = 0; k < dst.n; ++k) static_cast<uint4*>(dst.p[k])[i] = v;
  }
}

// The same with a source that is not 16-byte aligned where the destinations are: each thread
// assembles its 16-byte piece from four word loads (a warp still reads 512 contiguous bytes) so
// that the stores that cross NVLink stay 16 bytes wide.
template <int U>
__global__ void __launch_bounds__(256)
peer_scatter_shift_kernel(const uint32_t* __restrict__ src, size_t n16, const __grid_constant__ PeerPtrs dst) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  auto piece = [&](size_t j) {
    const uint32_t* w = src + 4 * j;
    return make_uint4(__ldcs(w), __ldcs(w + 1), __ldcs(w + 2), __ldcs(w + 3));
  };
  for (; i + (U - 1) * stride < n16; i += U * stride) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = piece(i + u * stride);
    for (int k = 0; k < dst.n; ++k) {
      uint4* d = static_cast<uint4*>(dst.p[k]);
#pragma unroll
      for (int u = 0; u < U; ++u) d[i + u * stride] = v[u];
    }
  }
  for (; i < n16; i += stride) {
    const uint4 v = piece(i);
    for (int k = 0; k < dst.n; ++k) static_cast<uint4*>(dst.p[k])[i] = v;
  }
}

__global__ void __launch_bounds__(256)
peer_scatter_words_kernel(const uint32_t* __restrict__ src, size_t n4, const __grid_constant__ PeerPtrs dst) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const uint32_t v = __ldcs(src + i);
    for (int k = 0; k < dst.n; ++k) static_cast<uint32_t*>(dst.p[k])[i] = v;
  }
}

int scatter_blocks() {
  // The NVLink ports, not the SMs, bound this kernel: 74 blocks already reach the rate of 592
  // (measured with three peers: 635 against 658 GB/s received per GPU), so one block per SM keeps
  // the links busy and leaves most of every SM to the kernels that run beside it.
  // SPARSETIR_SCATTER_BLOCKS overrides.
  static const int n = [] {
    const char* e = getenv("SPARSETIR_SCATTER_BLOCKS");
    const int v = e ? atoi(e) : 0;
    return v > 0 ? v : kNumSMs;
  }();
  return n;
}

}  // namespace
}  // namespace sptir

extern "C" int sparsetir_peer_scatter(int device_id, void* stream, const void* src, size_t bytes,
                                      int n_peers, void* const* peer_dst) {
  using namespace sptir;
  if (n_peers < 0 || n_peers > SPARSETIR_MAX_PEERS)
    return fail("sparsetir_peer_scatter: %d peers, at most %d", n_peers, SPARSETIR_MAX_PEERS);
  if (bytes % 4) return fail("sparsetir_peer_scatter: %zu bytes is not a whole number of 4-byte words", bytes);
  if (bytes == 0 || n_peers == 0) return 0;
  if (src == nullptr || peer_dst == nullptr) return fail("sparsetir_peer_scatter: null pointer");
  if (use_device(device_id) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PeerPtrs dst{};
  dst.n = n_peers;
  const uintptr_t s = reinterpret_cast<uintptr_t>(src);
  if (s % 4) return fail("sparsetir_peer_scatter: source not 4-byte aligned");
  // the destinations are cut at 16-byte boundaries when they all sit alike; the source then is
  // either aligned with them (vector loads) or not (four word loads per piece)
  bool alike = true;
  for (int k = 0; k < n_peers; ++k) {
    if (peer_dst[k] == nullptr) return fail("sparsetir_peer_scatter: destination %d is null", k);
    const uintptr_t d = reinterpret_cast<uintptr_t>(peer_dst[k]);
    if (d % 4) return fail("sparsetir_peer_scatter: destination %d not 4-byte aligned", k);
    alike = alike && (d % 16 == reinterpret_cast<uintptr_t>(peer_dst[0]) % 16);
    dst.p[k] = peer_dst[k];
  }
  const int blocks = scatter_blocks();
  if (!alike) {
    peer_scatter_words_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint32_t*>(src), bytes / 4, dst);
    SPTIR_LAUNCH_OK("peer_scatter_words_kernel");
    return 0;
  }
  // words up to the destinations' first 16-byte boundary, the 16-byte body, the words after it
  const size_t d0 = reinterpret_cast<uintptr_t>(peer_dst[0]) % 16;
  const size_t head = d0 ? ((16 - d0) < bytes ? (16 - d0) : bytes) : 0;
  const size_t body = (bytes - head) / 16 * 16;
  const size_t tail = bytes - head - body;
  auto shifted = [&](size_t off) {
    PeerPtrs q = dst;
    for (int k = 0; k < q.n; ++k) q.p[k] = static_cast<char*>(q.p[k]) + off;
    return q;
  };
  if (head) {
    peer_scatter_words_kernel<<<1, 32, 0, st>>>(static_cast<const uint32_t*>(src), head / 4, dst);
    SPTIR_LAUNCH_OK("peer_scatter_words_kernel");
  }
  if (body) {
    const size_t n16 = body / 16;
    const size_t want = (n16 + 256 * 4 - 1) / (256 * 4);
    const int grid = static_cast<int>(want < static_cast<size_t>(blocks) ? want : blocks);
    const char* from = static_cast<const char*>(src) + head;
    if (reinterpret_cast<uintptr_t>(from) % 16 == 0)
      peer_scatter_kernel<4><<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(from), n16, shifted(head));
    else
      peer_scatter_shift_kernel<4><<<grid, 256, 0, st>>>(reinterpret_cast<const uint32_t*>(from), n16,
                                                         shifted(head));
    SPTIR_LAUNCH_OK("peer_scatter_kernel");
  }
  if (tail) {
    peer_scatter_words_kernel<<<1, 32, 0, st>>>(
        reinterpret_cast<const uint32_t*>(static_cast<const char*>(src) + head + body), tail / 4,
        shifted(head + body));
    SPTIR_LAUNCH_OK("peer_scatter_words_kernel");
  }
  return 0;
}
