// Shared host-side plumbing of the library: thread-local error string, per-device stream
// table, launch checking.  Nothing here allocates device memory.
#ifndef SPARSETIR_B200_COMMON_H_
#define SPARSETIR_B200_COMMON_H_

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "sparsetir_b200.h"

namespace sptir {

// Records a printf-style message for sparsetir_get_last_error and returns -1, so that
// `return fail("...")` mirrors the reference's "set last error, return -1" protocol
// (src/runtime/c_runtime_api.cc:371-386).
int fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

// Makes `device_id` current (the generated reference stub does the same through
// __tvm_set_device, src/tir/transforms/make_packed_api.cc:286-305).
int use_device(int device_id);

cudaStream_t stream_for(int device_id);

// Scratch memory for kernels that need an intermediate buffer: one grow-only allocation per
// (device, stream), kept until the library is unloaded, so that steady-state calls allocate
// nothing.  Calls that use it on the same stream are ordered by the stream; calls on different
// streams get different buffers.  Returns nullptr (after recording the error) when the device
// cannot provide `bytes`.  Growing an existing buffer frees the old one, which synchronises the
// device once.
void* workspace(int device_id, cudaStream_t stream, size_t bytes);

// The same for counters and flags that kernels find at zero and leave at zero: the buffer is
// cleared (on `stream`) when it is allocated, and every kernel that uses it restores the zeros
// before it ends, so steady-state calls neither allocate nor clear.
void* zeroed_workspace(int device_id, cudaStream_t stream, size_t bytes);

// Deep checks of index arrays before a launch (validate.cu): enabled by SPARSETIR_VALIDATE=1 or
// sparsetir_set_validate(1).  Each returns 0, or -1 after recording which array is wrong where;
// they synchronise `st`.  nnz < 0 skips the check of the last row pointer.
bool validate_enabled();
int validate_indptr(const char* op, const char* what, const int32_t* indptr, long long rows,
                    long long nnz, cudaStream_t st);
int validate_range(const char* op, const char* what, const int32_t* ids, long long count,
                   long long bound, cudaStream_t st);
int validate_csr(const char* op, const int32_t* indptr, long long rows, const int32_t* indices,
                 long long nnz, long long cols, cudaStream_t st);

// Copies of an output array on other GPUs (peer-mapped): a kernel that takes one stores every
// finished element also at the same offset from (its own output pointer + delta[k]).  n = 0 for a
// plain call.  Filled by peer_table().
struct PeerOut {
  long long delta[SPARSETIR_MAX_PEERS];  // bytes from this GPU's output to peer k's copy of it
  int n;
};

// Checks the peer addresses of a *_peers entry point and turns them into offsets from `own`;
// every copy must sit like `own` with respect to `align` bytes.  Returns 0 or -1 (error recorded).
int peer_table(const char* fn, const void* own, int n_peers, void* const* peers, size_t align, PeerOut* out);

constexpr int kNumSMs = 148;  // B200

inline int ceil_div(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

}  // namespace sptir

#define SPTIR_CUDA_OK(expr)                                                                  \
  do {                                                                                       \
    cudaError_t err__ = (expr);                                                              \
    if (err__ != cudaSuccess)                                                                \
      return ::sptir::fail("CUDA error %s at %s:%d: %s", cudaGetErrorName(err__), __FILE__,  \
                           __LINE__, cudaGetErrorString(err__));                             \
  } while (0)

// After a kernel launch: report launch-configuration errors without synchronising.
#define SPTIR_LAUNCH_OK(name)                                                                \
  do {                                                                                       \
    cudaError_t err__ = cudaGetLastError();                                                  \
    if (err__ != cudaSuccess)                                                                \
      return ::sptir::fail("launch of %s failed: %s (%s)", name, cudaGetErrorName(err__),    \
                           cudaGetErrorString(err__));                                       \
  } while (0)

#endif  // SPARSETIR_B200_COMMON_H_
