// Optional deep checks of the index arrays an operator is about to walk.
//
// The reference's generated host stub checks shapes, dtypes and devices only
// (src/tir/transforms/arg_binder.cc:152-282); a wrong index then reads or writes out of bounds
// on the device.  With SPARSETIR_VALIDATE=1 in the environment (or sparsetir_set_validate(1)) every
// operator entry point first runs the kernels below over its structure arrays: row pointers start
// at 0, never decrease and end at the number of stored entries; column ids, row ids and relation
// ids lie inside their ranges.  The first violation is recorded in a device word (no trap, no
// assert: the context stays usable), the call synchronises its stream, reads the word and returns
// -1 with a message naming the array and the position.  A debugging aid: it costs a pass over the
// index arrays and a synchronisation per call, and cannot run while the stream is being captured.
#include <atomic>
#include <cstdlib>

#include "common.h"

namespace sptir {
namespace {

// [0]: error code (0 = none), [1]: position, [2]: offending value
__device__ unsigned long long g_violation[3];

enum : unsigned long long { kOk = 0, kBadStart = 1, kDecreasing = 2, kBadEnd = 3, kOutOfRange = 4 };

__device__ __forceinline__ void report(unsigned long long code, long long pos, long long value) {
  if (atomicCAS(&g_violation[0], 0ull, code) == 0ull) {
    g_violation[1] = static_cast<unsigned long long>(pos);
    g_violation[2] = static_cast<unsigned long long>(value);
  }
}

__global__ void check_indptr_kernel(const int32_t* __restrict__ indptr, long long rows, long long nnz) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i <= rows; i += stride) {
    const int32_t v = indptr[i];
    if (i == 0 && v != 0) report(kBadStart, 0, v);
    if (i == rows && nnz >= 0 && v != nnz) report(kBadEnd, i, v);
    if (i < rows && indptr[i + 1] < v) report(kDecreasing, i + 1, indptr[i + 1]);
  }
}

__global__ void check_range_kernel(const int32_t* __restrict__ ids, long long count, long long bound) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    const int32_t v = ids[i];
    if (v < 0 || v >= bound) report(kOutOfRange, i, v);
  }
}

std::atomic<int> g_validate{-1};  // -1: not decided yet (environment), 0 / 1

int grid_for(long long n) {
  const long long blocks = (n + 255) / 256;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 8 * kNumSMs ? 8 * kNumSMs : blocks));
}

int begin_check(cudaStream_t st) {
  static const unsigned long long zeros[3] = {0, 0, 0};
  SPTIR_CUDA_OK(cudaMemcpyToSymbolAsync(g_violation, zeros, sizeof(zeros), 0, cudaMemcpyHostToDevice, st));
  return 0;
}

// Reads the violation word back; `what` names the array that was checked.
int end_check(const char* op, const char* what, cudaStream_t st) {
  unsigned long long v[3] = {0, 0, 0};
  SPTIR_CUDA_OK(cudaMemcpyFromSymbolAsync(v, g_violation, sizeof(v), 0, cudaMemcpyDeviceToHost, st));
  SPTIR_CUDA_OK(cudaStreamSynchronize(st));
  const long long pos = static_cast<long long>(v[1]), val = static_cast<long long>(v[2]);
  switch (v[0]) {
    case kOk: return 0;
    case kBadStart: return fail("%s: %s[0] is %lld, expected 0", op, what, val);
    case kDecreasing: return fail("%s: %s decreases at position %lld (value %lld)", op, what, pos, val);
    case kBadEnd: return fail("%s: %s[%lld] is %lld, not the number of stored entries", op, what, pos, val);
    default: return fail("%s: %s[%lld] = %lld is out of range", op, what, pos, val);
  }
}

}  // namespace

bool validate_enabled() {
  int v = g_validate.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = std::getenv("SPARSETIR_VALIDATE");
    v = (e != nullptr && e[0] != '\0' && e[0] != '0') ? 1 : 0;
    g_validate.store(v, std::memory_order_relaxed);
  }
  return v == 1;
}

int validate_indptr(const char* op, const char* what, const int32_t* indptr, long long rows,
                    long long nnz, cudaStream_t st) {
  if (rows < 0 || indptr == nullptr) return 0;
  if (begin_check(st) != 0) return -1;
  check_indptr_kernel<<<grid_for(rows + 1), 256, 0, st>>>(indptr, rows, nnz);
  SPTIR_LAUNCH_OK("check_indptr_kernel");
  return end_check(op, what, st);
}

int validate_range(const char* op, const char* what, const int32_t* ids, long long count,
                   long long bound, cudaStream_t st) {
  if (count <= 0 || ids == nullptr) return 0;
  if (begin_check(st) != 0) return -1;
  check_range_kernel<<<grid_for(count), 256, 0, st>>>(ids, count, bound);
  SPTIR_LAUNCH_OK("check_range_kernel");
  return end_check(op, what, st);
}

int validate_csr(const char* op, const int32_t* indptr, long long rows, const int32_t* indices,
                 long long nnz, long long cols, cudaStream_t st) {
  if (validate_indptr(op, "indptr", indptr, rows, nnz, st) != 0) return -1;
  return validate_range(op, "indices", indices, nnz, cols, st);
}

}  // namespace sptir

extern "C" int sparsetir_set_validate(int on) {
  sptir::g_validate.store(on ? 1 : 0, std::memory_order_relaxed);
  return 0;
}
