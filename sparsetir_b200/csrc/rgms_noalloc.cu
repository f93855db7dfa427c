// RGMS for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need the operator: a
// serving or real-time loop whose rules forbid allocator calls after start-up (an allocation
// can block for milliseconds and synchronises the device), or a process whose device memory has
// been handed over entirely to another framework's pool, so that a second allocator would fail
// or fragment it.  The regular sparsetir_rgms keeps its intermediate (one aggregated feature
// row per (relation, destination) pair) in a scratch buffer that the library allocates on first
// use and grows on demand.  This entry point runs the same two launches with the intermediate
// in a fixed array that is part of the library image instead, so no call of it allocates.
//
// The price is a size limit and sharing: the array holds kMaxRows rows of 64 floats (32 MiB on
// every GPU that loads the library, until the process exits), and every call on a device uses
// the same array.  Two calls that overlap on the GPU (different streams, no ordering between
// them) would overwrite each other's intermediate: order them.  The first call on a device
// looks up the array's device address (cudaGetSymbolAddress), and with it the CUDA runtime loads
// this module's image on that device — that is when the 32 MiB come into being.  So make that
// first call at start-up, while device memory is still free, and before any stream capture.
#include <mutex>

#include "common.h"

namespace sptir {

// defined in csrmm.cu and rgms_tc.cu
int csrmm_impl(const float* a, const float* b, float* c, const int32_t* indptr, const int32_t* indices,
               int m, int n, int feat, int nnz, int device_id, void* stream, bool hub_rows);
int rgms_tc_launch(const float* a, const float* w, const float* x, float* y,
                   const int32_t* indptr_i, const int32_t* indices_i, const int32_t* indptr_j,
                   const int32_t* indices_j, int num_rels, int feat, int nnz_i,
                   const float* z, cudaStream_t stream);

namespace {

constexpr int kFeat = 64;
constexpr int kMaxRows = 131072;  // (relation, destination) pairs, i.e. nnz_i
constexpr int kMaxDevices = 64;

// The intermediate Z[nnz_i, 64].  In host code this name is only a handle for the runtime's
// symbol table, never a device address: the address is fetched once per device below.
static __device__ __align__(256) float g_rgms_scratch[static_cast<size_t>(kMaxRows) * kFeat];

std::mutex g_mutex;
float* g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the CURRENT device (must be `device_id`).
int scratch_address(int device_id, float** out) {
  if (device_id < 0 || device_id >= kMaxDevices) return fail("sparsetir_rgms_noalloc: bad device id %d", device_id);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_ptr[device_id] == nullptr) {
    void* p = nullptr;
    SPTIR_CUDA_OK(cudaGetSymbolAddress(&p, g_rgms_scratch));
    g_scratch_ptr[device_id] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[device_id];
  return 0;
}

}  // namespace
}  // namespace sptir

extern "C" int sparsetir_rgms_noalloc(const float* a, const float* w, const float* x, float* y,
                                      const int32_t* indptr_i, const int32_t* indices_i,
                                      const int32_t* indptr_j, const int32_t* indices_j, int m,
                                      int n, int num_rels, int feat, int nnz_i, int nnz_j,
                                      int device_id, void* stream) {
  using namespace sptir;
  (void)m;
  if (num_rels < 0 || nnz_i < 0 || nnz_j < 0 || n < 0) return fail("sparsetir_rgms_noalloc: negative size");
  if (feat != kFeat)
    return fail("sparsetir_rgms_noalloc: feat_size must be %d, got %d (use sparsetir_rgms)", kFeat, feat);
  if (nnz_i > kMaxRows)
    return fail("sparsetir_rgms_noalloc: nnz_i = %d exceeds the built-in scratch of %d rows "
                "(use sparsetir_rgms, which allocates)", nnz_i, kMaxRows);
  if (nnz_i == 0 || num_rels == 0) return 0;
  if (!w || !x || !y || !indptr_i || !indices_i || !indptr_j || (nnz_j > 0 && (!a || !indices_j)))
    return fail("sparsetir_rgms_noalloc: null pointer argument");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w)) & 15u)
    return fail("sparsetir_rgms_noalloc: x, y and w must be 16-byte aligned");
  if (use_device(device_id) != 0) return -1;
  float* z = nullptr;
  if (scratch_address(device_id, &z) != 0) return -1;
  // launch 1: Z = A_csf * X, every one of the nnz_i rows is written (rows without entries get
  // zeros), so nothing left in the array by an earlier call is ever read
  if (sptir::csrmm_impl(a, x, z, indptr_j, indices_j, nnz_i, n, kFeat, nnz_j, device_id, stream, /*hub_rows=*/false) != 0)
    return -1;
  // launch 2: Y[I[i], :] += Z[i, :] * W_r^T on the tensor cores
  const int rc = rgms_tc_launch(a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, kFeat,
                                nnz_i, z, static_cast<cudaStream_t>(stream));
  if (rc > 0) return fail("sparsetir_rgms_noalloc: shape not handled by the tensor-core kernel");
  return rc;
}
