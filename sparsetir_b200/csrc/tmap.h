// Host-side construction of TMA tensor maps (CUtensorMap) for 2-D row-major arrays.
// cuTensorMapEncodeTiled lives in the driver library; it is looked up through the runtime
// (cudaGetDriverEntryPoint), so the shared library keeps no link-time dependency on libcuda.
#ifndef SPARSETIR_B200_TMAP_H_
#define SPARSETIR_B200_TMAP_H_

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common.h"

namespace sptir {

// Describes `rows` x `cols` elements (row stride `row_stride_bytes`, a multiple of 16) and a
// box of `box_rows` x `box_cols`; the box row (box_cols * element size) must equal the swizzle
// width for the swizzled modes.  Returns 0, or -1 with the error message set.
inline int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base,
                        uint64_t cols, uint64_t rows, uint64_t row_stride_bytes, uint32_t box_cols,
                        uint32_t box_rows, CUtensorMapSwizzle swizzle) {
  using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode) return fail("cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = encode(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code %d", static_cast<int>(rc));
  return 0;
}

}  // namespace sptir
#endif  // SPARSETIR_B200_TMAP_H_
