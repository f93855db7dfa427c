// Tensor-core (tcgen05) RGMS path.  Placeholder until the kernel lands: reports every shape as
// unsupported so that the caller takes the CUDA-core kernel.
#include "common.h"

namespace sptir {
int rgms_tc_launch(const float*, const float*, const float*, float*, const int32_t*, const int32_t*,
                   const int32_t*, const int32_t*, int, int, int, cudaStream_t) {
  return 1;
}
}  // namespace sptir
