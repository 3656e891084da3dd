#include "rowpar.h"

namespace hb {

bool rowpar_fused_supported(const hb_world*, int64_t, int64_t, int64_t) { return false; }
size_t rowpar_fused_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }
int rowpar_fused(hb_world*, cudaStream_t, void*, void*, const void*, const void*, const void*,
                 const void*, int64_t, int64_t, int64_t, float, hb_algo, void*) {
  return fail(HB_ERR_INVALID_ARG, "fused row-parallel kernel not available for this shape");
}

}  // namespace hb
