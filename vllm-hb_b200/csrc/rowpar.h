// Internal interface of the row-parallel projection (rowpar.cu).
#pragma once

#include "comm.h"
#include "common.h"

namespace hb {

// One of HB_ROWPAR_* (the form hb_fused_rowparallel takes for this world, shape and algo)
// or a negative error.
int rowpar_form(const hb_world* w, int64_t M, int64_t N, int64_t K_local, hb_algo algo);
size_t rowpar_workspace_bytes(int64_t M, int64_t N, int64_t K_local);
int rowpar_run(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* X, const void* W,
               const void* resid_in, const void* norm_w, int64_t M, int64_t N, int64_t K_local, float eps,
               hb_algo algo, void* workspace);

}  // namespace hb
