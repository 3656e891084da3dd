// Internal interface of the row-parallel projection (fused and unfused forms).
#pragma once

#include "comm.h"
#include "common.h"

namespace hb {

size_t rowpar_unfused_workspace_bytes(int64_t M, int64_t N, int64_t K_local);
int rowpar_unfused(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* X,
                   const void* W, const void* resid_in, const void* norm_w, int64_t M, int64_t N,
                   int64_t K_local, float eps, hb_algo algo, void* workspace);

bool rowpar_fused_supported(const hb_world* w, int64_t M, int64_t N, int64_t K_local);
size_t rowpar_fused_workspace_bytes(int64_t M, int64_t N, int64_t K_local);
int rowpar_fused(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* X,
                 const void* W, const void* resid_in, const void* norm_w, int64_t M, int64_t N,
                 int64_t K_local, float eps, hb_algo algo, void* workspace);

}  // namespace hb
