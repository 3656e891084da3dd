// hb_gemm: the public GEMM entry point.  bf16 problems with K % 64 == 0 go to the
// tcgen05 kernel, everything else to the CUDA-core kernel.
#include "common.h"
#include "gemm.h"

extern "C" {

size_t hb_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, hb_dtype dtype) {
  if (!hb::gemm_tc_supported(M, N, K, dtype)) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  hb::TcGemmPlan plan;
  // operands only matter for the tensor maps; any aligned non-null address will do here
  alignas(16) static char dummy[16];
  if (hb::gemm_tc_plan(&plan, dummy, dummy, M, N, K, hb::kEpiStore, false, dev) != HB_OK) return 0;
  return plan.splits > 1 ? plan.workspace_bytes() : 0;
}

int hb_gemm(void* stream, void* Y, const void* X, const void* W, int64_t M, int64_t N, int64_t K,
            hb_dtype dtype, void* workspace) {
  HB_CHECK_ARG(Y && X && W, "hb_gemm: null pointer");
  HB_CHECK_ARG(hb::dtype_valid(dtype), "hb_gemm: bad dtype");
  HB_CHECK_ARG(M >= 0 && N >= 0 && K > 0, "hb_gemm: bad shape");
  if (M == 0 || N == 0) return HB_OK;
  auto st = (cudaStream_t)stream;
  if (hb::gemm_tc_supported(M, N, K, dtype)) {
    int dev = 0;
    HB_CUDA_CHECK(cudaGetDevice(&dev));
    hb::TcGemmPlan plan;
    int rc = hb::gemm_tc_plan(&plan, X, W, M, N, K, hb::kEpiStore, false, dev);
    if (rc) return rc;
    return hb::gemm_tc_run(plan, st, Y, N, workspace, nullptr);
  }
  return hb::gemm_simt(st, Y, X, W, M, N, K, dtype, false);
}

}  // extern "C"
