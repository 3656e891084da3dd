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

extern "C" {

size_t hb_gemm_ex_workspace_bytes(int64_t M, int64_t N, int64_t K, int epilogue, int force_splits) {
  if (!hb::gemm_tc_supported(M, N, K, HB_BF16)) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  hb::TcGemmPlan plan;
  alignas(16) static char dummy[16];
  if (hb::gemm_tc_plan(&plan, dummy, dummy, M, N, K, epilogue, false, dev, force_splits) != HB_OK) return 0;
  return plan.workspace_bytes();
}

int hb_gemm_ex(void* stream, void* Y, const void* X, const void* W, int64_t M, int64_t N,
               int64_t K, int epilogue, int out_f32, int force_splits, void* workspace) {
  HB_CHECK_ARG(Y && X && W, "hb_gemm_ex: null pointer");
  HB_CHECK_ARG(epilogue == hb::kEpiStore || epilogue == hb::kEpiSwiGLU, "hb_gemm_ex: unknown epilogue %d", epilogue);
  HB_CHECK_ARG(hb::gemm_tc_supported(M, N, K, HB_BF16),
               "hb_gemm_ex: bf16 with K %% 64 == 0 only (M=%lld N=%lld K=%lld)", (long long)M,
               (long long)N, (long long)K);
  int dev = 0;
  HB_CUDA_CHECK(cudaGetDevice(&dev));
  hb::TcGemmPlan plan;
  int rc = hb::gemm_tc_plan(&plan, X, W, M, N, K, epilogue, out_f32 != 0, dev, force_splits);
  if (rc) return rc;
  return hb::gemm_tc_run(plan, (cudaStream_t)stream, Y, plan.N, workspace, nullptr);
}

}  // extern "C"
