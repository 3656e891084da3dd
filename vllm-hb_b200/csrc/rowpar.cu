// hb_fused_rowparallel: row-parallel projection + sum over ranks + residual + RMSNorm.
//
// Two implementations live behind the entry point:
//   - the UNFUSED sequence  GEMM -> all-reduce -> add + RMSNorm  (three launches), which
//     is what the reference runs (src/engine/arch/llama_tp.rs:327,533-552) and is kept
//     as the measured baseline (algo = HB_ALGO_NCCL uses ncclAllReduce for the middle
//     step, as src/parallel/comm.rs:83-166 does);
//   - the fused kernel of rowpar_fused.cu (one launch per rank).
#include "comm.h"
#include "common.h"
#include "gemm.h"
#include "rowpar.h"

namespace hb {

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

size_t rowpar_unfused_workspace_bytes(int64_t M, int64_t N, int64_t K_local) {
  size_t ws = align256((size_t)M * N * 2);
  ws += hb_gemm_workspace_bytes(M, N, K_local, HB_BF16);
  return ws + 256;
}

int rowpar_unfused(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* X,
                   const void* W, const void* resid_in, const void* norm_w, int64_t M, int64_t N,
                   int64_t K_local, float eps, hb_algo algo, void* workspace) {
  uint8_t* base = (uint8_t*)workspace;
  void* partial = base;
  void* gemm_ws = base + align256((size_t)M * N * 2);
  int rc = hb_gemm(st, partial, X, W, M, N, K_local, HB_BF16, gemm_ws);
  if (rc) return rc;
  if (w && w->ws > 1) {
    rc = world_all_reduce(w, st, partial, (size_t)M * N, HB_BF16, algo);
    if (rc) return rc;
  }
  return hb_add_rms_norm(st, normed_out, resid_out, partial, resid_in, norm_w, M, N, eps, HB_BF16);
}

}  // namespace hb

extern "C" {

size_t hb_fused_rowparallel_workspace_bytes(int64_t M, int64_t N, int64_t K_local) {
  if (M <= 0 || N <= 0 || K_local <= 0) return 0;
  return std::max(hb::rowpar_unfused_workspace_bytes(M, N, K_local),
                  hb::rowpar_fused_workspace_bytes(M, N, K_local));
}

int hb_fused_rowparallel(hb_world* w, void* stream, void* normed_out, void* resid_out,
                         const void* X, const void* W, const void* resid_in, const void* norm_w,
                         int64_t M, int64_t N, int64_t K_local, float eps, hb_algo algo,
                         void* workspace) {
  HB_CHECK_ARG(resid_out && X && W && resid_in && workspace, "hb_fused_rowparallel: null pointer");
  HB_CHECK_ARG(!normed_out || norm_w, "hb_fused_rowparallel: normed_out needs a norm weight");
  HB_CHECK_ARG(M > 0 && N > 0 && K_local > 0, "hb_fused_rowparallel: bad shape");
  auto st = (cudaStream_t)stream;
  if (algo != HB_ALGO_NCCL && hb::rowpar_fused_supported(w, M, N, K_local))
    return hb::rowpar_fused(w, st, normed_out, resid_out, X, W, resid_in, norm_w, M, N, K_local, eps,
                            algo, workspace);
  return hb::rowpar_unfused(w, st, normed_out, resid_out, X, W, resid_in, norm_w, M, N, K_local, eps,
                            algo, workspace);
}

}  // extern "C"
