// hb_fused_rowparallel: row-parallel projection + sum over ranks + residual + RMSNorm,
//
//   resid_out  = resid_in + SUM_ranks( X_r . W_r^T )
//   normed_out = rms_norm(resid_out; norm_w, eps)
//
// the steps o_proj/down_proj -> all_reduce -> residual -> next norm of the reference
// (src/engine/arch/llama_tp.rs:327,533-552 and :339,563-571,517-522).  Four forms, picked
// by world size, shape and `algo`, and reported by hb_fused_rowparallel_form():
//   HB_ROWPAR_SINGLE   one rank: tcgen05 GEMM, then add + RMSNorm.
//   HB_ROWPAR_PUSH     the GEMM epilogue pushes every 128-feature tile of its partial over
//                      NVLink into the staging of the rank that reduces that column slice and
//                      raises the tile's arrival flag (gemm_tc.cu, kEpiPush); one peer-memory
//                      kernel then sums its slices, adds the residual, returns the reduced
//                      slices to all ranks and normalises (ar_norm.cu).  Two launches; the
//                      first hop of the all-reduce is inside the GEMM.
//   HB_ROWPAR_EXCHANGE tcgen05 GEMM to a local partial, then the same peer-memory kernel
//                      doing both hops (one-shot for small messages).
//   HB_ROWPAR_NCCL     GEMM -> ncclAllReduce -> add + RMSNorm: the reference's sequence
//                      (src/parallel/comm.rs:83-166), kept as the measured baseline.
//   HB_ROWPAR_MULTIMEM the GEMM writes its partial into the world's multicast window; one
//                      kernel reduces inside the NVLink switch, adds the residual and
//                      normalises (ar_multimem.cu).
#include "rowpar.h"

#include <algorithm>

#include "comm.h"
#include "common.h"
#include "gemm.h"

namespace hb {

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Plans the GEMM with the push epilogue; false when the shape cannot take that form.
static bool plan_push(TcGemmPlan* pl, const hb_world* w, const void* X, const void* W, int64_t M, int64_t N,
                      int64_t K_local) {
  if (!w || w->ws < 2 || !push_exchange_supported(w, M, N, HB_BF16)) return false;
  if (!gemm_tc_supported(M, N, K_local, HB_BF16)) return false;
  if (gemm_tc_plan(pl, X, W, M, N, K_local, kEpiPush, false, w->device) != HB_OK) return false;
  const int rb = gemm_tc_push_row_block(*pl);
  return rb > 0 && ((M + rb - 1) / rb) * (N / 128) <= kMaxPushFlags;
}

int rowpar_form(const hb_world* w, int64_t M, int64_t N, int64_t K_local, hb_algo algo) {
  if (M < 1 || N < 1 || K_local < 1) return fail(HB_ERR_INVALID_ARG, "fused row-parallel: bad shape");
  if (!w || w->ws == 1) return HB_ROWPAR_SINGLE;
  if (algo == HB_ALGO_NCCL) return HB_ROWPAR_NCCL;
  if (algo == HB_ALGO_MULTIMEM) {
    if (mm_ar_add_norm_supported(w, M, N, HB_BF16)) return HB_ROWPAR_MULTIMEM;
    return fail(HB_ERR_INVALID_ARG,
                "fused row-parallel: HB_ALGO_MULTIMEM needs a multicast window (hb_world_attach_multicast) that "
                "holds %lld x %lld bf16, rows <= 256, N a multiple of 8 * ranks", (long long)M, (long long)N);
  }
  if (!w->attached) return fail(HB_ERR_INVALID_ARG, "fused row-parallel: world not attached to its peers yet");
  if (algo == HB_ALGO_AUTO || algo == HB_ALGO_TWO_SHOT) {
    // two hops pay once one hop of everything would bring 4 MiB into every rank (comm.h)
    const bool two_hop = algo == HB_ALGO_TWO_SHOT || exchange_two_hops(w->ws, (size_t)M * N * 2);
    alignas(16) static char dummy[16];
    TcGemmPlan pl;
    if (two_hop && plan_push(&pl, w, dummy, dummy, M, N, K_local)) return HB_ROWPAR_PUSH;
  }
  if (ar_add_norm_supported(w, M, N, HB_BF16)) return HB_ROWPAR_EXCHANGE;
  return fail(HB_ERR_INVALID_ARG,
              "fused row-parallel: %lld x %lld is outside the exchange kernel's range (rows <= 256, rows of at "
              "most 32 KiB in multiples of 16 bytes); use HB_ALGO_NCCL", (long long)M, (long long)N);
}

size_t rowpar_workspace_bytes(int64_t M, int64_t N, int64_t K_local) {
  size_t ws = align256((size_t)M * N * 2);  // the local partial of the forms that keep one
  ws += hb_gemm_workspace_bytes(M, N, K_local, HB_BF16);
  return ws + 256;
}

int rowpar_run(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* X, const void* W,
               const void* resid_in, const void* norm_w, int64_t M, int64_t N, int64_t K_local, float eps,
               hb_algo algo, void* workspace) {
  const int form = rowpar_form(w, M, N, K_local, algo);
  if (form < 0) return form;
  if (w) HB_CUDA_CHECK(cudaSetDevice(w->device));
  uint8_t* base = (uint8_t*)workspace;
  void* partial = base;
  void* gemm_ws = base + align256((size_t)M * N * 2);
  int rc;
  if (form == HB_ROWPAR_PUSH) {
    TcGemmPlan pl;
    if (!plan_push(&pl, w, X, W, M, N, K_local)) return fail(HB_ERR_INVALID_ARG, "fused row-parallel: plan changed");
    TcNormLink link;
    link.push_peers = w->peer;
    link.push_ranks = w->ws;
    link.push_rank = w->rank;
    link.push_spin = w->wait_limit;
    if ((rc = gemm_tc_run(pl, st, nullptr, N, gemm_ws, nullptr, &link))) return rc;
    PushGeometry geo{gemm_tc_push_row_block(pl), (int)(N / 128 / w->ws)};
    return world_ar_add_norm(w, st, normed_out, resid_out, nullptr, resid_in, norm_w, M, N, eps, HB_BF16,
                             HB_ALGO_TWO_SHOT, &geo);
  }
  if (form == HB_ROWPAR_MULTIMEM) partial = mm_partial_ptr(w);  // the GEMM writes into the window
  if ((rc = hb_gemm(st, partial, X, W, M, N, K_local, HB_BF16, gemm_ws))) return rc;
  if (form == HB_ROWPAR_MULTIMEM)
    return world_mm_ar_add_norm(w, st, normed_out, resid_out, partial, resid_in, norm_w, M, N, eps, HB_BF16);
  if (form == HB_ROWPAR_EXCHANGE)
    return world_ar_add_norm(w, st, normed_out, resid_out, partial, resid_in, norm_w, M, N, eps, HB_BF16,
                             algo == HB_ALGO_TWO_SHOT ? HB_ALGO_AUTO : algo);
  if (form == HB_ROWPAR_NCCL && (rc = world_all_reduce(w, st, partial, (size_t)M * N, HB_BF16, HB_ALGO_NCCL))) return rc;
  return hb_add_rms_norm(st, normed_out, resid_out, partial, resid_in, norm_w, M, N, eps, HB_BF16);
}

}  // namespace hb

extern "C" {

size_t hb_fused_rowparallel_workspace_bytes(int64_t M, int64_t N, int64_t K_local) {
  if (M <= 0 || N <= 0 || K_local <= 0) return 0;
  return hb::rowpar_workspace_bytes(M, N, K_local);
}

int hb_fused_rowparallel_form(const hb_world* w, int64_t M, int64_t N, int64_t K_local, hb_algo algo) {
  return hb::rowpar_form(w, M, N, K_local, algo);
}

int hb_fused_rowparallel(hb_world* w, void* stream, void* normed_out, void* resid_out,
                         const void* X, const void* W, const void* resid_in, const void* norm_w,
                         int64_t M, int64_t N, int64_t K_local, float eps, hb_algo algo,
                         void* workspace) {
  HB_CHECK_ARG(resid_out && X && W && resid_in && workspace, "hb_fused_rowparallel: null pointer");
  HB_CHECK_ARG(!normed_out || norm_w, "hb_fused_rowparallel: normed_out needs a norm weight");
  HB_CHECK_ARG(M > 0 && N > 0 && K_local > 0, "hb_fused_rowparallel: bad shape");
  return hb::rowpar_run(w, (cudaStream_t)stream, normed_out, resid_out, X, W, resid_in, norm_w, M, N, K_local,
                        eps, algo, workspace);
}

}  // extern "C"
