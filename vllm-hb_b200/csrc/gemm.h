// Internal GEMM interface: Y[M,N] = X[M,K] . W[N,K]^T (+ fused epilogues).
#pragma once

#include <cuda.h>

#include "common.h"

namespace hb {

// CUDA-core kernel, any dtype/shape.
int gemm_simt(cudaStream_t st, void* Y, const void* X, const void* W, int64_t M, int64_t N,
              int64_t K, hb_dtype dtype, bool out_f32);

// What the tensor-core kernel does with the finished fp32 tile.
enum TcEpilogue : int {
  kEpiStore = 0,     // Y = acc (bf16, or f32 when out_f32)
  kEpiSwiGLU = 1,    // W rows are [gate tile | up tile] pairs: Y = silu(gate) * up, N_out = N/2
  kEpiResidual = 2,  // deferred RMSNorm producer (cluster plans only), see TcNormLink
  kEpiPush = 3,      // row-parallel partial pushed into the reducing ranks' staging, see TcNormLink
};

// Deferred RMSNorm between two GEMMs of a single-rank decode step.  Instead of a separate
// add + norm kernel between a row-parallel projection P and the projection C that consumes
// the normalised activations, P's epilogue (kEpiResidual) writes
//     h  = resid + Y                      (the new residual, in place in `resid`)
//     Y' = h * norm_w                     (what C reads as its X operand)
//     rowsq[m][tile] = sum over the tile's 128 features of h[m]^2
// and C multiplies batch row m of its accumulator by rsqrt(sum_tiles rowsq[m][.] / n + eps)
// before its own epilogue:  (h * r * w) . W^T == r * ((h * w) . W^T).  The only numerical
// difference from normalising first is where the single bf16 rounding of the activations
// falls (h*w instead of h*r*w).
struct TcNormLink {
  // producer side (kEpiResidual)
  void* resid = nullptr;           // [M, N] bf16, read and overwritten with h
  const void* norm_w = nullptr;    // [N] bf16
  float* rowsq_out = nullptr;      // [M, rowsq_stride] fp32
  // consumer side
  const float* rowsq_in = nullptr; // [M, rowsq_stride] fp32 written by the producer
  int rowsq_tiles = 0;             // entries to sum per row = producer's N / 128
  int rowsq_stride = 0;
  float n = 1.f, eps = 0.f;        // mean over n features
  // independent of the norm: scale of batch row m after the activation, per group of output
  // tiles (mixture of experts: group = expert, post_scale[m * post_groups + group])
  const float* post_scale = nullptr;
  int post_groups = 0, post_tiles_per_group = 0;
  // independent of the norm: RoPE and the paged KV write in the epilogue of the q|k|v
  // projection (cluster plans, bf16, head_dim 128 so that an output tile is one head).
  // Query heads are rotated and stored to Y as usual; key heads are rotated and written to
  // slot kv_slots[m] of k_cache, value heads copied to v_cache, and neither is stored to Y.
  // rope_cs[m * 64 + i] = (cos, sin) of row m's position times frequency i, rounded to bf16
  // (rope_table() in ops.h); caches are [num_blocks, n_kv_heads, 16, 128].
  const float2* rope_cs = nullptr;
  const int64_t* kv_slots = nullptr;
  void* k_cache = nullptr;
  void* v_cache = nullptr;
  int n_q_heads = 0, n_kv_heads = 0;
  int64_t num_blocks = 0;
  // kEpiPush (cluster plans, bf16): the first hop of the all-reduce that follows a
  // row-parallel projection happens here.  Rank q of push_ranks reduces the q-th column slice
  // of the [M, N] result; a CTA that has staged its [rows][128] tile writes it with 16-byte
  // stores straight into rank q's staging (peer memory over NVLink, or this rank's own) and
  // raises the tile's arrival flag there with a system-scope release.  Nothing is written to
  // Y.  The consumer is world_ar_add_norm(..., staged) in ar_norm.cu.  push_peers are the
  // staging bases of all ranks (hb_world::peer), push_spin the poll limit of the one wait
  // (peers done with the previous exchange).
  void* const* push_peers = nullptr;
  int push_ranks = 0, push_rank = 0;
  uint32_t push_spin = 0;
  // independent of everything above: the GEMM announces its own completion to all ranks (the
  // exchange through the NVLink switch, ar_multimem.cu, then starts without an arrival hop of
  // its own).  The CTA that finishes last — counted in ready_ctas, which wraps back to zero —
  // increments ready_calls (local, read by the exchange kernel as the number of calls so far)
  // and adds 1 to the arrival counter of every rank through its multicast address.
  uint32_t* ready_mc = nullptr;
  uint32_t* ready_calls = nullptr;
  uint32_t* ready_ctas = nullptr;
};

// A launch plan for one (M, N, K) problem: tensor maps are encoded once and passed by
// value to the kernel, so a plan can be replayed inside a CUDA graph.
struct TcGemmPlan {
  CUtensorMap tm_w;  // A operand: W [N, K], box 128 x 64
  CUtensorMap tm_x;  // B operand: X [M, K], box m_pad x 64
  int64_t M = 0, N = 0, K = 0;
  int m_pad = 0;      // UMMA N (multiple of 16, <= 256)
  int m_tiles = 0;    // ceil(M / m_pad)
  int n_tiles = 0;    // ceil(N / 128)
  int splits = 1;     // split-K factor
  bool cluster = false;  // the splits of a tile form a thread-block cluster (on-chip reduction)
  bool recv_dedicated = false;  // cluster: the exchange's receive area lies behind the pipeline buffers
  int stages = 0;
  int tmem_cols = 0;
  size_t smem_bytes = 0;
  int epilogue = kEpiStore;
  bool out_f32 = false;
  bool tma_store = false;  // output rows are 16-byte multiples: bulk tensor stores
  // scratch layout inside the caller's workspace
  size_t ws_partials_bytes = 0;  // fp32 [m_tiles*n_tiles*splits][m_pad][128]
  size_t ws_counters_bytes = 0;  // int32 [m_tiles*n_tiles] (zero between calls)
  size_t workspace_bytes() const { return ws_partials_bytes + ws_counters_bytes + 16; }
};

bool gemm_tc_supported(int64_t M, int64_t N, int64_t K, hb_dtype dtype);
// X and W must be 16-byte aligned device pointers; they are baked into the plan.
int gemm_tc_plan(TcGemmPlan* plan, const void* X, const void* W, int64_t M, int64_t N, int64_t K,
                 int epilogue, bool out_f32, int device, int force_splits = 0);
// Y row stride ldy in elements.  workspace: plan.workspace_bytes(), zeroed once.
// err_flag (device int, may be null) is set non-zero when a bounded wait ran out.
// True when `plan` can carry the RoPE + KV-write epilogue of TcNormLink.
bool gemm_tc_rope_epilogue_ok(const TcGemmPlan& plan);
// Batch rows per arrival flag of a kEpiPush plan (the PushGeometry::row_block its consumer
// needs): the rows a cluster partner owns, or the whole batch tile of an unsplit plan; 0 when
// the plan cannot push.
int gemm_tc_push_row_block(const TcGemmPlan& plan);
int gemm_tc_run(const TcGemmPlan& plan, cudaStream_t st, void* Y, int64_t ldy, void* workspace,
                int* err_flag, const TcNormLink* link = nullptr);

}  // namespace hb
