// Internal view of a tensor-parallel world (one rank's side).
#pragma once

#include "common.h"

// Layout of every rank's staging buffer (all ranks use the same offsets, so a peer's
// flag or data slot is peer_base + the same offset):
//   [0, kFlagBytes)         flags and counters
//   [kFlagBytes, size)      data area (partials pushed by peers, reduced slices)
namespace hb {

constexpr int kMaxCommCtas = 128;
constexpr size_t kFlagBytes = 64 * 1024;
constexpr int kMaxFusedTiles = 256;  // N <= 32768 in the fused row-parallel kernel
constexpr int kMaxPushFlags = 4096;  // row blocks x ranks x tiles per slice of one pushed projection

struct CommFlags {
  // written by peers (release, system scope), polled locally
  uint32_t done[HB_MAX_RANKS];                      // calls completed by rank p
  uint32_t arrive1[kMaxCommCtas][HB_MAX_RANKS];     // per-CTA: partials pushed
  uint32_t arrive2[kMaxCommCtas][HB_MAX_RANKS];     // per-CTA: reduced slice pushed
  uint32_t pflag[kMaxFusedTiles * HB_MAX_RANKS];    // fused kernel: partial of tile t from rank p landed
  uint32_t gflag[kMaxFusedTiles];                   // fused kernel: reduced tile t (+ row sums) landed
  uint32_t sflag[kMaxFusedTiles * HB_MAX_RANKS];    // exchange + norm kernel: reduced slice of row t from rank p landed
  uint32_t tflag[kMaxPushFlags];                    // GEMM push epilogue: tile of a slice for a row block landed
  // local only
  uint32_t seq;        // collectives completed on this rank
  uint32_t finished;   // CTAs of the running kernel that are done
  int32_t status;      // 0 or HB_ERR_TIMEOUT
  uint32_t local_tiles_done;  // fused kernel, single-rank barrier
};
static_assert(sizeof(CommFlags) <= kFlagBytes, "flag block too large");

// The same operation with the sum done inside the NVLink switch (ar_multimem.cu); needs a
// multicast window.  mm_partial_ptr: where inside the window a GEMM leaves its partial so that
// nothing has to be copied.
bool mm_ar_add_norm_supported(const hb_world* w, int64_t M, int64_t N, hb_dtype dtype);
void* mm_partial_ptr(const hb_world* w);
// gemm_signals: the GEMM that wrote the partial (into the window) announced its completion to
// all ranks itself (TcNormLink::ready_mc, counters from mm_gemm_signal): the kernel skips its
// own arrival hop.
int world_mm_ar_add_norm(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* partial,
                         const void* resid_in, const void* norm_w, int64_t M, int64_t N, float eps, hb_dtype dtype,
                         bool gemm_signals = false);
void mm_gemm_signal(const hb_world* w, uint32_t** ready_mc, uint32_t** calls, uint32_t** ctas);

}  // namespace hb

namespace hb {
// Crossover of the exchange algorithms on peer memory.  One hop of everything ((R-1) x bytes
// inbound per rank) against two hops of slices (2 (R-1)/R x bytes, a second flag wait): the
// second hop pays once the inbound volume of the first form reaches about 4 MB (measured at
// four ranks, rows of 16 KB: one-shot 24.7 us against 27.5 at 1 MB per rank, 31.9 against
// 30.2 at 2 MB; at eight ranks two-shot was ahead from 1 MB per rank).  Two ranks: never.
inline bool exchange_two_hops(int ranks, size_t bytes) {
  return ranks > 2 && (size_t)(ranks - 1) * bytes >= ((size_t)4 << 20);
}
}  // namespace hb

struct hb_world {
  int ws = 1, rank = 0, device = 0;
  cudaStream_t stream = nullptr;
  size_t staging_bytes = 0;
  void* local = nullptr;              // this rank's staging (cudaMalloc)
  void* peer[HB_MAX_RANKS] = {};      // peer[rank] == local
  bool ipc_open[HB_MAX_RANKS] = {};   // peer[p] came from cudaIpcOpenMemHandle
  bool owns_local = true;
  bool attached = false;
  void* nccl = nullptr;               // ncclComm_t when hb_world_init_nccl ran
  // window mapped into a multicast object by the caller (hb_world_attach_multicast): this rank's
  // ordinary address, the multicast address, size
  void* mc_local = nullptr;
  void* mc_base = nullptr;
  size_t mc_bytes = 0;
  uint32_t wait_limit = 1u << 22;     // polls before a device-side wait on a peer flag gives up
  int32_t* host_status = nullptr;     // pinned mirror for hb_world_status
};

namespace hb {

// In-place all-reduce on `st`; the building block of hb_all_reduce and of the engine.
int world_all_reduce(hb_world* w, cudaStream_t st, void* buf, size_t count, hb_dtype dtype,
                     hb_algo algo);
// All-reduce of `partial` + residual add + RMSNorm in one kernel (ar_norm.cu); the values
// of world_all_reduce followed by hb_add_rms_norm.
bool ar_add_norm_supported(const hb_world* w, int64_t M, int64_t N, hb_dtype dtype);
// How a GEMM epilogue pushed its partial into the reducers' staging (gemm_tc.cu, kEpiPush):
// tiles of 128 features x row_block batch rows; every rank's column slice is
// tiles_per_slice tiles wide.
struct PushGeometry {
  int row_block = 0;
  int tiles_per_slice = 0;
};
// True when a [M, N] row-parallel projection on this world can leave through the push epilogue.
bool push_exchange_supported(const hb_world* w, int64_t M, int64_t N, hb_dtype dtype);
// staged != null: `partial` is ignored, the slices were pushed by the GEMM (two-shot form).
int world_ar_add_norm(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* partial,
                      const void* resid_in, const void* norm_w, int64_t M, int64_t N, float eps,
                      hb_dtype dtype, hb_algo algo, const PushGeometry* staged = nullptr);

}  // namespace hb
