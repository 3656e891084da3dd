// All-reduce + residual add + RMSNorm with the reduction done INSIDE the NVLink switch
// (NVLink SHARP; PTX `multimem`): the same operation as ar_norm.cu —
//
//   s          = SUM_ranks partial_r          (fp32 accumulation in the switch, rounded once to bf16)
//   resid_out  = resid_in + s                 (rounded to bf16)
//   normed_out = resid_out * rsqrt(mean(resid_out^2) + eps) * norm_w
//
// (TpLlamaBackend::forward between a row-parallel projection and the next column-parallel one,
// src/engine/arch/llama_tp.rs:533-552 and :563-571,517-522) — but instead of R-1 peer stores per
// hop, a rank issues ONE load that the switch answers with the sum over all ranks' copies
// (multimem.ld_reduce) and ONE store that the switch delivers to all ranks (multimem.st).
//
// The caller maps one window of hb_world_multicast_bytes() on every rank into a multicast
// object and hands over this rank's ordinary address of it and the multicast address
// (hb_world_attach_multicast).  Window layout, same offsets on every rank:
//   [0, 64 KB)      arrival counters per batch row, written by every rank through
//                   multimem.red.add: `ready` (this rank's partial is complete) and `gathered`
//                   (this rank's reduced slice has been delivered everywhere)
//   then            partial [rows][hidden] bf16: the row-parallel GEMM writes here
//   then            gather  [rows][hidden] bf16: reduced slices from all ranks
//
// One CTA per batch row (the row statistic never leaves the CTA; a CTA waits only for the CTA
// of the same row on the other ranks, never for a CTA of its own grid):
//   A  ready[row] += 1 on every rank (one multimem.red, release), wait until the local copy
//      shows all R ranks: every rank's GEMM has completed (stream order on each rank).
//   B  this rank's column slice of the row: multimem.ld_reduce -> + residual -> multimem.st
//      into the gather area of all ranks.
//   C  gathered[row] += 1 everywhere (release), wait for R ranks.
//   D  the full row from the local gather area -> resid_out, row scale, normed_out.
// Counters only grow, by exactly R per call in which the row takes part, and a row's previous
// call has completed everywhere before anybody starts the next one: a CTA reads both counters
// before it adds to `ready` and waits for the next multiple of R (R is a power of two, so this
// survives the 32-bit wrap); nothing is reset between calls and calls may differ in their
// number of rows.  A rank leaves a call only after every rank's CTAs have passed C, i.e. after
// all loads of its partial and all stores into its gather area have completed: one partial and
// one gather area suffice.
// The sum's order inside the switch is not the rank order of ar_norm.cu, so the two kernels
// agree to bf16 rounding, not bit for bit; all ranks still hold identical rows (one rank
// computes each slice for everybody).  Every wait is bounded.
#include "comm.h"
#include "peer_sync.cuh"
#include "tc_core.cuh"

#include <cstring>

namespace hb {

constexpr int kMmThreads = 256;   // as rms_norm_vec_kernel: same vector assignment and sum order
constexpr int kMmMaxVec = 8;
constexpr int kMmMaxRows = 256;

struct MmCounters {       // window offset 0
  // written by every rank through the multicast address
  uint32_t ready[kMmMaxRows];
  uint32_t gathered[kMmMaxRows];
  uint32_t ready_all;     // arrivals signalled by the producing GEMM itself (TcNormLink::ready_mc)
  uint32_t pad[31];
  // local only, never addressed through the multicast window
  uint32_t gemm_calls;    // launches of a signalling GEMM on this rank so far
  uint32_t gemm_ctas;     // CTAs of the running GEMM that are done
};
static_assert(sizeof(MmCounters) <= kFlagBytes, "multicast counters too large");

__device__ __forceinline__ uint4 mm_ld_reduce_bf16x8(const void* mc) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc)
               : "memory");
  return r;
}
__device__ __forceinline__ void mm_st_bf16x8(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void mm_red_add_release(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

struct MmParams {
  uint8_t* uc;           // this rank's window
  uint8_t* mc;           // the multicast window
  int64_t partial_off, gather_off;  // byte offsets inside the window
  const void* resid_in;  // [M, N]
  void* resid_out;       // [M, N] (may alias resid_in)
  void* normed_out;      // [M, N] or null
  const void* norm_w;    // [N]
  int32_t* status;       // the world's status word
  int ws, rank, M;
  int64_t row_vecs;      // N * 2 / 16
  int64_t slice_vecs;    // row_vecs / R
  float eps, n_feat;
  uint32_t spin;
  int gemm_signals;      // the producing GEMM has announced this rank's partial (ready_all / gemm_calls)
};

template <int VPT>
__global__ void __launch_bounds__(kMmThreads)
mm_ar_add_norm_kernel(const MmParams p) {
  typedef __nv_bfloat16 T;
  constexpr int N = 8;
  __shared__ float s_red[33];
  const int tid = threadIdx.x, row = blockIdx.x, R = p.ws, me = p.rank;
  MmCounters* cnt = reinterpret_cast<MmCounters*>(p.uc);
  MmCounters* cnt_mc = reinterpret_cast<MmCounters*>(p.mc);
  const int64_t rv = p.row_vecs, sv = p.slice_vecs;
  const uint4* rin = reinterpret_cast<const uint4*>(p.resid_in) + (int64_t)row * rv;
  uint4* rout = reinterpret_cast<uint4*>(p.resid_out) + (int64_t)row * rv;

  // what does not come from a peer is requested before the first wait
  uint4 wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int64_t v = tid + (int64_t)i * kMmThreads;
    wv[i] = make_uint4(0, 0, 0, 0);
    if (v < rv && p.normed_out) wv[i] = reinterpret_cast<const uint4*>(p.norm_w)[v];
  }
  // this rank's slice of the row: vectors [me * sv, (me + 1) * sv), thread t takes t, t + 256, ...
  constexpr int SPT = VPT;  // slice vectors per thread never exceed row vectors per thread
  uint4 rs[SPT];
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    const int64_t v = tid + (int64_t)i * kMmThreads;
    rs[i] = make_uint4(0, 0, 0, 0);
    if (v < sv) rs[i] = rin[(int64_t)me * sv + v];
  }

  // The GEMM that follows in the stream carries a programmatic launch edge: released here, it
  // becomes resident and requests its first weight stages while this kernel talks to its peers
  // (it still waits for this kernel's completion before it reads the activations).  Measured at
  // four ranks: 15.59 -> 15.41 ms per 70B decode step; giving THIS kernel such an edge to the
  // GEMM before it was slower (16.03 ms).
  pdl_launch_dependents();
  // A. this rank's partial is complete (the GEMM is an earlier kernel of the stream): tell
  // everybody, wait for everybody.  Both targets come from the counters as they stand before
  // this rank's own arrival: each may already hold up to R-1 arrivals of this call (peers can
  // be ahead, by a whole phase when the GEMMs signal), never this rank's own, so rounding down
  // to a multiple of R and adding R is exact.
  bool ok = true;
  __shared__ uint32_t s_target_c;
  const uint32_t mask = ~(uint32_t)(R - 1);
  // (a thread of another warp fetches the second counter meanwhile: two L2 round trips side by side)
  if (tid == 32) s_target_c = (peer_ld_acquire(&cnt->gathered[row]) & mask) + (uint32_t)R;
  if (tid == 0) {
    if (p.gemm_signals) {
      // the GEMM's last CTA has counted this call locally and told all ranks: every rank has
      // made the same number of such calls, so R times this rank's count is the target
      const uint32_t calls = *reinterpret_cast<volatile uint32_t*>(&cnt->gemm_calls);
      ok = peer_wait_ge(&cnt->ready_all, calls * (uint32_t)R, p.spin);
    } else {
      const uint32_t target_a = (peer_ld_acquire(&cnt->ready[row]) & mask) + (uint32_t)R;
      mm_red_add_release(&cnt_mc->ready[row], 1u);
      ok = peer_wait_ge(&cnt->ready[row], target_a, p.spin);
    }
  }
  bool all_ok = __syncthreads_and(ok ? 1 : 0) != 0;

  // B. reduce this rank's slice in the switch, add the residual, deliver to all ranks
  if (all_ok) {
    const int64_t base = (int64_t)row * rv + (int64_t)me * sv;
    const uint4* part_mc = reinterpret_cast<const uint4*>(p.mc + p.partial_off) + base;
    uint4* gath_mc = reinterpret_cast<uint4*>(p.mc + p.gather_off) + base;
    uint4 sum[SPT];
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      const int64_t v = tid + (int64_t)i * kMmThreads;
      sum[i] = make_uint4(0, 0, 0, 0);
      if (v < sv) sum[i] = mm_ld_reduce_bf16x8(part_mc + v);
    }
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      const int64_t v = tid + (int64_t)i * kMmThreads;
      if (v < sv) {
        const T* se = reinterpret_cast<const T*>(&sum[i]);
        const T* re = reinterpret_cast<const T*>(&rs[i]);
        uint4 h;
        T* he = reinterpret_cast<T*>(&h);
#pragma unroll
        for (int j = 0; j < N; ++j) he[j] = __float2bfloat16_rn(__bfloat162float(re[j]) + __bfloat162float(se[j]));
        mm_st_bf16x8(gath_mc + v, h);
      }
    }
  }
  __syncthreads();  // orders every thread's multicast stores before the release below

  // C. this rank's slice has been sent: tell everybody, wait for everybody's
  ok = true;
  if (all_ok && tid == 0) {
    mm_red_add_release(&cnt_mc->gathered[row], 1u);
    ok = peer_wait_ge(&cnt->gathered[row], s_target_c, p.spin);
  }
  all_ok = __syncthreads_and((all_ok && ok) ? 1 : 0) != 0;

  // D. the full row, row scale and normalised row (numerics of rms_norm_vec_kernel)
  uint4 hv[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) hv[i] = make_uint4(0, 0, 0, 0);
  if (all_ok) {
    const uint4* src = reinterpret_cast<const uint4*>(p.uc + p.gather_off) + (int64_t)row * rv;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t v = tid + (int64_t)i * kMmThreads;
      if (v < rv) hv[i] = __ldcg(src + v);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t v = tid + (int64_t)i * kMmThreads;
      if (v < rv) {
        rout[v] = hv[i];
        const T* he = reinterpret_cast<const T*>(&hv[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float h = __bfloat162float(he[j]);
          ss += h * h;
        }
      }
    }
  }
  ss = block_sum(ss, s_red);
  if (all_ok && p.normed_out) {
    const float scale = rsqrtf(ss / p.n_feat + p.eps);
    uint4* nout = reinterpret_cast<uint4*>(p.normed_out) + (int64_t)row * rv;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t v = tid + (int64_t)i * kMmThreads;
      if (v < rv) {
        const T* he = reinterpret_cast<const T*>(&hv[i]);
        const T* we = reinterpret_cast<const T*>(&wv[i]);
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < N; ++j) oe[j] = __float2bfloat16_rn(__bfloat162float(he[j]) * scale * __bfloat162float(we[j]));
        nout[v] = o;
      }
    }
  }

  if (tid == 0 && !all_ok) atomicExch(p.status, HB_ERR_TIMEOUT);
}

size_t mm_window_bytes(int64_t max_rows, int64_t hidden) {
  return kFlagBytes + 2 * (size_t)max_rows * (size_t)hidden * 2;
}

bool mm_ar_add_norm_supported(const hb_world* w, int64_t M, int64_t N, hb_dtype dtype) {
  if (!w || w->ws < 2 || (w->ws & (w->ws - 1)) || !w->mc_base || dtype != HB_BF16) return false;
  if (M < 1 || M > kMmMaxRows || N % ((int64_t)8 * w->ws)) return false;
  if (N / 8 > (int64_t)kMmMaxVec * kMmThreads) return false;
  return mm_window_bytes(M, N) <= w->mc_bytes;
}

void* mm_partial_ptr(const hb_world* w) { return w->mc_local ? (uint8_t*)w->mc_local + kFlagBytes : nullptr; }

void mm_gemm_signal(const hb_world* w, uint32_t** ready_mc, uint32_t** calls, uint32_t** ctas) {
  MmCounters* loc = reinterpret_cast<MmCounters*>(w->mc_local);
  *ready_mc = &reinterpret_cast<MmCounters*>(w->mc_base)->ready_all;
  *calls = &loc->gemm_calls;
  *ctas = &loc->gemm_ctas;
}

int world_mm_ar_add_norm(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* partial,
                         const void* resid_in, const void* norm_w, int64_t M, int64_t N, float eps, hb_dtype dtype,
                         bool gemm_signals) {
  if (!mm_ar_add_norm_supported(w, M, N, dtype))
    return fail(HB_ERR_INVALID_ARG,
                "all_reduce_add_rms_norm (multimem): needs an attached multicast window, bf16 rows of a multiple of "
                "%d features and at most %d rows (%lld x %lld given)", 8 * (w ? w->ws : 1), kMmMaxRows, (long long)M,
                (long long)N);
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!partial || !al16(partial) || !al16(resid_in) || !al16(resid_out) || !al16(normed_out) || !al16(norm_w))
    return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: buffers must be non-null and 16-byte aligned");
  if (normed_out && !norm_w) return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: normed_out needs a weight");
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  // a partial that is not already in the window is copied there (the engine's GEMMs write into it)
  if (gemm_signals && partial != mm_partial_ptr(w))
    return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm (multimem): a GEMM that signals writes into the window");
  if (partial != mm_partial_ptr(w))
    HB_CUDA_CHECK(cudaMemcpyAsync(mm_partial_ptr(w), partial, (size_t)M * N * 2, cudaMemcpyDeviceToDevice, st));
  MmParams p;
  memset(&p, 0, sizeof(p));
  p.uc = (uint8_t*)w->mc_local;
  p.mc = (uint8_t*)w->mc_base;
  p.partial_off = (int64_t)kFlagBytes;
  // the gather area follows a partial area sized for the window's capacity, so that the offsets
  // do not depend on the call's row count
  p.gather_off = (int64_t)kFlagBytes + (int64_t)((w->mc_bytes - kFlagBytes) / 2 / 16 * 16);
  p.resid_in = resid_in; p.resid_out = resid_out; p.normed_out = normed_out; p.norm_w = norm_w;
  p.status = &reinterpret_cast<CommFlags*>(w->local)->status;
  p.ws = w->ws; p.rank = w->rank; p.M = (int)M;
  p.row_vecs = N / 8;
  p.slice_vecs = p.row_vecs / w->ws;
  p.eps = eps;
  p.n_feat = (float)N;
  p.spin = w->wait_limit;
  p.gemm_signals = gemm_signals ? 1 : 0;
  const int64_t vpt = (p.row_vecs + kMmThreads - 1) / kMmThreads;
  if (vpt <= 1) mm_ar_add_norm_kernel<1><<<(unsigned)M, kMmThreads, 0, st>>>(p);
  else if (vpt <= 2) mm_ar_add_norm_kernel<2><<<(unsigned)M, kMmThreads, 0, st>>>(p);
  else if (vpt <= 4) mm_ar_add_norm_kernel<4><<<(unsigned)M, kMmThreads, 0, st>>>(p);
  else mm_ar_add_norm_kernel<8><<<(unsigned)M, kMmThreads, 0, st>>>(p);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace hb

extern "C" {

size_t hb_world_multicast_bytes(int64_t max_rows, int64_t hidden) {
  if (max_rows < 1 || hidden < 1) return 0;
  return hb::mm_window_bytes(max_rows, hidden);
}

int hb_world_attach_multicast(hb_world* w, void* local_ptr, void* multicast_ptr, size_t bytes) {
  HB_CHECK_ARG(w && local_ptr && multicast_ptr, "hb_world_attach_multicast: null argument");
  HB_CHECK_ARG(w->ws > 1, "hb_world_attach_multicast: a single-rank world exchanges nothing");
  HB_CHECK_ARG(bytes >= hb::kFlagBytes + 4096 && !(reinterpret_cast<uintptr_t>(local_ptr) & 15) &&
                   !(reinterpret_cast<uintptr_t>(multicast_ptr) & 15),
               "hb_world_attach_multicast: the window must be 16-byte aligned and hold at least one row");
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  // counters and local words start at zero; the caller separates attach and first use by a
  // barrier over all ranks
  HB_CUDA_CHECK(cudaMemset(local_ptr, 0, hb::kFlagBytes));
  HB_CUDA_CHECK(cudaDeviceSynchronize());
  w->mc_local = local_ptr;
  w->mc_base = multicast_ptr;
  w->mc_bytes = bytes;
  return HB_OK;
}

int hb_world_detach_multicast(hb_world* w) {
  HB_CHECK_ARG(w, "hb_world_detach_multicast: null world");
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  HB_CUDA_CHECK(cudaDeviceSynchronize());
  w->mc_local = w->mc_base = nullptr;
  w->mc_bytes = 0;
  return HB_OK;
}

int hb_world_has_multicast(const hb_world* w) { return w && w->mc_base ? 1 : 0; }

void* hb_world_multicast_partial(const hb_world* w) { return w ? hb::mm_partial_ptr(w) : nullptr; }

}  // extern "C"
