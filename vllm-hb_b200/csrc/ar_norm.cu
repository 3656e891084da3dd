// All-reduce + residual add + RMSNorm in one kernel per rank:
//
//   s          = SUM_ranks partial_r          (fp32 in rank order, rounded once to T)
//   resid_out  = resid_in + s                 (rounded to T)
//   normed_out = resid_out * rsqrt(mean(resid_out^2) + eps) * norm_w
//
// i.e. what TpLlamaBackend::forward does between a row-parallel projection and the next
// column-parallel one (src/engine/arch/llama_tp.rs:533-552 and :563-571,517-522), where the
// reference runs an NCCL all-reduce, peer copies, an add and a norm kernel.  The values
// are the ones of hb_all_reduce followed by hb_add_rms_norm, bit for bit.
//
// One CTA per batch row, so the row statistics never leave the CTA and no CTA waits for
// another CTA of its own grid.  Same peer-memory protocol as the all-reduce kernel (push
// with 128-bit stores, system-scope release flags, device-resident sequence numbers, the
// per-rank "done" flags guarding the staging area):
//   one-shot : every rank pushes row r of its partial to every peer; every rank reduces
//              and normalises every row.
//   two-shot : row r is reduced by rank r % R only, which pushes the new residual row to
//              its peers; every rank then normalises the row it received.
// Every wait is bounded; on expiry the kernel records HB_ERR_TIMEOUT in the world's status
// word and returns.
#include "comm.h"

#include <cstring>

namespace hb {

// Thread count, vector assignment (v = tid + i * threads) and the order of the row
// sum are those of rms_norm_vec_kernel (norm.cu), so that the normalised row is
// bit-identical to hb_add_rms_norm's.
constexpr int kAnThreads = 256;
constexpr int kAnMaxVec = 8;  // 16-byte vectors per thread kept in registers
constexpr uint32_t kAnSpin = 1u << 22;

__device__ __forceinline__ uint32_t an_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void an_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool an_wait_ge(const uint32_t* p, uint32_t target) {
  for (uint32_t it = 0; it < kAnSpin; ++it) {
    if ((int32_t)(an_ld_acquire(p) - target) >= 0) return true;
    if (it > 64) __nanosleep(40);
  }
  return false;
}

// Optional phase timestamps (compiled in with -DHB_TC_TRACE only): the CTA of one row this
// rank reduces and of one row it only receives record the global timer at six points of
// every call, in a ring indexed by the call's sequence number; hb_debug_an_trace() copies
// the ring out.
#ifdef HB_TC_TRACE
constexpr int kAnTraceCalls = 2048, kAnTraceSlots = 8;
static __device__ unsigned long long g_an_trace[kAnTraceCalls * 2 * kAnTraceSlots];
__device__ __forceinline__ void an_trace(int which, uint32_t seq, int slot) {
  if (which < 0 || threadIdx.x != 0) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  g_an_trace[((seq % kAnTraceCalls) * 2 + which) * kAnTraceSlots + slot] = t;
}
#define AN_TRACE(slot) an_trace(tr_which, seq, slot)
#else
#define AN_TRACE(slot)
#endif

struct ArNormParams {
  void* peer[HB_MAX_RANKS];
  const void* partial;   // [M, N] this rank's partial
  const void* resid_in;  // [M, N]
  void* resid_out;       // [M, N] (may alias resid_in)
  void* normed_out;      // [M, N] or null
  const void* norm_w;    // [N]
  int ws, rank, two_shot;
  int M;
  int64_t row_vecs;      // N * sizeof(T) / 16
  int rows_own;          // two-shot: rows a rank reduces = ceil(M / R); one-shot: M
  int64_t gather_off;    // two-shot: vector offset of the gathered rows inside the data area
  float eps;
  float n_feat;
  int pdl;               // let the next kernel of the stream start its prologue while this one waits for peers
};

// VPT = 16-byte vectors per thread (row_vecs <= VPT * kAnThreads).  Everything a CTA needs
// that does not come from a peer (its partial row, the residual row, the norm weight) is
// requested before the first wait and arrives while the CTA waits; the staged rows of the
// peers are read with all loads of a source in flight together.
template <typename T, int VPT>
__global__ void __launch_bounds__(kAnThreads)
ar_add_norm_kernel(const ArNormParams p) {
  constexpr int N = 16 / sizeof(T);
  __shared__ uint32_t s_seq;
  __shared__ float s_red[33];
  // Most of this kernel is waiting for peers.  The next kernel of the stream (a GEMM that
  // prefetches its weights before its own dependency wait) may become resident meanwhile.
  // This grid itself touches nothing, the sequence number included, before every earlier
  // kernel of the stream has completed.
  if (p.pdl) pdl_trigger();
  pdl_grid_wait();
  const int tid = threadIdx.x, row = blockIdx.x, R = p.ws, me = p.rank;
  CommFlags* fl = reinterpret_cast<CommFlags*>(p.peer[me]);
  auto flags_of = [&](int q) { return reinterpret_cast<CommFlags*>(p.peer[q]); };
  auto data_of = [&](int q) { return reinterpret_cast<uint4*>((uint8_t*)p.peer[q] + kFlagBytes); };
  const int64_t rv = p.row_vecs;
  const uint4* part = reinterpret_cast<const uint4*>(p.partial) + (int64_t)row * rv;
  const uint4* rin = reinterpret_cast<const uint4*>(p.resid_in) + (int64_t)row * rv;
  uint4* rout = reinterpret_cast<uint4*>(p.resid_out) + (int64_t)row * rv;
  const int owner = p.two_shot ? row % R : me;
  const int slot = p.two_shot ? row / R : row;
  const bool reducer = owner == me;

  uint4 pv[VPT], rr[VPT], wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int64_t v = tid + (int64_t)i * kAnThreads;
    pv[i] = rr[i] = wv[i] = make_uint4(0, 0, 0, 0);
    if (v < rv) {
      pv[i] = part[v];
      if (reducer) rr[i] = rin[v];
      if (p.normed_out) wv[i] = reinterpret_cast<const uint4*>(p.norm_w)[v];
    }
  }

  if (tid == 0) s_seq = *reinterpret_cast<volatile uint32_t*>(&fl->seq);
  __syncthreads();
  const uint32_t seq = s_seq, target = seq + 1;
#ifdef HB_TC_TRACE
  const int tr_which = row == me % p.M ? 0 : (row == (me + 1) % p.M ? 1 : -1);
#endif
  AN_TRACE(0);

  // A. peers must be done with the previous collective before their staging is written
  bool ok = true;
  if (tid < R && tid != me) ok = an_wait_ge(&fl->done[tid], seq);
  bool all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
  AN_TRACE(1);

  // B. push this rank's partial row to its reducer(s)
  if (all_ok) {
    for (int q = 0; q < R; ++q) {
      if (q == me || (p.two_shot && q != owner)) continue;
      uint4* dst = data_of(q) + ((int64_t)me * p.rows_own + slot) * rv;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int64_t v = tid + (int64_t)i * kAnThreads;
        if (v < rv) dst[v] = pv[i];
      }
    }
    __syncthreads();  // orders every thread's stores before the flag threads' release stores
    if (tid < R && tid != me && (!p.two_shot || tid == owner))
      an_st_release(&flags_of(tid)->pflag[row * HB_MAX_RANKS + me], target);
  }
  AN_TRACE(2);

  // C. the new residual row, kept in registers
  uint4 hv[VPT];
  if (all_ok && reducer) {
    ok = true;
    if (tid < R && tid != me) ok = an_wait_ge(&fl->pflag[row * HB_MAX_RANKS + tid], target);
    all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
    AN_TRACE(3);
    if (all_ok) {
      const uint4* mine = data_of(me) + (int64_t)slot * rv;
      const int64_t src_stride = (int64_t)p.rows_own * rv;
      float acc[VPT][N];
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < N; ++j) acc[i][j] = 0.f;
      // fp32 sum in rank order, this rank's own partial in its place
#pragma unroll(VPT >= 8 ? 2 : 4)
      for (int src = 0; src < R; ++src) {
        uint4 x[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int64_t v = tid + (int64_t)i * kAnThreads;
          x[i] = pv[i];
          if (src != me && v < rv) x[i] = __ldcg(mine + src * src_stride + v);
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const T* e = reinterpret_cast<const T*>(&x[i]);
#pragma unroll
          for (int j = 0; j < N; ++j) acc[i][j] += to_f32<T>(e[j]);
        }
      }
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int64_t v = tid + (int64_t)i * kAnThreads;
        const T* re = reinterpret_cast<const T*>(&rr[i]);
        T* he = reinterpret_cast<T*>(&hv[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float s = to_f32<T>(from_f32<T>(acc[i][j]));     // the all-reduce rounds once
          he[j] = from_f32<T>(to_f32<T>(re[j]) + s);             // the sum is materialised in T
        }
        if (v < rv) rout[v] = hv[i];
      }
      if (p.two_shot) {
        for (int q = 0; q < R; ++q) {
          if (q == me) continue;
          uint4* dst = data_of(q) + p.gather_off + (int64_t)row * rv;
#pragma unroll
          for (int i = 0; i < VPT; ++i) {
            const int64_t v = tid + (int64_t)i * kAnThreads;
            if (v < rv) dst[v] = hv[i];
          }
        }
        __syncthreads();
        if (tid < R && tid != me) an_st_release(&flags_of(tid)->gflag[row], target);
      }
      AN_TRACE(4);
    }
  } else if (all_ok) {
    // D. two-shot, a row reduced elsewhere: wait for the gathered row
    ok = true;
    if (tid == 0) ok = an_wait_ge(&fl->gflag[row], target);
    all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
    AN_TRACE(3);
    if (all_ok) {
      const uint4* src = data_of(me) + p.gather_off + (int64_t)row * rv;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int64_t v = tid + (int64_t)i * kAnThreads;
        hv[i] = make_uint4(0, 0, 0, 0);
        if (v < rv) hv[i] = __ldcg(src + v);
      }
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int64_t v = tid + (int64_t)i * kAnThreads;
        if (v < rv) rout[v] = hv[i];
      }
    }
  }

  // row scale and the normalised row (numerics of rms_norm_vec_kernel: per thread the
  // squares are summed vector by vector, element by element)
  float ss = 0.f;
  if (all_ok) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int64_t v = tid + (int64_t)i * kAnThreads;
      if (v < rv) {
        const T* he = reinterpret_cast<const T*>(&hv[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float h = to_f32<T>(he[j]);
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
      const int64_t v = tid + (int64_t)i * kAnThreads;
      if (v < rv) {
        const T* he = reinterpret_cast<const T*>(&hv[i]);
        const T* we = reinterpret_cast<const T*>(&wv[i]);
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < N; ++j) oe[j] = from_f32<T>(to_f32<T>(he[j]) * scale * to_f32<T>(we[j]));
        nout[v] = o;
      }
    }
  }

  // E. the last CTA publishes "this rank is done with call `target`"
  __syncthreads();
  AN_TRACE(5);
  if (tid == 0) {
    if (!all_ok) atomicExch(&fl->status, HB_ERR_TIMEOUT);
    __threadfence();
    const uint32_t prev = atomicAdd(&fl->finished, 1u);
    if (prev == gridDim.x - 1) {
      fl->finished = 0;
      *reinterpret_cast<volatile uint32_t*>(&fl->seq) = target;
      __threadfence_system();
      for (int q = 0; q < R; ++q)
        if (q != me) an_st_release(&flags_of(q)->done[me], target);
    }
  }
}

template <typename T, int VPT>
static cudaError_t launch_ar_add_norm(const ArNormParams& p, bool secondary, cudaStream_t st) {
  if (secondary) return launch_pdl(ar_add_norm_kernel<T, VPT>, dim3((unsigned)p.M), dim3(kAnThreads), 0, st, p);
  ar_add_norm_kernel<T, VPT><<<(unsigned)p.M, kAnThreads, 0, st>>>(p);
  return cudaGetLastError();
}

bool ar_add_norm_supported(const hb_world* w, int64_t M, int64_t N, hb_dtype dtype) {
  if (!w || w->ws < 2 || !w->attached || !dtype_valid(dtype)) return false;
  const size_t row_bytes = (size_t)N * dtype_size(dtype);
  if (M < 1 || M > kMaxFusedTiles || row_bytes % 16) return false;
  if ((int64_t)(row_bytes / 16) > (int64_t)kAnMaxVec * kAnThreads) return false;
  return true;
}

int world_ar_add_norm(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* partial,
                      const void* resid_in, const void* norm_w, int64_t M, int64_t N, float eps,
                      hb_dtype dtype, hb_algo algo) {
  if (!ar_add_norm_supported(w, M, N, dtype))
    return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: unsupported shape %lld x %lld or world", (long long)M,
                (long long)N);
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al16(partial) || !al16(resid_in) || !al16(resid_out) || !al16(normed_out) || !al16(norm_w))
    return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: buffers must be 16-byte aligned");
  if (normed_out && !norm_w) return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: normed_out needs a weight");
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  const int R = w->ws;
  const size_t row_bytes = (size_t)N * dtype_size(dtype);
  bool two = algo == HB_ALGO_TWO_SHOT;
  if (algo == HB_ALGO_AUTO) two = R > 2 && (size_t)M * row_bytes > 128 * 1024;
  ArNormParams p;
  memset(&p, 0, sizeof(p));
  for (int q = 0; q < R; ++q) p.peer[q] = w->peer[q];
  p.partial = partial; p.resid_in = resid_in; p.resid_out = resid_out; p.normed_out = normed_out; p.norm_w = norm_w;
  p.ws = R; p.rank = w->rank; p.two_shot = two ? 1 : 0;
  p.M = (int)M;
  p.row_vecs = (int64_t)(row_bytes / 16);
  p.rows_own = two ? (int)((M + R - 1) / R) : (int)M;
  p.gather_off = (int64_t)R * p.rows_own * p.row_vecs;
  p.eps = eps;
  p.n_feat = (float)N;
  // Programmatic edges around this kernel measured slower than full serialisation inside
  // the decode graph (70B shape, 2 ranks, 40 layers: 10.85 ms serialised, 10.89 with the
  // edge to the next kernel, 11.05 with the edge from the previous one, 11.15 with both),
  // so they are opt-in.  HB_AR_PDL: 0 = serialised (default), 1 = both edges, 2 = only the
  // edge to the next kernel, 3 = only the edge from the previous one.
  static const int mode = [] { const char* e = getenv("HB_AR_PDL"); return e ? atoi(e) : 0; }();
  const bool secondary = pdl_enabled() && (mode == 1 || mode == 3);
  p.pdl = pdl_enabled() && (mode == 1 || mode == 2) ? 1 : 0;
  const size_t need = ((size_t)p.gather_off + (two ? (size_t)M * p.row_vecs : 0)) * 16;
  if (need > w->staging_bytes)
    return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: needs %zu bytes of staging, world has %zu", need,
                w->staging_bytes);
  const int64_t vpt = (p.row_vecs + kAnThreads - 1) / kAnThreads;
  HB_DISPATCH_DTYPE(dtype, T, {
    if (vpt <= 1) HB_CUDA_CHECK((launch_ar_add_norm<T, 1>(p, secondary, st)));
    else if (vpt <= 2) HB_CUDA_CHECK((launch_ar_add_norm<T, 2>(p, secondary, st)));
    else if (vpt <= 4) HB_CUDA_CHECK((launch_ar_add_norm<T, 4>(p, secondary, st)));
    else HB_CUDA_CHECK((launch_ar_add_norm<T, 8>(p, secondary, st)));
  });
  return HB_OK;
}

}  // namespace hb

#ifdef HB_TC_TRACE
extern "C" int hb_debug_an_trace(unsigned long long* host_out, int n_calls) {
  if (n_calls > hb::kAnTraceCalls) n_calls = hb::kAnTraceCalls;
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(host_out, hb::g_an_trace,
                                   sizeof(unsigned long long) * n_calls * 2 * hb::kAnTraceSlots);
}
#endif

extern "C" {

int hb_all_reduce_add_rms_norm(hb_world* w, void* stream, void* normed_out, void* resid_out, const void* partial,
                               const void* resid_in, const void* norm_w, int64_t rows, int64_t hidden, float eps,
                               hb_dtype dtype, hb_algo algo) {
  HB_CHECK_ARG(w && resid_out && partial && resid_in, "hb_all_reduce_add_rms_norm: null argument");
  return hb::world_ar_add_norm(w, stream ? (cudaStream_t)stream : w->stream, normed_out, resid_out, partial, resid_in,
                               norm_w, rows, hidden, eps, dtype, algo);
}

}  // extern "C"
