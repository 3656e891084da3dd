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
//   two-shot : rank q reduces the q-th column slice of EVERY row (each row's CTA pushes the
//              other R-1 slices of its partial to their reducers, sums its own slice, pushes
//              the result to its peers and collects theirs); every rank then normalises the
//              full row.  All CTAs of all ranks do the same amount of work in both hops.
// Every wait is bounded; on expiry the kernel records HB_ERR_TIMEOUT in the world's status
// word and returns.
#include "comm.h"
#include "peer_sync.cuh"

#include <cstring>

namespace hb {

// Thread count, vector assignment (v = tid + i * threads) and the order of the row
// sum are those of rms_norm_vec_kernel (norm.cu), so that the normalised row is
// bit-identical to hb_add_rms_norm's.
constexpr int kAnThreads = 256;
constexpr int kAnMaxVec = 8;  // 16-byte vectors per thread kept in registers

__device__ __forceinline__ void an_st_release(uint32_t* p, uint32_t v) { peer_st_release(p, v); }
__device__ __forceinline__ bool an_wait_ge(const uint32_t* p, uint32_t target, uint32_t limit) {
  return peer_wait_ge(p, target, limit);
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
  int64_t slice_vecs;    // two-shot: vectors of every row one rank reduces = ceil(row_vecs / R)
  int64_t gather_off;    // two-shot: vector offset of the gathered rows inside the data area
  float eps;
  float n_feat;
  uint32_t spin;         // polls before a wait gives up
  // staged != 0 (two-shot only): the partial slices are already on their way into the
  // reducers' staging, pushed by the epilogue of the GEMM that computed them (gemm_tc.cu,
  // kEpiPush), one 128-feature tile of `row_block` batch rows at a time; the arrival of
  // tile ti of the slice from rank src for row block b is tflag[(b * R + src) * tiles + ti].
  int staged, row_block, tiles_per_slice;
};

// VPT = 16-byte vectors per thread (row_vecs <= VPT * kAnThreads).  Everything a CTA needs
// that does not come from a peer (its partial row, the residual row, the norm weight) is
// requested before the first wait and arrives while the CTA waits; the staged vectors of
// the peers are read with all loads in flight together.
//
// Staging (data area of every rank, same offsets everywhere):
//   one-shot : [source rank][row][row_vecs]
//   two-shot : [source rank][row][slice_vecs]  partial slices pushed to their reducer,
//              then at gather_off [row][row_vecs] the reduced slices pushed back.
// Two-shot splits every row by COLUMNS: rank q reduces vectors [q*slice_vecs, (q+1)*slice_vecs)
// of all rows, so the CTA of a row does 1/R of that row's summing on every rank (none idles
// while a few reduce whole rows) and each hop moves slice-sized messages between all pairs.
template <typename T, int VPT>
__global__ void __launch_bounds__(kAnThreads)
ar_add_norm_kernel(const ArNormParams p) {
  constexpr int N = 16 / sizeof(T);
  __shared__ uint32_t s_seq;
  __shared__ float s_red[33];
  // Launched the ordinary way: programmatic edges around this kernel (the next GEMM resident
  // and prefetching while this one waits for its peers) were measured slower inside the decode
  // graph, by 0.4 % to 2.8 % per step.
  const int tid = threadIdx.x, row = blockIdx.x, R = p.ws, me = p.rank;
  CommFlags* fl = reinterpret_cast<CommFlags*>(p.peer[me]);
  auto flags_of = [&](int q) { return reinterpret_cast<CommFlags*>(p.peer[q]); };
  auto data_of = [&](int q) { return reinterpret_cast<uint4*>((uint8_t*)p.peer[q] + kFlagBytes); };
  const int64_t rv = p.row_vecs, sv = p.slice_vecs;
  const uint4* part = reinterpret_cast<const uint4*>(p.partial) + (int64_t)row * rv;
  const uint4* rin = reinterpret_cast<const uint4*>(p.resid_in) + (int64_t)row * rv;
  uint4* rout = reinterpret_cast<uint4*>(p.resid_out) + (int64_t)row * rv;
  // owner of vector v: everybody reduces everything (one-shot) or the slice's rank (two-shot)
  auto mine_to_reduce = [&](int64_t v) { return !p.two_shot || (int)(v / sv) == me; };

  uint4 pv[VPT], rr[VPT], wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int64_t v = tid + (int64_t)i * kAnThreads;
    pv[i] = rr[i] = wv[i] = make_uint4(0, 0, 0, 0);
    if (v < rv) {
      if (!p.staged) pv[i] = part[v];
      if (mine_to_reduce(v)) rr[i] = rin[v];
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
  // (staged: the GEMM epilogue waited for that before it pushed)
  bool ok = true;
  if (!p.staged && tid < R && tid != me) ok = an_wait_ge(&fl->done[tid], seq, p.spin);
  bool all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
  AN_TRACE(1);

  // B. push this rank's partial row: all of it to every peer (one-shot), each slice to its
  // reducer (two-shot)
  if (all_ok && !p.staged) {
    if (!p.two_shot) {
      for (int q = 0; q < R; ++q) {
        if (q == me) continue;
        uint4* dst = data_of(q) + ((int64_t)me * p.M + row) * rv;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int64_t v = tid + (int64_t)i * kAnThreads;
          if (v < rv) dst[v] = pv[i];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int64_t v = tid + (int64_t)i * kAnThreads;
        if (v < rv) {
          const int q = (int)(v / sv);
          if (q != me) data_of(q)[((int64_t)me * p.M + row) * sv + (v - (int64_t)q * sv)] = pv[i];
        }
      }
    }
    __syncthreads();  // orders every thread's stores before the flag threads' release stores
    if (tid < R && tid != me) an_st_release(&flags_of(tid)->pflag[row * HB_MAX_RANKS + me], target);
  }
  AN_TRACE(2);

  // C. wait for the peers' partials of this row, sum what this rank reduces
  uint4 hv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) hv[i] = make_uint4(0, 0, 0, 0);
  if (all_ok) {
    ok = true;
    if (p.staged) {
      // every tile of this rank's slice, from every rank (this one included)
      const int n_flags = R * p.tiles_per_slice, b = row / p.row_block;
      for (int f = tid; f < n_flags; f += kAnThreads) ok = ok && an_wait_ge(&fl->tflag[b * n_flags + f], target, p.spin);
    } else if (tid < R && tid != me) {
      ok = an_wait_ge(&fl->pflag[row * HB_MAX_RANKS + tid], target, p.spin);
    }
    all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
  }
  AN_TRACE(3);
  if (all_ok) {
    const uint4* mine = data_of(me);
    // vector v of source rank `src` in this rank's staging
    const int64_t src_stride = (int64_t)p.M * (p.two_shot ? sv : rv);
    const int64_t row_off = (int64_t)row * (p.two_shot ? sv : rv) - (p.two_shot ? (int64_t)me * sv : 0);
    // groups of at most four vectors per thread: all their staged loads are in flight together
    constexpr int G = VPT < 4 ? VPT : 4;
#pragma unroll
    for (int i0 = 0; i0 < VPT; i0 += G) {
      uint4 x[G][HB_MAX_RANKS];
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        const int i = i0 + gi;
        const int64_t v = tid + (int64_t)i * kAnThreads;
        const bool red = v < rv && mine_to_reduce(v);
#pragma unroll
        for (int src = 0; src < HB_MAX_RANKS; ++src) {
          x[gi][src] = pv[i];
          if (red && src < R && (src != me || p.staged)) x[gi][src] = __ldcg(mine + src * src_stride + row_off + v);
        }
      }
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        const int i = i0 + gi;
        const int64_t v = tid + (int64_t)i * kAnThreads;
        if (v < rv && mine_to_reduce(v)) {
          // fp32 sum in rank order, this rank's own partial in its place
          float acc[N];
#pragma unroll
          for (int j = 0; j < N; ++j) acc[j] = 0.f;
#pragma unroll
          for (int src = 0; src < HB_MAX_RANKS; ++src) {
            if (src < R) {
              const T* e = reinterpret_cast<const T*>(&x[gi][src]);
#pragma unroll
              for (int j = 0; j < N; ++j) acc[j] += to_f32<T>(e[j]);
            }
          }
          const T* re = reinterpret_cast<const T*>(&rr[i]);
          T* he = reinterpret_cast<T*>(&hv[i]);
#pragma unroll
          for (int j = 0; j < N; ++j) {
            const float s = to_f32<T>(from_f32<T>(acc[j]));      // the all-reduce rounds once
            he[j] = from_f32<T>(to_f32<T>(re[j]) + s);           // the sum is materialised in T
          }
          rout[v] = hv[i];
          if (p.two_shot) {
            // the reduced slice goes back to every peer
            for (int q = 0; q < R; ++q)
              if (q != me) data_of(q)[p.gather_off + (int64_t)row * rv + v] = hv[i];
          }
        }
      }
    }
    AN_TRACE(4);
    if (p.two_shot) {
      __syncthreads();
      if (tid < R && tid != me) an_st_release(&flags_of(tid)->sflag[row * HB_MAX_RANKS + me], target);
      // D. the slices of this row reduced elsewhere
      ok = true;
      if (tid < R && tid != me) ok = an_wait_ge(&fl->sflag[row * HB_MAX_RANKS + tid], target, p.spin);
      all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
      if (all_ok) {
        const uint4* src = mine + p.gather_off + (int64_t)row * rv;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int64_t v = tid + (int64_t)i * kAnThreads;
          if (v < rv && !mine_to_reduce(v)) {
            hv[i] = __ldcg(src + v);
            rout[v] = hv[i];
          }
        }
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
static cudaError_t launch_ar_add_norm(const ArNormParams& p, cudaStream_t st) {
  ar_add_norm_kernel<T, VPT><<<(unsigned)p.M, kAnThreads, 0, st>>>(p);
  return cudaGetLastError();
}

bool push_exchange_supported(const hb_world* w, int64_t M, int64_t N, hb_dtype dtype) {
  // bf16 rows whose rank slices are whole 128-feature GEMM tiles; staging for the pushed
  // slices and the gathered rows
  if (!ar_add_norm_supported(w, M, N, dtype) || dtype != HB_BF16) return false;
  if (N % ((int64_t)w->ws * 128)) return false;
  return (size_t)2 * M * N * 2 <= w->staging_bytes;
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
                      hb_dtype dtype, hb_algo algo, const PushGeometry* staged) {
  if (algo == HB_ALGO_MULTIMEM) {
    if (staged) return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: the switch reduction takes no pushed partials");
    return world_mm_ar_add_norm(w, st, normed_out, resid_out, partial, resid_in, norm_w, M, N, eps, dtype);
  }
  if (!ar_add_norm_supported(w, M, N, dtype))
    return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: unsupported shape %lld x %lld or world", (long long)M,
                (long long)N);
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (staged) {
    if (!push_exchange_supported(w, M, N, dtype) || staged->row_block < 1 || staged->tiles_per_slice < 1 ||
        (int64_t)staged->tiles_per_slice * 128 * w->ws != N ||
        ((M + staged->row_block - 1) / staged->row_block) * w->ws * staged->tiles_per_slice > kMaxPushFlags)
      return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: bad geometry for partials pushed by the GEMM");
  } else if (!partial) {
    return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: null partial");
  }
  if (!al16(partial) || !al16(resid_in) || !al16(resid_out) || !al16(normed_out) || !al16(norm_w))
    return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: buffers must be 16-byte aligned");
  if (normed_out && !norm_w) return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: normed_out needs a weight");
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  const int R = w->ws;
  const size_t row_bytes = (size_t)N * dtype_size(dtype);
  bool two = algo == HB_ALGO_TWO_SHOT || staged;
  if (algo == HB_ALGO_AUTO) two = staged || exchange_two_hops(R, (size_t)M * row_bytes);
  ArNormParams p;
  memset(&p, 0, sizeof(p));
  for (int q = 0; q < R; ++q) p.peer[q] = w->peer[q];
  p.partial = partial; p.resid_in = resid_in; p.resid_out = resid_out; p.normed_out = normed_out; p.norm_w = norm_w;
  p.ws = R; p.rank = w->rank; p.two_shot = two ? 1 : 0;
  p.M = (int)M;
  p.row_vecs = (int64_t)(row_bytes / 16);
  p.slice_vecs = two ? (p.row_vecs + R - 1) / R : p.row_vecs;
  p.gather_off = (int64_t)R * M * p.slice_vecs;
  p.eps = eps;
  p.n_feat = (float)N;
  p.spin = w->wait_limit;
  if (staged) {
    p.staged = 1;
    p.row_block = staged->row_block;
    p.tiles_per_slice = staged->tiles_per_slice;
  }
  const size_t need = ((size_t)p.gather_off + (two ? (size_t)M * p.row_vecs : 0)) * 16;
  if (need > w->staging_bytes)
    return fail(HB_ERR_INVALID_ARG, "all_reduce_add_rms_norm: needs %zu bytes of staging, world has %zu", need,
                w->staging_bytes);
  const int64_t vpt = (p.row_vecs + kAnThreads - 1) / kAnThreads;
  HB_DISPATCH_DTYPE(dtype, T, {
    if (vpt <= 1) HB_CUDA_CHECK((launch_ar_add_norm<T, 1>(p, st)));
    else if (vpt <= 2) HB_CUDA_CHECK((launch_ar_add_norm<T, 2>(p, st)));
    else if (vpt <= 4) HB_CUDA_CHECK((launch_ar_add_norm<T, 4>(p, st)));
    else HB_CUDA_CHECK((launch_ar_add_norm<T, 8>(p, st)));
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
                               norm_w, rows, hidden, eps, dtype, algo, nullptr);
}

}  // extern "C"
