// Tensor-parallel world and the peer-memory all-reduce.
//
// Replaces TpWorld / nccl_all_reduce (src/parallel/world.rs:95-213,
// src/parallel/comm.rs:83-166).  Every rank owns one staging buffer that all peers can
// address (peer access inside one process, CUDA IPC between processes); all ranks use
// the same layout, so "slot X on rank p" is peer[p] + offset(X).
//
// One kernel per rank per collective.  Data moves by PUSH: a rank writes its partial
// straight into the consumer's staging with 128-bit stores over NVLink (posted writes:
// no round trip), then raises a flag there with a system-scope release store; the
// consumer polls its own memory with acquire loads.
//   one-shot : every rank pushes its whole partial to every peer, each rank sums all R
//              partials locally.  (R-1)*bytes per direction, one flag hop.
//   two-shot : rank r pushes slice s to rank s (reduce-scatter), rank s sums its slice
//              and pushes the result to everybody (all-gather).  2(R-1)/R*bytes, two hops.
// Partials are summed in rank order 0,1,.. in fp32 and rounded once
// (src/parallel/comm.rs:54-58 adds in the same order, rounding each partial sum).
//
// Reuse of the staging area is guarded by a per-rank "calls completed" flag that the
// last CTA of each kernel publishes to all peers; the next kernel waits for it before
// its first push.  All sequence numbers live in device memory, so a captured CUDA graph
// can replay the kernel.  Every wait is bounded; on expiry the kernel records
// HB_ERR_TIMEOUT in the status word and returns.
#include "comm.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <vector>

namespace hb {

constexpr int kArThreads = 512;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until *p >= target (flags only grow). false when the limit ran out.
__device__ __forceinline__ bool wait_ge(const uint32_t* p, uint32_t target, uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if ((int32_t)(ld_acquire_sys(p) - target) >= 0) return true;
    if (it > 64) __nanosleep(40);
  }
  return false;
}

struct ArParams {
  void* peer[HB_MAX_RANKS];
  void* buf;
  int ws, rank;
  int two_shot;
  int64_t total_vecs;   // 16-byte vectors in the message
  int64_t slice_vecs;   // two-shot: vectors per rank slice (one-shot: == total_vecs)
  int64_t vecs_per_cta; // sub-range of a slice handled by one CTA
  uint32_t spin;        // polls before a wait gives up
};

template <typename T>
__device__ __forceinline__ void acc_vec(float (&acc)[16 / sizeof(T)], const uint4& raw) {
  constexpr int N = 16 / sizeof(T);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] += to_f32<T>(e[i]);
}

template <typename T>
__global__ void __launch_bounds__(kArThreads)
all_reduce_kernel(const ArParams p) {
  constexpr int N = 16 / sizeof(T);
  __shared__ uint32_t s_seq;
  const int tid = threadIdx.x, b = blockIdx.x, R = p.ws, me = p.rank;
  CommFlags* fl = reinterpret_cast<CommFlags*>(p.peer[me]);
  auto peer_flags = [&](int q) { return reinterpret_cast<CommFlags*>(p.peer[q]); };
  auto peer_data = [&](int q) { return reinterpret_cast<uint4*>((uint8_t*)p.peer[q] + kFlagBytes); };
  uint4* buf = reinterpret_cast<uint4*>(p.buf);

  if (tid == 0) s_seq = *reinterpret_cast<volatile uint32_t*>(&fl->seq);
  __syncthreads();
  const uint32_t seq = s_seq, target = seq + 1;

  // A. every peer must have finished consuming the previous collective's data
  bool ok = true;
  if (tid < R && tid != me) ok = wait_ge(&fl->done[tid], seq, p.spin);
  bool all_ok = __syncthreads_and(ok ? 1 : 0) != 0;

  const int64_t v0 = (int64_t)b * p.vecs_per_cta;
  const int64_t v1 = min(v0 + p.vecs_per_cta, p.slice_vecs);

  if (all_ok) {
    // B. push
    if (!p.two_shot) {
      // slot[src] holds total_vecs vectors
      for (int64_t v = v0 + tid; v < v1; v += kArThreads) {
        const uint4 x = buf[v];
        for (int q = 0; q < R; ++q)
          if (q != me) peer_data(q)[(int64_t)me * p.slice_vecs + v] = x;
      }
    } else {
      for (int s = 0; s < R; ++s) {
        if (s == me) continue;
        uint4* dst = peer_data(s) + (int64_t)me * p.slice_vecs;  // slot1[src = me] on rank s
        for (int64_t v = v0 + tid; v < v1; v += kArThreads) {
          const int64_t g = (int64_t)s * p.slice_vecs + v;
          if (g < p.total_vecs) dst[v] = buf[g];
        }
      }
    }
    // bar.sync + the flag threads' system-scope release store publish every thread's stores
    __syncthreads();
    if (tid < R && tid != me) st_release_sys(&peer_flags(tid)->arrive1[b][me], target);
    ok = true;
    if (tid < R && tid != me) ok = wait_ge(&fl->arrive1[b][tid], target, p.spin);
    all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
  }

  if (all_ok) {
    // C. reduce this CTA's sub-range (of the whole message, or of slice `me`)
    const uint4* mine = peer_data(me);
    const int64_t base = p.two_shot ? (int64_t)me * p.slice_vecs : 0;
    for (int64_t v = v0 + tid; v < v1; v += kArThreads) {
      const int64_t g = base + v;
      if (g >= p.total_vecs) continue;
      float acc[N];
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = 0.f;
      for (int src = 0; src < R; ++src) {
        const uint4 x = (src == me) ? buf[g] : __ldcg(mine + (int64_t)src * p.slice_vecs + v);
        acc_vec<T>(acc, x);
      }
      uint4 r;
      T* e = reinterpret_cast<T*>(&r);
#pragma unroll
      for (int i = 0; i < N; ++i) e[i] = from_f32<T>(acc[i]);
      buf[g] = r;
      if (p.two_shot) {
        // slot2[slice me] on every peer sits after the R slot1 areas
        for (int q = 0; q < R; ++q)
          if (q != me) peer_data(q)[(int64_t)(R + me) * p.slice_vecs + v] = r;
      }
    }
    if (p.two_shot) {
      __syncthreads();
      if (tid < R && tid != me) st_release_sys(&peer_flags(tid)->arrive2[b][me], target);
      ok = true;
      if (tid < R && tid != me) ok = wait_ge(&fl->arrive2[b][tid], target, p.spin);
      all_ok = __syncthreads_and(ok ? 1 : 0) != 0;
      if (all_ok) {
        // D. gather the other ranks' reduced slices
        for (int s = 0; s < R; ++s) {
          if (s == me) continue;
          const uint4* src = mine + (int64_t)(R + s) * p.slice_vecs;
          for (int64_t v = v0 + tid; v < v1; v += kArThreads) {
            const int64_t g = (int64_t)s * p.slice_vecs + v;
            if (g < p.total_vecs) buf[g] = __ldcg(src + v);
          }
        }
      }
    }
  }

  // E. the last CTA publishes "this rank is done with call `target`"
  __syncthreads();
  if (tid == 0) {
    if (!all_ok) atomicExch(&fl->status, HB_ERR_TIMEOUT);
    __threadfence();
    const uint32_t prev = atomicAdd(&fl->finished, 1u);
    if (prev == gridDim.x - 1) {
      fl->finished = 0;
      *reinterpret_cast<volatile uint32_t*>(&fl->seq) = target;
      __threadfence_system();
      for (int q = 0; q < R; ++q)
        if (q != me) st_release_sys(&peer_flags(q)->done[me], target);
    }
  }
}

// ----------------------------------------------------------------------- NCCL
struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

static NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
    api.AllReduce = (decltype(api.AllReduce))dlsym(h, "ncclAllReduce");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
    api.ok = api.GetUniqueId && api.CommInitRank && api.AllReduce && api.CommDestroy;
  });
  return &api;
}

static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int world_all_reduce(hb_world* w, cudaStream_t st, void* buf, size_t count, hb_dtype dtype,
                     hb_algo algo) {
  if (!w) return fail(HB_ERR_INVALID_ARG, "all_reduce: null world");
  if (!dtype_valid(dtype)) return fail(HB_ERR_UNSUPPORTED_DTYPE, "all_reduce: unsupported dtype %d", (int)dtype);
  if (count == 0) return fail(HB_ERR_EMPTY, "all_reduce: shard is empty");
  if (!buf) return fail(HB_ERR_INVALID_ARG, "all_reduce: null buffer");
  if (w->ws == 1) return HB_OK;  // single shard is a passthrough (src/parallel/comm.rs:50)
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  if (algo == HB_ALGO_NCCL) {
    NcclApi* api = nccl_api();
    if (!w->nccl || !api->ok) return fail(HB_ERR_NCCL, "all_reduce: NCCL communicator not initialised");
    const ncclDataType_t dt = dtype == HB_F32 ? ncclFloat32 : dtype == HB_F16 ? ncclFloat16 : ncclBfloat16;
    ncclResult_t r = api->AllReduce(buf, buf, count, dt, ncclSum, (ncclComm_t)w->nccl, st);
    if (r != ncclSuccess)
      return fail(HB_ERR_NCCL, "ncclAllReduce: %s", api->GetErrorString ? api->GetErrorString(r) : "error");
    return HB_OK;
  }
  if (algo == HB_ALGO_MULTIMEM)
    return fail(HB_ERR_INVALID_ARG, "all_reduce: HB_ALGO_MULTIMEM exists for hb_all_reduce_add_rms_norm and hb_fused_rowparallel only");
  if ((int)algo < 0 || (int)algo > HB_ALGO_MULTIMEM) return fail(HB_ERR_INVALID_ARG, "all_reduce: unknown algorithm %d", (int)algo);
  if (!w->attached) return fail(HB_ERR_INVALID_ARG, "all_reduce: world not attached to its peers yet");
  const size_t bytes = count * dtype_size(dtype);
  if (bytes % 16 || (reinterpret_cast<uintptr_t>(buf) & 15))
    return fail(HB_ERR_INVALID_ARG, "all_reduce: buffer must be 16-byte aligned and a multiple of 16 bytes");
  const int R = w->ws;
  bool two = algo == HB_ALGO_TWO_SHOT;
  if (algo == HB_ALGO_AUTO) two = exchange_two_hops(R, bytes);
  ArParams p;
  memset(&p, 0, sizeof(p));
  for (int q = 0; q < R; ++q) p.peer[q] = w->peer[q];
  p.buf = buf;
  p.ws = R;
  p.rank = w->rank;
  p.two_shot = two ? 1 : 0;
  p.spin = w->wait_limit;
  p.total_vecs = (int64_t)(bytes / 16);
  p.slice_vecs = two ? (p.total_vecs + R - 1) / R : p.total_vecs;
  const size_t need = (size_t)p.slice_vecs * 16 * (two ? 2 * R : R);
  if (need > w->staging_bytes)
    return fail(HB_ERR_INVALID_ARG, "all_reduce: message of %zu bytes needs %zu bytes of staging, world has %zu",
                bytes, need, w->staging_bytes);
  // one CTA per 8 KiB of a slice, at most kMaxCommCtas
  int ctas = (int)std::min<int64_t>(kMaxCommCtas, std::max<int64_t>(1, (p.slice_vecs + 511) / 512));
  p.vecs_per_cta = (p.slice_vecs + ctas - 1) / ctas;
  ctas = (int)((p.slice_vecs + p.vecs_per_cta - 1) / p.vecs_per_cta);
  HB_DISPATCH_DTYPE(dtype, T, { all_reduce_kernel<T><<<ctas, kArThreads, 0, st>>>(p); });
  HB_LAUNCH_CHECK();
  return HB_OK;
}

static int world_alloc(hb_world* w, int ws, int rank, int device, size_t staging_bytes) {
  if (ws < 1 || ws > HB_MAX_RANKS)
    return fail(HB_ERR_INVALID_ARG, "tensor_parallel_size=%d outside [1, %d]", ws, HB_MAX_RANKS);
  if (rank < 0 || rank >= ws) return fail(HB_ERR_INVALID_ARG, "rank %d outside [0, %d)", rank, ws);
  const int ndev = hb_device_count();
  if (device < 0 || device >= ndev)
    return fail(HB_ERR_CUDA, "tensor_parallel_size=%d: CUDA device %d requested but only %d CUDA device(s) detected",
                ws, device, ndev);
  w->ws = ws; w->rank = rank; w->device = device;
  w->staging_bytes = round_up(staging_bytes ? staging_bytes : (size_t)64 << 20, 4096);
  HB_CUDA_CHECK(cudaSetDevice(device));
  HB_CUDA_CHECK(cudaMalloc(&w->local, kFlagBytes + w->staging_bytes));
  HB_CUDA_CHECK(cudaMemset(w->local, 0, kFlagBytes + w->staging_bytes));
  HB_CUDA_CHECK(cudaStreamCreateWithFlags(&w->stream, cudaStreamNonBlocking));
  HB_CUDA_CHECK(cudaMallocHost((void**)&w->host_status, sizeof(int32_t)));
  *w->host_status = 0;
  w->peer[rank] = w->local;
  w->attached = (ws == 1);
  HB_CUDA_CHECK(cudaDeviceSynchronize());
  return HB_OK;
}

}  // namespace hb

extern "C" {

int hb_world_create_rank(int world_size, int rank, int device, size_t staging_bytes,
                         hb_world** out) {
  HB_CHECK_ARG(out, "hb_world_create_rank: null output");
  hb_world* w = new hb_world;
  int rc = hb::world_alloc(w, world_size, rank, device, staging_bytes);
  if (rc) { hb_world_free(w); return rc; }
  *out = w;
  return HB_OK;
}

int hb_world_create_local(int n, const int* device_ids, size_t staging_bytes,
                          hb_world** worlds_out) {
  HB_CHECK_ARG(worlds_out, "hb_world_create_local: null output");
  HB_CHECK_ARG(n >= 1 && n <= HB_MAX_RANKS, "tensor_parallel_size=%d outside [1, %d]", n, HB_MAX_RANKS);
  const int ndev = hb_device_count();
  // Without an explicit device list rank i runs on device i and n devices must exist
  // (world.rs:108-114).  An explicit list may name a device more than once (ranks that share
  // a GPU: useful for exercising the protocol, not for speed).
  if (n > 1 && !device_ids && ndev < n)
    return hb::fail(HB_ERR_CUDA,
                    "tensor_parallel_size=%d requested but only %d CUDA device(s) detected. "
                    "Use tensor_parallel_size 1 for single-GPU.", n, ndev);
  std::vector<hb_world*> ws(n, nullptr);
  int rc = HB_OK;
  for (int i = 0; i < n && !rc; ++i) {
    ws[i] = new hb_world;
    rc = hb::world_alloc(ws[i], n, i, device_ids ? device_ids[i] : i, staging_bytes);
  }
  for (int i = 0; i < n && !rc; ++i) {
    cudaSetDevice(ws[i]->device);
    for (int j = 0; j < n && !rc; ++j) {
      if (i == j) continue;
      if (ws[i]->device == ws[j]->device) { ws[i]->peer[j] = ws[j]->local; continue; }
      int can = 0;
      cudaDeviceCanAccessPeer(&can, ws[i]->device, ws[j]->device);
      if (!can) { rc = hb::fail(HB_ERR_CUDA, "device %d cannot access device %d", ws[i]->device, ws[j]->device); break; }
      cudaError_t ce = cudaDeviceEnablePeerAccess(ws[j]->device, 0);
      if (ce != cudaSuccess && ce != cudaErrorPeerAccessAlreadyEnabled) {
        rc = hb::fail(HB_ERR_CUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(ce));
        break;
      }
      cudaGetLastError();
      ws[i]->peer[j] = ws[j]->local;
    }
    ws[i]->attached = true;
  }
  if (rc) {
    for (auto* w : ws) hb_world_free(w);
    return rc;
  }
  for (int i = 0; i < n; ++i) worlds_out[i] = ws[i];
  return HB_OK;
}

int hb_world_ipc_handle(hb_world* w, void* handle_out) {
  HB_CHECK_ARG(w && handle_out, "hb_world_ipc_handle: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == HB_IPC_HANDLE_BYTES, "IPC handle size");
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  cudaIpcMemHandle_t h;
  HB_CUDA_CHECK(cudaIpcGetMemHandle(&h, w->local));
  memcpy(handle_out, &h, sizeof(h));
  return HB_OK;
}

int hb_world_attach(hb_world* w, const void* all_handles) {
  HB_CHECK_ARG(w && all_handles, "hb_world_attach: null argument");
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  for (int q = 0; q < w->ws; ++q) {
    if (q == w->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const uint8_t*)all_handles + (size_t)q * HB_IPC_HANDLE_BYTES, sizeof(h));
    void* p = nullptr;
    HB_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    w->peer[q] = p;
    w->ipc_open[q] = true;
  }
  w->attached = true;
  return HB_OK;
}

int hb_world_attach_ptrs(hb_world* w, void* const* peer_ptrs) {
  HB_CHECK_ARG(w && peer_ptrs, "hb_world_attach_ptrs: null argument");
  for (int q = 0; q < w->ws; ++q) {
    HB_CHECK_ARG(peer_ptrs[q], "hb_world_attach_ptrs: null pointer for rank %d", q);
    if (q == w->rank) {
      if (peer_ptrs[q] != w->local) {
        // adopt the caller's buffer as this rank's staging
        HB_CUDA_CHECK(cudaSetDevice(w->device));
        if (w->owns_local && w->local) cudaFree(w->local);
        w->local = peer_ptrs[q];
        w->owns_local = false;
        HB_CUDA_CHECK(cudaMemset(w->local, 0, hb::kFlagBytes));
        HB_CUDA_CHECK(cudaDeviceSynchronize());
      }
      w->peer[q] = w->local;
    } else {
      w->peer[q] = peer_ptrs[q];
    }
  }
  w->attached = true;
  return HB_OK;
}

int hb_nccl_unique_id(void* id_out) {
  HB_CHECK_ARG(id_out, "hb_nccl_unique_id: null output");
  static_assert(sizeof(ncclUniqueId) == HB_NCCL_ID_BYTES, "NCCL id size");
  hb::NcclApi* api = hb::nccl_api();
  if (!api->ok) return hb::fail(HB_ERR_NCCL, "libnccl.so.2 could not be loaded");
  ncclUniqueId id;
  ncclResult_t r = api->GetUniqueId(&id);
  if (r != ncclSuccess) return hb::fail(HB_ERR_NCCL, "ncclGetUniqueId failed (%d)", (int)r);
  memcpy(id_out, &id, sizeof(id));
  return HB_OK;
}

int hb_world_init_nccl(hb_world* w, const void* id) {
  HB_CHECK_ARG(w && id, "hb_world_init_nccl: null argument");
  hb::NcclApi* api = hb::nccl_api();
  if (!api->ok) return hb::fail(HB_ERR_NCCL, "libnccl.so.2 could not be loaded");
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof(uid));
  ncclComm_t comm = nullptr;
  ncclResult_t r = api->CommInitRank(&comm, w->ws, uid, w->rank);
  if (r != ncclSuccess)
    return hb::fail(HB_ERR_NCCL, "NCCL communicator init failed: %s",
                    api->GetErrorString ? api->GetErrorString(r) : "error");
  w->nccl = comm;
  return HB_OK;
}

int hb_world_free(hb_world* w) {
  if (!w) return HB_OK;
  cudaSetDevice(w->device);
  cudaDeviceSynchronize();
  if (w->nccl && hb::nccl_api()->ok) hb::nccl_api()->CommDestroy((ncclComm_t)w->nccl);
  for (int q = 0; q < HB_MAX_RANKS; ++q)
    if (w->ipc_open[q] && w->peer[q]) cudaIpcCloseMemHandle(w->peer[q]);
  if (w->owns_local && w->local) cudaFree(w->local);
  if (w->stream) cudaStreamDestroy(w->stream);
  if (w->host_status) cudaFreeHost(w->host_status);
  cudaGetLastError();
  delete w;
  return HB_OK;
}

int hb_world_size(const hb_world* w) { return w ? w->ws : HB_ERR_INVALID_ARG; }
int hb_world_rank(const hb_world* w) { return w ? w->rank : HB_ERR_INVALID_ARG; }
int hb_world_device(const hb_world* w) { return w ? w->device : HB_ERR_INVALID_ARG; }
int hb_world_is_single(const hb_world* w) { return w ? (w->ws == 1 ? 1 : 0) : HB_ERR_INVALID_ARG; }
size_t hb_world_staging_bytes(const hb_world* w) { return w ? w->staging_bytes : 0; }
void* hb_world_stream(const hb_world* w) { return w ? (void*)w->stream : nullptr; }

int hb_world_status(hb_world* w) {
  HB_CHECK_ARG(w, "hb_world_status: null world");
  if (!w->local) return HB_OK;
  HB_CUDA_CHECK(cudaSetDevice(w->device));
  hb::CommFlags* fl = (hb::CommFlags*)w->local;
  HB_CUDA_CHECK(cudaMemcpy(w->host_status, &fl->status, sizeof(int32_t), cudaMemcpyDeviceToHost));
  const int s = *w->host_status;
  if (s) {
    // reading the status clears it: the next collective reports for itself
    HB_CUDA_CHECK(cudaMemset(&fl->status, 0, sizeof(int32_t)));
    hb::set_error("a bounded wait on a peer flag ran out (status %d)", s);
  }
  return s;
}

int hb_world_set_wait_limit(hb_world* w, uint32_t polls) {
  HB_CHECK_ARG(w, "hb_world_set_wait_limit: null world");
  w->wait_limit = polls ? polls : (1u << 22);
  return HB_OK;
}


int hb_all_reduce(hb_world* w, void* stream, void* buf, size_t count, hb_dtype dtype,
                  hb_algo algo) {
  return hb::world_all_reduce(w, (cudaStream_t)stream, buf, count, dtype, algo);
}

}  // extern "C"
