// Fused row-parallel projection: ONE kernel per rank computes
//
//   resid_out  = resid_in + SUM_ranks( X_r[M,Kl] . W_r[N,Kl]^T )
//   normed_out = resid_out * rsqrt(mean(resid_out^2) + eps) * norm_w
//
// i.e. o_proj / down_proj -> all_reduce -> residual add -> next RMSNorm of the layer
// loop (src/engine/arch/llama_tp.rs:327,533-552 and :339,563-571,517-522), which the
// reference runs as a library GEMM, an NCCL all-reduce, peer copies and a norm kernel.
//
// Phases of a CTA = (128-feature tile t, K split s):
//   1. tcgen05 mainloop (TMA -> shared memory -> UMMA, fp32 accumulator in tensor
//      memory), exactly the decode GEMM: the weight slab is the UMMA A operand.
//   2. split-K: partials meet in local scratch; the last CTA of a tile goes on as the
//      tile's "finisher", the others exit.
//   3. the finisher rounds the rank's partial tile to bf16 (the reference's partials are
//      bf16 tensors), stages it in shared memory and PUSHES it with coalesced 128-bit
//      stores into the staging buffer of the tile's reducer rank(s) over NVLink, then
//      raises pflag[t][me] there.  two-shot: the reducer of tile t is rank t/(T/R);
//      one-shot: every rank reduces every tile (one NVLink hop, R-1 times the bytes).
//   4. a reducer waits for the R-1 remote partials of its tile, sums all R in rank
//      order in fp32 on top of the residual, rounds, writes resid_out, accumulates the
//      per-row sum of squares of the rounded tile, and (two-shot) pushes the reduced
//      tile and the row sums to every peer, then raises gflag[t] everywhere.
//   5. every finisher waits until all T tiles (hence all row sums) are present locally,
//      computes the row scales and writes its tile of normed_out (non-reducers also copy
//      the gathered tile into resid_out).
// Flags carry the device-resident call sequence number, so a captured CUDA graph can
// replay the kernel; staging reuse is guarded by the per-rank "done" flags shared with
// the all-reduce kernel.  The grid is launched cooperatively (all CTAs co-resident)
// because finishers wait for other CTAs of the same grid.  All waits are bounded.
#include <algorithm>
#include <mutex>

#include "comm.h"
#include "gemm.h"
#include "rowpar.h"
#include "tc_core.cuh"

namespace hb {

constexpr uint32_t kFusedFlagSpin = 1u << 22;

struct FusedParams {
  int M, N, m_pad, splits, stages, tmem_cols, k_chunks, n_tiles;
  int ws, rank, two_shot, tiles_own;   // tiles_own: tiles a reducer owns (T/R or T)
  float eps;
  const __nv_bfloat16* resid_in;
  __nv_bfloat16* resid_out;
  __nv_bfloat16* normed_out;           // may be null
  const __nv_bfloat16* norm_w;
  float* partials;                     // split-K scratch [tile][split][m_pad][128] fp32
  int* counters;                       // [n_tiles], zero between launches
  void* peer[HB_MAX_RANKS];            // staging base of every rank (flags + data)
  int64_t tile_bytes;                  // M * 128 * 2
  int64_t gather_off, rowsq_off;       // byte offsets inside the data area
};

__device__ __forceinline__ uint32_t f_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void f_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool f_wait_ge(const uint32_t* p, uint32_t target) {
  for (uint32_t it = 0; it < kFusedFlagSpin; ++it) {
    if ((int32_t)(f_ld_acquire(p) - target) >= 0) return true;
    if (it > 32) __nanosleep(32);
  }
  return false;
}
__device__ __forceinline__ void bf16x8_to_f32(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float (&f)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}

__global__ void __launch_bounds__(kTcThreads, 1)
rowpar_fused_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    const FusedParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kMaxStages];
  __shared__ __align__(8) uint64_t s_done;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_last;
  __shared__ uint32_t s_seq;
  __shared__ float s_rowsq[256];
  __shared__ float s_rs[256];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x / p.splits;
  const int split = blockIdx.x % p.splits;
  const int base_c = p.k_chunks / p.splits, rem_c = p.k_chunks % p.splits;
  const int kc0 = split * base_c + min(split, rem_c);
  const int n_kc = base_c + (split < rem_c ? 1 : 0);

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));  // generic view of the same bytes
  const uint32_t a_bytes = kTileN * kTileK * 2;
  const uint32_t b_bytes = (uint32_t)p.m_pad * kTileK * 2;
  const uint32_t stage_bytes = a_bytes + b_bytes;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    mbar_init(smem_u32(&s_done), 1);
    s_abort = 0;
    s_last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;

  // ------------------------------------------------------------ 1. mainloop
  if (warp == 0) {
    if (lane == 0) {
      int armed = 0;
      for (int i = 0; i < n_kc; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        if (i >= p.stages && !mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, &s_abort)) break;
        const uint32_t full = smem_u32(&s_full[s]);
        const uint32_t sa = smem_base + s * stage_bytes;
        mbar_expect_tx(full, stage_bytes);
        const int kx = (kc0 + i) * kTileK;
        tma_load_2d(sa, &tm_w, kx, tile * kTileN, full);
        tma_load_2d(sa + a_bytes, &tm_x, kx, 0, full);
        armed = i + 1;
      }
      if (s_abort) {
        for (int i = max(0, armed - p.stages); i < armed; ++i) {
          const int s = i % p.stages;
          const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
          for (uint32_t it = 0; it < kSpinLimit && !mbar_try(smem_u32(&s_full[s]), ph); ++it) {
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(p.m_pad);
      bool ok = true;
      for (int i = 0; i < n_kc && ok; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        ok = mbar_wait(smem_u32(&s_full[s]), ph, &s_abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_base + s * stage_bytes;
        const uint64_t a_desc = make_smem_desc(sa);
        const uint64_t b_desc = make_smem_desc(sa + a_bytes);
#pragma unroll
        for (int k = 0; k < kTileK / kUmmaK; ++k)
          umma_bf16(tmem_base, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc,
                    (i > 0 || k > 0) ? 1u : 0u);
        tc_commit(smem_u32(&s_empty[s]));
      }
      if (ok) tc_commit(smem_u32(&s_done));
    }
    __syncwarp();
  }

  const bool have_acc = mbar_wait(smem_u32(&s_done), 0, &s_abort);
  tc_fence_after();
  const int row = warp * 32 + lane;  // accumulator row = feature inside the tile
  const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
  bool ok_all = __syncthreads_and(have_acc ? 1 : 0) != 0;
  bool finisher = ok_all;

  // ------------------------------------------------------------ 2. split-K
  if (ok_all && p.splits > 1) {
    float* mine = p.partials + ((int64_t)tile * p.splits + split) * (int64_t)p.m_pad * kTileN;
    for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
      float v[16];
      tmem_ld16(t_lane + c0, v);
#pragma unroll
      for (int j = 0; j < 16; ++j) mine[(int64_t)(c0 + j) * kTileN + row] = v[j];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int prev = atomicAdd(&p.counters[tile], 1);
      s_last = (prev == p.splits - 1);
      if (s_last) p.counters[tile] = 0;
    }
    __syncthreads();
    finisher = s_last != 0;
    if (finisher) __threadfence();
  }

  CommFlags* fl = reinterpret_cast<CommFlags*>(p.peer[p.rank]);
  bool proto_ok = true;

  if (finisher) {
    const int R = p.ws, me = p.rank, T = p.n_tiles;
    __nv_bfloat16* tile_s = reinterpret_cast<__nv_bfloat16*>(smem_gen);  // [M][128] bf16
    uint4* tile_u4 = reinterpret_cast<uint4*>(smem_gen);
    const int n_u4 = p.M * 16;  // 16-byte vectors in the tile

    // ---- 3a. this rank's partial tile, rounded to bf16, into shared memory
    if (p.splits == 1) {
      for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
        float v[16];
        tmem_ld16(t_lane + c0, v);
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c0 + j < p.M) tile_s[(c0 + j) * kTileN + row] = __float2bfloat16_rn(v[j]);
      }
    } else {
      const float* base = p.partials + (int64_t)tile * p.splits * (int64_t)p.m_pad * kTileN + row;
      const int64_t sstride = (int64_t)p.m_pad * kTileN;
      for (int m0 = 0; m0 < p.M; m0 += 8) {
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 0.f;
        for (int s = 0; s < p.splits; ++s) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (m0 + j < p.M) g[j] += __ldcg(base + s * sstride + (int64_t)(m0 + j) * kTileN);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (m0 + j < p.M) tile_s[(m0 + j) * kTileN + row] = __float2bfloat16_rn(g[j]);
      }
    }
    if (tid == 0) s_seq = *reinterpret_cast<volatile uint32_t*>(&fl->seq);
    __syncthreads();
    const uint32_t seq = s_seq, target = seq + 1;

    const int owner = p.two_shot ? tile / p.tiles_own : me;
    const bool reducer = !p.two_shot || owner == me;
    const int t_slot = p.two_shot ? tile - owner * p.tiles_own : tile;
    auto data_of = [&](int q) { return (uint8_t*)p.peer[q] + kFlagBytes; };
    auto flags_of = [&](int q) { return reinterpret_cast<CommFlags*>(p.peer[q]); };
    auto part_slot = [&](int q, int src, int slot) {
      return reinterpret_cast<uint4*>(data_of(q) + ((int64_t)src * p.tiles_own + slot) * p.tile_bytes);
    };

    if (R > 1) {
      // ---- A. peers must be done with the previous collective before their staging is written
      bool ok = true;
      if (tid < R && tid != me) ok = f_wait_ge(&fl->done[tid], seq);
      proto_ok = __syncthreads_and(ok ? 1 : 0) != 0;
      // ---- 3b. push the partial to the reducer(s)
      if (proto_ok) {
        for (int q = 0; q < R; ++q) {
          if (q == me || (p.two_shot && q != owner)) continue;
          uint4* dst = part_slot(q, me, t_slot);
          for (int i = tid; i < n_u4; i += kTcThreads) dst[i] = tile_u4[i];
        }
        __threadfence_system();
        __syncthreads();
        if (tid < R && tid != me && (!p.two_shot || tid == owner))
          f_st_release(&flags_of(tid)->pflag[tile * HB_MAX_RANKS + me], target);
      }
    }

    // ---- 4. reduce
    if (proto_ok && reducer) {
      if (R > 1) {
        bool ok = true;
        if (tid < R && tid != me) ok = f_wait_ge(&fl->pflag[tile * HB_MAX_RANKS + tid], target);
        proto_ok = __syncthreads_and(ok ? 1 : 0) != 0;
      }
      if (proto_ok) {
        for (int i0 = 0; i0 < n_u4; i0 += kTcThreads) {
          const int i = i0 + tid;
          float ss = 0.f;
          if (i < n_u4) {
            const int m = i >> 4, c = i & 15;
            const int64_t g_off = (int64_t)m * p.N + tile * kTileN + c * 8;
            float acc[8], t8[8];
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(p.resid_in + g_off), acc);
            for (int src = 0; src < R; ++src) {
              const uint4 raw = (src == me) ? tile_u4[i] : __ldcg(part_slot(me, src, t_slot) + i);
              bf16x8_to_f32(raw, t8);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] += t8[j];
            }
            const uint4 out = f32_to_bf16x8(acc);
            bf16x8_to_f32(out, t8);  // the norm sees the rounded residual
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += t8[j] * t8[j];
            tile_u4[i] = out;
            *reinterpret_cast<uint4*>(p.resid_out + g_off) = out;
          }
          // 16 consecutive lanes hold one batch row of the tile
#pragma unroll
          for (int o = 8; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (i < n_u4 && (i & 15) == 0) s_rowsq[i >> 4] = ss;
        }
        __syncthreads();
        float* my_rowsq = reinterpret_cast<float*>(data_of(me) + p.rowsq_off) + (int64_t)tile * p.M;
        for (int m = tid; m < p.M; m += kTcThreads) my_rowsq[m] = s_rowsq[m];
        if (R > 1 && p.two_shot) {
          for (int q = 0; q < R; ++q) {
            if (q == me) continue;
            uint4* dst = reinterpret_cast<uint4*>(data_of(q) + p.gather_off + (int64_t)tile * p.tile_bytes);
            for (int i = tid; i < n_u4; i += kTcThreads) dst[i] = tile_u4[i];
            float* rq = reinterpret_cast<float*>(data_of(q) + p.rowsq_off) + (int64_t)tile * p.M;
            for (int m = tid; m < p.M; m += kTcThreads) rq[m] = s_rowsq[m];
          }
        }
        __threadfence_system();
        __syncthreads();
        if (tid == 0) f_st_release(&fl->gflag[tile], target);
        if (R > 1 && p.two_shot && tid < R && tid != me) f_st_release(&flags_of(tid)->gflag[tile], target);
      }
    }

    // ---- 5. all tiles present -> row scales -> normalise this tile
    if (proto_ok) {
      bool ok = true;
      for (int t2 = tid; t2 < T; t2 += kTcThreads) ok = ok && f_wait_ge(&fl->gflag[t2], target);
      proto_ok = __syncthreads_and(ok ? 1 : 0) != 0;
    }
    if (proto_ok) {
      const float* rowsq = reinterpret_cast<const float*>(data_of(me) + p.rowsq_off);
      for (int m = tid; m < p.M; m += kTcThreads) {
        float s = 0.f;
        for (int t2 = 0; t2 < T; ++t2) s += __ldcg(rowsq + (int64_t)t2 * p.M + m);
        s_rs[m] = rsqrtf(s / (float)p.N + p.eps);
      }
      if (!reducer) {
        const uint4* src = reinterpret_cast<const uint4*>(data_of(me) + p.gather_off + (int64_t)tile * p.tile_bytes);
        for (int i = tid; i < n_u4; i += kTcThreads) {
          const uint4 v = __ldcg(src + i);
          tile_u4[i] = v;
          const int m = i >> 4, c = i & 15;
          *reinterpret_cast<uint4*>(p.resid_out + (int64_t)m * p.N + tile * kTileN + c * 8) = v;
        }
      }
      __syncthreads();
      if (p.normed_out) {
        for (int i = tid; i < n_u4; i += kTcThreads) {
          const int m = i >> 4, c = i & 15;
          float h[8], w8[8];
          bf16x8_to_f32(tile_u4[i], h);
          bf16x8_to_f32(*reinterpret_cast<const uint4*>(p.norm_w + tile * kTileN + c * 8), w8);
          const float r = s_rs[m];
#pragma unroll
          for (int j = 0; j < 8; ++j) h[j] = h[j] * r * w8[j];
          *reinterpret_cast<uint4*>(p.normed_out + (int64_t)m * p.N + tile * kTileN + c * 8) = f32_to_bf16x8(h);
        }
      }
    }

    // ---- E. the last finisher closes the collective
    __syncthreads();
    if (tid == 0) {
      if (!proto_ok) atomicExch(&fl->status, HB_ERR_TIMEOUT);
      __threadfence();
      const uint32_t prev = atomicAdd(&fl->finished, 1u);
      if (prev == (uint32_t)T - 1) {
        fl->finished = 0;
        *reinterpret_cast<volatile uint32_t*>(&fl->seq) = target;
        __threadfence_system();
        for (int q = 0; q < R; ++q)
          if (q != me) f_st_release(&flags_of(q)->done[me], target);
      }
    }
  } else if (!ok_all && tid == 0) {
    atomicExch(&fl->status, HB_ERR_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

// ------------------------------------------------------------------------ host
// Layout of the caller's workspace (zero-initialised once, left clean by every call):
//   [0, 64K)          split-K tile counters
//   [64K, 128K)       flag block   } single-rank only: the memory that a multi-rank
//   [128K, 384K)      row sums     } world keeps in its staging buffer
//   [384K, ...)       split-K fp32 partials
// All offsets are fixed, so calls of different shapes may share one workspace.
constexpr size_t kFusedRowsqBytes = (size_t)kMaxFusedTiles * 256 * sizeof(float);
constexpr size_t kFusedPartialsOff = kCounterBlockBytes + kFlagBytes + kFusedRowsqBytes;

struct FusedPlan {
  TcGemmPlan g;        // tensor maps and tile geometry (epilogue unused)
  int splits = 1;
  int capacity = 0;    // co-resident CTAs of the kernel on this device
  size_t partials_bytes = 0;
};

static int fused_capacity(int device, size_t smem_bytes, int* out) {
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  static bool attr_done[64] = {false};
  if (device >= 0 && device < 64 && !attr_done[device]) {
    HB_CUDA_CHECK(cudaFuncSetAttribute(rowpar_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       224 * 1024));
    attr_done[device] = true;
  }
  int per_sm = 0;
  HB_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rowpar_fused_kernel, kTcThreads,
                                                              smem_bytes));
  DeviceInfo di;
  int rc = device_info(device, &di);
  if (rc) return rc;
  *out = per_sm * di.sm_count;
  return HB_OK;
}

static int fused_plan(FusedPlan* fp, const void* X, const void* W, int64_t M, int64_t N, int64_t Kl,
                      int device) {
  int rc = gemm_tc_plan(&fp->g, X, W, M, N, Kl, kEpiStore, false, device, 1);
  if (rc) return rc;
  if ((rc = fused_capacity(device, fp->g.smem_bytes, &fp->capacity))) return rc;
  // tensor memory: two CTAs per SM at most share the 512 columns
  const int k_chunks = (int)(Kl / kTileK);
  // same rule as the plain GEMM: a split through global scratch pays off only for few
  // tiles with a deep K
  int s = (fp->g.n_tiles <= 40 && k_chunks >= 128) ? 2 : 1;
  if (const char* ev = getenv("HB_FUSED_SPLITS")) s = std::max(1, std::min(std::min(atoi(ev), 4), k_chunks));
  while (s > 1 && fp->g.n_tiles * s > fp->capacity) --s;
  fp->splits = s;
  fp->partials_bytes = s > 1 ? (size_t)fp->g.n_tiles * s * fp->g.m_pad * kTileN * sizeof(float) : 0;
  return HB_OK;
}

bool rowpar_fused_supported(const hb_world* w, int64_t M, int64_t N, int64_t K_local) {
  if (M < 1 || M > 256 || N % kTileN != 0 || N / kTileN > kMaxFusedTiles) return false;
  if (K_local < kTileK || K_local % kTileK != 0) return false;
  if (w && w->ws > 1 && !w->attached) return false;
  return true;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t rowpar_fused_workspace_bytes(int64_t M, int64_t N, int64_t K_local) {
  if (!rowpar_fused_supported(nullptr, M, N, K_local)) return 0;
  const size_t m_pad = (size_t)std::max<int64_t>(16, (M + 15) / 16 * 16);
  const size_t tiles = (size_t)(N / kTileN);
  // bound on the partials for any split factor the plan may choose (<= 4)
  return kFusedPartialsOff + tiles * 4 * m_pad * kTileN * sizeof(float) + 256;
}

int rowpar_fused(hb_world* w, cudaStream_t st, void* normed_out, void* resid_out, const void* X,
                 const void* W, const void* resid_in, const void* norm_w, int64_t M, int64_t N,
                 int64_t K_local, float eps, hb_algo algo, void* workspace) {
  int device = 0;
  if (w) { device = w->device; HB_CUDA_CHECK(cudaSetDevice(device)); }
  else HB_CUDA_CHECK(cudaGetDevice(&device));
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al16(resid_in) || !al16(resid_out) || !al16(normed_out) || !al16(norm_w) || !al16(workspace))
    return fail(HB_ERR_INVALID_ARG, "fused row-parallel: buffers must be 16-byte aligned");
  FusedPlan fp;
  int rc = fused_plan(&fp, X, W, M, N, K_local, device);
  if (rc) return rc;
  const int R = w ? w->ws : 1;
  const int T = fp.g.n_tiles;
  FusedParams p;
  memset(&p, 0, sizeof(p));
  p.M = (int)M; p.N = (int)N; p.m_pad = fp.g.m_pad; p.splits = fp.splits; p.stages = fp.g.stages;
  p.tmem_cols = fp.g.tmem_cols; p.k_chunks = (int)(K_local / kTileK); p.n_tiles = T;
  p.ws = R; p.rank = w ? w->rank : 0;
  p.eps = eps;
  p.resid_in = (const __nv_bfloat16*)resid_in;
  p.resid_out = (__nv_bfloat16*)resid_out;
  p.normed_out = (__nv_bfloat16*)normed_out;
  p.norm_w = (const __nv_bfloat16*)norm_w;
  uint8_t* wsb = (uint8_t*)workspace;
  p.counters = (int*)wsb;
  p.partials = (float*)(wsb + kFusedPartialsOff);
  p.tile_bytes = (int64_t)M * kTileN * 2;
  bool two = false;
  if (R > 1) {
    two = algo == HB_ALGO_TWO_SHOT || (algo == HB_ALGO_AUTO && R > 2 && (size_t)M * N * 2 >= 256 * 1024);
    if (T % R != 0) two = false;
  }
  p.two_shot = two ? 1 : 0;
  p.tiles_own = two ? T / R : T;
  const size_t part_area = (size_t)R * p.tiles_own * p.tile_bytes;
  p.gather_off = (int64_t)align_up(part_area, 256);
  p.rowsq_off = p.gather_off + (int64_t)align_up(two ? (size_t)T * p.tile_bytes : 0, 256);
  const size_t need = (size_t)p.rowsq_off + (size_t)T * M * sizeof(float);
  if (R > 1) {
    if (need > w->staging_bytes)
      return fail(HB_ERR_INVALID_ARG, "fused row-parallel: needs %zu bytes of staging, world has %zu", need,
                  w->staging_bytes);
    for (int q = 0; q < R; ++q) p.peer[q] = w->peer[q];
  } else {
    // single rank: flag block and row sums live in the caller's workspace
    p.peer[0] = wsb + kCounterBlockBytes;
    p.gather_off = 0;
    p.rowsq_off = 0;
  }
  if (T * fp.splits > fp.capacity)
    return fail(HB_ERR_INVALID_ARG, "fused row-parallel: %d tiles do not fit the %d co-resident CTAs", T,
                fp.capacity);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(T * fp.splits));
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = fp.g.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  HB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, rowpar_fused_kernel, fp.g.tm_w, fp.g.tm_x, p));
  return HB_OK;
}

}  // namespace hb
