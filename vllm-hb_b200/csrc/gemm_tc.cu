// bf16 GEMM for decode shapes on 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
//   Y[M,N] = X[M,K] . W[N,K]^T        M = batch (1..256 per tile), weights [out,in]
//
// Decode is weight streaming: the whole of W is read once per step and M is small.
// So the operands are swapped: a 128-row slab of W is the UMMA "A" operand (M=128)
// and the batch X is the "B" operand (UMMA N = batch padded to 16).  Both are K-major,
// which is how they already lie in memory, so TMA drops 128x64 and m_padx64 bf16
// boxes with the 128-byte swizzle straight into shared memory and tcgen05.mma reads
// them through shared-memory descriptors; the fp32 accumulator [128 x m_pad] lives in
// tensor memory.  Split-K spreads a weight matrix with few row slabs over all SMs:
// every CTA owns (slab, K range).  The partners of a slab form a thread-block cluster:
// CTA r owns the batch rows [r*m_pad/S, (r+1)*m_pad/S) of the tile, receives the other
// partners' accumulator columns for those rows through distributed shared memory, adds
// them in split order (deterministic) and runs the epilogue; the output tile leaves
// through one bulk tensor store.  Plans that cannot form a cluster write fp32 partials
// to global scratch and the last CTA to arrive for a slab sums them.
// Epilogues: store (bf16 / fp32), SwiGLU over [gate ; up] slabs, residual add with the
// deferred RMSNorm (producer and consumer side, TcNormLink), RoPE + paged KV write for
// the q|k|v projection, per-expert routing weight.
// The kernel is launched programmatically: it requests its first weight stages before
// griddepcontrol.wait (weights never depend on the previous kernel), activations after.
//
// CTA = 4 warps.  Warp 0 lane 0 issues TMA, warp 1 lane 0 issues MMAs, all four warps
// read the accumulator (warp w owns TMEM lanes 32w..32w+31 = output features).
// Every wait is bounded: on expiry the kernel raises *err_flag, lets outstanding
// copies land, frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <mutex>

#include "comm.h"
#include "common.h"
#include "gemm.h"
#include "peer_sync.cuh"
#include "tc_core.cuh"

namespace hb {

struct TcParams {
  int M, N;                 // N = weight rows (for SwiGLU: rows of gate == rows of up)
  int m_pad, splits, stages, tmem_cols;
  int k_chunks;             // K / 64
  int n_tiles;
  int epilogue, out_f32;
  int64_t ldy;
  int up_row_offset;        // SwiGLU: first row of the up projection inside W
  int cluster;              // split-K partners form a thread-block cluster of `splits` CTAs
  int tma_store;            // the output leaves through bulk tensor stores (tm_y is valid)
  // Deferred RMSNorm (see TcNormLink in gemm.h).  Producer (epilogue kEpiResidual, cluster
  // form only): h = resid + Y, written through tm_h; Y' = h * norm_w written through tm_y;
  // row sums of h^2 over this tile's 128 features to rowsq_out[row * rowsq_stride + tile].
  // Consumer (rowsq_in != null): every accumulator column (batch row) is multiplied by
  // rsqrt(sum over rowsq_tiles entries / rs_n + rs_eps) before the epilogue.
  const __nv_bfloat16* norm_w;
  float* rowsq_out;
  const float* rowsq_in;
  int rowsq_stride, rowsq_tiles;
  float rs_inv_n, rs_eps;
  // Mixture of experts: output tile t belongs to expert t / post_tiles_per_group; after the
  // activation every batch row m is multiplied by post_scale[m * post_groups + expert].
  const float* post_scale;
  int post_groups, post_tiles_per_group;
  // RoPE + paged KV write (see TcNormLink): tile t is head t of the [q|k|v] row.
  const float2* rope_cs;
  const int64_t* kv_slots;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  int rope_nq, rope_nkv;
  int64_t kv_num_blocks;
  // kEpiPush (see TcNormLink): staging bases of all ranks, this rank, tiles and 16-byte
  // vectors per rank slice, poll limit
  void* push_peer[HB_MAX_RANKS];
  int push_R, push_me, push_T;
  int64_t push_sv;
  uint32_t push_spin;
  uint32_t* ready_mc;       // see TcNormLink::ready_mc
  uint32_t* ready_calls;
  uint32_t* ready_ctas;
  int recv_dedicated;       // cluster plans: the receive area of the exchange lies behind the pipeline buffers
  void* Y;
  float* partials;
  int* counters;
  int* err_flag;
  int trace_id;             // trace build only: slot of this launch in the launch ring
};

// Optional phase timestamps (compiled in with -DHB_TC_TRACE only): every CTA records
// the global timer at eight points of its life into a device array that
// hb_debug_tc_trace() copies out.
#ifdef HB_TC_TRACE
constexpr int kTraceCtas = 4096, kTraceSlots = 16;
static __device__ unsigned long long g_tc_trace[kTraceCtas * kTraceSlots];
__device__ __forceinline__ void tc_trace(int slot) {
  const int cta = blockIdx.y * gridDim.x + blockIdx.x;
  if (cta >= kTraceCtas) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  g_tc_trace[cta * kTraceSlots + slot] = t;
  if (slot == 0) {
    unsigned sm;
    asm volatile("mov.u32 %0, %smid;" : "=r"(sm));
    g_tc_trace[cta * kTraceSlots + 9] = sm;
    g_tc_trace[cta * kTraceSlots + 8] = (unsigned long long)clock64();
  }
  if (slot == 7) g_tc_trace[cta * kTraceSlots + 15] = (unsigned long long)clock64();
}
#define TC_TRACE(cond, slot) do { if (cond) tc_trace(slot); } while (0)
// One record per launch (slot = launch number at issue time, so the launches of a replayed
// graph keep their slots): start of CTA (0,0), latest exit of any CTA, N and K.
constexpr int kLaunchRing = 1024;
static __device__ unsigned long long g_tc_launch[kLaunchRing * 4];
// what: 0 = kernel entry, 1 = exit, 3 = the producer thread has passed its dependency wait
// (the previous kernel of the stream has completed)
__device__ __forceinline__ void tc_launch_trace(int id, int what, int n, int k) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  if (what == 1) {
    atomicMax(&g_tc_launch[id * 4 + 1], t);
  } else if (blockIdx.x == 0 && blockIdx.y == 0) {
    g_tc_launch[id * 4 + what] = t;
    if (what == 0) g_tc_launch[id * 4 + 2] = ((unsigned long long)(unsigned)n << 32) | (unsigned)k;
  }
}
#define TC_LAUNCH_TRACE(what) do { if (tid == 0) tc_launch_trace(p.trace_id, what, p.N, p.k_chunks * kTileK); } while (0)
#else
#define TC_TRACE(cond, slot) do { } while (0)
#define TC_LAUNCH_TRACE(what) do { } while (0)
#endif

// kEpiPush: the first hop of the all-reduce.  The CTA's staged bf16 tile [n_rows][128] (batch
// rows row0.. of output tile `tile`) goes with 16-byte stores into the staging of the rank
// that reduces this tile's column slice (peer memory over NVLink, or this rank's own), then
// the arrival flag of (row block, this rank, tile of the slice) is raised there with a
// system-scope release.  Every thread of the CTA calls it.
__device__ __forceinline__ void push_tile(const TcParams& p, const uint8_t* staged, int row0, int n_rows, int tile,
                                          int row_block, uint32_t seq, int tid) {
  const int R = p.push_R, me = p.push_me, T = p.push_T;
  const int q = tile / T, ti = tile % T;
  uint4* dst = reinterpret_cast<uint4*>((uint8_t*)p.push_peer[q] + kFlagBytes) +
               ((int64_t)me * p.M + row0) * p.push_sv + ti * 16;
  const uint4* src = reinterpret_cast<const uint4*>(staged);
  for (int idx = tid; idx < n_rows * 16; idx += kTcThreads) {
    const int rr = idx >> 4, vv = idx & 15;
    if (row0 + rr < p.M) dst[(int64_t)rr * p.push_sv + vv] = src[idx];
  }
  __syncthreads();  // orders every thread's stores before the release below
  if (tid == 0)
    peer_st_release(&reinterpret_cast<CommFlags*>(p.push_peer[q])->tflag[(row_block * R + me) * T + ti], seq + 1);
}

// ----------------------------------------------------------------------- kernel
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
               const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_h,
               const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kMaxStages];
  __shared__ __align__(8) uint64_t s_done;
  __shared__ __align__(8) uint64_t s_recv;   // split-K exchange: bytes of the partners' partials landed
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_last;
  __shared__ uint32_t s_seq;
  __shared__ int s_push_ok;
  __shared__ __align__(8) uint64_t s_resid;  // residual tile landed (kEpiResidual)
  __shared__ float s_rscale[256];            // row scales of the deferred norm (consumer)
  __shared__ float s_pscale[256];            // row scales applied after the activation (MoE weights)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool swiglu = p.epilogue == kEpiSwiGLU;
  const int n_acc = swiglu ? 2 : 1;
  TC_TRACE(tid == 0, 0);
  TC_LAUNCH_TRACE(0);

  // work unit: blockIdx.x = tile * splits + split, blockIdx.y = batch tile
  const int tile = blockIdx.x / p.splits;
  const int split = p.cluster ? (int)cluster_ctarank() : blockIdx.x % p.splits;
  const int m_tile = blockIdx.y;
  const int base_c = p.k_chunks / p.splits, rem_c = p.k_chunks % p.splits;
  const int kc0 = split * base_c + min(split, rem_c);
  const int n_kc = base_c + (split < rem_c ? 1 : 0);

  // shared memory carve-up (1024-byte aligned: the swizzle pattern repeats every 1024 B)
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_bytes = kTileN * kTileK * 2;  // 16 KB per weight slab
  const uint32_t b_bytes = (uint32_t)p.m_pad * kTileK * 2;
  const uint32_t stage_bytes = a_bytes * n_acc + b_bytes;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    mbar_init(smem_u32(&s_done), 1);
    mbar_init(smem_u32(&s_resid), 1);
    mbar_init(smem_u32(&s_recv), 1);
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
  if (p.cluster && p.splits > 1) {
    // exchange barrier: armed with the bytes the S-1 partners will send.  With a dedicated
    // receive area partners may send before this CTA is done streaming, so the cluster must
    // know the barrier is initialised: everybody arrives here and waits just before the
    // first remote store, by which time the barrier has long completed.
    if (tid == 0)
      mbar_expect_tx(smem_u32(&s_recv),
                     (uint32_t)(p.splits - 1) * (uint32_t)(n_acc * (p.m_pad / p.splits) * kTileN * 4));
    if (p.recv_dedicated) cluster_arrive_release();
  }
  TC_TRACE(tid == 0, 1);
  // (The next kernel is released once this CTA's accumulator is complete, below, not here: its
  // CTAs hold their pipeline's shared memory from the moment they are resident.)
  if (!(warp == 0 && lane == 0)) pdl_wait();  // the producer waits after its weight prefetch

  if (warp >= 2 && p.rowsq_in) {
    // deferred norm: scale of every batch row of this tile column, from the row sums the
    // producing GEMM left per 128-feature tile (fixed summation order)
    for (int i = tid - 64; i < p.m_pad; i += 64) {
      const int m = blockIdx.y * p.m_pad + i;
      float sc = 1.f;
      if (m < p.M) {
        // rows are padded to a multiple of four entries that stay zero: 128-bit loads,
        // all in flight at once, summed in a fixed order
        const float4* rq = reinterpret_cast<const float4*>(p.rowsq_in + (int64_t)m * p.rowsq_stride);
        const int n4 = (p.rowsq_tiles + 3) >> 2;
        float a = 0.f;
#pragma unroll 8
        for (int t4 = 0; t4 < n4; ++t4) {
          const float4 v = __ldcg(rq + t4);
          a += (v.x + v.y) + (v.z + v.w);
        }
        sc = rsqrtf(a * p.rs_inv_n + p.rs_eps);
      }
      s_rscale[i] = sc;
    }
  }
  if (warp == 3 && p.epilogue == kEpiPush) {
    // push epilogue: while the weights stream, learn the number of the coming exchange and
    // make sure every peer is done reading the staging of the previous one (the previous
    // exchange kernel of this rank has completed: griddepcontrol.wait above)
    CommFlags* fl = reinterpret_cast<CommFlags*>(p.push_peer[p.push_me]);
    const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(&fl->seq);
    bool okp = true;
    if (lane < p.push_R && lane != p.push_me) okp = peer_wait_ge(&fl->done[lane], seq, p.push_spin);
    okp = __all_sync(0xffffffffu, okp);
    if (lane == 0) {
      s_seq = seq;
      s_push_ok = okp ? 1 : 0;
    }
  }
  if (warp >= 2 && p.post_scale) {
    const int grp = (blockIdx.x / p.splits) / p.post_tiles_per_group;
    for (int i = tid - 64; i < p.m_pad; i += 64) {
      const int m = blockIdx.y * p.m_pad + i;
      s_pscale[i] = m < p.M ? __ldcg(p.post_scale + (int64_t)m * p.post_groups + grp) : 0.f;
    }
  }
  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------- TMA producer
      int armed = 0;  // k-chunks whose copies were issued
      const uint64_t w_policy = l2_policy_evict_first();
      // every weight byte is read once per launch: it may leave L2 first (measured +1 % on the
      // 8B decode step against the default policy)
      auto load_w = [&](uint32_t dst, int kx, int row, uint32_t bar) {
        tma_load_2d_hint(dst, &tm_w, kx, row, bar, w_policy);
      };
      // Weights never depend on the previous kernel: the first stages' weight slabs are
      // requested before waiting for it; activations only afterwards.
      const int pre = min(p.stages, n_kc);
      for (int i = 0; i < pre; ++i) {
        const uint32_t full = smem_u32(&s_full[i]);
        const uint32_t sa = smem_base + i * stage_bytes;
        mbar_expect_tx(full, stage_bytes);
        const int kx = (kc0 + i) * kTileK;
        load_w(sa, kx, tile * kTileN, full);
        if (swiglu) load_w(sa + a_bytes, kx, p.up_row_offset + tile * kTileN, full);
      }
      // (Requesting further chunks into L2 at this point was measured harmful: -2 % to -7 % per
      // decode step after HBM-bound kernels, no gain after an NVLink exchange.  Requesting the
      // NEXT kernel's weights into L2 once this CTA has issued its last load, so that HBM works
      // through the tail (a linear prefix of 8-32 MB, or per CTA of the next kernel the 1-4
      // chunks after the stages it fetches by itself): within +-0.4 % per step, -1.5 % and worse
      // from 8 chunks or 64 MB: neither the tail nor the restart of the stream waits for HBM.  With the weights already resident in L2 the 8B q|k|v projection takes
      // 15.7 us instead of 17.6: the time is L2-to-SM transport and the serial chain of the tail.)
      pdl_wait();
      TC_LAUNCH_TRACE(3);
      for (int i = 0; i < pre; ++i) {
        tma_load_2d(smem_base + i * stage_bytes + a_bytes * n_acc, &tm_x, (kc0 + i) * kTileK, m_tile * p.m_pad,
                    smem_u32(&s_full[i]));
      }
      armed = pre;
      for (int i = pre; i < n_kc; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, &s_abort)) break;
        const uint32_t full = smem_u32(&s_full[s]);
        const uint32_t sa = smem_base + s * stage_bytes;
        mbar_expect_tx(full, stage_bytes);
        const int kx = (kc0 + i) * kTileK;
        load_w(sa, kx, tile * kTileN, full);
        if (swiglu) load_w(sa + a_bytes, kx, p.up_row_offset + tile * kTileN, full);
        tma_load_2d(sa + a_bytes * n_acc, &tm_x, kx, m_tile * p.m_pad, full);
        armed = i + 1;
      }
      if (s_abort) {
        // let every issued copy land before this CTA's shared memory can be reused
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
      // ------------------------------------------------------------ MMA issuer
      const uint32_t idesc = make_idesc(p.m_pad);
      bool ok = true;
      for (int i = 0; i < n_kc && ok; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        ok = mbar_wait(smem_u32(&s_full[s]), ph, &s_abort);
        if (!ok) break;
        TC_TRACE(i == 0, 2);
        tc_fence_after();
        const uint32_t sa = smem_base + s * stage_bytes;
        const uint64_t b_desc = make_smem_desc(sa + a_bytes * n_acc);
#pragma unroll
        for (int acc = 0; acc < 2; ++acc) {
          if (acc < n_acc) {
            const uint64_t a_desc = make_smem_desc(sa + acc * a_bytes);
#pragma unroll
            for (int k = 0; k < kTileK / kUmmaK; ++k) {
              // advancing K by 16 elements = 32 bytes inside the swizzled row
              umma_bf16(tmem_base + acc * p.m_pad, a_desc + (uint64_t)(k * 2),
                        b_desc + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
            }
          }
        }
        tc_commit(smem_u32(&s_empty[s]));  // frees the stage once these MMAs have read it
      }
      // only this thread polls for the accumulator; the other 127 sleep at the CTA
      // barrier below
      if (ok) {
        tc_commit(smem_u32(&s_done));
        ok = mbar_wait(smem_u32(&s_done), 0, &s_abort);
      }
      if (!ok) s_abort = 1;
      // The next kernel may become resident now: it requests its first weight stages while this
      // kernel exchanges, sums and stores, i.e. while HBM would otherwise idle.  Releasing it at
      // the start of this kernel instead (resident and holding shared memory for the whole
      // stream) measured 4.36 against 4.32 ms per 8B decode step; after the last load was
      // issued, or half-way through the stream, in between.
      pdl_launch_dependents();
      TC_TRACE(true, 3);
    }
    __syncwarp();
  }

  // ---------------------------------------------------------------- epilogue
  const int row = warp * 32 + lane;              // accumulator row = output feature
  const int n_glob = tile * kTileN + row;
  const int m_base = m_tile * p.m_pad;
  const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
  __syncthreads();
  tc_fence_after();
  const bool ok_all = s_abort == 0;
  TC_TRACE(tid == 0, 4);

  // Output tiles are staged in the (now idle) pipeline buffers as [batch row][128
  // features] and leave through bulk tensor stores: one instruction per box instead of
  // a 2- or 4-byte store per element (measured: 16 scalar store instructions per warp
  // cost 1-2 us at the end of every GEMM).
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  if (p.cluster && p.splits > 1) {
    // ---- split-K inside a thread-block cluster: the partners exchange accumulator
    // columns through distributed shared memory.  CTA r of the cluster owns the batch
    // rows (accumulator columns) [r*CW, (r+1)*CW) of the tile for all 128 features;
    // everybody sends the columns it does not own to their owner, the owner adds the S
    // partials in split order (deterministic) and runs the epilogue for its rows.
    // The cluster barrier is reached unconditionally.  (The same exchange through global
    // scratch in L2 — plain stores by the partners, ld.global.cg by the owner, one cluster
    // barrier less — was measured 0.5 to 2 us slower per launch on every decode shape.)
    const int S = p.splits, CW = p.m_pad / S;          // CW is a multiple of 4
    // receive area [S-1][n_acc][CW/4][128 features][4 columns]: behind the pipeline buffers
    // (dedicated: partners send as soon as THEIR accumulator is complete) or over them (a
    // cluster barrier first tells everybody that all pipelines are idle); the staged output
    // lies over the pipeline buffers either way
    const int slot_floats = n_acc * CW * kTileN;
    const uint32_t recv_off = p.recv_dedicated ? (uint32_t)p.stages * stage_bytes : 0u;
    float* recv = reinterpret_cast<float*>(smem_gen + recv_off);
    const uint32_t out_off = p.recv_dedicated ? 0u : (uint32_t)((S - 1) * slot_floats) * 4u;  // staged output [CW][128]
    const bool residual = p.epilogue == kEpiResidual;
    const uint32_t tile_b = (uint32_t)CW * kTileN * 2u;   // one staged bf16 tile
    const uint32_t h_off = out_off + tile_b;              // kEpiResidual: new residual [CW][128]
    const uint32_t resid_off = h_off + tile_b;            // kEpiResidual: residual tile read by TMA
    if (residual && tid == 0 && ok_all) {
      // this CTA's own pipeline buffers are idle: fetch the residual tile while the partners
      // catch up and exchange (rows past the batch read as zeros)
      const uint32_t bar = smem_u32(&s_resid);
      mbar_expect_tx(bar, tile_b);
      tma_load_2d(smem_base + resid_off, &tm_h, tile * kTileN, m_base + split * CW, bar);
    }
    if (p.recv_dedicated) cluster_wait_acquire();  // every partner's exchange barrier is initialised
    else cluster_sync_all();                       // every partner's pipeline buffers are idle from here on
    TC_TRACE(tid == 0, 5);
    if (ok_all) {
      const uint32_t bar_local = smem_u32(&s_recv);
      for (int acc = 0; acc < n_acc; ++acc) {
        for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
          // groups this CTA owns entirely stay in tensor memory (uniform over the CTA)
          if (c0 / CW == split && (c0 + 15) / CW == split) continue;
          float v[16];
          tmem_ld16(t_lane + acc * p.m_pad + c0, v);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            // four columns at a time: 16-byte remote stores, a warp fills 512 contiguous bytes
            const int c = c0 + 4 * q, owner = c / CW;
            if (owner != split) {
              const int slot = split < owner ? split : split - 1;
              const uint32_t local =
                  smem_base + recv_off +
                  (uint32_t)(slot * slot_floats + ((acc * (CW >> 2) + ((c % CW) >> 2)) * kTileN + row) * 4) * 4u;
              st_async_v4(cluster_map(local, (uint32_t)owner), v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3],
                          cluster_map(bar_local, (uint32_t)owner));
            }
          }
        }
      }
    }
    // the partners' columns: every 16-byte store above reports to its owner's barrier, which
    // completes when all (S-1) partial slices have landed.  No CTA leaves before it has
    // received everything addressed to it, so no store can arrive at a CTA that has exited.
    const bool ok_recv = ok_all && mbar_wait(smem_u32(&s_recv), 0, &s_abort);
    TC_TRACE(tid == 0, 6);
    bool resid_ok = true;
    const float w_norm = (residual && n_glob < p.N) ? __bfloat162float(p.norm_w[n_glob]) : 0.f;
    if (ok_recv) {
      const int c_lo = split * CW;
      for (int c0 = c_lo & ~15; c0 < c_lo + CW; c0 += 16) {
        float own[16], own_u[16], g[16], u[16];
        tmem_ld16(t_lane + c0, own);
        if (swiglu) tmem_ld16(t_lane + p.m_pad + c0, own_u);
        TC_TRACE(tid == 0 && c0 == (c_lo & ~15), 13);
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] = u[j] = 0.f;
        // partials are added in split order (deterministic); the 16 columns are
        // independent chains, so the loads and the activation overlap
        for (int src = 0; src < S; ++src) {
          if (src == split) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              g[j] += own[j];
              if (swiglu) u[j] += own_u[j];
            }
          } else {
            const float* rs = recv + (src < split ? src : src - 1) * slot_floats;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int cl = c0 + 4 * q - c_lo;
              if (cl >= 0 && cl < CW) {
                const float4 t = *reinterpret_cast<const float4*>(rs + ((cl >> 2) * kTileN + row) * 4);
                g[4 * q] += t.x; g[4 * q + 1] += t.y; g[4 * q + 2] += t.z; g[4 * q + 3] += t.w;
                if (swiglu) {
                  const float4 t2 =
                      *reinterpret_cast<const float4*>(rs + (((CW >> 2) + (cl >> 2)) * kTileN + row) * 4);
                  u[4 * q] += t2.x; u[4 * q + 1] += t2.y; u[4 * q + 2] += t2.z; u[4 * q + 3] += t2.w;
                }
              }
            }
          }
        }
        TC_TRACE(tid == 0 && c0 == (c_lo & ~15), 14);
        // (Requesting all partners' pieces of a four-column group before the first addition, and
        // two tensor-memory loads per wait in the send loop, took the kernel from 96 to 178
        // registers and made it SLOWER: q|k|v of the 8B shape 16.5 -> 17.5 us.)
        if (p.rowsq_in) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float rs_ = s_rscale[c0 + j];
            g[j] *= rs_;
            u[j] *= rs_;
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] = swiglu ? silu_f(g[j]) * u[j] : g[j];
        if (p.post_scale) {
#pragma unroll
          for (int j = 0; j < 16; ++j) g[j] *= s_pscale[c0 + j];
        }
        if (residual) {
          // h = resid + Y (both rounded to bf16 as the reference materialises them); the
          // norm weight is applied here, the row scale by the GEMM that consumes Y'
          if (c0 == (c_lo & ~15)) {
            const bool landed = mbar_wait(smem_u32(&s_resid), 0, &s_abort);
            resid_ok = resid_ok && landed;
          }
          const __nv_bfloat16* rs_tile = reinterpret_cast<const __nv_bfloat16*>(smem_gen + resid_off);
          __nv_bfloat16* hs = reinterpret_cast<__nv_bfloat16*>(smem_gen + h_off);
          __nv_bfloat16* ts = reinterpret_cast<__nv_bfloat16*>(smem_gen + out_off);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int cl = c0 + j - c_lo;
            if (cl >= 0 && cl < CW) {
              const float y = __bfloat162float(__float2bfloat16_rn(g[j]));
              const __nv_bfloat16 h = __float2bfloat16_rn(__bfloat162float(rs_tile[cl * kTileN + row]) + y);
              hs[cl * kTileN + row] = h;
              ts[cl * kTileN + row] = __float2bfloat16_rn(__bfloat162float(h) * w_norm);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int cl = c0 + j - c_lo;
            if (cl >= 0 && cl < CW) {
              if (p.out_f32) reinterpret_cast<float*>(smem_gen + out_off)[cl * kTileN + row] = g[j];
              else reinterpret_cast<__nv_bfloat16*>(smem_gen + out_off)[cl * kTileN + row] = __float2bfloat16_rn(g[j]);
            }
          }
        }
      }
      fence_async_smem();
    }
    TC_TRACE(tid == 0, 10);
    const bool tail_ok = __syncthreads_and((ok_recv && resid_ok) ? 1 : 0) != 0;
    TC_TRACE(tid == 0, 11);
    if (tail_ok && residual) {
      // sum of squares of every new residual row over this tile's 128 features: a warp per
      // row, four values per lane, fixed order
      const __nv_bfloat16* hs = reinterpret_cast<const __nv_bfloat16*>(smem_gen + h_off);
      for (int cl = warp; cl < CW; cl += kTcThreads / 32) {
        const uint2 raw = *reinterpret_cast<const uint2*>(hs + cl * kTileN + lane * 4);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
        float ss = (a.x * a.x + a.y * a.y) + (b.x * b.x + b.y * b.y);
        ss = warp_sum(ss);
        const int m = m_base + split * CW + cl;
        if (lane == 0 && m < p.M) p.rowsq_out[(int64_t)m * p.rowsq_stride + tile] = ss;
      }
    }
    bool store_y = true;
    if (p.rope_cs) {
      // the staged tile is one head for this CTA's CW batch rows: rotate query and key heads
      // (pairs (i, i + 64), values as rounded to bf16 above), send key and value heads
      // straight to their cache slots
      __nv_bfloat16* ts = reinterpret_cast<__nv_bfloat16*>(smem_gen + out_off);
      const int head = tile, row0 = m_base + split * CW;
      if (tail_ok && head < p.rope_nq + p.rope_nkv) {
        for (int idx = tid; idx < CW * 64; idx += kTcThreads) {
          const int cl = idx >> 6, i = idx & 63, m = row0 + cl;
          if (m < p.M) {
            const float2 cs = __ldg(p.rope_cs + (int64_t)m * 64 + i);
            const float x1 = __bfloat162float(ts[cl * kTileN + i]), x2 = __bfloat162float(ts[cl * kTileN + 64 + i]);
            float o1, o2;
            rope_rotate(x1, x2, cs.x, cs.y, &o1, &o2);
            ts[cl * kTileN + i] = __float2bfloat16_rn(o1);
            ts[cl * kTileN + 64 + i] = __float2bfloat16_rn(o2);
          }
        }
      }
      if (head < p.rope_nq) fence_async_smem();
      __syncthreads();
      if (head >= p.rope_nq) {
        store_y = false;
        if (tail_ok) {
          const bool is_k = head < p.rope_nq + p.rope_nkv;
          __nv_bfloat16* cache = is_k ? p.k_cache : p.v_cache;
          const int kvh = head - p.rope_nq - (is_k ? 0 : p.rope_nkv);
          for (int idx = tid; idx < CW * 16; idx += kTcThreads) {
            const int cl = idx >> 4, v = idx & 15, m = row0 + cl;
            if (m < p.M) {
              const int64_t slot = __ldg(p.kv_slots + m);
              if (slot >= 0 && slot < p.kv_num_blocks * HB_BLOCK_SIZE) {
                const int64_t blk = slot / HB_BLOCK_SIZE, off = slot % HB_BLOCK_SIZE;
                __nv_bfloat16* dst = cache + ((blk * p.rope_nkv + kvh) * HB_BLOCK_SIZE + off) * (int64_t)kTileN;
                reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(ts + cl * kTileN)[v];
              }
            }
          }
        }
      }
    }
    if (p.epilogue == kEpiPush) {
      // ---- first hop of the all-reduce: the staged bf16 tile goes to the rank that reduces
      // this tile's column slice (16-byte stores into its staging over NVLink, or into this
      // rank's own), then the tile's arrival flag is raised there
      store_y = false;
      // s_seq / s_push_ok were written by warp 3 before the epilogue's first CTA barrier
      if (tail_ok && s_push_ok != 0) {
        const int row0 = m_base + split * CW;
        push_tile(p, smem_gen + out_off, row0, CW, tile, row0 / CW, s_seq, tid);
      } else if (tid == 0 && tail_ok) {
        atomicExch(&reinterpret_cast<CommFlags*>(p.push_peer[p.push_me])->status, HB_ERR_TIMEOUT);
        if (p.err_flag) atomicExch(p.err_flag, HB_ERR_TIMEOUT);
      }
    }
    if (tail_ok && store_y && tid == 0 && m_base + split * CW < p.M) {
      tma_store_2d(&tm_y, smem_base + out_off, tile * kTileN, m_base + split * CW);
      if (residual) tma_store_2d(&tm_h, smem_base + h_off, tile * kTileN, m_base + split * CW);
      tma_store_commit();
      tma_store_wait_read();
    }
    if (!tail_ok && ok_all && tid == 0 && p.err_flag) atomicExch(p.err_flag, HB_ERR_TIMEOUT);
    TC_TRACE(tid == 0, 12);
    if (!ok_all && tid == 0 && p.err_flag) atomicExch(p.err_flag, HB_ERR_TIMEOUT);
  } else if (ok_all && p.splits == 1 && p.tma_store) {
    // ---- one CTA per tile: 16 batch rows per box, as many boxes in flight as the
    // pipeline buffers hold
    const uint32_t elt = p.out_f32 ? 4u : 2u;
    const uint32_t grp_bytes = 16u * kTileN * elt;
    const int G = p.m_pad / 16;
    const int nbuf = min(G, (int)((uint32_t)p.stages * stage_bytes / grp_bytes));
    for (int g0 = 0; g0 < G; g0 += nbuf) {
      if (g0 > 0) {
        if (tid == 0) tma_store_wait_read();
        __syncthreads();
      }
      const int g1 = min(G, g0 + nbuf);
      for (int g = g0; g < g1; ++g) {
        float v[16];
        tmem_ld16(t_lane + g * 16, v);
        if (p.rowsq_in) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] *= s_rscale[g * 16 + j];
        }
        if (swiglu) {
          float u[16];
          tmem_ld16(t_lane + p.m_pad + g * 16, u);
          if (p.rowsq_in) {
#pragma unroll
            for (int j = 0; j < 16; ++j) u[j] *= s_rscale[g * 16 + j];
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = silu_f(v[j]) * u[j];
        }
        if (p.post_scale) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] *= s_pscale[g * 16 + j];
        }
        uint8_t* dst = smem_gen + (uint32_t)(g - g0) * grp_bytes;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (p.out_f32) reinterpret_cast<float*>(dst)[j * kTileN + row] = v[j];
          else reinterpret_cast<__nv_bfloat16*>(dst)[j * kTileN + row] = __float2bfloat16_rn(v[j]);
        }
      }
      fence_async_smem();
      __syncthreads();
      if (p.epilogue == kEpiPush) {
        // the whole [m_pad][128] tile is staged at once (the host checks that it fits): push it
        if (s_push_ok != 0) {
          push_tile(p, smem_gen, m_base, p.m_pad, tile, m_tile, s_seq, tid);
        } else if (tid == 0) {
          atomicExch(&reinterpret_cast<CommFlags*>(p.push_peer[p.push_me])->status, HB_ERR_TIMEOUT);
          if (p.err_flag) atomicExch(p.err_flag, HB_ERR_TIMEOUT);
        }
      } else if (tid == 0) {
        for (int g = g0; g < g1; ++g)
          if (m_base + g * 16 < p.M)
            tma_store_2d(&tm_y, smem_base + (uint32_t)(g - g0) * grp_bytes, tile * kTileN, m_base + g * 16);
        tma_store_commit();
      }
    }
    if (tid == 0) tma_store_wait_read();
  } else if (ok_all) {
    if (p.splits == 1) {
      for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
        float v[16];
        tmem_ld16(t_lane + c0, v);
        if (swiglu) {
          float u[16];
          tmem_ld16(t_lane + p.m_pad + c0, u);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = silu_f(v[j]) * u[j];
        }
        if (n_glob < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m_base + c0 + j;
            if (m < p.M) {
              if (p.out_f32) ((float*)p.Y)[(int64_t)m * p.ldy + n_glob] = v[j];
              else ((__nv_bfloat16*)p.Y)[(int64_t)m * p.ldy + n_glob] = __float2bfloat16_rn(v[j]);
            }
          }
        }
      }
    } else {
      // fp32 partial -> scratch [unit][acc][m][128]; lanes write consecutive floats
      const int64_t unit = ((int64_t)m_tile * p.n_tiles + tile) * p.splits;
      float* mine = p.partials + (unit + split) * (int64_t)(n_acc * p.m_pad) * kTileN;
      for (int acc = 0; acc < n_acc; ++acc) {
        for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
          float v[16];
          tmem_ld16(t_lane + acc * p.m_pad + c0, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) mine[(int64_t)(acc * p.m_pad + c0 + j) * kTileN + row] = v[j];
        }
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int prev = atomicAdd(&p.counters[m_tile * p.n_tiles + tile], 1);
        s_last = (prev == p.splits - 1);
      }
      __syncthreads();
      if (s_last) {
        __threadfence();
        const float* base = p.partials + unit * (int64_t)(n_acc * p.m_pad) * kTileN;
        const int64_t sstride = (int64_t)(n_acc * p.m_pad) * kTileN;
        const int m_lim = min(p.m_pad, p.M - m_base);
        // eight batch rows at a time: 8 (16 with SwiGLU) independent loads are in
        // flight per split instead of one dependent chain per row
        for (int m0 = 0; m0 < m_lim; m0 += 8) {
          float g[8], u[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] = u[j] = 0.f;
          for (int s = 0; s < p.splits; ++s) {
            const float* ps = base + s * sstride + row;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (m0 + j < m_lim) {
                g[j] += __ldcg(ps + (int64_t)(m0 + j) * kTileN);
                if (swiglu) u[j] += __ldcg(ps + (int64_t)(p.m_pad + m0 + j) * kTileN);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int m = m0 + j;
            if (m < m_lim && n_glob < p.N) {
              const float r = swiglu ? silu_f(g[j]) * u[j] : g[j];
              if (p.out_f32) ((float*)p.Y)[(int64_t)(m_base + m) * p.ldy + n_glob] = r;
              else ((__nv_bfloat16*)p.Y)[(int64_t)(m_base + m) * p.ldy + n_glob] = __float2bfloat16_rn(r);
            }
          }
        }
        if (tid == 0) p.counters[m_tile * p.n_tiles + tile] = 0;  // ready for the next launch
      }
    }
  } else if (tid == 0 && p.err_flag) {
    atomicExch(p.err_flag, HB_ERR_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  if (p.ready_mc && tid == 0) {
    // this CTA's output is written (its bulk stores were issued by this thread, everybody
    // else's plain stores precede the barrier above); the last CTA of the grid tells all ranks
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __threadfence();
    const unsigned total = gridDim.x * gridDim.y;
    if (atomicInc(p.ready_ctas, total - 1) == total - 1) {
      __threadfence();
      atomicAdd(p.ready_calls, 1u);
      asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.ready_mc), "r"(1u) : "memory");
    }
  }
  TC_TRACE(tid == 0, 7);
  TC_LAUNCH_TRACE(1);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

// ------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

// 2-D bf16 row-major [rows, cols] tensor, box [box_rows, 64 cols], 128-byte swizzle.
static int encode_map(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t cols, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(HB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(HB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return HB_OK;
}

// Output map: [rows, cols] elements of elt bytes, row stride ld elements, box
// [box_rows, 128 cols], no swizzle (the kernel stages rows of 128 features densely).
static int encode_out_map(CUtensorMap* tm, void* ptr, int64_t rows, int64_t cols, int64_t ld, bool f32,
                          int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(HB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const cuuint64_t elt = f32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * elt};
  cuuint32_t box[2] = {(cuuint32_t)kTileN, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(HB_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with code %d", (int)r);
  return HB_OK;
}

bool gemm_tc_supported(int64_t M, int64_t N, int64_t K, hb_dtype dtype) {
  return dtype == HB_BF16 && M >= 1 && N >= 1 && K >= kTileK && K % kTileK == 0 &&
         N < (1ll << 30) && M < (1ll << 30);
}

static int pick_splits(int units, int k_chunks, int slots) {
  // Measured on B200: a split through global scratch costs one fp32 accumulator tile
  // (128 x m_pad x 4 B) written and read back per extra CTA, which outweighs the gain
  // unless the K range per CTA is long and the batch small.  So: split in two only
  // for few tiles with a deep K (the 8B down_proj: 32 tiles x 224 chunks, 94 -> 76 us).
  (void)slots;
  if (units * 4 <= 160 && k_chunks >= 128) return 2;
  return 1;
}

// Split factor when the partners reduce on chip (thread-block cluster + distributed
// shared memory).  One SM draws at most ~34 GB/s of weights from HBM (measured), so
// every GEMM wants at least one CTA on each SM: the smallest power of two that
// covers the SMs, at most 8 (portable cluster size), each CTA keeping >= 4 K chunks.
static int pick_cluster_splits(int units, int k_chunks, int sm_count) {
  int s = 1;
  const int cap = 8;  // portable cluster size
  while (s < cap && units * s < sm_count && k_chunks / (s * 2) >= 4) s *= 2;
  return s;
}

int gemm_tc_plan(TcGemmPlan* plan, const void* X, const void* W, int64_t M, int64_t N, int64_t K,
                 int epilogue, bool out_f32, int device, int force_splits) {

  if (!gemm_tc_supported(M, N, K, HB_BF16))
    return fail(HB_ERR_INVALID_ARG, "gemm_tc: unsupported shape M=%lld N=%lld K=%lld", (long long)M,
                (long long)N, (long long)K);
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return fail(HB_ERR_INVALID_ARG, "gemm_tc: operands must be 16-byte aligned");
  DeviceInfo di;
  int rc = device_info(device, &di);
  if (rc) return rc;
  if (di.cc_major != 10)
    return fail(HB_ERR_CUDA, "gemm_tc: device %d is sm_%d%d, this library is built for sm_100a",
                device, di.cc_major, di.cc_minor);
  TcGemmPlan& pl = *plan;
  pl.M = M; pl.K = K;
  pl.epilogue = epilogue;
  pl.out_f32 = out_f32;
  const int n_acc = epilogue == kEpiSwiGLU ? 2 : 1;
  if (epilogue == kEpiSwiGLU && N % 2) return fail(HB_ERR_INVALID_ARG, "gemm_tc: SwiGLU needs even N");
  const int64_t n_rows = epilogue == kEpiSwiGLU ? N / 2 : N;  // output features
  pl.N = n_rows;
  // At most 128 batch rows per tile: a 256-row tile doubles the activation traffic per weight
  // byte and the exchange per CTA (measured at M = 256: 8192 x 3584 38.0 -> 24.9 us, 8192 x 4096
  // 40.7 -> 26.7 us with two tiles of 128 rows).
  const int m_cap = 128;
  const int64_t m_eff = std::min<int64_t>(M, m_cap);
  pl.m_pad = (int)std::max<int64_t>(16, (m_eff + 15) / 16 * 16);
  pl.n_tiles = (int)((n_rows + kTileN - 1) / kTileN);
  const int k_chunks = (int)(K / kTileK);
  const bool want_cluster = true;  // split-K partners reduce on chip; global scratch only where a cluster cannot form
  const bool tuned = want_cluster && force_splits <= 0;
  // Few weights under a wide batch (o_proj and q|k|v at high tensor-parallel degrees): the
  // split-K exchange moves 128 x m_pad fp32 per CTA through the SM-to-SM network, which at
  // m_pad = 128 costs more than the matrix takes to stream.  Two batch tiles of 64 rows read
  // the weight tile twice (the second time from L2) and need no, or a smaller, exchange
  // (measured: 8192 x 1024 at M = 128 15.4 -> 11.1 us, 1280 x 8192 19.0 -> 16.4 us).
  bool m_split = false;
  if (tuned && n_acc == 1 && pl.m_pad >= 128 && (int64_t)pl.n_tiles * k_chunks <= 2048 &&
      (epilogue == kEpiStore || epilogue == kEpiPush)) {
    pl.m_pad = 64;
    m_split = true;
  }
  pl.m_tiles = (int)((M + pl.m_pad - 1) / pl.m_pad);
  const int units = pl.n_tiles * pl.m_tiles;
  const int acc_cols = pl.m_pad * n_acc;
  pl.tmem_cols = acc_cols <= 32 ? 32 : acc_cols <= 64 ? 64 : acc_cols <= 128 ? 128 : acc_cols <= 256 ? 256 : 512;
  const size_t stage = (size_t)kTileN * kTileK * 2 * n_acc + (size_t)pl.m_pad * kTileK * 2;
  // Two pipeline depths: ~110 KB, so that two CTAs share an SM and one's epilogue hides under
  // the other's loads, or ~200 KB with the SM to itself.
  const size_t small_budget = 110 * 1024, big_budget = 200 * 1024;
  auto stages_for = [&](size_t budget) { return (int)std::max<size_t>(2, std::min<size_t>(kMaxStages, budget / stage)); };
  const int small_stages = stages_for(small_budget);
  const int big_stages = (size_t)stages_for(big_budget) * stage + 1024 <= di.smem_optin ? stages_for(big_budget) : small_stages;
  if ((size_t)small_stages * stage + 1024 > di.smem_optin)
    return fail(HB_ERR_INVALID_ARG, "gemm_tc: needs %zu bytes of shared memory", (size_t)small_stages * stage + 1024);
  const int slots = di.sm_count * 2;
  bool big = false;
  if (force_splits > 0) {
    pl.splits = std::min(force_splits, k_chunks);
  } else if (!want_cluster) {
    pl.splits = pick_splits(units, k_chunks, slots);
  } else if (tuned && n_acc == 2 && units <= di.sm_count) {
    // SwiGLU tiles carry two weight slabs per stage: the 110 KB budget holds two stages, too
    // shallow to keep HBM busy.  One CTA per SM with the deep pipeline, and the largest split
    // that still fits one wave (measured: 14336 x 8192 at M = 128 68.6 -> 51.0 us)
    int sp = 1;
    while (sp * 2 <= 8 && units * sp * 2 <= di.sm_count && k_chunks / (sp * 4) >= 4) sp *= 2;
    pl.splits = sp;
    big = true;
  } else if (m_split) {
    // split K only while a CTA would stream more than 512 KB or the SMs are not covered
    int sp = 1;
    auto cta_bytes = [&](int s_) { return (size_t)(kTileN + pl.m_pad) * (size_t)(k_chunks / s_) * kTileK * 2; };
    while (sp < 8 && k_chunks / (sp * 2) >= 4 &&
           (units * sp * 5 < di.sm_count * 4 || (cta_bytes(sp) > 512 * 1024 && units * sp < di.sm_count)))
      sp *= 2;
    pl.splits = sp;
  } else {
    pl.splits = pick_cluster_splits(units, k_chunks, di.sm_count);
  }
  // (Partner counts that are not powers of two, with shares of the batch rows that differ by
  // four rows, were built and measured to cover more SMs where 28 tiles x 4 partners leave 36 of
  // 148 idle: clusters of five do not pack into the GPCs - 28 of them are not resident together -
  // and the 7168 x 8192 SwiGLU GEMM at M = 128 went from 32.4 to 59.9 us; three partners for the
  // 8B q|k|v projection 18.1 against 16.5 us with four.  Removed again.)
  // a grid of at most one CTA per SM gains nothing from leaving room for a second one
  if (tuned && units * pl.splits <= di.sm_count) big = true;
  pl.stages = big ? big_stages : small_stages;
  // cluster form: power-of-two size <= 8 whose receive buffers fit the pipeline's
  // shared memory; anything else reduces through global scratch
  pl.cluster = false;
  // the output leaves through bulk tensor stores when its rows are 16-byte multiples
  const size_t out_elt = out_f32 ? 4 : 2;
  pl.tma_store = ((size_t)n_rows * out_elt) % 16 == 0;
  auto recv_fits = [&](int sp) {
    // received partials [sp-1][n_acc][m_pad/sp][128] fp32 + the staged output [m_pad/sp][128]
    const size_t cw = (size_t)pl.m_pad / sp;
    const size_t extra = epilogue == kEpiResidual ? 2 * cw * kTileN * 2 : 0;  // new residual + fetched residual
    return (size_t)(sp - 1) * n_acc * cw * kTileN * sizeof(float) + cw * kTileN * out_elt + extra <=
           (size_t)pl.stages * stage;
  };
  if (want_cluster && pl.splits > 1 && pl.tma_store) {
    // The exchange buffers of a wide batch (or of the two SwiGLU accumulators) may not
    // fit the two-CTAs-per-SM budget.  When a split factor yields at most one CTA per SM
    // anyway, it may take the deep pipeline instead of being halved: a matrix with few row
    // slabs needs the splits to reach the SMs.
    if (force_splits <= 0) {
      while (pl.splits > 1) {
        if (pl.m_pad / pl.splits >= 4 && pl.m_pad % (4 * pl.splits) == 0) {
          pl.stages = big ? big_stages : small_stages;
          if (recv_fits(pl.splits)) break;
          if (big_stages > small_stages && (int64_t)units * pl.splits <= di.sm_count) {
            pl.stages = big_stages;
            if (recv_fits(pl.splits)) break;
          }
        }
        pl.splits /= 2;
      }
      if (pl.splits == 1) pl.stages = (tuned && units <= di.sm_count) ? big_stages : small_stages;
    }
    // every partner owns m_pad / splits batch rows, exchanged four at a time
    pl.cluster = pl.splits > 1 && pl.splits <= 8 && (pl.splits & (pl.splits - 1)) == 0 &&
                 pl.m_pad % (4 * pl.splits) == 0 && recv_fits(pl.splits);
  }
  // Where the budget leaves at least three stages beside it, the receive area of the exchange
  // gets shared memory of its own behind the pipeline: partners then send without waiting for
  // this CTA's pipeline to drain (one cluster barrier less in the tail).
  pl.recv_dedicated = false;
  size_t recv_bytes = 0;
  if (pl.cluster) {
    const size_t cw = (size_t)pl.m_pad / pl.splits;
    recv_bytes = (size_t)(pl.splits - 1) * n_acc * cw * kTileN * sizeof(float);
    const size_t staged = cw * kTileN * out_elt + (epilogue == kEpiResidual ? 2 * cw * kTileN * 2 : 0);
    const size_t budget = (pl.stages == big_stages && big_stages > small_stages) ? big_budget : small_budget;
    const int st_d = budget > recv_bytes ? (int)std::min<size_t>(kMaxStages, (budget - recv_bytes) / stage) : 0;
    if (st_d >= 3 && staged <= (size_t)st_d * stage) {
      pl.recv_dedicated = true;
      pl.stages = st_d;
    } else {
      recv_bytes = 0;
    }
  }
  pl.smem_bytes = pl.stages * stage + recv_bytes + 1024;
  // The tile counters sit in a block of FIXED size at the start of the workspace, so
  // that plans of different shapes sharing one workspace never see each other's
  // partials where they expect zeroed counters.
  if (!pl.cluster && (size_t)units * sizeof(int) > kCounterBlockBytes) pl.splits = 1;
  pl.ws_partials_bytes = (pl.splits > 1 && !pl.cluster) ? (size_t)units * pl.splits * n_acc * pl.m_pad * kTileN * sizeof(float) : 0;
  pl.ws_counters_bytes = (pl.splits > 1 && !pl.cluster) ? kCounterBlockBytes : 0;
  // opt in to the large dynamic shared memory window once per device (here, not at
  // launch, so that launches stay legal inside a stream capture)
  {
    int cur = 0;
    HB_CUDA_CHECK(cudaGetDevice(&cur));
    static bool dev_done[64] = {false};
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (cur >= 0 && cur < 64 && !dev_done[cur]) {
      // 227 KiB per CTA minus the kernel's static shared memory (barriers, flags, row scales)
      HB_CUDA_CHECK(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         224 * 1024));
      dev_done[cur] = true;
    }
  }
  rc = encode_map(&pl.tm_w, W, N, K, kTileN);
  if (rc) return rc;
  rc = encode_map(&pl.tm_x, X, M, K, pl.m_pad);
  return rc;
}

int gemm_tc_push_row_block(const TcGemmPlan& pl) {
  if (pl.epilogue != kEpiPush || pl.out_f32 || !pl.tma_store) return 0;
  if (pl.cluster && pl.splits > 1) return pl.m_pad / pl.splits;
  // one CTA per tile: the whole [m_pad][128] bf16 tile must fit the pipeline buffers
  const size_t stage = (size_t)kTileN * kTileK * 2 + (size_t)pl.m_pad * kTileK * 2;
  if (pl.splits == 1 && (size_t)pl.m_pad * kTileN * 2 <= (size_t)pl.stages * stage) return pl.m_pad;
  return 0;
}

bool gemm_tc_rope_epilogue_ok(const TcGemmPlan& pl) {
  return pl.cluster && pl.splits > 1 && pl.tma_store && !pl.out_f32 && pl.epilogue == kEpiStore &&
         pl.N % kTileN == 0;
}

int gemm_tc_run(const TcGemmPlan& pl, cudaStream_t st, void* Y, int64_t ldy, void* workspace,
                int* err_flag, const TcNormLink* link) {
  if (pl.splits > 1 && !pl.cluster && !workspace)
    return fail(HB_ERR_INVALID_ARG, "gemm_tc: split-K plan needs a workspace of %zu bytes",
                pl.workspace_bytes());
  TcParams p;
  memset(&p, 0, sizeof(p));
#ifdef HB_TC_TRACE
  static std::atomic<int> launch_no{0};
  p.trace_id = launch_no.fetch_add(1) % kLaunchRing;
#endif
  p.M = (int)pl.M; p.N = (int)pl.N;
  p.m_pad = pl.m_pad; p.splits = pl.splits; p.stages = pl.stages; p.tmem_cols = pl.tmem_cols;
  p.k_chunks = (int)(pl.K / kTileK);
  p.n_tiles = pl.n_tiles;
  p.epilogue = pl.epilogue; p.out_f32 = pl.out_f32 ? 1 : 0;
  p.ldy = ldy;
  p.up_row_offset = (int)pl.N;
  p.Y = Y;
  // counters first (16-byte aligned block), partials after
  p.counters = (int*)workspace;
  p.partials = workspace ? (float*)((uint8_t*)workspace + pl.ws_counters_bytes) : nullptr;
  p.err_flag = err_flag;
  p.cluster = pl.cluster ? 1 : 0;
  p.recv_dedicated = pl.recv_dedicated ? 1 : 0;
  CUtensorMap tm_y;
  memset(&tm_y, 0, sizeof(tm_y));
  const size_t y_elt = pl.out_f32 ? 4 : 2;
  const bool push = pl.epilogue == kEpiPush;
  const bool y_ok = push || ((reinterpret_cast<uintptr_t>(Y) & 15) == 0 && ((size_t)ldy * y_elt) % 16 == 0);
  if (pl.cluster && !y_ok)
    return fail(HB_ERR_INVALID_ARG, "gemm_tc: output must be 16-byte aligned with rows of a multiple of 16 bytes");
  p.tma_store = (pl.tma_store && y_ok && (pl.cluster || pl.splits == 1)) ? 1 : 0;
  if (push) {
    const int R = link ? link->push_ranks : 0;
    const int rb = gemm_tc_push_row_block(pl);
    if (rb < 1 || pl.out_f32 || !link || !link->push_peers || R < 2 || R > HB_MAX_RANKS ||
        link->push_rank < 0 || link->push_rank >= R || pl.N % ((int64_t)R * kTileN) ||
        (int64_t)((pl.M + rb - 1) / rb) * (pl.N / kTileN) > kMaxPushFlags)
      return fail(HB_ERR_INVALID_ARG, "gemm_tc: the push epilogue needs bf16 output staged as whole tiles and rank slices of whole tiles");
    for (int q = 0; q < R; ++q) p.push_peer[q] = link->push_peers[q];
    p.push_R = R;
    p.push_me = link->push_rank;
    p.push_T = (int)(pl.N / kTileN / R);
    p.push_sv = (int64_t)p.push_T * 16;
    p.push_spin = link->push_spin ? link->push_spin : (1u << 22);
  }
  if (p.tma_store && !push) {
    const int box_rows = pl.cluster ? pl.m_pad / pl.splits : 16;
    int rc = encode_out_map(&tm_y, Y, pl.M, pl.N, ldy, pl.out_f32, box_rows);
    if (rc) return rc;
  }
  CUtensorMap tm_h;
  memset(&tm_h, 0, sizeof(tm_h));
  if (pl.epilogue == kEpiResidual) {
    if (!pl.cluster || !p.tma_store || pl.out_f32 || !link || !link->resid || !link->norm_w || !link->rowsq_out)
      return fail(HB_ERR_INVALID_ARG, "gemm_tc: the residual epilogue needs a cluster plan, bf16 output and a norm link");
    if ((reinterpret_cast<uintptr_t>(link->resid) & 15) || link->rowsq_stride < pl.n_tiles)
      return fail(HB_ERR_INVALID_ARG, "gemm_tc: bad residual buffer or row-sum stride");
    int rc = encode_out_map(&tm_h, link->resid, pl.M, pl.N, ldy, false, pl.m_pad / pl.splits);
    if (rc) return rc;
    p.norm_w = (const __nv_bfloat16*)link->norm_w;
    p.rowsq_out = link->rowsq_out;
    p.rowsq_stride = link->rowsq_stride;
  }
  if (link && link->post_scale) {
    if (!p.tma_store || (pl.splits > 1 && !pl.cluster) || link->post_tiles_per_group < 1)
      return fail(HB_ERR_INVALID_ARG, "gemm_tc: post-activation row scaling needs the bulk-store epilogue");
    p.post_scale = link->post_scale;
    p.post_groups = link->post_groups;
    p.post_tiles_per_group = link->post_tiles_per_group;
  }
  if (link && link->rope_cs) {
    if (!gemm_tc_rope_epilogue_ok(pl) || !p.tma_store || !link->kv_slots || !link->k_cache || !link->v_cache ||
        pl.N != (int64_t)(link->n_q_heads + 2 * link->n_kv_heads) * kTileN)
      return fail(HB_ERR_INVALID_ARG, "gemm_tc: the RoPE epilogue needs a cluster plan over [q|k|v] heads of 128");
    p.rope_cs = link->rope_cs;
    p.kv_slots = link->kv_slots;
    p.k_cache = (__nv_bfloat16*)link->k_cache;
    p.v_cache = (__nv_bfloat16*)link->v_cache;
    p.rope_nq = link->n_q_heads;
    p.rope_nkv = link->n_kv_heads;
    p.kv_num_blocks = link->num_blocks;
  }
  if (link && link->ready_mc) {
    if (!link->ready_calls || !link->ready_ctas)
      return fail(HB_ERR_INVALID_ARG, "gemm_tc: the completion signal needs its two local counters");
    p.ready_mc = link->ready_mc;
    p.ready_calls = link->ready_calls;
    p.ready_ctas = link->ready_ctas;
  }
  if (link && link->rowsq_in) {
    if (!p.tma_store || (pl.splits > 1 && !pl.cluster))
      return fail(HB_ERR_INVALID_ARG, "gemm_tc: row scaling needs the bulk-store epilogue");
    p.rowsq_in = link->rowsq_in;
    p.rowsq_tiles = link->rowsq_tiles;
    p.rowsq_stride = link->rowsq_stride;
    p.rs_inv_n = 1.0f / link->n;
    p.rs_eps = link->eps;
  }
  dim3 grid((unsigned)(pl.n_tiles * pl.splits), (unsigned)pl.m_tiles);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  static const bool use_pdl = [] { const char* e = getenv("HB_PDL"); return !(e && e[0] == '0'); }();
  if (use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (pl.cluster) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)pl.splits;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  HB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_tc_kernel, pl.tm_w, pl.tm_x, tm_y, tm_h, p));
  return HB_OK;
}

}  // namespace hb

#ifdef HB_TC_TRACE
extern "C" int hb_debug_tc_launches(unsigned long long* host_out, int n) {
  if (n > hb::kLaunchRing) n = hb::kLaunchRing;
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(host_out, hb::g_tc_launch, sizeof(unsigned long long) * n * 4);
}
extern "C" int hb_debug_tc_trace(unsigned long long* host_out, int n_ctas) {
  if (n_ctas > hb::kTraceCtas) n_ctas = hb::kTraceCtas;
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(host_out, hb::g_tc_trace, sizeof(unsigned long long) * n_ctas * hb::kTraceSlots);
}
#endif
