// Fused row-parallel projection: ONE kernel per rank computes
//
//   resid_out  = resid_in + SUM_ranks( X_r[M,Kl] . W_r[N,Kl]^T )
//   normed_out = resid_out * rsqrt(mean(resid_out^2) + eps) * norm_w
//
// i.e. o_proj / down_proj -> all_reduce -> residual add -> next RMSNorm of the layer
// loop (src/engine/arch/llama_tp.rs:327,533-552 and :339,563-571,517-522), which the
// reference runs as a library GEMM, an NCCL all-reduce, peer copies and a norm kernel.
//
// Phases of a CTA = (128-feature tile t, K split s); the S splits of a tile form a
// thread-block cluster:
//   1. tcgen05 mainloop (TMA -> shared memory -> UMMA, fp32 accumulator in tensor
//      memory), exactly the decode GEMM: the weight slab is the UMMA A operand.
//   2. split-K on chip: CTA s owns the batch rows [s*CW, (s+1)*CW), CW = m_pad/S, of the
//      tile for all 128 features — the "unit" t*S+s; partners send it their accumulator
//      columns through distributed shared memory (16-byte stores) and it adds the S
//      partials in split order.
//   3. every CTA rounds its unit of the rank's partial to bf16 (the reference's partials
//      are bf16 tensors), keeps it in shared memory and PUSHES it with coalesced 128-bit
//      stores into the staging buffer of the unit's reducer rank(s) over NVLink, then
//      raises pflag[u][me] there.  two-shot: the reducer of unit u is rank u/(U/R);
//      one-shot: every rank reduces every unit (one NVLink hop, R-1 times the bytes).
//   4. a reducer waits for the R-1 remote partials of its unit, sums all R in rank
//      order in fp32 on top of the residual, rounds, writes resid_out, accumulates the
//      sum of squares of the unit's rows over its 128 features, and (two-shot) pushes the
//      reduced unit and the row sums to every peer, then raises gflag[u] everywhere.
//   5. every CTA waits until the units of ITS batch rows are present locally for every
//      tile (N/128 flags), sums their row sums into the row scales and writes its unit
//      of normed_out (non-reducers also copy the gathered unit into resid_out).
// Flags carry the device-resident call sequence number, so a captured CUDA graph can
// replay the kernel; staging reuse is guarded by the per-rank "done" flags shared with
// the all-reduce kernel.  CTAs wait for other CTAs of the same grid, so the grid never
// exceeds the number of CTAs the device can hold at once.  All waits are bounded.
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
  int64_t tile_bytes;                  // one unit: (m_pad / splits) * 128 * 2
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
  __shared__ uint32_t s_seq;
  __shared__ float s_rowsq[256];
  __shared__ float s_rs[256];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x / p.splits;
  const int split = p.splits > 1 ? (int)cluster_ctarank() : 0;
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
  pdl_launch_dependents();
  if (!(warp == 0 && lane == 0)) pdl_wait();

  // ------------------------------------------------------------ 1. mainloop
  if (warp == 0) {
    if (lane == 0) {
      int armed = 0;
      // weight slabs of the first stages are requested before the previous kernel is
      // known to be finished; activations only after pdl_wait()
      const int pre = min(p.stages, n_kc);
      for (int i = 0; i < pre; ++i) {
        const uint32_t full = smem_u32(&s_full[i]);
        mbar_expect_tx(full, stage_bytes);
        tma_load_2d(smem_base + i * stage_bytes, &tm_w, (kc0 + i) * kTileK, tile * kTileN, full);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem_base + i * stage_bytes + a_bytes, &tm_x, (kc0 + i) * kTileK, 0, smem_u32(&s_full[i]));
      armed = pre;
      for (int i = pre; i < n_kc; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, &s_abort)) break;
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
      // only this thread polls for the accumulator; the other 127 sleep at the CTA
      // barrier below
      if (ok) {
        tc_commit(smem_u32(&s_done));
        ok = mbar_wait(smem_u32(&s_done), 0, &s_abort);
      }
      if (!ok) s_abort = 1;
    }
    __syncwarp();
  }

  const int row = warp * 32 + lane;  // accumulator row = feature inside the 128-wide tile
  const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
  __syncthreads();
  tc_fence_after();
  const bool ok_all = s_abort == 0;

  // ------------------------------------------------------------ 2. split-K in the cluster
  // CTA r of the cluster owns the batch rows [r*CW, (r+1)*CW) of the tile for all 128
  // features = "unit" tile*S + r.  Partners send the accumulator columns they do not
  // own to the owner through distributed shared memory (16-byte stores, four columns at
  // a time); the owner adds the S partials in split order, rounds to bf16 (the
  // reference's partials are bf16 tensors) and leaves its unit [CW][128] in shared memory.
  const int S = p.splits, CW = p.m_pad / S;
  float* recv = reinterpret_cast<float*>(smem_gen);  // [S-1][CW/4][128 features][4 columns] fp32
  const int slot_floats = CW * kTileN;
  const uint32_t recv_bytes = (uint32_t)((S - 1) * slot_floats * 4);
  __nv_bfloat16* unit_s = reinterpret_cast<__nv_bfloat16*>(smem_gen + recv_bytes);  // [CW][128] bf16
  uint4* unit_u4 = reinterpret_cast<uint4*>(smem_gen + recv_bytes);
  const int r0 = split * CW;                          // first batch row of the unit
  const int rows_valid = max(0, min(CW, p.M - r0));   // rows of the unit inside the batch
  if (S > 1) {
    cluster_sync_all();  // every partner's pipeline buffers are idle from here on
    if (ok_all) {
      for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
        if (c0 / CW == split && (c0 + 15) / CW == split) continue;  // uniform over the CTA
        float v[16];
        tmem_ld16(t_lane + c0, v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c = c0 + 4 * q, owner = c / CW;
          if (owner != split) {
            const int slot = split < owner ? split : split - 1;
            const uint32_t local =
                smem_base + (uint32_t)(slot * slot_floats + (((c % CW) >> 2) * kTileN + row) * 4) * 4u;
            st_cluster_v4(cluster_map(local, (uint32_t)owner), v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
        }
      }
    }
    cluster_sync_all();  // release/acquire: columns sent above are visible to their owner
  }
  if (ok_all) {
    for (int c0 = r0 & ~15; c0 < r0 + CW; c0 += 16) {
      float own[16], g[16];
      tmem_ld16(t_lane + c0, own);
#pragma unroll
      for (int j = 0; j < 16; ++j) g[j] = 0.f;
      for (int src = 0; src < S; ++src) {
        if (src == split) {
#pragma unroll
          for (int j = 0; j < 16; ++j) g[j] += own[j];
        } else {
          const float* rs = recv + (src < split ? src : src - 1) * slot_floats;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int cl = c0 + 4 * q - r0;
            if (cl >= 0 && cl < CW) {
              const float4 t = *reinterpret_cast<const float4*>(rs + ((cl >> 2) * kTileN + row) * 4);
              g[4 * q] += t.x; g[4 * q + 1] += t.y; g[4 * q + 2] += t.z; g[4 * q + 3] += t.w;
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int cl = c0 + j - r0;
        if (cl >= 0 && cl < CW) unit_s[cl * kTileN + row] = __float2bfloat16_rn(g[j]);
      }
    }
  }
  __syncthreads();

  // ------------------------------------------------------------ 3..5 unit protocol
  CommFlags* fl = reinterpret_cast<CommFlags*>(p.peer[p.rank]);
  bool proto_ok = ok_all;
  const int R = p.ws, me = p.rank;
  const int unit = tile * S + split, U = p.n_tiles * S;
  const int t_stride = (p.n_tiles + 3) & ~3;  // row stride of the [batch row][tile] row-sum table
  constexpr int lpr = kTileN / 8;            // 16-byte vectors (lanes) per batch row of the unit
  const int n_u4 = rows_valid * lpr;
  const int n0 = tile * kTileN;              // first feature of the unit
  if (tid == 0) s_seq = *reinterpret_cast<volatile uint32_t*>(&fl->seq);
  __syncthreads();
  const uint32_t seq = s_seq, target = seq + 1;
  const int owner_rank = p.two_shot ? unit / p.tiles_own : me;
  const bool reducer = !p.two_shot || owner_rank == me;
  const int u_slot = p.two_shot ? unit - owner_rank * p.tiles_own : unit;
  auto data_of = [&](int q) { return (uint8_t*)p.peer[q] + kFlagBytes; };
  auto flags_of = [&](int q) { return reinterpret_cast<CommFlags*>(p.peer[q]); };
  auto part_slot = [&](int q, int src, int slot) {
    return reinterpret_cast<uint4*>(data_of(q) + ((int64_t)src * p.tiles_own + slot) * p.tile_bytes);
  };

  if (R > 1) {
    // ---- A. peers must be done with the previous collective before their staging is written
    bool ok = true;
    if (tid < R && tid != me) ok = f_wait_ge(&fl->done[tid], seq);
    proto_ok = __syncthreads_and((ok && proto_ok) ? 1 : 0) != 0;
    // ---- 3. push this rank's partial of the unit to its reducer(s), coalesced 128-bit stores
    if (proto_ok) {
      for (int q = 0; q < R; ++q) {
        if (q == me || (p.two_shot && q != owner_rank)) continue;
        uint4* dst = part_slot(q, me, u_slot);
        for (int i = tid; i < n_u4; i += kTcThreads) dst[i] = unit_u4[i];
      }
      // bar.sync orders every thread's stores before the flag threads; their system-scope
      // release store is cumulative over them (no fence per thread needed)
      __syncthreads();
      if (tid < R && tid != me && (!p.two_shot || tid == owner_rank))
        f_st_release(&flags_of(tid)->pflag[unit * HB_MAX_RANKS + me], target);
    }
  }

  // ---- 4. reduce over ranks (rank order, fp32) on top of the residual
  if (proto_ok && reducer) {
    if (R > 1) {
      bool ok = true;
      if (tid < R && tid != me) ok = f_wait_ge(&fl->pflag[unit * HB_MAX_RANKS + tid], target);
      proto_ok = __syncthreads_and(ok ? 1 : 0) != 0;
    }
    if (proto_ok) {
      // 16 consecutive lanes hold one batch row of the unit (256 bytes)
      for (int i0 = 0; i0 < n_u4; i0 += kTcThreads) {
        const int i = i0 + tid;
        float ss = 0.f;
        if (i < n_u4) {
          const int m = r0 + i / lpr, c = i % lpr;
          const int64_t g_off = (int64_t)m * p.N + n0 + c * 8;
          float acc[8], t8[8];
          bf16x8_to_f32(*reinterpret_cast<const uint4*>(p.resid_in + g_off), acc);
          for (int src = 0; src < R; ++src) {
            const uint4 raw = (src == me) ? unit_u4[i] : __ldcg(part_slot(me, src, u_slot) + i);
            bf16x8_to_f32(raw, t8);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += t8[j];
          }
          const uint4 out = f32_to_bf16x8(acc);
          bf16x8_to_f32(out, t8);  // the norm sees the rounded residual
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += t8[j] * t8[j];
          unit_u4[i] = out;
          *reinterpret_cast<uint4*>(p.resid_out + g_off) = out;
        }
        for (int o = lpr >> 1; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (i < n_u4 && (i % lpr) == 0) s_rowsq[i / lpr] = ss;
      }
      __syncthreads();
      // row sums are kept [batch row][tile] (tile fastest) so that a reader sums a row
      // with 128-bit loads
      float* my_rowsq = reinterpret_cast<float*>(data_of(me) + p.rowsq_off) + tile;
      for (int m = tid; m < rows_valid; m += kTcThreads) my_rowsq[(int64_t)(r0 + m) * t_stride] = s_rowsq[m];
      if (R > 1 && p.two_shot) {
        for (int q = 0; q < R; ++q) {
          if (q == me) continue;
          uint4* dst = reinterpret_cast<uint4*>(data_of(q) + p.gather_off + (int64_t)unit * p.tile_bytes);
          for (int i = tid; i < n_u4; i += kTcThreads) dst[i] = unit_u4[i];
          float* rq = reinterpret_cast<float*>(data_of(q) + p.rowsq_off) + tile;
          for (int m = tid; m < rows_valid; m += kTcThreads) rq[(int64_t)(r0 + m) * t_stride] = s_rowsq[m];
        }
      }
      __syncthreads();
      if (tid == 0) f_st_release(&fl->gflag[unit], target);
      if (R > 1 && p.two_shot && tid < R && tid != me) f_st_release(&flags_of(tid)->gflag[unit], target);
    }
  }

  // ---- 5. the units of this row group are present for every tile -> row scales ->
  //         normalise this unit
  if (proto_ok) {
    bool ok = true;
    for (int t2 = tid; t2 < p.n_tiles; t2 += kTcThreads) ok = ok && f_wait_ge(&fl->gflag[t2 * S + split], target);
    proto_ok = __syncthreads_and(ok ? 1 : 0) != 0;
  }
  if (proto_ok) {
    // sum of squares of the unit's batch rows over all tiles: tpr threads per row, 128-bit
    // loads, partials combined in a fixed order
    const float* rowsq = reinterpret_cast<const float*>(data_of(me) + p.rowsq_off);
    int tpr = 1;  // power of two, tpr * CW <= 128
    while (tpr < 32 && tpr * 2 * CW <= kTcThreads) tpr *= 2;
    const int t4_total = t_stride >> 2;
    for (int m0 = 0; m0 < CW; m0 += kTcThreads / tpr) {
      const int m = m0 + tid / tpr, part = tid % tpr;
      float a = 0.f;
      if (m < rows_valid) {
        const float4* r4 = reinterpret_cast<const float4*>(rowsq + (int64_t)(r0 + m) * t_stride);
        for (int i = part; i < t4_total; i += tpr) {
          const float4 v = __ldcg(r4 + i);
          const int t2 = i << 2;  // entries past the last tile are never written: mask them
          a += ((t2 < p.n_tiles ? v.x : 0.f) + (t2 + 1 < p.n_tiles ? v.y : 0.f)) +
               ((t2 + 2 < p.n_tiles ? v.z : 0.f) + (t2 + 3 < p.n_tiles ? v.w : 0.f));
        }
      }
      for (int o = tpr >> 1; o >= 1; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (m < rows_valid && part == 0) s_rs[m] = rsqrtf(a / (float)p.N + p.eps);
    }
    if (!reducer) {
      const uint4* src = reinterpret_cast<const uint4*>(data_of(me) + p.gather_off + (int64_t)unit * p.tile_bytes);
      for (int i = tid; i < n_u4; i += kTcThreads) {
        const uint4 v = __ldcg(src + i);
        unit_u4[i] = v;
        const int m = r0 + i / lpr, c = i % lpr;
        *reinterpret_cast<uint4*>(p.resid_out + (int64_t)m * p.N + n0 + c * 8) = v;
      }
    }
    __syncthreads();
    if (p.normed_out) {
      for (int i = tid; i < n_u4; i += kTcThreads) {
        const int ml = i / lpr, c = i % lpr;
        float h[8], w8[8];
        bf16x8_to_f32(unit_u4[i], h);
        bf16x8_to_f32(*reinterpret_cast<const uint4*>(p.norm_w + n0 + c * 8), w8);
        const float r = s_rs[ml];
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = h[j] * r * w8[j];
        *reinterpret_cast<uint4*>(p.normed_out + (int64_t)(r0 + ml) * p.N + n0 + c * 8) = f32_to_bf16x8(h);
      }
    }
  }

  // ---- E. the last CTA closes the collective
  __syncthreads();
  if (tid == 0) {
    if (!proto_ok) atomicExch(&fl->status, HB_ERR_TIMEOUT);
    __threadfence();
    const uint32_t prev = atomicAdd(&fl->finished, 1u);
    if (prev == (uint32_t)U - 1) {
      fl->finished = 0;
      *reinterpret_cast<volatile uint32_t*>(&fl->seq) = target;
      __threadfence_system();
      for (int q = 0; q < R; ++q)
        if (q != me) f_st_release(&flags_of(q)->done[me], target);
    }
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
// Layout of the caller's workspace (zero-initialised once, left clean by every call);
// only a single-rank call uses it, for what a multi-rank world keeps in its staging:
//   [0, 64K)      flag block
//   [64K, 320K)   row sums [batch row][tile]
// All offsets are fixed, so calls of different shapes may share one workspace.
constexpr size_t kFusedRowsqBytes = (size_t)kMaxFusedTiles * 256 * sizeof(float);

struct FusedPlan {
  TcGemmPlan g;        // tensor maps and tile geometry (epilogue unused)
  int splits = 1;      // cluster size S: power of two, <= 8
  int capacity = 0;    // co-resident CTAs of the kernel on this device
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
  fp->g.splits = 1;
  fp->g.cluster = false;
  if ((rc = fused_capacity(device, fp->g.smem_bytes, &fp->capacity))) return rc;
  DeviceInfo di;
  if ((rc = device_info(device, &di))) return rc;
  const int k_chunks = (int)(Kl / kTileK);
  const int T = fp->g.n_tiles;
  const size_t pipe_bytes = fp->g.smem_bytes - 1024;
  auto fits = [&](int s) {
    // a partner owns m_pad / s batch rows, exchanged four at a time
    if (fp->g.m_pad % (4 * s) != 0) return false;
    const size_t cw = (size_t)fp->g.m_pad / s;
    const size_t recv = (size_t)(s - 1) * cw * kTileN * sizeof(float);
    const size_t unit = cw * kTileN * 2;
    // units are capped by the flag arrays; a cluster leaves a little slack in the
    // co-residency bound because its CTAs must land in one GPC
    return recv + unit <= pipe_bytes && T * s <= kMaxFusedTiles && T * s <= fp->capacity - (s > 1 ? 8 : 0);
  };
  // at least one CTA per SM when possible (one SM draws ~34 GB/s from HBM at most)
  int s = 1;
  while (s < 8 && T * s < di.sm_count && k_chunks / (s * 2) >= 4 && fits(s * 2)) s *= 2;
  if (const char* ev = getenv("HB_FUSED_SPLITS")) {
    const int want = atoi(ev);
    if ((want == 1 || want == 2 || want == 4 || want == 8) && want <= k_chunks && fits(want)) s = want;
  }
  if (!fits(s)) return fail(HB_ERR_INVALID_ARG, "fused row-parallel: %d tiles do not fit the device", T);
  fp->splits = s;
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
  return kFlagBytes + kFusedRowsqBytes + 256;
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
  const int T = fp.g.n_tiles, S = fp.splits, U = T * S;
  FusedParams p;
  memset(&p, 0, sizeof(p));
  p.M = (int)M; p.N = (int)N; p.m_pad = fp.g.m_pad; p.splits = S; p.stages = fp.g.stages;
  p.tmem_cols = fp.g.tmem_cols; p.k_chunks = (int)(K_local / kTileK); p.n_tiles = T;
  p.ws = R; p.rank = w ? w->rank : 0;
  p.eps = eps;
  p.resid_in = (const __nv_bfloat16*)resid_in;
  p.resid_out = (__nv_bfloat16*)resid_out;
  p.normed_out = (__nv_bfloat16*)normed_out;
  p.norm_w = (const __nv_bfloat16*)norm_w;
  uint8_t* wsb = (uint8_t*)workspace;
  p.tile_bytes = (int64_t)(fp.g.m_pad / S) * kTileN * 2;  // one unit: [m_pad / S batch rows][128] bf16
  bool two = false;
  if (R > 1) {
    two = algo == HB_ALGO_TWO_SHOT || (algo == HB_ALGO_AUTO && R > 2 && (size_t)M * N * 2 >= 256 * 1024);
    if (U % R != 0) two = false;
  }
  p.two_shot = two ? 1 : 0;
  p.tiles_own = two ? U / R : U;  // units a reducer rank owns
  const size_t part_area = (size_t)R * p.tiles_own * p.tile_bytes;
  p.gather_off = (int64_t)align_up(part_area, 256);
  p.rowsq_off = p.gather_off + (int64_t)align_up(two ? (size_t)U * p.tile_bytes : 0, 256);
  const size_t need = (size_t)p.rowsq_off + (size_t)((T + 3) & ~3) * fp.g.m_pad * sizeof(float);
  if (R > 1) {
    if (need > w->staging_bytes)
      return fail(HB_ERR_INVALID_ARG, "fused row-parallel: needs %zu bytes of staging, world has %zu", need,
                  w->staging_bytes);
    for (int q = 0; q < R; ++q) p.peer[q] = w->peer[q];
  } else {
    // single rank: flag block and row sums live in the caller's workspace
    p.peer[0] = wsb;
    p.gather_off = 0;
    p.rowsq_off = 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)U);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = fp.g.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (S > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)S;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  static const bool use_pdl = [] { const char* e = getenv("HB_PDL"); return !(e && e[0] == '0'); }();
  if (use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  } else if (S == 1) {
    attr[na].id = cudaLaunchAttributeCooperative;  // co-residency checked by the driver
    attr[na].val.cooperative = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (S > 1) {
    // CTAs of this grid wait for one another: every cluster must be resident at once
    int max_clusters = 0;
    HB_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&max_clusters, rowpar_fused_kernel, &cfg));
    if (U / S > max_clusters)
      return fail(HB_ERR_INVALID_ARG, "fused row-parallel: %d clusters of %d CTAs, device holds %d at once",
                  U / S, S, max_clusters);
  }
  HB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, rowpar_fused_kernel, fp.g.tm_w, fp.g.tm_x, p));
  return HB_OK;
}

}  // namespace hb
