// Paged GQA decode attention on tensor cores (bf16, head_dim 128, up to 16 query heads
// per kv head).  Same contract and pool layout as the CUDA-core kernel in attention.cu
// (src/engine/arch/llama_tp.rs:264-324): out = softmax(q k^T / sqrt(d)) v over the
// sequence's block table, partials + log-sum-exp merge when the KV range is split.
//
// Decode attention is a stream of K and V rows read once.  With 4-8 query heads per
// kv head the CUDA-core kernel needs ~750 issued instructions per 8 KB of KV, which is
// about what the SMs can issue at HBM speed; here the two products run as
// mma.sync.m16n8k16 (the query heads padded to the 16 MMA rows), which cuts the issue
// count per KV block about sevenfold, and the KV blocks arrive by TMA:
//
//   CTA = (sequence, kv head, KV split), NW = 2, 4 or 8 warps.  Warp w owns the blocks
//   b0+w, b0+w+NW, ... of the CTA's range and keeps its own online-softmax state, so
//   the main loop has no CTA-wide barrier.  Each warp has a ring of kAttnStages
//   stages; one stage holds a block's K and V ([16 tokens][128] bf16 each) as four
//   [16 x 64] boxes with the 128-byte swizzle, so that ldmatrix reads them without
//   bank conflicts.  Lane 0 issues the four TMA loads of a block on the stage's
//   mbarrier; the warp waits for it, computes S = Q K^T (16 MMAs), the online softmax
//   in fp32, O += P V (16 MMAs, P rounded to bf16), and refills the stage.
//   At the end the warps merge their (m, l, O) through shared memory.
//   When the caller bounds the tokens that the preceding kernels write (the engine's
//   step), the ring is filled with older blocks before griddepcontrol.wait.
//   Prefill chunks (q_group > 1): the rows of the batch are consecutive positions of ONE
//   sequence; a CTA then takes q_group of them, the 16 MMA rows holding q_group positions x
//   n_rep heads, each row with its own causal limit, so that the sequence's K and V are read
//   once per q_group positions instead of once per position (src/engine/arch/llama_tp.rs:
//   313-316: the causal mask of a multi-token forward).
//
// Every wait is bounded: on expiry the CTA raises *err_flag (when given), writes NaN
// to its outputs, lets outstanding copies land and returns.
#include <climits>
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "common.h"
#include "tc_core.cuh"

namespace hb {

constexpr int kAttnStages = 3;
constexpr int kAttnStageBytes = 8192;  // K lo | K hi | V lo | V hi, 2 KB each
constexpr int kAttnHD = 128;
// shared memory of a CTA of NW warps (the merge scratch [NW][16][132] floats fits inside)
constexpr size_t mma_attn_smem(int nw) { return (size_t)nw * kAttnStages * kAttnStageBytes + 1024; }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                              uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D[16x8] += A[16x16] . B[16x8], bf16 operands, fp32 accumulate.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int NW>
__global__ void __launch_bounds__(NW * 32)
paged_attn_mma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                      float* __restrict__ part_ml, const __nv_bfloat16* __restrict__ q,
                      const int32_t* __restrict__ block_tables, const int32_t* __restrict__ ctx_lens, int hq,
                      int hkv, int nrep, int64_t max_blocks, int64_t num_blocks, int n_splits, float scale,
                      int64_t q_stride, int window, int* err_flag, int fresh, int q_group, int n_rows) {
  constexpr int kMmaAttnWarps = NW, kMmaAttnThreads = NW * 32;
  // fresh >= 0: at most `fresh` tokens at the end of every sequence were written by the
  // kernels right before this one (the current step's K/V); every earlier block of the pool
  // is final, so its copies may start before those kernels have completed.  The context
  // lengths and block tables are step inputs, not products of a kernel.
  const bool early = fresh >= 0;
  if (!early) pdl_grid_wait();
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kMmaAttnWarps][kAttnStages];
  __shared__ int s_abort;

  const int split = blockIdx.x, kvh = blockIdx.y;
  // the CTA's batch rows: [seq, seq + n_q); row seq + j holds position j of the group
  const int64_t seq = (int64_t)blockIdx.z * q_group;
  const int n_q = min(q_group, n_rows - (int)seq);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;  // MMA fragment coordinates

  // a context longer than the table row can describe is cut to the row (the table of the
  // next sequence, or memory past the allocation, is never indexed)
  const int ctx_cap = (int)min(max_blocks * HB_BLOCK_SIZE, (int64_t)INT_MAX);
  auto ctx_of = [&](int j) { return max(0, min(ctx_lens[seq + j], ctx_cap)); };
  // MMA row r of the padded 16-row tile = (position r / nrep of the group, head r % nrep)
  const int j_lo = g / nrep, j_hi = (g + 8) / nrep;
  const bool row_lo = j_lo < n_q, row_hi = j_hi < n_q;
  const int ctx_lo = row_lo ? ctx_of(j_lo) : 0, ctx_hi = row_hi ? ctx_of(j_hi) : 0;
  const int ctx = ctx_of(n_q - 1);   // the longest context of the group (contexts grow with j)
  const int nblk = (ctx + HB_BLOCK_SIZE - 1) / HB_BLOCK_SIZE;
  // sliding window (src/engine/arch/mixtral.rs:155-176): the query at position c-1 sees the
  // keys ki with c-1-ki < window; the group's first row reaches furthest back
  const int first_tok = window > 0 ? max(0, ctx_of(0) - window) : 0;
  const int first_lo = window > 0 ? max(0, ctx_lo - window) : 0, first_hi = window > 0 ? max(0, ctx_hi - window) : 0;
  const int first_blk = first_tok / HB_BLOCK_SIZE;
  const int bps = (nblk - first_blk + n_splits - 1) / n_splits;
  const int b0 = first_blk + split * bps;
  const int b1 = min(nblk, b0 + bps);
  // this warp's blocks: b0 + warp + NW i, i < n_w
  const int n_w = (b1 - b0 - warp + kMmaAttnWarps - 1) > 0 ? (b1 - b0 - warp + kMmaAttnWarps - 1) / kMmaAttnWarps : 0;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring = smem_base + (uint32_t)(warp * kAttnStages) * kAttnStageBytes;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  if (tid == 0) s_abort = 0;
  if (lane == 0) {
    for (int s = 0; s < kAttnStages; ++s) mbar_init(smem_u32(&s_full[warp][s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  // ---- block table entries of this warp, 32 at a time, one per lane
  const int32_t* table = block_tables + seq * max_blocks;
  int tab_base = 0;
  int32_t tab = 0;
  auto load_tab = [&](int base) {
    tab_base = base;
    const int i = base + lane;
    tab = i < n_w ? table[b0 + warp + kMmaAttnWarps * i] : 0;
  };
  // Whole warp calls; lane 0 issues block i of this warp into stage i % kAttnStages.
  auto issue = [&](int i) {
    if (i >= tab_base + 32) load_tab(i);
    int64_t phys = __shfl_sync(0xffffffffu, tab, i - tab_base);
    if (phys < 0 || phys >= num_blocks) phys = 0;  // never read outside the pool
    if (lane == 0) {
      const int s = i % kAttnStages;
      const uint32_t bar = smem_u32(&s_full[warp][s]);
      const uint32_t dst = ring + (uint32_t)s * kAttnStageBytes;
      const int row = (int)((phys * hkv + kvh) * HB_BLOCK_SIZE);
      mbar_expect_tx(bar, kAttnStageBytes);
      tma_load_2d(dst, &tm_k, 0, row, bar);
      tma_load_2d(dst + 2048, &tm_k, 64, row, bar);
      tma_load_2d(dst + 4096, &tm_v, 0, row, bar);
      tma_load_2d(dst + 6144, &tm_v, 64, row, bar);
    }
  };
  load_tab(0);
  int issued = 0;
  if (early) {
    // blocks [0, stable) were complete before this step began
    const int stable = max(0, ctx_of(0) - fresh) / HB_BLOCK_SIZE;
    for (; issued < min(kAttnStages, n_w); ++issued) {
      if (b0 + warp + kMmaAttnWarps * issued >= stable) break;
      issue(issued);
    }
    pdl_grid_wait();
  }
  for (; issued < min(kAttnStages, n_w); ++issued) issue(issued);


  // ---- query fragments: rows g and g+8 of the padded 16-head tile, all 8 k-steps
  uint32_t qa[8][4];
  {
    const __nv_bfloat16* q0 = q + (seq + j_lo) * q_stride + ((int64_t)kvh * nrep + g % nrep) * kAttnHD;
    const __nv_bfloat16* q1 = q + (seq + j_hi) * q_stride + ((int64_t)kvh * nrep + (g + 8) % nrep) * kAttnHD;
    const bool h0 = row_lo, h1 = row_hi;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int col = ks * 16 + 2 * t;
      qa[ks][0] = h0 ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
      qa[ks][1] = h1 ? *reinterpret_cast<const uint32_t*>(q1 + col) : 0u;
      qa[ks][2] = h0 ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
      qa[ks][3] = h1 ? *reinterpret_cast<const uint32_t*>(q1 + col + 8) : 0u;
    }
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  int done = 0;
  bool ok = true;
  for (int i = 0; i < n_w; ++i) {
    const int s = i % kAttnStages;
    const uint32_t ph = (uint32_t)(i / kAttnStages) & 1u;
    ok = mbar_wait(smem_u32(&s_full[warp][s]), ph, &s_abort);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    done = i + 1;
    const uint32_t base = ring + (uint32_t)s * kAttnStageBytes;
    const int blk = b0 + warp + kMmaAttnWarps * i;
    const int tok0 = blk * HB_BLOCK_SIZE;
    const int nvalid = min(HB_BLOCK_SIZE, ctx - tok0);
    if (nvalid < HB_BLOCK_SIZE) {
      // V rows past the context may hold anything (NaN included): zero them.  A row's
      // eight 16-byte chunks are permuted inside the row, so whole rows can be cleared.
      uint8_t* vb = smem_gen + (base - smem_base) + 4096;
      for (int c = lane; c < (HB_BLOCK_SIZE - nvalid) * 16; c += 32) {
        const int r = nvalid + c / 16, half = (c / 8) & 1, ch = c & 7;
        *reinterpret_cast<uint4*>(vb + half * 2048 + r * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
      }
      __syncwarp();
    }

    // ---- S[16 heads x 16 tokens] = Q K^T
    float sc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
      const int r = nt * 8 + (lane & 7);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int cidx = q4 * 4 + (lane >> 3);
        const uint32_t addr =
            base + (uint32_t)((cidx >> 3) * 2048 + r * 128 + (((cidx & 7) ^ (r & 7)) << 4));
        uint32_t k0, k1, k2, k3;
        ldsm_x4(addr, k0, k1, k2, k3);
        mma_bf16_16816(sc[nt], qa[2 * q4], k0, k1);
        mma_bf16_16816(sc[nt], qa[2 * q4 + 1], k2, k3);
      }
    }
    // ---- online softmax (rows g and g+8), fp32
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = tok0 + nt * 8 + 2 * t + (e & 1);
        // elements 0, 1 belong to row g, elements 2, 3 to row g + 8: each with its own limits
        const bool vis = e < 2 ? (tok < ctx_lo && tok >= first_lo) : (tok < ctx_hi && tok >= first_hi);
        const float v = vis ? sc[nt][e] * scale : -INFINITY;
        sc[nt][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    // (a row of a group may see none of a block's tokens: its maximum then stays where it was,
    // possibly still -inf, and the block adds nothing to it)
    const float m0n = fmaxf(m0, mx0), m1n = fmaxf(m1, mx1);
    const float a0 = (m0 == -INFINITY) ? 0.f : __expf(m0 - m0n);
    const float a1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - m1n);
    m0 = m0n; m1 = m1n;
    l0 *= a0; l1 *= a1;
#pragma unroll
    for (int nd = 0; nd < 16; ++nd) {
      o[nd][0] *= a0; o[nd][1] *= a0;
      o[nd][2] *= a1; o[nd][3] *= a1;
    }
    uint32_t pa[4];
    {
      float p[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        p[nt][0] = sc[nt][0] == -INFINITY ? 0.f : __expf(sc[nt][0] - m0);
        p[nt][1] = sc[nt][1] == -INFINITY ? 0.f : __expf(sc[nt][1] - m0);
        p[nt][2] = sc[nt][2] == -INFINITY ? 0.f : __expf(sc[nt][2] - m1);
        p[nt][3] = sc[nt][3] == -INFINITY ? 0.f : __expf(sc[nt][3] - m1);
        l0 += p[nt][0] + p[nt][1];
        l1 += p[nt][2] + p[nt][3];
      }
      pa[0] = pack_bf16(p[0][0], p[0][1]);
      pa[1] = pack_bf16(p[0][2], p[0][3]);
      pa[2] = pack_bf16(p[1][0], p[1][1]);
      pa[3] = pack_bf16(p[1][2], p[1][3]);
    }
    // ---- O[16 heads x 128] += P V
    {
      const int mi = lane >> 3;
      const int r = (mi & 1) * 8 + (lane & 7);
#pragma unroll
      for (int nd2 = 0; nd2 < 8; ++nd2) {
        const int cidx = nd2 * 2 + (mi >> 1);
        const uint32_t addr =
            base + 4096u + (uint32_t)((cidx >> 3) * 2048 + r * 128 + (((cidx & 7) ^ (r & 7)) << 4));
        uint32_t v0, v1, v2, v3;
        ldsm_x4_trans(addr, v0, v1, v2, v3);
        mma_bf16_16816(o[2 * nd2], pa, v0, v1);
        mma_bf16_16816(o[2 * nd2 + 1], pa, v2, v3);
      }
    }
    __syncwarp();  // every lane has read the stage
    if (issued < n_w) { issue(issued); ++issued; }
  }
  if (!ok) {
    // let the copies already issued land before the shared memory is given back
    for (int i = done; i < issued; ++i) {
      const uint32_t bar = smem_u32(&s_full[warp][i % kAttnStages]);
      const uint32_t ph = (uint32_t)(i / kAttnStages) & 1u;
      for (uint32_t it = 0; it < kSpinLimit && !mbar_try(bar, ph); ++it) {
      }
    }
  }

  // The next kernel (the o_proj GEMM) may become resident from here on, not from the start: its
  // CTAs hold 100-200 KB of shared memory each while they wait, which the CTAs of this grid
  // that are not resident yet would otherwise miss (measured 4.386 -> 4.367 ms per 8B decode step).
  pdl_trigger();
  // ---- merge the four warps: (m, l, O) per head through shared memory
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();  // all rings are idle
  constexpr int kOStride = kAttnHD + 4;
  float* s_o = reinterpret_cast<float*>(smem_gen);             // [4][16][kOStride]
  float* s_ml = s_o + kMmaAttnWarps * 16 * kOStride;           // [4][16][2]
#pragma unroll
  for (int nd = 0; nd < 16; ++nd) {
    *reinterpret_cast<float2*>(s_o + (warp * 16 + g) * kOStride + nd * 8 + 2 * t) = make_float2(o[nd][0], o[nd][1]);
    *reinterpret_cast<float2*>(s_o + (warp * 16 + g + 8) * kOStride + nd * 8 + 2 * t) = make_float2(o[nd][2], o[nd][3]);
  }
  if (t == 0) {
    s_ml[(warp * 16 + g) * 2] = m0;
    s_ml[(warp * 16 + g) * 2 + 1] = l0;
    s_ml[(warp * 16 + g + 8) * 2] = m1;
    s_ml[(warp * 16 + g + 8) * 2 + 1] = l1;
  }
  __syncthreads();
  const bool failed = s_abort != 0;
  if (failed && tid == 0 && err_flag) atomicExch(err_flag, HB_ERR_TIMEOUT);
  for (int idx = tid; idx < n_q * nrep * kAttnHD; idx += kMmaAttnThreads) {
    const int h = idx / kAttnHD, d = idx % kAttnHD;   // h = MMA row = (position h / nrep, head h % nrep)
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaAttnWarps; ++w) M = fmaxf(M, s_ml[(w * 16 + h) * 2]);
    float ov = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kMmaAttnWarps; ++w) {
      const float mw = s_ml[(w * 16 + h) * 2];
      const float wt = (mw == -INFINITY) ? 0.f : __expf(mw - M);
      ov += wt * s_o[(w * 16 + h) * kOStride + d];
      l += wt * s_ml[(w * 16 + h) * 2 + 1];
    }
    if (failed) { ov = __int_as_float(0x7fc00000); l = 1.f; }
    const int64_t head = (seq + h / nrep) * hq + (int64_t)kvh * nrep + h % nrep;
    if (n_splits == 1) {
      out[head * kAttnHD + d] = __float2bfloat16_rn(l > 0.f ? ov / l : 0.f);
    } else {
      part_o[(head * n_splits + split) * kAttnHD + d] = ov;
      if (d == 0) {
        part_ml[(head * n_splits + split) * 2 + 0] = M;
        part_ml[(head * n_splits + split) * 2 + 1] = l;
      }
    }
  }
}

// ------------------------------------------------------------------------ host
typedef CUresult (*AttnEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AttnEncodeFn attn_encode_fn() {
  static AttnEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = (AttnEncodeFn)sym;
  });
  return fn;
}

// The pool of one layer as a 2-D tensor [num_blocks * n_kv_heads * 16 rows, 128], box
// [16 rows, 64 columns], 128-byte swizzle.
static int encode_pool_map(CUtensorMap* tm, const void* pool, int64_t num_blocks, int hkv) {
  AttnEncodeFn enc = attn_encode_fn();
  if (!enc) return fail(HB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {(cuuint64_t)kAttnHD, (cuuint64_t)(num_blocks * hkv * HB_BLOCK_SIZE)};
  cuuint64_t strides[1] = {(cuuint64_t)kAttnHD * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)HB_BLOCK_SIZE};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(HB_ERR_CUDA, "cuTensorMapEncodeTiled (KV pool) failed with code %d", (int)r);
  return HB_OK;
}

bool paged_attention_mma_supported(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                   int nrep, int head_dim, int64_t num_blocks, int hkv, hb_dtype dtype) {
  if (dtype != HB_BF16 || head_dim != kAttnHD || nrep < 1 || nrep > 16) return false;
  if ((reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15)) return false;
  if ((reinterpret_cast<uintptr_t>(q) & 3) || (q_stride & 1)) return false;
  if (num_blocks * hkv * HB_BLOCK_SIZE >= (1ll << 31)) return false;  // TMA row coordinate is an int
  return true;
}

// Opts the kernels in to their dynamic shared memory; once per device, outside any
// stream capture (the engine calls it when it is created).
int paged_attention_mma_prepare() {
  static std::mutex mu;
  static bool done[64] = {false};
  int dev = 0;
  HB_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 64 && !done[dev]) {
    HB_CUDA_CHECK(cudaFuncSetAttribute(paged_attn_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)mma_attn_smem(4)));
    HB_CUDA_CHECK(cudaFuncSetAttribute(paged_attn_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)mma_attn_smem(2)));
    HB_CUDA_CHECK(cudaFuncSetAttribute(paged_attn_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)mma_attn_smem(8)));
    done[dev] = true;
  }
  return HB_OK;
}

int paged_attention_mma(cudaStream_t st, void* out, float* part_o, float* part_ml, const void* q,
                        int64_t q_stride, const void* k_cache, const void* v_cache, const int32_t* block_tables,
                        const int32_t* ctx_lens, int64_t n_seqs, int hq, int hkv, int64_t max_blocks,
                        int64_t num_blocks, int n_splits, int window, int* err_flag, int fresh, int q_group) {
  int rc = paged_attention_mma_prepare();
  const int nrep_ = hq / hkv;
  if (q_group < 1 || q_group * nrep_ > 16) return fail(HB_ERR_INVALID_ARG, "paged attention: %d positions x %d heads exceed the 16 rows of a tile", q_group, nrep_);
  const int n_rows = (int)n_seqs;
  if (rc) return rc;
  CUtensorMap tm_k, tm_v;
  if ((rc = encode_pool_map(&tm_k, k_cache, num_blocks, hkv))) return rc;
  if ((rc = encode_pool_map(&tm_v, v_cache, num_blocks, hkv))) return rc;
  dim3 grid((unsigned)n_splits, (unsigned)hkv, (unsigned)((n_seqs + q_group - 1) / q_group));
  const float scale = 1.0f / sqrtf((float)kAttnHD);
  // Two CTAs of four warps fit an SM, or four of two warps (same bytes in flight).
  // When the grid is larger than one wave of the former, the smaller CTAs keep every
  // unit resident at once instead of leaving a partial second wave.
  DeviceInfo di;
  int device = 0;
  HB_CUDA_CHECK(cudaGetDevice(&device));
  if ((rc = device_info(device, &di))) return rc;
  const int64_t ctas = (int64_t)n_splits * hkv * ((n_seqs + q_group - 1) / q_group);
  // ... and a grid that does not even fill the SMs takes eight warps per CTA: two warps per
  // scheduler hide each other's MMA and softmax latency (70B TP=8 shape: 17.2 against 21.0 us)
  const int nw = ctas > 2 * (int64_t)di.sm_count ? 2 : (ctas <= (int64_t)di.sm_count ? 8 : 4);
  if (nw == 8) {
    HB_CUDA_CHECK(launch_pdl(paged_attn_mma_kernel<8>, grid, dim3(256), mma_attn_smem(8), st, tm_k, tm_v,
                             (__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q, block_tables, ctx_lens, hq,
                             hkv, hq / hkv, max_blocks, num_blocks, n_splits, scale, q_stride, window, err_flag, fresh, q_group, n_rows));
    return HB_OK;
  }
  if (nw == 2) {
    HB_CUDA_CHECK(launch_pdl(paged_attn_mma_kernel<2>, grid, dim3(64), mma_attn_smem(2), st, tm_k, tm_v,
                             (__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q, block_tables, ctx_lens, hq,
                             hkv, hq / hkv, max_blocks, num_blocks, n_splits, scale, q_stride, window, err_flag, fresh, q_group, n_rows));
  } else {
    HB_CUDA_CHECK(launch_pdl(paged_attn_mma_kernel<4>, grid, dim3(128), mma_attn_smem(4), st, tm_k, tm_v,
                             (__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q, block_tables, ctx_lens, hq,
                             hkv, hq / hkv, max_blocks, num_blocks, n_splits, scale, q_stride, window, err_flag, fresh, q_group, n_rows));
  }
  return HB_OK;
}

}  // namespace hb
