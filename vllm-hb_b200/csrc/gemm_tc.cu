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
// every CTA owns (slab, K range), writes its fp32 partial to scratch, and the last
// CTA to arrive for a slab sums the partials in split order (deterministic) and runs
// the epilogue.
//
// CTA = 4 warps.  Warp 0 lane 0 issues TMA, warp 1 lane 0 issues MMAs, all four warps
// read the accumulator (warp w owns TMEM lanes 32w..32w+31 = output features).
// Every wait is bounded: on expiry the kernel raises *err_flag, lets outstanding
// copies land, frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <cstring>
#include <mutex>

#include "common.h"
#include "gemm.h"
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
  int packed;               // weights stored tile-major: [n_tile][k_chunk][128][64]
  int stagger;              // rotate the K walk per tile
  int cluster;              // split-K partners form a thread-block cluster of `splits` CTAs
  void* Y;
  float* partials;
  int* counters;
  int* err_flag;
};

// ----------------------------------------------------------------------- kernel
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
               const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kMaxStages];
  __shared__ __align__(8) uint64_t s_done;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool swiglu = p.epilogue == kEpiSwiGLU;
  const int n_acc = swiglu ? 2 : 1;

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

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------- TMA producer
      int armed = 0;  // k-chunks whose copies were issued
      for (int i = 0; i < n_kc; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        if (i >= p.stages && !mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, &s_abort)) break;
        const uint32_t full = smem_u32(&s_full[s]);
        const uint32_t sa = smem_base + s * stage_bytes;
        mbar_expect_tx(full, stage_bytes);
        // tiles walk their K range from different starting chunks so that the CTAs do
        // not all ask L2 for the same slice of X at the same moment
        const int ci = p.stagger ? (i + tile * 5) % n_kc : i;
        const int kx = (kc0 + ci) * kTileK;
        if (p.packed) tma_load_2d(sa, &tm_w, 0, (tile * p.k_chunks + kc0 + ci) * kTileN, full);
        else tma_load_2d(sa, &tm_w, kx, tile * kTileN, full);
        if (swiglu) tma_load_2d(sa + a_bytes, &tm_w, kx, p.up_row_offset + tile * kTileN, full);
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
      if (ok) tc_commit(smem_u32(&s_done));
    }
    __syncwarp();
  }

  // ---------------------------------------------------------------- epilogue
  const bool have_acc = mbar_wait(smem_u32(&s_done), 0, &s_abort);
  tc_fence_after();
  const int row = warp * 32 + lane;              // accumulator row = output feature
  const int n_glob = tile * kTileN + row;
  const int m_base = m_tile * p.m_pad;
  const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
  const bool ok_all = __syncthreads_and(have_acc ? 1 : 0) != 0;

  if (p.cluster && p.splits > 1) {
    // ---- split-K inside a thread-block cluster: the partners exchange accumulator rows
    // through distributed shared memory.  CTA r of the cluster owns the features
    // [r*FW, (r+1)*FW) of the tile; everybody sends the rows it does not own to their
    // owner, the owner adds the S partials in split order (deterministic) and runs the
    // epilogue for its rows.  Both cluster barriers are reached unconditionally.
    const int S = p.splits, FW = kTileN / S;
    const int owner = row / FW, f_loc = row % FW;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    float* recv = reinterpret_cast<float*>(smem_gen);  // [S-1][n_acc][m_pad][FW]
    const int slot_floats = n_acc * p.m_pad * FW;
    // tcgen05.ld is warp-collective: whole warps take the branches below, lanes are
    // masked only at the stores
    const int own_lo = (warp * 32) / FW, own_hi = (warp * 32 + 31) / FW;
    const bool warp_sends = !(own_lo == split && own_hi == split);
    const bool warp_owns = own_lo <= split && split <= own_hi;
    cluster_sync_all();  // every partner's pipeline buffers are idle from here on
    if (ok_all && warp_sends) {
      const int slot = split < owner ? split : split - 1;
      const uint32_t dst0 = cluster_map(smem_base + (uint32_t)(slot * slot_floats + f_loc) * 4u, (uint32_t)owner);
      for (int acc = 0; acc < n_acc; ++acc) {
        for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
          float v[16];
          tmem_ld16(t_lane + acc * p.m_pad + c0, v);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (owner != split) st_cluster_f32(dst0 + (uint32_t)((acc * p.m_pad + c0 + j) * FW) * 4u, v[j]);
        }
      }
    }
    cluster_sync_all();  // release/acquire: the rows sent above are visible to their owner
    if (ok_all && warp_owns) {
      for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
        float own[16], own_u[16], g[16], u[16];
        tmem_ld16(t_lane + c0, own);
        if (swiglu) tmem_ld16(t_lane + p.m_pad + c0, own_u);
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] = u[j] = 0.f;
        for (int src = 0; src < S; ++src) {
          if (src == split) {
#pragma unroll
            for (int j = 0; j < 16; ++j) { g[j] += own[j]; if (swiglu) u[j] += own_u[j]; }
          } else {
            const float* rs = recv + (src < split ? src : src - 1) * slot_floats + f_loc;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              g[j] += rs[(c0 + j) * FW];
              if (swiglu) u[j] += rs[(p.m_pad + c0 + j) * FW];
            }
          }
        }
        if (n_glob < p.N && owner == split) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m_base + c0 + j;
            if (m < p.M) {
              const float r = swiglu ? silu_f(g[j]) * u[j] : g[j];
              if (p.out_f32) ((float*)p.Y)[(int64_t)m * p.ldy + n_glob] = r;
              else ((__nv_bfloat16*)p.Y)[(int64_t)m * p.ldy + n_glob] = __float2bfloat16_rn(r);
            }
          }
        }
      }
    }
    if (!ok_all && tid == 0 && p.err_flag) atomicExch(p.err_flag, HB_ERR_TIMEOUT);
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
  while (s < 8 && units * s < sm_count && k_chunks / (s * 2) >= 4) s *= 2;
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
  const int m_cap = n_acc == 2 ? 128 : 256;
  const int64_t m_eff = std::min<int64_t>(M, m_cap);
  pl.m_pad = (int)std::max<int64_t>(16, (m_eff + 15) / 16 * 16);
  pl.m_tiles = (int)((M + pl.m_pad - 1) / pl.m_pad);
  pl.n_tiles = (int)((n_rows + kTileN - 1) / kTileN);
  const int acc_cols = pl.m_pad * n_acc;
  pl.tmem_cols = acc_cols <= 32 ? 32 : acc_cols <= 64 ? 64 : acc_cols <= 128 ? 128 : acc_cols <= 256 ? 256 : 512;
  const size_t stage = (size_t)kTileN * kTileK * 2 * n_acc + (size_t)pl.m_pad * kTileK * 2;
  // two CTAs per SM when the stages allow it, so one CTA's epilogue hides under the
  // other's loads
  size_t budget = 110 * 1024;
  if (const char* ev = getenv("HB_TC_SMEM_KB")) budget = (size_t)atoi(ev) * 1024;  // experiment knob
  pl.stages = (int)std::max<size_t>(2, std::min<size_t>(kMaxStages, budget / stage));
  pl.smem_bytes = pl.stages * stage + 1024;
  if (pl.smem_bytes > di.smem_optin)
    return fail(HB_ERR_INVALID_ARG, "gemm_tc: needs %zu bytes of shared memory", pl.smem_bytes);
  const int ctas_per_sm = std::max(1, std::min<int>((int)(di.smem_optin / pl.smem_bytes), 512 / pl.tmem_cols));
  const int k_chunks = (int)(K / kTileK);
  const int slots = di.sm_count * std::min(ctas_per_sm, 2);
  const char* cl_env = getenv("HB_TC_CLUSTER");
  const bool want_cluster = !(cl_env && cl_env[0] == '0');
  if (force_splits > 0) pl.splits = std::min(force_splits, k_chunks);
  else if (want_cluster) pl.splits = pick_cluster_splits(pl.n_tiles * pl.m_tiles, k_chunks, di.sm_count);
  else pl.splits = pick_splits(pl.n_tiles * pl.m_tiles, k_chunks, slots);
  // cluster form: power-of-two size <= 8 whose receive buffers fit the pipeline's
  // shared memory; anything else reduces through global scratch
  pl.cluster = false;
  auto recv_fits = [&](int sp) {
    return (size_t)(sp - 1) * n_acc * pl.m_pad * (kTileN / sp) * sizeof(float) <= (size_t)pl.stages * stage;
  };
  if (want_cluster && pl.splits > 1) {
    if (force_splits <= 0)
      while (pl.splits > 1 && !recv_fits(pl.splits)) pl.splits /= 2;
    pl.cluster = pl.splits > 1 && pl.splits <= 8 && (pl.splits & (pl.splits - 1)) == 0 && recv_fits(pl.splits);
  }
  const size_t units = (size_t)pl.m_tiles * pl.n_tiles;
  // The tile counters sit in a block of FIXED size at the start of the workspace, so
  // that plans of different shapes sharing one workspace never see each other's
  // partials where they expect zeroed counters.
  if (!pl.cluster && units * sizeof(int) > kCounterBlockBytes) pl.splits = 1;
  pl.ws_partials_bytes = (pl.splits > 1 && !pl.cluster) ? units * pl.splits * n_acc * pl.m_pad * kTileN * sizeof(float) : 0;
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
      // 227 KiB per CTA minus the kernel's static shared memory (barriers, flags)
      HB_CUDA_CHECK(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         226 * 1024));
      dev_done[cur] = true;
    }
  }
  if (getenv("HB_TC_PACKED")) rc = encode_map(&pl.tm_w, W, N * (K / kTileK), kTileK, kTileN);  // speed experiment
  else rc = encode_map(&pl.tm_w, W, N, K, kTileN);
  if (rc) return rc;
  rc = encode_map(&pl.tm_x, X, M, K, pl.m_pad);
  return rc;
}

int gemm_tc_run(const TcGemmPlan& pl, cudaStream_t st, void* Y, int64_t ldy, void* workspace,
                int* err_flag) {
  if (pl.splits > 1 && !pl.cluster && !workspace)
    return fail(HB_ERR_INVALID_ARG, "gemm_tc: split-K plan needs a workspace of %zu bytes",
                pl.workspace_bytes());
  TcParams p;
  p.M = (int)pl.M; p.N = (int)pl.N;
  p.m_pad = pl.m_pad; p.splits = pl.splits; p.stages = pl.stages; p.tmem_cols = pl.tmem_cols;
  p.k_chunks = (int)(pl.K / kTileK);
  p.n_tiles = pl.n_tiles;
  p.epilogue = pl.epilogue; p.out_f32 = pl.out_f32 ? 1 : 0;
  p.ldy = ldy;
  p.up_row_offset = (int)pl.N;
  p.packed = getenv("HB_TC_PACKED") ? 1 : 0;
  p.Y = Y;
  // counters first (16-byte aligned block), partials after
  p.counters = (int*)workspace;
  p.partials = workspace ? (float*)((uint8_t*)workspace + pl.ws_counters_bytes) : nullptr;
  p.err_flag = err_flag;
  p.cluster = pl.cluster ? 1 : 0;
  { const char* sg = getenv("HB_TC_STAGGER"); p.stagger = (sg && sg[0] == '1') ? 1 : 0; }  // measured: no gain, off
  dim3 grid((unsigned)(pl.n_tiles * pl.splits), (unsigned)pl.m_tiles);
  if (pl.cluster) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = pl.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)pl.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    HB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_tc_kernel, pl.tm_w, pl.tm_x, p));
  } else {
    gemm_tc_kernel<<<grid, kTcThreads, pl.smem_bytes, st>>>(pl.tm_w, pl.tm_x, p);
    HB_LAUNCH_CHECK();
  }
  return HB_OK;
}

}  // namespace hb
