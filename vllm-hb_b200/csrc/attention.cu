// Paged GQA decode attention (one query token per sequence).
//
// Work unit = (sequence, kv head, KV split).  A CTA of four warps streams its share of
// the sequence's 16-token KV blocks through the block table with 128-bit loads, each K
// and V row being read ONCE for all n_rep query heads that share the kv head
// (query head j uses kv head j / n_rep, src/engine/arch/llama_tp.rs:264-279; the
// reference materialises n_rep expanded copies instead).  Scores q.k/sqrt(d), an
// online softmax and the weighted sum of V all accumulate in fp32
// (src/engine/arch/llama_tp.rs:304-324 computes the softmax in the tensor dtype).
// With n_splits > 1 the CTAs write (m, l, unnormalised o) partials that a small merge
// kernel combines by log-sum-exp.
//
// Pool layout per layer: [num_blocks, n_kv_heads, 16, head_dim].
#include <climits>
#include <cfloat>
#include <mutex>

#include "common.h"

namespace hb {

constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = 4;
constexpr int kChunkBlocks = 16;                         // KV blocks per softmax chunk
constexpr int kChunkTokens = kChunkBlocks * HB_BLOCK_SIZE;  // 256

// Sum P values across the LPR lanes of a row group so that each lane ends with P/LPR
// complete sums: v[i] (i < P/LPR) is the total of original index
// (lane % LPR) * (P/LPR) + i.  P + P/2 + ... shuffles instead of P * log2(LPR).
template <int P, int LPR>
__device__ __forceinline__ void reduce_scatter(float (&v)[P], int lane_in_group) {
  static_assert(P % LPR == 0, "P must be a multiple of the group width");
  int cnt = P;
#pragma unroll
  for (int o = LPR / 2; o >= 1; o >>= 1) {
    const int half = cnt / 2;
    const bool upper = (lane_in_group & o) != 0;
#pragma unroll
    for (int i = 0; i < P / 2; ++i) {
      if (i < half) {
        const float send = upper ? v[i] : v[i + half];
        const float keep = upper ? v[i + half] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
      }
    }
    cnt = half;
  }
}

template <typename T, int HD, int NREP>
__global__ void __launch_bounds__(kAttnThreads)
paged_attn_kernel(T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                  const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc,
                  const int32_t* __restrict__ block_tables, const int32_t* __restrict__ ctx_lens,
                  int hq, int hkv, int64_t max_blocks, int64_t num_blocks, int n_splits,
                  float scale, int64_t q_stride, int window) {
  pdl_trigger();
  constexpr int N = Vec16<T>::N;       // elements per 16-byte vector
  constexpr int LPR = HD / N;          // lanes covering one row
  constexpr int RPP = 32 / LPR;        // rows per warp pass
  constexpr int PB = HB_BLOCK_SIZE / RPP;  // passes per KV block
  // heads padded so that a block's partial sums are a multiple of the group width
  constexpr int NH = (PB * NREP) % LPR == 0 ? NREP : (LPR / PB);
  constexpr int P = PB * NH;
  constexpr int OUTS = P / LPR;        // finished scores per lane per block
  static_assert(LPR <= 32 && 32 % LPR == 0, "unsupported head_dim / dtype");
  static_assert(P % LPR == 0 && NH >= NREP, "bad padding");

  __shared__ float s_p[NREP][kChunkTokens];
  __shared__ float s_red[kAttnWarps][NREP];
  __shared__ float s_acc[kAttnWarps][NREP][HD];

  const int split = blockIdx.x, kvh = blockIdx.y;
  const int64_t seq = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = lane % LPR, grp = lane / LPR;

  // a context longer than the table row can describe is cut to the row (the table of the
  // next sequence, or memory past the allocation, is never indexed)
  const int ctx = max(0, min(ctx_lens[seq], (int)min(max_blocks * HB_BLOCK_SIZE, (int64_t)INT_MAX)));
  const int nblk = (ctx + HB_BLOCK_SIZE - 1) / HB_BLOCK_SIZE;
  // sliding window (src/engine/arch/mixtral.rs:155-176): keys ki with ctx-1-ki < window
  const int first_tok = window > 0 ? max(0, ctx - window) : 0;
  const int first_blk = first_tok / HB_BLOCK_SIZE;
  const int bps = (nblk - first_blk + n_splits - 1) / n_splits;
  const int b0 = first_blk + split * bps;
  const int b1 = min(nblk, b0 + bps);

  // query slices, pre-scaled by 1/sqrt(d)
  float qf[NH][N];
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    if (h < NREP) {
      Vec16<T> qv;
      qv.load(q + seq * q_stride + ((int64_t)kvh * NREP + h) * HD + c * N);
      qv.unpack(qf[h]);
#pragma unroll
      for (int j = 0; j < N; ++j) qf[h][j] *= scale;
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j) qf[h][j] = 0.f;
    }
  }

  float m_run[NREP], l_loc[NREP], acc[NREP][N];
#pragma unroll
  for (int h = 0; h < NREP; ++h) {
    m_run[h] = -INFINITY;
    l_loc[h] = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) acc[h][j] = 0.f;
  }
  const int32_t* table = block_tables + seq * max_blocks;

  for (int cb = b0; cb < b1; cb += kChunkBlocks) {
    const int nb = min(kChunkBlocks, b1 - cb);

    // ---- phase 1: scores of this chunk into shared memory
    for (int bi = warp; bi < nb; bi += kAttnWarps) {
      int64_t phys = table[cb + bi];
      if (phys < 0 || phys >= num_blocks) phys = 0;  // never read outside the pool
      const T* kb = kc + ((phys * hkv + kvh) * HB_BLOCK_SIZE) * (int64_t)HD;
      Vec16<T> kv[PB];
#pragma unroll
      for (int p = 0; p < PB; ++p) kv[p].load(kb + (p * RPP + grp) * HD + c * N);
      float part[P];
#pragma unroll
      for (int p = 0; p < PB; ++p) {
        float kf[N];
        kv[p].unpack(kf);
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          float s = 0.f;
#pragma unroll
          for (int j = 0; j < N; ++j) s = fmaf(qf[h][j], kf[j], s);
          part[p * NH + h] = s;
        }
      }
      reduce_scatter<P, LPR>(part, c);
#pragma unroll
      for (int i = 0; i < OUTS; ++i) {
        const int idx = c * OUTS + i;  // = p * NH + h
        const int p = idx / NH, h = idx % NH;
        if (h < NREP) {
          const int tok_in_blk = p * RPP + grp;
          const int tok = (cb + bi) * HB_BLOCK_SIZE + tok_in_blk;
          s_p[h][bi * HB_BLOCK_SIZE + tok_in_blk] = (tok < ctx && tok >= first_tok) ? part[i] : -INFINITY;
        }
      }
    }
    __syncthreads();

    // ---- chunk maximum per head, rescale the running state
    const int ntok = nb * HB_BLOCK_SIZE;
    float cmax[NREP];
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
      float v = -INFINITY;
      for (int t = tid; t < ntok; t += kAttnThreads) v = fmaxf(v, s_p[h][t]);
      v = warp_max(v);
      if (lane == 0) s_red[warp][h] = v;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
      float v = s_red[0][h];
#pragma unroll
      for (int w = 1; w < kAttnWarps; ++w) v = fmaxf(v, s_red[w][h]);
      cmax[h] = v;
    }
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
      const float m_new = fmaxf(m_run[h], cmax[h]);
      const float alpha = (m_run[h] == -INFINITY) ? 0.f : __expf(m_run[h] - m_new);
      m_run[h] = m_new;
      l_loc[h] *= alpha;
#pragma unroll
      for (int j = 0; j < N; ++j) acc[h][j] *= alpha;
      for (int t = tid; t < ntok; t += kAttnThreads) {
        const float e = __expf(s_p[h][t] - m_new);  // exp(-inf) = 0 for masked tokens
        s_p[h][t] = e;
        l_loc[h] += e;
      }
    }
    __syncthreads();

    // ---- phase 2: acc += p * V
    for (int bi = warp; bi < nb; bi += kAttnWarps) {
      int64_t phys = table[cb + bi];
      if (phys < 0 || phys >= num_blocks) phys = 0;
      const T* vb = vc + ((phys * hkv + kvh) * HB_BLOCK_SIZE) * (int64_t)HD;
      Vec16<T> vv[PB];
#pragma unroll
      for (int p = 0; p < PB; ++p) vv[p].load(vb + (p * RPP + grp) * HD + c * N);
#pragma unroll
      for (int p = 0; p < PB; ++p) {
        const int tok_in_blk = p * RPP + grp;
        const int tok = (cb + bi) * HB_BLOCK_SIZE + tok_in_blk;
        float vf[N];
        vv[p].unpack(vf);
        if (tok >= ctx) {  // slots past the context may hold anything, NaN included
#pragma unroll
          for (int j = 0; j < N; ++j) vf[j] = 0.f;
        }
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
          const float pw = s_p[h][bi * HB_BLOCK_SIZE + tok_in_blk];
#pragma unroll
          for (int j = 0; j < N; ++j) acc[h][j] = fmaf(pw, vf[j], acc[h][j]);
        }
      }
    }
    __syncthreads();
  }

  // ---- combine: row groups inside the warp, then the four warps
#pragma unroll
  for (int h = 0; h < NREP; ++h) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float v = acc[h][j];
#pragma unroll
      for (int o = LPR; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[h][j] = v;
    }
    float l = warp_sum(l_loc[h]);
    if (lane == 0) s_red[warp][h] = l;
    if (grp == 0) {
#pragma unroll
      for (int j = 0; j < N; ++j) s_acc[warp][h][c * N + j] = acc[h][j];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < NREP * HD; idx += kAttnThreads) {
    const int h = idx / HD, d = idx % HD;
    float o = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      o += s_acc[w][h][d];
      l += s_red[w][h];
    }
    const int64_t head = seq * hq + (int64_t)kvh * NREP + h;
    if (n_splits == 1) {
      out[head * HD + d] = from_f32<T>(l > 0.f ? o / l : 0.f);
    } else {
      part_o[(head * n_splits + split) * HD + d] = o;
      if (d == 0) {
        part_ml[(head * n_splits + split) * 2 + 0] = m_run[h];
        part_ml[(head * n_splits + split) * 2 + 1] = l;
      }
    }
  }
}

// out = sum_s exp(m_s - M) o_s / sum_s exp(m_s - M) l_s, one warp-sized CTA per head.
template <typename T>
__global__ void attn_merge_kernel(T* __restrict__ out, const float* __restrict__ part_o,
                                  const float* __restrict__ part_ml, int n_splits, int hd) {
  pdl_trigger();
  const int64_t head = blockIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(head * n_splits + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float m = part_ml[(head * n_splits + s) * 2];
    const float w = (m == -INFINITY) ? 0.f : __expf(m - M);
    L += w * part_ml[(head * n_splits + s) * 2 + 1];
  }
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float m = part_ml[(head * n_splits + s) * 2];
      const float w = (m == -INFINITY) ? 0.f : __expf(m - M);
      o += w * part_o[(head * n_splits + s) * hd + d];
    }
    out[head * hd + d] = from_f32<T>(L > 0.f ? o / L : 0.f);
  }
}

template <typename T, int HD, int NREP>
static int launch_attn(cudaStream_t st, T* out, float* part_o, float* part_ml, const T* q,
                       const T* kc, const T* vc, const int32_t* bt, const int32_t* cl,
                       int64_t n_seqs, int hq, int hkv, int64_t max_blocks, int64_t num_blocks,
                       int n_splits, int64_t q_stride, int window) {
  dim3 grid((unsigned)n_splits, (unsigned)hkv, (unsigned)n_seqs);
  const float scale = 1.0f / sqrtf((float)HD);
  paged_attn_kernel<T, HD, NREP><<<grid, kAttnThreads, 0, st>>>(
      out, part_o, part_ml, q, kc, vc, bt, cl, hq, hkv, max_blocks, num_blocks, n_splits, scale,
      q_stride, window);
  HB_LAUNCH_CHECK();
  if (n_splits > 1) {
    attn_merge_kernel<T><<<(unsigned)(n_seqs * hq), HD <= 64 ? 64 : 128, 0, st>>>(
        out, part_o, part_ml, n_splits, HD);
    HB_LAUNCH_CHECK();
  }
  return HB_OK;
}

template <typename T, int HD>
static int dispatch_nrep(int nrep, cudaStream_t st, T* out, float* po, float* pml, const T* q,
                         const T* kc, const T* vc, const int32_t* bt, const int32_t* cl,
                         int64_t n_seqs, int hq, int hkv, int64_t mb, int64_t nb, int ns, int64_t qs, int win) {
  switch (nrep) {
    case 1: return launch_attn<T, HD, 1>(st, out, po, pml, q, kc, vc, bt, cl, n_seqs, hq, hkv, mb, nb, ns, qs, win);
    case 2: return launch_attn<T, HD, 2>(st, out, po, pml, q, kc, vc, bt, cl, n_seqs, hq, hkv, mb, nb, ns, qs, win);
    case 4: return launch_attn<T, HD, 4>(st, out, po, pml, q, kc, vc, bt, cl, n_seqs, hq, hkv, mb, nb, ns, qs, win);
    case 8: return launch_attn<T, HD, 8>(st, out, po, pml, q, kc, vc, bt, cl, n_seqs, hq, hkv, mb, nb, ns, qs, win);
    default:
      return fail(HB_ERR_INVALID_ARG,
                  "hb_paged_decode_attention: n_q_heads/n_kv_heads = %d not in {1,2,4,8}", nrep);
  }
}

// Tensor-core kernel (attention_mma.cu): bf16, head_dim 128, up to 16 query heads per kv head.
bool paged_attention_mma_supported(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                   int nrep, int head_dim, int64_t num_blocks, int hkv, hb_dtype dtype);
int paged_attention_mma(cudaStream_t st, void* out, float* part_o, float* part_ml, const void* q,
                        int64_t q_stride, const void* k_cache, const void* v_cache, const int32_t* block_tables,
                        const int32_t* ctx_lens, int64_t n_seqs, int hq, int hkv, int64_t max_blocks,
                        int64_t num_blocks, int n_splits, int window, int* err_flag, int fresh, int q_group);

// Internal entry: q rows may sit inside a wider [q|k|v] projection buffer.  err_flag
// (device int, may be null) is raised when a bounded wait of the tensor-core kernel ran out.
int paged_attention(cudaStream_t st, void* out, const void* q, int64_t q_stride, const void* k_cache,
                    const void* v_cache, const int32_t* block_tables, const int32_t* ctx_lens,
                    int64_t n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                    int64_t max_blocks_per_seq, int64_t num_blocks, int n_splits, void* workspace,
                    hb_dtype dtype, int* err_flag, int window, int fresh_tokens, int q_group) {
  if (n_seqs == 0) return HB_OK;
  const int nrep = n_q_heads / n_kv_heads;
  float* po = (float*)workspace;
  float* pml = po ? po + (size_t)n_seqs * n_q_heads * n_splits * head_dim : nullptr;
  static const bool force_simt = [] { const char* e = getenv("HB_ATTN"); return e && e[0] == 's'; }();
  if (!force_simt && paged_attention_mma_supported(q, q_stride, k_cache, v_cache, nrep, head_dim, num_blocks,
                                                   n_kv_heads, dtype)) {
    int rc = paged_attention_mma(st, out, po, pml, q, q_stride, k_cache, v_cache, block_tables, ctx_lens, n_seqs,
                                 n_q_heads, n_kv_heads, max_blocks_per_seq, num_blocks, n_splits, window, err_flag,
                                 fresh_tokens, q_group);
    if (rc) return rc;
    if (n_splits > 1) {
      attn_merge_kernel<__nv_bfloat16><<<(unsigned)(n_seqs * n_q_heads), 128, 0, st>>>(
          (__nv_bfloat16*)out, po, pml, n_splits, head_dim);
      HB_LAUNCH_CHECK();
    }
    return HB_OK;
  }
  HB_DISPATCH_DTYPE(dtype, T, {
    if (head_dim == 128)
      return (dispatch_nrep<T, 128>(nrep, st, (T*)out, po, pml, (const T*)q, (const T*)k_cache,
                                    (const T*)v_cache, block_tables, ctx_lens, n_seqs, n_q_heads,
                                    n_kv_heads, max_blocks_per_seq, num_blocks, n_splits, q_stride, window));
    if (head_dim == 64)
      return (dispatch_nrep<T, 64>(nrep, st, (T*)out, po, pml, (const T*)q, (const T*)k_cache,
                                   (const T*)v_cache, block_tables, ctx_lens, n_seqs, n_q_heads,
                                   n_kv_heads, max_blocks_per_seq, num_blocks, n_splits, q_stride, window));
    return fail(HB_ERR_INVALID_ARG, "paged attention: head_dim %d not in {64,128}", head_dim);
  });
  return HB_OK;
}

}  // namespace hb

extern "C" {

size_t hb_attention_workspace_bytes(int64_t n_seqs, int n_q_heads, int head_dim, int n_splits) {
  if (n_splits <= 1 || n_seqs <= 0) return 0;
  return (size_t)n_seqs * n_q_heads * n_splits * (head_dim + 2) * sizeof(float);
}

int hb_paged_decode_attention(void* stream, void* out, const void* q, const void* k_cache,
                              const void* v_cache, const int32_t* block_tables,
                              const int32_t* ctx_lens, int64_t n_seqs, int n_q_heads,
                              int n_kv_heads, int head_dim, int64_t max_blocks_per_seq,
                              int64_t num_blocks, int n_splits, void* workspace, hb_dtype dtype) {
  HB_CHECK_ARG(out && q && k_cache && v_cache && block_tables && ctx_lens,
               "hb_paged_decode_attention: null pointer");
  HB_CHECK_ARG(n_seqs >= 0 && n_seqs <= 65535, "hb_paged_decode_attention: n_seqs %lld out of range",
               (long long)n_seqs);
  HB_CHECK_ARG(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0,
               "hb_paged_decode_attention: n_q_heads must be a multiple of n_kv_heads");
  HB_CHECK_ARG(n_splits >= 1 && n_splits <= 64, "hb_paged_decode_attention: n_splits out of range");
  HB_CHECK_ARG(n_splits == 1 || workspace, "hb_paged_decode_attention: workspace needed for splits");
  HB_CHECK_ARG(max_blocks_per_seq > 0 && num_blocks > 0, "hb_paged_decode_attention: bad block counts");
  return hb::paged_attention((cudaStream_t)stream, out, q, (int64_t)n_q_heads * head_dim, k_cache,
                             v_cache, block_tables, ctx_lens, n_seqs, n_q_heads, n_kv_heads,
                             head_dim, max_blocks_per_seq, num_blocks, n_splits, workspace, dtype, nullptr, 0, -1, 1);
}

int hb_paged_decode_attention_window(void* stream, void* out, const void* q, const void* k_cache,
                                     const void* v_cache, const int32_t* block_tables,
                                     const int32_t* ctx_lens, int64_t n_seqs, int n_q_heads,
                                     int n_kv_heads, int head_dim, int64_t max_blocks_per_seq,
                                     int64_t num_blocks, int n_splits, void* workspace, int sliding_window,
                                     hb_dtype dtype) {
  HB_CHECK_ARG(out && q && k_cache && v_cache && block_tables && ctx_lens,
               "hb_paged_decode_attention_window: null pointer");
  HB_CHECK_ARG(n_seqs >= 0 && n_seqs <= 65535, "hb_paged_decode_attention_window: n_seqs %lld out of range",
               (long long)n_seqs);
  HB_CHECK_ARG(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0,
               "hb_paged_decode_attention_window: n_q_heads must be a multiple of n_kv_heads");
  HB_CHECK_ARG(n_splits >= 1 && n_splits <= 64, "hb_paged_decode_attention_window: n_splits out of range");
  HB_CHECK_ARG(n_splits == 1 || workspace, "hb_paged_decode_attention_window: workspace needed for splits");
  HB_CHECK_ARG(max_blocks_per_seq > 0 && num_blocks > 0, "hb_paged_decode_attention_window: bad block counts");
  HB_CHECK_ARG(sliding_window >= 0, "hb_paged_decode_attention_window: negative window");
  return hb::paged_attention((cudaStream_t)stream, out, q, (int64_t)n_q_heads * head_dim, k_cache,
                             v_cache, block_tables, ctx_lens, n_seqs, n_q_heads, n_kv_heads, head_dim,
                             max_blocks_per_seq, num_blocks, n_splits, workspace, dtype, nullptr, sliding_window, -1, 1);
}

}  // extern "C"

// ---------------------------------------------------------------------------------
// Split-KV decode attention for callers that cannot allocate device memory.
//
// The split partials (unnormalised outputs and the (max, sum) pairs) live in a
// file-scope device array instead of a caller-provided workspace.  Every GPU that
// loads this library carries the array until the process exits.
namespace hb {

constexpr size_t kStaticAttnScratchBytes = 8u << 20;  // 8 MiB per device
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticAttnScratchBytes];

// In host code `g_attn_static_scratch` is only a handle for the runtime, not a device
// address: the address is asked for once per device, with that device current.
static int static_attn_scratch(void** out) {
  static std::mutex mu;
  static void* cached[64] = {nullptr};
  int dev = 0;
  HB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(HB_ERR_INVALID_ARG, "device %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* ptr = nullptr;
    HB_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_attn_static_scratch));
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return HB_OK;
}

}  // namespace hb

extern "C" {

size_t hb_paged_decode_attention_static_max_bytes(void) { return hb::kStaticAttnScratchBytes; }

int hb_paged_decode_attention_static(void* stream, void* out, const void* q, const void* k_cache,
                                     const void* v_cache, const int32_t* block_tables,
                                     const int32_t* ctx_lens, int64_t n_seqs, int n_q_heads,
                                     int n_kv_heads, int head_dim, int64_t max_blocks_per_seq,
                                     int64_t num_blocks, int n_splits, hb_dtype dtype) {
  HB_CHECK_ARG(out && q && k_cache && v_cache && block_tables && ctx_lens,
               "hb_paged_decode_attention_static: null pointer");
  HB_CHECK_ARG(n_seqs >= 0 && n_seqs <= 65535, "hb_paged_decode_attention_static: n_seqs %lld out of range",
               (long long)n_seqs);
  HB_CHECK_ARG(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0,
               "hb_paged_decode_attention_static: n_q_heads must be a multiple of n_kv_heads");
  HB_CHECK_ARG(n_splits >= 1 && n_splits <= 64, "hb_paged_decode_attention_static: n_splits out of range");
  HB_CHECK_ARG(max_blocks_per_seq > 0 && num_blocks > 0, "hb_paged_decode_attention_static: bad block counts");
  const size_t need = hb_attention_workspace_bytes(n_seqs, n_q_heads, head_dim, n_splits);
  if (need > hb::kStaticAttnScratchBytes)
    return hb::fail(HB_ERR_INVALID_ARG,
                    "hb_paged_decode_attention_static: %lld sequences x %d heads x %d splits need %zu bytes of "
                    "split scratch, the built-in array holds %zu; use fewer splits or "
                    "hb_paged_decode_attention with a workspace of your own",
                    (long long)n_seqs, n_q_heads, n_splits, need, hb::kStaticAttnScratchBytes);
  void* scratch = nullptr;
  int rc = hb::static_attn_scratch(&scratch);
  if (rc) return rc;
  return hb::paged_attention((cudaStream_t)stream, out, q, (int64_t)n_q_heads * head_dim, k_cache, v_cache,
                             block_tables, ctx_lens, n_seqs, n_q_heads, n_kv_heads, head_dim,
                             max_blocks_per_seq, num_blocks, n_splits, scratch, dtype, nullptr, 0, -1, 1);
}

}  // extern "C"
