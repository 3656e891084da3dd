// Engine-internal kernels: fused RoPE + paged KV write on the [q|k|v] projection row,
// device-side weight initialisation, dtype conversion.
#include "common.h"
#include "ops.h"

namespace hb {

constexpr int kRkThreads = 128;

// One CTA per token.  Row layout: [q (nq*hd) | k (nkv*hd) | v (nkv*hd)].
// q is rotated in place; rotated k and the untouched v go to slot_mapping[t] of the
// pool [num_blocks, nkv, 16, hd].  The rotation is the one of hb_rope (cos/sin in f32,
// rounded to T, apply_rope src/engine/arch/llama_tp.rs:112-152); K is cached after RoPE
// (src/engine/arch/llama_tp.rs:242-259).
template <typename T>
__global__ void __launch_bounds__(kRkThreads)
rope_kv_kernel(T* __restrict__ qkv, T* __restrict__ kc, T* __restrict__ vc,
               const int32_t* __restrict__ positions, const int64_t* __restrict__ slots,
               const float* __restrict__ inv_freq, int nq, int nkv, int hd, int64_t num_blocks) {
  __shared__ float s_cos[256];
  __shared__ float s_sin[256];
  pdl_trigger();
  pdl_grid_wait();
  constexpr int N = Vec16<T>::N;
  const int64_t t = blockIdx.x;
  const int half = hd >> 1;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += kRkThreads) {
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    s_cos[i] = to_f32<T>(from_f32<T>(c));
    s_sin[i] = to_f32<T>(from_f32<T>(s));
  }
  __syncthreads();
  const int64_t row_len = (int64_t)(nq + 2 * nkv) * hd;
  T* row = qkv + t * row_len;
  const int64_t slot = slots[t];
  const bool store = slot >= 0 && slot < num_blocks * HB_BLOCK_SIZE;
  const int64_t blk = store ? slot / HB_BLOCK_SIZE : 0, off = store ? slot % HB_BLOCK_SIZE : 0;
  const int vph = half / N;  // vector pairs per head
  // q heads and k heads: rotate
  for (int idx = threadIdx.x; idx < (nq + nkv) * vph; idx += kRkThreads) {
    const int h = idx / vph, v = idx % vph;
    T* base = row + (int64_t)h * hd;  // k heads follow the q heads directly
    Vec16<T> a, b;
    a.load(base + v * N);
    b.load(base + half + v * N);
    float x1[N], x2[N], o1[N], o2[N];
    a.unpack(x1);
    b.unpack(x2);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      rope_rotate(x1[j], x2[j], s_cos[v * N + j], s_sin[v * N + j], &o1[j], &o2[j]);
    }
    a.pack(o1);
    b.pack(o2);
    if (h < nq) {
      a.store(base + v * N);
      b.store(base + half + v * N);
    } else if (store) {
      T* dst = kc + (((blk * nkv + (h - nq)) * HB_BLOCK_SIZE + off) * (int64_t)hd);
      a.store(dst + v * N);
      b.store(dst + half + v * N);
    }
  }
  // v heads: copy
  if (store) {
    const int vecs = hd / N;
    for (int idx = threadIdx.x; idx < nkv * vecs; idx += kRkThreads) {
      const int h = idx / vecs, v = idx % vecs;
      Vec16<T> a;
      a.load(row + (int64_t)(nq + nkv + h) * hd + v * N);
      a.store(vc + (((blk * nkv + h) * HB_BLOCK_SIZE + off) * (int64_t)hd) + v * N);
    }
  }
}

int rope_kv_write(cudaStream_t st, void* qkv, void* k_cache, void* v_cache,
                  const int32_t* positions, const int64_t* slot_mapping, const float* inv_freq,
                  int64_t n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                  int64_t num_blocks, hb_dtype dtype) {
  if (n_tokens == 0) return HB_OK;
  if (head_dim % 2 || head_dim / 2 > 256)
    return fail(HB_ERR_INVALID_ARG, "rope_kv_write: head_dim %d unsupported", head_dim);
  HB_DISPATCH_DTYPE(dtype, T, {
    if ((head_dim / 2) % Vec16<T>::N != 0)
      return fail(HB_ERR_INVALID_ARG, "rope_kv_write: head_dim %d too small for 128-bit vectors",
                  head_dim);
    HB_CUDA_CHECK(launch_pdl(rope_kv_kernel<T>, dim3((unsigned)n_tokens), dim3(kRkThreads), 0, st, (T*)qkv,
                             (T*)k_cache, (T*)v_cache, positions, slot_mapping, inv_freq, n_q_heads, n_kv_heads,
                             head_dim, num_blocks));
  });
  return HB_OK;
}

// (cos, sin) of position[t] * inv_freq[i], rounded to T like rope_kv_kernel rounds them:
// computed once per decode step for the GEMM epilogue that rotates q and k (TcNormLink).
template <typename T>
__global__ void rope_table_kernel(float2* __restrict__ table, const int32_t* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int64_t n_tokens, int half) {
  pdl_trigger();
  pdl_grid_wait();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_tokens * half) return;
  const int64_t t = idx / half;
  const int i = (int)(idx % half);
  float s, c;
  sincosf((float)positions[t] * inv_freq[i], &s, &c);
  table[idx] = make_float2(to_f32<T>(from_f32<T>(c)), to_f32<T>(from_f32<T>(s)));
}

int rope_table(cudaStream_t st, float2* table, const int32_t* positions, const float* inv_freq,
               int64_t n_tokens, int head_dim, hb_dtype dtype) {
  if (n_tokens == 0) return HB_OK;
  const int half = head_dim / 2;
  const int64_t total = n_tokens * half;
  HB_DISPATCH_DTYPE(dtype, T, {
    HB_CUDA_CHECK(launch_pdl(rope_table_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, table,
                             positions, inv_freq, n_tokens, half));
  });
  return HB_OK;
}

// ------------------------------------------------------------ weight initialisation
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ dst, int64_t rows, int64_t cols, int64_t row0,
                                   int64_t col0, int64_t g_cols, uint64_t key, float std, int64_t dst_ld) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * cols) return;
  const int64_t r = idx / cols, c = idx % cols;
  const uint64_t g = (uint64_t)((row0 + r) * g_cols + (col0 + c));
  const uint64_t z = splitmix64(key ^ splitmix64(g));
  const float u1 = ((float)(z >> 40) + 1.0f) * (1.0f / 16777216.0f);        // (0, 1]
  const float u2 = ((float)((z >> 16) & 0xFFFFFF) + 0.5f) * (1.0f / 16777216.0f);
  const float n = sqrtf(-2.0f * __logf(u1)) * __cosf(6.28318530717958647692f * u2);
  dst[r * dst_ld + c] = from_f32<T>(n * std);
}

template <typename T>
__global__ void fill_const_kernel(T* __restrict__ dst, int64_t n, float v) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n) dst[idx] = from_f32<T>(v);
}

template <typename T>
__global__ void to_f32_kernel(float* __restrict__ dst, const T* __restrict__ src, int64_t n, int64_t cols,
                              int64_t src_ld) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n) dst[idx] = to_f32<T>(src[(idx / cols) * src_ld + idx % cols]);
}

// dst[r * dst_ld + c] = convert(src[r * cols + c]) for a dense [rows, cols] source
template <typename TD, typename TS>
__global__ void convert_2d_kernel(TD* __restrict__ dst, const TS* __restrict__ src, int64_t n, int64_t cols,
                                  int64_t dst_ld) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n) dst[(idx / cols) * dst_ld + idx % cols] = from_f32<TD>(to_f32<TS>(src[idx]));
}

int convert_2d(cudaStream_t st, void* dst, hb_dtype dst_dtype, int64_t dst_ld, const void* src, hb_dtype src_dtype,
               int64_t rows, int64_t cols) {
  const int64_t n = rows * cols;
  if (n == 0) return HB_OK;
  if (dst_ld <= 0) dst_ld = cols;
  const unsigned grid = (unsigned)((n + 255) / 256);
  HB_DISPATCH_DTYPE(dst_dtype, TD, {
    switch (src_dtype) {
      case HB_F32: convert_2d_kernel<TD, float><<<grid, 256, 0, st>>>((TD*)dst, (const float*)src, n, cols, dst_ld); break;
      case HB_F16: convert_2d_kernel<TD, __half><<<grid, 256, 0, st>>>((TD*)dst, (const __half*)src, n, cols, dst_ld); break;
      case HB_BF16: convert_2d_kernel<TD, __nv_bfloat16><<<grid, 256, 0, st>>>((TD*)dst, (const __nv_bfloat16*)src, n, cols, dst_ld); break;
      default: return fail(HB_ERR_UNSUPPORTED_DTYPE, "unsupported source dtype %d", (int)src_dtype);
    }
  });
  HB_LAUNCH_CHECK();
  return HB_OK;
}

int fill_normal(cudaStream_t st, void* dst, hb_dtype dtype, int64_t rows, int64_t cols,
                int64_t row0, int64_t col0, int64_t g_cols, uint64_t seed, uint64_t tensor_id,
                float std, int64_t dst_ld) {
  const int64_t n = rows * cols;
  if (dst_ld <= 0) dst_ld = cols;
  if (n == 0) return HB_OK;
  const uint64_t key = seed * 0xD1342543DE82EF95ull + tensor_id * 0x9E3779B97F4A7C15ull + 1;
  HB_DISPATCH_DTYPE(dtype, T, {
    fill_normal_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>((T*)dst, rows, cols, row0,
                                                                      col0, g_cols, key, std, dst_ld);
  });
  HB_LAUNCH_CHECK();
  return HB_OK;
}

int fill_const(cudaStream_t st, void* dst, hb_dtype dtype, int64_t n, float value) {
  if (n == 0) return HB_OK;
  HB_DISPATCH_DTYPE(dtype, T, {
    fill_const_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>((T*)dst, n, value);
  });
  HB_LAUNCH_CHECK();
  return HB_OK;
}

int to_f32(cudaStream_t st, float* dst, const void* src, hb_dtype dtype, int64_t n, int64_t cols, int64_t src_ld) {
  if (n == 0) return HB_OK;
  if (cols <= 0) cols = n;
  if (src_ld <= 0) src_ld = cols;
  HB_DISPATCH_DTYPE(dtype, T, {
    to_f32_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(dst, (const T*)src, n, cols, src_ld);
  });
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace hb
