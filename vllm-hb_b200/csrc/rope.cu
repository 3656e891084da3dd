// Rotary position embedding.
//
// hb_rope: one CTA per token.  The token's cos/sin row is computed once in f32 from
// positions[t] * inv_freq[i], rounded to the tensor dtype (apply_rope casts its tables
// with to_dtype, src/engine/arch/llama_tp.rs:132-133) and shared by all q and k heads
// of the token; every thread then rotates 128-bit vector pairs (d, d + head_dim/2).
// q and k carry their own head counts, so GQA is handled (the reference's fused
// rope_inplace kernel indexes k with the q head count, kernels/rope.cu:83).
//
// hb_rope_cos_sin: the calling convention of rope_single_{f32,f16}
// (kernels/rope.cu:19-63): tables pre-sliced by the caller, position = token % seq_len.
#include "common.h"

namespace hb {

constexpr int kRopeThreads = 128;
constexpr int kMaxHalf = 256;  // head_dim <= 512

template <typename T>
__global__ void __launch_bounds__(kRopeThreads)
rope_kernel(T* __restrict__ q, T* __restrict__ k, const int32_t* __restrict__ positions,
            const float* __restrict__ inv_freq, int nq, int nkv, int head_dim) {
  __shared__ float s_cos[kMaxHalf];
  __shared__ float s_sin[kMaxHalf];
  const int64_t t = blockIdx.x;
  const int half = head_dim >> 1;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += kRopeThreads) {
    const float f = pos * inv_freq[i];
    float s, c;
    sincosf(f, &s, &c);
    s_cos[i] = to_f32<T>(from_f32<T>(c));
    s_sin[i] = to_f32<T>(from_f32<T>(s));
  }
  __syncthreads();

  constexpr int N = Vec16<T>::N;
  const int heads = nq + (k ? nkv : 0);
  if (half % N == 0) {
    const int vph = half / N;  // vector pairs per head
    for (int idx = threadIdx.x; idx < heads * vph; idx += kRopeThreads) {
      const int h = idx / vph, v = idx % vph;
      T* base = (h < nq) ? q + (t * nq + h) * head_dim : k + (t * nkv + (h - nq)) * head_dim;
      Vec16<T> a, b;
      a.load(base + v * N);
      b.load(base + half + v * N);
      float x1[N], x2[N], o1[N], o2[N];
      a.unpack(x1);
      b.unpack(x2);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float c = s_cos[v * N + j], s = s_sin[v * N + j];
        o1[j] = x1[j] * c - x2[j] * s;
        o2[j] = x1[j] * s + x2[j] * c;
      }
      a.pack(o1);
      b.pack(o2);
      a.store(base + v * N);
      b.store(base + half + v * N);
    }
  } else {
    for (int idx = threadIdx.x; idx < heads * half; idx += kRopeThreads) {
      const int h = idx / half, d = idx % half;
      T* base = (h < nq) ? q + (t * nq + h) * head_dim : k + (t * nkv + (h - nq)) * head_dim;
      const float x1 = to_f32<T>(base[d]), x2 = to_f32<T>(base[d + half]);
      const float c = s_cos[d], s = s_sin[d];
      base[d] = from_f32<T>(x1 * c - x2 * s);
      base[d + half] = from_f32<T>(x1 * s + x2 * c);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kRopeThreads)
rope_cos_sin_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ cos_t,
                    const T* __restrict__ sin_t, int64_t seq_len, int head_dim) {
  const int64_t token = blockIdx.x;  // over batch*heads*seq
  const int half = head_dim >> 1;
  const int64_t t = token % seq_len;
  const T* xi = x + token * head_dim;
  T* yo = out + token * head_dim;
  for (int d = threadIdx.x; d < half; d += kRopeThreads) {
    const float x0 = to_f32<T>(xi[d]), x1 = to_f32<T>(xi[d + half]);
    const float c = to_f32<T>(cos_t[t * half + d]), s = to_f32<T>(sin_t[t * half + d]);
    yo[d] = from_f32<T>(x0 * c - x1 * s);
    yo[d + half] = from_f32<T>(x0 * s + x1 * c);
  }
}

}  // namespace hb

extern "C" {

int hb_rope_inv_freq(float theta, int head_dim, float* out) {
  HB_CHECK_ARG(out && head_dim > 0 && head_dim % 2 == 0, "hb_rope_inv_freq: bad head_dim %d",
               head_dim);
  const int half = head_dim / 2;
  for (int i = 0; i < half; ++i)
    out[i] = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
  return HB_OK;
}

int hb_rope(void* stream, void* q, void* k, const int32_t* positions, const float* inv_freq,
            int64_t n_tokens, int n_q_heads, int n_kv_heads, int head_dim, hb_dtype dtype) {
  HB_CHECK_ARG(q && positions && inv_freq, "hb_rope: null pointer");
  HB_CHECK_ARG(head_dim > 0 && head_dim % 2 == 0 && head_dim / 2 <= hb::kMaxHalf,
               "hb_rope: head_dim %d must be even and <= %d", head_dim, 2 * hb::kMaxHalf);
  HB_CHECK_ARG(n_q_heads > 0 && (!k || n_kv_heads > 0), "hb_rope: bad head counts");
  HB_CHECK_ARG(n_tokens >= 0 && n_tokens < (1ll << 31), "hb_rope: bad n_tokens");
  if (n_tokens == 0) return HB_OK;
  HB_CHECK_ARG((reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(k) & 15) == 0,
               "hb_rope: q and k must be 16-byte aligned");
  HB_DISPATCH_DTYPE(dtype, T, {
    const bool vec_ok = ((head_dim / 2) % hb::Vec16<T>::N == 0);
    (void)vec_ok;
    hb::rope_kernel<T><<<(unsigned)n_tokens, hb::kRopeThreads, 0, (cudaStream_t)stream>>>(
        (T*)q, (T*)k, positions, inv_freq, n_q_heads, n_kv_heads, head_dim);
  });
  HB_LAUNCH_CHECK();
  return HB_OK;
}

int hb_rope_cos_sin(void* stream, void* out, const void* x, const void* cos_table,
                    const void* sin_table, int64_t batch_heads, int64_t seq_len, int head_dim,
                    hb_dtype dtype) {
  HB_CHECK_ARG(out && x && cos_table && sin_table, "hb_rope_cos_sin: null pointer");
  HB_CHECK_ARG(head_dim > 0 && head_dim % 2 == 0, "hb_rope_cos_sin: head_dim must be even");
  HB_CHECK_ARG(batch_heads >= 0 && seq_len > 0 && batch_heads * seq_len < (1ll << 31),
               "hb_rope_cos_sin: bad shape");
  if (batch_heads == 0) return HB_OK;
  HB_DISPATCH_DTYPE(dtype, T, {
    hb::rope_cos_sin_kernel<T><<<(unsigned)(batch_heads * seq_len), hb::kRopeThreads, 0,
                                 (cudaStream_t)stream>>>((T*)out, (const T*)x, (const T*)cos_table,
                                                         (const T*)sin_table, seq_len, head_dim);
  });
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // extern "C"
