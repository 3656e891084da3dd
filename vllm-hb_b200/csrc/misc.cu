// Small memory-bound ops of the decode step: SwiGLU gate, embedding gather, argmax.
#include <cfloat>

#include "common.h"

namespace hb {

// out[m,i] = silu(g[m,i]) * u[m,i], gate_up row = [gate(inter) | up(inter)].
// silu(z) = z * sigmoid(z) in fp32, product rounded once
// (ffn_partial, src/engine/arch/llama_tp.rs:333-339).
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t M,
                                int64_t inter) {
  constexpr int N = Vec16<T>::N;
  const int64_t vper = inter / N;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * vper) return;
  const int64_t m = idx / vper, v = idx % vper;
  Vec16<T> g, u;
  g.load(gu + m * 2 * inter + v * N);
  u.load(gu + m * 2 * inter + inter + v * N);
  float a[N], b[N];
  g.unpack(a);
  u.unpack(b);
#pragma unroll
  for (int j = 0; j < N; ++j) a[j] = (a[j] / (1.f + __expf(-a[j]))) * b[j];
  g.pack(a);
  g.store(out + m * inter + v * N);
}

template <typename T>
__global__ void silu_mul_scalar_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t M,
                                       int64_t inter) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * inter) return;
  const int64_t m = idx / inter, i = idx % inter;
  const float a = to_f32<T>(gu[m * 2 * inter + i]);
  const float b = to_f32<T>(gu[m * 2 * inter + inter + i]);
  out[idx] = from_f32<T>((a / (1.f + __expf(-a))) * b);
}

template <typename V>
__global__ void embed_kernel(V* __restrict__ out, const V* __restrict__ table,
                             const uint32_t* __restrict__ ids, int64_t row_v, int64_t vocab) {
  const int64_t t = blockIdx.x;
  uint32_t id = ids[t];
  if (id >= vocab) id = (uint32_t)(vocab - 1);  // never read outside the table
  const V* src = table + (int64_t)id * row_v;
  V* dst = out + t * row_v;
  for (int64_t i = threadIdx.x; i < row_v; i += blockDim.x) dst[i] = src[i];
}

// First index of the maximum of each row (ties -> lowest index).
template <typename T>
__global__ void __launch_bounds__(1024)
argmax_kernel(uint32_t* __restrict__ out, const T* __restrict__ logits, int64_t vocab) {
  __shared__ float s_val[32];
  __shared__ uint32_t s_idx[32];
  const T* row = logits + (int64_t)blockIdx.x * vocab;
  float best = -FLT_MAX;
  uint32_t bi = 0xffffffffu;
  // NaN never wins; strictly greater keeps the earliest index within a thread (a thread
  // visits its elements in increasing index order on both paths)
  auto take = [&](float v, int64_t i) {
    if (v > best || bi == 0xffffffffu) {
      if (v == v) { best = v; bi = (uint32_t)i; }
    }
  };
  constexpr int N = Vec16<T>::N;
  if (vocab % N == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // 128-bit loads, four independent ones in flight per thread
    const int64_t nvec = vocab / N;
    const int64_t step = blockDim.x;
    for (int64_t v0 = threadIdx.x; v0 < nvec; v0 += 4 * step) {
      Vec16<T> a[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + u * step < nvec) a[u].load(row + (v0 + u * step) * N);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (v0 + u * step < nvec) {
          float f[N];
          a[u].unpack(f);
#pragma unroll
          for (int j = 0; j < N; ++j) take(f[j], (v0 + u * step) * N + j);
        }
      }
    }
  } else {
    for (int64_t i = threadIdx.x; i < vocab; i += blockDim.x) take(to_f32<T>(row[i]), i);
  }
  auto better = [](float v, uint32_t i, float bv, uint32_t bidx) {
    return (i != 0xffffffffu) && (bidx == 0xffffffffu || v > bv || (v == bv && i < bidx));
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) { s_val[wid] = best; s_idx[wid] = bi; }
  __syncthreads();
  if (wid == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? s_val[lane] : -FLT_MAX;
    bi = lane < nw ? s_idx[lane] : 0xffffffffu;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = (bi == 0xffffffffu) ? 0u : bi;
  }
}

}  // namespace hb

extern "C" {

int hb_silu_mul(void* stream, void* out, const void* gate_up, int64_t M, int64_t inter,
                hb_dtype dtype) {
  HB_CHECK_ARG(out && gate_up, "hb_silu_mul: null pointer");
  HB_CHECK_ARG(M >= 0 && inter > 0, "hb_silu_mul: bad shape");
  if (M == 0) return HB_OK;
  auto st = (cudaStream_t)stream;
  HB_DISPATCH_DTYPE(dtype, T, {
    constexpr int N = hb::Vec16<T>::N;
    const bool vec = inter % N == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(gate_up) & 15) == 0;
    if (vec) {
      const int64_t total = M * (inter / N);
      hb::silu_mul_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
          (T*)out, (const T*)gate_up, M, inter);
    } else {
      const int64_t total = M * inter;
      hb::silu_mul_scalar_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
          (T*)out, (const T*)gate_up, M, inter);
    }
  });
  HB_LAUNCH_CHECK();
  return HB_OK;
}

int hb_embed(void* stream, void* out, const void* table, const uint32_t* ids, int64_t n_tokens,
             int64_t hidden, int64_t vocab, hb_dtype dtype) {
  HB_CHECK_ARG(out && table && ids, "hb_embed: null pointer");
  HB_CHECK_ARG(hb::dtype_valid(dtype), "hb_embed: bad dtype");
  HB_CHECK_ARG(n_tokens >= 0 && hidden > 0 && vocab > 0, "hb_embed: bad shape");
  if (n_tokens == 0) return HB_OK;
  auto st = (cudaStream_t)stream;
  const size_t row_bytes = (size_t)hidden * hb::dtype_size(dtype);
  const bool vec = row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(table) & 15) == 0;
  if (vec)
    hb::embed_kernel<uint4><<<(unsigned)n_tokens, 256, 0, st>>>((uint4*)out, (const uint4*)table,
                                                               ids, (int64_t)(row_bytes / 16), vocab);
  else if (hb::dtype_size(dtype) == 4)
    hb::embed_kernel<uint32_t><<<(unsigned)n_tokens, 256, 0, st>>>(
        (uint32_t*)out, (const uint32_t*)table, ids, hidden, vocab);
  else
    hb::embed_kernel<uint16_t><<<(unsigned)n_tokens, 256, 0, st>>>(
        (uint16_t*)out, (const uint16_t*)table, ids, hidden, vocab);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

int hb_argmax(void* stream, uint32_t* out, const void* logits, int64_t n, int64_t vocab,
              hb_dtype dtype) {
  HB_CHECK_ARG(out && logits, "hb_argmax: null pointer");
  HB_CHECK_ARG(n >= 0 && vocab > 0 && vocab < (1ll << 32), "hb_argmax: bad shape");
  if (n == 0) return HB_OK;
  HB_DISPATCH_DTYPE(dtype, T, {
    hb::argmax_kernel<T><<<(unsigned)n, 1024, 0, (cudaStream_t)stream>>>(out, (const T*)logits,
                                                                        vocab);
  });
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // extern "C"
