// Sparse mixture-of-experts routing for the decode step (Mixtral):
// SparseMoeBlock::forward, src/engine/arch/mixtral.rs:371-430.
//
// The reference routes on the host: softmax(x . Wg^T) over the experts, top-k by
// descending probability, weights renormalised by their sum (floored at 1e-9), then one
// Expert::forward per (token, chosen expert) and a weighted fp32 sum.  Decode reads every
// expert's weights anyway once a few dozen tokens are in the batch, so the engine runs
// the experts as ONE pair of GEMMs over the concatenated expert weights
//   act[m, e*I + i] = silu(x . w1_e^T)[i] * (x . w3_e^T)[i]            (gate|up GEMM, N = 2*E*I)
//   out[m, :]       = SUM_e scale[m,e] * (act[m, e*I : (e+1)*I] . w2_e^T)   (down GEMM, K = E*I)
// with scale[m,e] the renormalised routing weight of a chosen expert and 0 otherwise:
// the scale is applied to the activations (moe_scale_kernel) and the down GEMM then
// accumulates all experts in fp32 in one pass.  These two kernels produce and apply
// scale[m,e].
#include <cfloat>

#include "common.h"
#include "ops.h"

namespace hb {

constexpr int kRouterThreads = 256;
constexpr int kMaxExperts = 64;

// One CTA per token: logits (fp32 accumulate, rounded to T like gate.forward's output),
// softmax (rounded to T like candle's softmax output), top-k, renormalise.
// Ties keep the lower expert index (the reference's sort_unstable_by leaves them open).
template <typename T>
__global__ void __launch_bounds__(kRouterThreads)
moe_router_kernel(float* __restrict__ scale, const T* __restrict__ x, const T* __restrict__ wg,
                  int64_t hidden, int n_experts, int top_k) {
  pdl_trigger();
  pdl_grid_wait();
  __shared__ float s_logit[kMaxExperts];
  constexpr int N = Vec16<T>::N;
  const int64_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = kRouterThreads / 32;
  const T* xr = x + m * hidden;
  const bool vec = hidden % N == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(wg) & 15) == 0;
  for (int e = warp; e < n_experts; e += n_warps) {
    const T* wr = wg + (int64_t)e * hidden;
    float acc = 0.f;
    if (vec) {
      for (int64_t v = lane; v < hidden / N; v += 32) {
        Vec16<T> a, b;
        a.load(xr + v * N);
        b.load(wr + v * N);
        float fa[N], fb[N];
        a.unpack(fa);
        b.unpack(fb);
#pragma unroll
        for (int j = 0; j < N; ++j) acc = fmaf(fa[j], fb[j], acc);
      }
    } else {
      for (int64_t i = lane; i < hidden; i += 32) acc = fmaf(to_f32<T>(xr[i]), to_f32<T>(wr[i]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) s_logit[e] = to_f32<T>(from_f32<T>(acc));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mx = -FLT_MAX;
    for (int e = 0; e < n_experts; ++e) mx = fmaxf(mx, s_logit[e]);
    float sum = 0.f;
    for (int e = 0; e < n_experts; ++e) {
      s_logit[e] = expf(s_logit[e] - mx);
      sum += s_logit[e];
    }
    for (int e = 0; e < n_experts; ++e) s_logit[e] = to_f32<T>(from_f32<T>(s_logit[e] / sum));
    // top-k by descending probability, lower index first among equals
    float chosen_w[kMaxExperts];
    int chosen[kMaxExperts];
    const int k = min(top_k, n_experts);
    float wsum = 0.f;
    for (int j = 0; j < k; ++j) {
      int best = -1;
      float bv = -1.f;
      for (int e = 0; e < n_experts; ++e) {
        bool taken = false;
        for (int q = 0; q < j; ++q) taken = taken || chosen[q] == e;
        if (!taken && s_logit[e] > bv) { bv = s_logit[e]; best = e; }
      }
      chosen[j] = best;
      chosen_w[j] = bv;
      wsum += bv;
    }
    float* out = scale + m * n_experts;
    for (int e = 0; e < n_experts; ++e) out[e] = 0.f;
    const float denom = fmaxf(wsum, 1e-9f);
    for (int j = 0; j < k; ++j) out[chosen[j]] = chosen_w[j] / denom;
  }
}

// act[m, e*I + i] *= scale[m, e], 128-bit vectors (I a multiple of the vector width).
template <typename T>
__global__ void moe_scale_kernel(T* __restrict__ act, const float* __restrict__ scale, int64_t inter,
                                 int n_experts) {
  pdl_trigger();
  pdl_grid_wait();
  constexpr int N = Vec16<T>::N;
  const int64_t m = blockIdx.x;
  const int64_t row = inter * n_experts;
  T* ar = act + m * row;
  const float* sr = scale + m * n_experts;
  if (inter % N == 0 && (reinterpret_cast<uintptr_t>(act) & 15) == 0) {
    for (int64_t v = threadIdx.x; v < row / N; v += blockDim.x) {
      const float s = sr[(v * N) / inter];
      Vec16<T> a;
      a.load(ar + v * N);
      float f[N];
      a.unpack(f);
#pragma unroll
      for (int j = 0; j < N; ++j) f[j] *= s;
      a.pack(f);
      a.store(ar + v * N);
    }
  } else {
    for (int64_t i = threadIdx.x; i < row; i += blockDim.x)
      ar[i] = from_f32<T>(to_f32<T>(ar[i]) * sr[i / inter]);
  }
}

int moe_route(cudaStream_t st, float* scale, const void* x, const void* w_gate, int64_t n_tokens,
              int64_t hidden, int n_experts, int top_k, hb_dtype dtype) {
  if (n_tokens == 0) return HB_OK;
  if (n_experts < 1 || n_experts > kMaxExperts || top_k < 1)
    return fail(HB_ERR_INVALID_ARG, "moe_route: %d experts / top-%d unsupported (1..%d experts)", n_experts,
                top_k, kMaxExperts);
  HB_DISPATCH_DTYPE(dtype, T, {
    HB_CUDA_CHECK(launch_pdl(moe_router_kernel<T>, dim3((unsigned)n_tokens), dim3(kRouterThreads), 0, st, scale,
                             (const T*)x, (const T*)w_gate, hidden, n_experts, top_k));
  });
  return HB_OK;
}

int moe_scale_act(cudaStream_t st, void* act, const float* scale, int64_t n_tokens, int64_t inter,
                  int n_experts, hb_dtype dtype) {
  if (n_tokens == 0) return HB_OK;
  HB_DISPATCH_DTYPE(dtype, T, {
    HB_CUDA_CHECK(launch_pdl(moe_scale_kernel<T>, dim3((unsigned)n_tokens), dim3(256), 0, st, (T*)act, scale, inter,
                             n_experts));
  });
  return HB_OK;
}

}  // namespace hb

extern "C" {

int hb_moe_route(void* stream, float* scale, const void* x, const void* w_gate, int64_t n_tokens,
                 int64_t hidden, int n_experts, int top_k, hb_dtype dtype) {
  HB_CHECK_ARG(scale && x && w_gate, "hb_moe_route: null pointer");
  HB_CHECK_ARG(n_tokens >= 0 && hidden > 0, "hb_moe_route: bad shape");
  return hb::moe_route((cudaStream_t)stream, scale, x, w_gate, n_tokens, hidden, n_experts, top_k, dtype);
}

}  // extern "C"
