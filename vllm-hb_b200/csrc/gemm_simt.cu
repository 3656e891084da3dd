// Y[M,N] = X[M,K] . W[N,K]^T on CUDA cores, any dtype and any shape.
//
// This is the coverage kernel: F32/F16 models (the reference's CPU and default CUDA
// dtypes, src/engine/dtype.rs:22-28), and bf16 shapes the tensor-core kernel does not
// take (K not a multiple of 64).  One warp per output column n streams W[n,:] once
// with 128-bit loads and keeps kMB rows of the batch in fp32 accumulators.
#include "common.h"
#include "gemm.h"

namespace hb {

constexpr int kSimtWarps = 8;
constexpr int kMB = 8;

template <typename T, typename OutT, bool VEC>
__global__ void __launch_bounds__(kSimtWarps * 32)
gemm_simt_kernel(OutT* __restrict__ Y, const T* __restrict__ X, const T* __restrict__ W, int64_t M,
                 int64_t N, int64_t K, int64_t ldy) {
  constexpr int NV = Vec16<T>::N;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t n = (int64_t)blockIdx.x * kSimtWarps + warp;
  const int64_t m0 = (int64_t)blockIdx.y * kMB;
  if (n >= N) return;
  const T* wr = W + n * K;
  float acc[kMB];
#pragma unroll
  for (int i = 0; i < kMB; ++i) acc[i] = 0.f;
  if (VEC) {
    for (int64_t k = (int64_t)lane * NV; k < K; k += 32 * NV) {
      Vec16<T> wv;
      wv.load(wr + k);
      float wf[NV];
      wv.unpack(wf);
#pragma unroll
      for (int i = 0; i < kMB; ++i) {
        if (m0 + i < M) {
          Vec16<T> xv;
          xv.load(X + (m0 + i) * K + k);
          float xf[NV];
          xv.unpack(xf);
#pragma unroll
          for (int j = 0; j < NV; ++j) acc[i] = fmaf(xf[j], wf[j], acc[i]);
        }
      }
    }
  } else {
    for (int64_t k = lane; k < K; k += 32) {
      const float wf = to_f32<T>(wr[k]);
#pragma unroll
      for (int i = 0; i < kMB; ++i)
        if (m0 + i < M) acc[i] = fmaf(to_f32<T>(X[(m0 + i) * K + k]), wf, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < kMB; ++i) {
    const float s = warp_sum(acc[i]);
    if (lane == 0 && m0 + i < M) Y[(m0 + i) * ldy + n] = from_f32<OutT>(s);
  }
}

template <typename T, typename OutT>
static int launch_simt(cudaStream_t st, OutT* Y, const T* X, const T* W, int64_t M, int64_t N,
                       int64_t K, int64_t ldy) {
  constexpr int NV = Vec16<T>::N;
  const bool vec = K % NV == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(W) & 15) == 0;
  dim3 grid((unsigned)((N + kSimtWarps - 1) / kSimtWarps), (unsigned)((M + kMB - 1) / kMB));
  if (vec)
    gemm_simt_kernel<T, OutT, true><<<grid, kSimtWarps * 32, 0, st>>>(Y, X, W, M, N, K, ldy);
  else
    gemm_simt_kernel<T, OutT, false><<<grid, kSimtWarps * 32, 0, st>>>(Y, X, W, M, N, K, ldy);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

int gemm_simt(cudaStream_t st, void* Y, const void* X, const void* W, int64_t M, int64_t N,
              int64_t K, hb_dtype dtype, bool out_f32) {
  if (M == 0 || N == 0) return HB_OK;
  HB_DISPATCH_DTYPE(dtype, T, {
    if (out_f32)
      return (launch_simt<T, float>(st, (float*)Y, (const T*)X, (const T*)W, M, N, K, N));
    return (launch_simt<T, T>(st, (T*)Y, (const T*)X, (const T*)W, M, N, K, N));
  });
  return HB_OK;
}

}  // namespace hb
