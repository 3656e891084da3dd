// RMSNorm and residual-add + RMSNorm.
//
// One CTA per row.  The row is read once with 128-bit loads and kept in registers
// (up to kMaxVec vectors per thread) between the sum-of-squares pass and the scale
// pass; the reference kernel reads x twice with scalar loads
// (kernels/rms_norm.cu:74-82 and :99-110).  Accumulation is fp32 with one rounding at
// the end, the numerics of rms_norm_f16_impl (kernels/rms_norm.cu:89-111).
#include "common.h"

namespace hb {

constexpr int kNormThreads = 256;
constexpr int kMaxVec = 8;

// ADD: x += resid first, write the sum (rounded to T) to resid_out, and normalise the
// rounded sum — the reference materialises h + attn_out in dtype before the norm
// (src/engine/arch/llama_tp.rs:536-544).
template <typename T, bool ADD>
__global__ void __launch_bounds__(kNormThreads)
rms_norm_vec_kernel(T* __restrict__ out, T* __restrict__ resid_out, const T* __restrict__ x,
                    const T* __restrict__ resid_in, const T* __restrict__ w, int64_t hidden,
                    float eps) {
  pdl_trigger();
  pdl_grid_wait();
  __shared__ float red[33];
  constexpr int N = Vec16<T>::N;
  const int64_t row = blockIdx.x;
  const int64_t nvec = hidden / N;
  const T* xr = x + row * hidden;
  T* yr = out ? out + row * hidden : nullptr;

  Vec16<T> cache[kMaxVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int64_t v = threadIdx.x + (int64_t)i * kNormThreads;
    if (v < nvec) {
      cache[i].load(xr + v * N);
      float f[N];
      cache[i].unpack(f);
      if (ADD) {
        Vec16<T> r;
        r.load(resid_in + row * hidden + v * N);
        float g[N];
        r.unpack(g);
#pragma unroll
        for (int j = 0; j < N; ++j) f[j] += g[j];
        cache[i].pack(f);       // round the sum to T ...
        cache[i].store(resid_out + row * hidden + v * N);
        cache[i].unpack(f);     // ... and normalise the rounded value
      }
#pragma unroll
      for (int j = 0; j < N; ++j) ss += f[j] * f[j];
    }
  }
  // Rows wider than the register cache: stream the rest (second read hits L2).
  for (int64_t v = threadIdx.x + (int64_t)kMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
    Vec16<T> a;
    a.load(xr + v * N);
    float f[N];
    a.unpack(f);
    if (ADD) {
      Vec16<T> r;
      r.load(resid_in + row * hidden + v * N);
      float g[N];
      r.unpack(g);
#pragma unroll
      for (int j = 0; j < N; ++j) f[j] += g[j];
      a.pack(f);
      a.store(resid_out + row * hidden + v * N);
      a.unpack(f);
    }
#pragma unroll
    for (int j = 0; j < N; ++j) ss += f[j] * f[j];
  }
  ss = block_sum(ss, red);
  if (!yr) return;
  const float scale = rsqrtf(ss / (float)hidden + eps);

#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int64_t v = threadIdx.x + (int64_t)i * kNormThreads;
    if (v < nvec) {
      float f[N], g[N];
      cache[i].unpack(f);
      Vec16<T> wv;
      wv.load(w + v * N);
      wv.unpack(g);
#pragma unroll
      for (int j = 0; j < N; ++j) f[j] = f[j] * scale * g[j];
      Vec16<T> o;
      o.pack(f);
      o.store(yr + v * N);
    }
  }
  for (int64_t v = threadIdx.x + (int64_t)kMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
    Vec16<T> a;
    a.load((ADD ? (const T*)resid_out + row * hidden : xr) + v * N);
    float f[N], g[N];
    a.unpack(f);
    Vec16<T> wv;
    wv.load(w + v * N);
    wv.unpack(g);
#pragma unroll
    for (int j = 0; j < N; ++j) f[j] = f[j] * scale * g[j];
    a.pack(f);
    a.store(yr + v * N);
  }
}

// Any hidden size / alignment: scalar loads.
template <typename T, bool ADD>
__global__ void __launch_bounds__(kNormThreads)
rms_norm_scalar_kernel(T* __restrict__ out, T* __restrict__ resid_out, const T* __restrict__ x,
                       const T* __restrict__ resid_in, const T* __restrict__ w, int64_t hidden,
                       float eps) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * hidden;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < hidden; i += kNormThreads) {
    float f = to_f32<T>(xr[i]);
    if (ADD) {
      T s = from_f32<T>(f + to_f32<T>(resid_in[row * hidden + i]));
      resid_out[row * hidden + i] = s;
      f = to_f32<T>(s);
    }
    ss += f * f;
  }
  ss = block_sum(ss, red);
  if (!out) return;
  const float scale = rsqrtf(ss / (float)hidden + eps);
  const T* src = ADD ? (const T*)resid_out + row * hidden : xr;
  for (int64_t i = threadIdx.x; i < hidden; i += kNormThreads)
    out[row * hidden + i] = from_f32<T>(to_f32<T>(src[i]) * scale * to_f32<T>(w[i]));
}

template <typename T, bool ADD>
static int launch_norm(cudaStream_t st, T* out, T* resid_out, const T* x, const T* resid_in,
                       const T* w, int64_t rows, int64_t hidden, float eps) {
  if (rows == 0) return HB_OK;
  constexpr int N = Vec16<T>::N;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = hidden % N == 0 && aligned(out) && aligned(x) && aligned(w) &&
                   (!ADD || (aligned(resid_out) && aligned(resid_in)));
  if (vec)
    HB_CUDA_CHECK(launch_pdl(rms_norm_vec_kernel<T, ADD>, dim3((unsigned)rows), dim3(kNormThreads), 0, st, out,
                             resid_out, x, resid_in, w, hidden, eps));
  else
    rms_norm_scalar_kernel<T, ADD><<<(unsigned)rows, kNormThreads, 0, st>>>(out, resid_out, x,
                                                                           resid_in, w, hidden, eps);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace hb

extern "C" {

int hb_rms_norm(void* stream, void* out, const void* x, const void* w, int64_t rows,
                int64_t hidden, float eps, hb_dtype dtype) {
  HB_CHECK_ARG(rows >= 0 && hidden > 0, "hb_rms_norm: bad shape rows=%lld hidden=%lld",
               (long long)rows, (long long)hidden);
  if (rows == 0) return HB_OK;
  HB_CHECK_ARG(out && x && w, "hb_rms_norm: null pointer");
  HB_CHECK_ARG(rows < (1ll << 31), "hb_rms_norm: too many rows");
  HB_DISPATCH_DTYPE(dtype, T,
                    return (hb::launch_norm<T, false>((cudaStream_t)stream, (T*)out, nullptr,
                                                      (const T*)x, nullptr, (const T*)w, rows,
                                                      hidden, eps)));
  return HB_OK;
}

int hb_add_rms_norm(void* stream, void* normed_out, void* resid_out, const void* x,
                    const void* resid_in, const void* w, int64_t rows, int64_t hidden, float eps,
                    hb_dtype dtype) {
  HB_CHECK_ARG(resid_out && x && resid_in, "hb_add_rms_norm: null pointer");
  HB_CHECK_ARG(!normed_out || w, "hb_add_rms_norm: normed_out needs a weight");
  HB_CHECK_ARG(rows >= 0 && hidden > 0, "hb_add_rms_norm: bad shape");
  HB_CHECK_ARG(rows < (1ll << 31), "hb_add_rms_norm: too many rows");
  HB_DISPATCH_DTYPE(dtype, T,
                    return (hb::launch_norm<T, true>((cudaStream_t)stream, (T*)normed_out,
                                                     (T*)resid_out, (const T*)x,
                                                     (const T*)resid_in, (const T*)w, rows, hidden,
                                                     eps)));
  return HB_OK;
}

}  // extern "C"
