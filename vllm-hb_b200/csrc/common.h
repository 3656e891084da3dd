// Internal helpers shared by every translation unit of libhb.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>

#include "../../include/hb.h"

namespace hb {

// Thread-local message behind hb_last_error().
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

inline size_t dtype_size(hb_dtype d) { return d == HB_F32 ? 4 : 2; }
inline bool dtype_valid(int d) { return d == HB_F32 || d == HB_F16 || d == HB_BF16; }

#define HB_CUDA_CHECK(expr)                                                              \
  do {                                                                                   \
    cudaError_t err__ = (expr);                                                          \
    if (err__ != cudaSuccess) {                                                          \
      cudaGetLastError(); /* clear the non-sticky error so later calls start clean */    \
      return ::hb::fail(HB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                     \
                        cudaGetErrorString(err__), __FILE__, __LINE__);                  \
    }                                                                                    \
  } while (0)

#define HB_CHECK_ARG(cond, ...)                                 \
  do {                                                          \
    if (!(cond)) return ::hb::fail(HB_ERR_INVALID_ARG, __VA_ARGS__); \
  } while (0)

#define HB_LAUNCH_CHECK() HB_CUDA_CHECK(cudaGetLastError())

#ifdef __CUDACC__
// Launch with programmatic stream serialisation: the grid may become resident while the
// preceding kernel of the stream is still draining, which hides the launch latency of
// the small kernels of a decode step.  The kernel must call pdl_grid_wait() before it
// touches global memory.  HB_PDL=0 launches normally.
inline bool pdl_enabled() {
  static const bool on = [] { const char* e = getenv("HB_PDL"); return !(e && e[0] == '0'); }();
  return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// Dispatch a generic lambda on the element type.
#define HB_DISPATCH_DTYPE(dtype, T, ...)                                   \
  switch (dtype) {                                                         \
    case HB_F32: { using T = float; __VA_ARGS__; break; }                  \
    case HB_F16: { using T = __half; __VA_ARGS__; break; }                 \
    case HB_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }         \
    default: return ::hb::fail(HB_ERR_UNSUPPORTED_DTYPE, "unsupported dtype %d", (int)(dtype)); \
  }

#ifdef __CUDACC__
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 16-byte vector of T: 4 floats or 8 half/bf16.
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ void load(const T* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void unpack(float (&f)[N]) const {
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = to_f32<T>(e[i]);
  }
  __device__ __forceinline__ void pack(const float (&f)[N]) {
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) e[i] = from_f32<T>(f[i]);
  }
};

// Programmatic dependent launch: lets a successor that was launched with the
// programmatic-serialisation attribute begin its prologue (it still waits for this
// grid to finish before it reads what this grid writes).  A no-op otherwise.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Blocks until the preceding grid of the stream has completed and its writes are
// visible; returns at once for a kernel launched without the attribute.  A kernel that
// launch_pdl() starts must pass here before its first global read or write.
__device__ __forceinline__ void pdl_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// One RoPE pair (x1, x2) = (element i, element i + head_dim/2) rotated by (c, s); every
// kernel that rotates uses this one expression so that they agree bit for bit.
__device__ __forceinline__ void rope_rotate(float x1, float x2, float c, float s, float* o1, float* o2) {
  *o1 = x1 * c - x2 * s;
  *o2 = x1 * s + x2 * c;
}
// Sum over the whole block; every thread gets the total. `smem` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* smem) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protect smem reuse between calls
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  float t = (lane < nwarps) ? smem[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
#endif  // __CUDACC__

// Device properties cached per device.
struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t smem_optin = 0;
  size_t l2_bytes = 0;
};
int device_info(int device, DeviceInfo* out);

}  // namespace hb
