// Device-side building blocks of the tcgen05 kernels: mbarrier / TMA / tcgen05 PTX
// wrappers, shared-memory and instruction descriptors.  Every wait is bounded.
#pragma once

#include <cuda.h>

#include "common.h"

namespace hb {

constexpr int kTileN = 128;       // weight rows per CTA tile = UMMA M
constexpr int kTileK = 64;        // bf16 elements per 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kMaxStages = 12;
constexpr int kTcThreads = 128;
constexpr uint32_t kSpinLimit = 1u << 21;
constexpr size_t kCounterBlockBytes = 64 * 1024;  // int32 counters of up to 16384 tiles


// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false when the limit ran out or another thread already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* s_abort) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 255u) == 255u && *s_abort) return false;
  }
  *s_abort = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tm), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// The same load with an L2 eviction policy (see l2_policy_*): weights are read once per step
// and should leave L2 first, the batch operand is re-read by every CTA and should stay.
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* tm, int x, int y,
                                                 uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst), "l"(tm), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// Bulk tensor store shared -> global (box of the tensor map at element coordinates
// x, y); rows and columns outside the tensor are clipped.  x * element size must be a
// multiple of 16 bytes and the coordinates non-negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(tm), "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once every committed store has finished READING shared memory (the buffer
// may be reused or the CTA may exit); the global writes complete with the grid.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Orders this thread's shared-memory writes before later async-proxy (TMA) reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 16 consecutive fp32 columns: thread i gets lane (base_lane + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows are 128 B,
// groups of 8 rows (1024 B) repeat along the M/N dimension (stride byte offset 1024).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);        // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                        // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                        // layout type: 128-byte swizzle
  return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, A and B K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kTileN >> 4) << 24);
}

// ---- programmatic dependent launch: a kernel launched with the attribute may start
// while its predecessor in the stream is still running; it must not touch memory the
// predecessor produces (or still reads) before pdl_wait() returns.  Both are no-ops for
// a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- thread-block cluster helpers (split-K partners exchange accumulators on chip)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t caddr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(caddr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t caddr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(caddr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
// 16-byte store into a partner CTA's shared memory that reports its bytes to an mbarrier of
// THAT CTA (both addresses already mapped into the partner's window): the receiver waits on
// its own barrier and needs no cluster-wide barrier or fence to see the data.
__device__ __forceinline__ void st_async_v4(uint32_t caddr, float a, float b, float c, float d, uint32_t cbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(caddr), "f"(a), "f"(b), "f"(c), "f"(d), "r"(cbar)
               : "memory");
}
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Every thread of every CTA of the cluster arrives; hardware barrier, always reached.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// silu(z) = z / (1 + e^-z) with the fast divide: the 16 activations of an accumulator
// group must not cost more than the group's loads (the IEEE divide is ~20 dependent
// instructions); the quotient is rounded to bf16 afterwards.
__device__ __forceinline__ float silu_f(float z) { return __fdividef(z, 1.f + __expf(-z)); }

}  // namespace hb
