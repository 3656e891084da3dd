// KV-cache slot writes (bit-exact copies).
//
// hb_kv_assign_contig restates kv_slot_assign_impl (kernels/kv_assign.cu:16-28):
//   buf[head*max_seq*hd + offset*hd + e] = src[head*hd + e]
// in place, 128 bits per thread when the row allows it.
//
// hb_kv_assign_paged writes K and V of a batch of tokens into the paged pool
// [num_blocks, nkv, 16, head_dim] at slot = block*16 + pos%16.
#include "common.h"

namespace hb {

template <typename V>
__global__ void kv_contig_kernel(V* __restrict__ buf, const V* __restrict__ src, int nkv,
                                 int64_t max_seq, int row_v, int64_t offset) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= nkv * row_v) return;
  const int head = tid / row_v, e = tid % row_v;
  buf[((int64_t)head * max_seq + offset) * row_v + e] = src[(int64_t)head * row_v + e];
}

// One thread per (token, kv head, vector); V is uint4 or a scalar element type.
template <typename V>
__global__ void kv_paged_kernel(V* __restrict__ kc, V* __restrict__ vc, const V* __restrict__ k,
                                const V* __restrict__ v, const int64_t* __restrict__ slots,
                                int64_t n_tokens, int nkv, int row_v, int64_t num_blocks) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t per_tok = (int64_t)nkv * row_v;
  if (tid >= n_tokens * per_tok) return;
  const int64_t t = tid / per_tok;
  const int rem = (int)(tid % per_tok);
  const int head = rem / row_v, e = rem % row_v;
  const int64_t slot = slots[t];
  if (slot < 0 || slot >= num_blocks * HB_BLOCK_SIZE) return;  // skipped / out of pool
  const int64_t blk = slot / HB_BLOCK_SIZE, off = slot % HB_BLOCK_SIZE;
  const int64_t dst = ((blk * nkv + head) * HB_BLOCK_SIZE + off) * row_v + e;
  kc[dst] = k[tid];
  if (vc) vc[dst] = v[tid];
}

}  // namespace hb

// One CTA per (pair, K or V): the whole block [nkv, 16, head_dim] of `src` is copied to
// `dst` inside the same pool with 16-byte loads and stores.  Pairs with an id outside the
// pool are skipped.
__global__ void kv_copy_blocks_kernel(uint4* __restrict__ kc, uint4* __restrict__ vc,
                                      const int64_t* __restrict__ pairs, int64_t block_vecs,
                                      int64_t num_blocks) {
  const int64_t src = pairs[2 * blockIdx.x], dst = pairs[2 * blockIdx.x + 1];
  if (src < 0 || dst < 0 || src >= num_blocks || dst >= num_blocks || src == dst) return;
  uint4* pool = blockIdx.y == 0 ? kc : vc;
  const uint4* s = pool + src * block_vecs;
  uint4* d = pool + dst * block_vecs;
  for (int64_t i = threadIdx.x; i < block_vecs; i += blockDim.x) d[i] = s[i];
}

namespace hb {

int kv_copy_blocks(cudaStream_t st, void* k_cache, void* v_cache, const int64_t* d_pairs, int64_t n_pairs,
                   int64_t block_bytes, int64_t num_blocks) {
  if (n_pairs <= 0) return HB_OK;
  if (block_bytes % 16) return fail(HB_ERR_INVALID_ARG, "kv_copy_blocks: block size must be a multiple of 16 bytes");
  kv_copy_blocks_kernel<<<dim3((unsigned)n_pairs, 2), 256, 0, st>>>((uint4*)k_cache, (uint4*)v_cache, d_pairs,
                                                                   block_bytes / 16, num_blocks);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace hb

extern "C" {

int hb_kv_assign_contig(void* stream, void* buf, const void* src, int nkv, int64_t max_seq,
                        int head_dim, int64_t offset, hb_dtype dtype) {
  HB_CHECK_ARG(buf && src, "hb_kv_assign_contig: null pointer");
  HB_CHECK_ARG(hb::dtype_valid(dtype), "hb_kv_assign_contig: bad dtype");
  HB_CHECK_ARG(nkv > 0 && head_dim > 0 && max_seq > 0, "hb_kv_assign_contig: bad shape");
  HB_CHECK_ARG(offset >= 0 && offset < max_seq,
               "hb_kv_assign_contig: offset %lld outside [0, %lld)", (long long)offset,
               (long long)max_seq);
  const size_t es = hb::dtype_size(dtype);
  const size_t row_bytes = (size_t)head_dim * es;
  auto st = (cudaStream_t)stream;
  const bool vec = row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(buf) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  if (vec) {
    const int row_v = (int)(row_bytes / 16);
    const int total = nkv * row_v;
    hb::kv_contig_kernel<uint4><<<(total + 127) / 128, 128, 0, st>>>((uint4*)buf, (const uint4*)src,
                                                                    nkv, max_seq, row_v, offset);
  } else if (es == 4) {
    const int total = nkv * head_dim;
    hb::kv_contig_kernel<uint32_t><<<(total + 127) / 128, 128, 0, st>>>(
        (uint32_t*)buf, (const uint32_t*)src, nkv, max_seq, head_dim, offset);
  } else {
    const int total = nkv * head_dim;
    hb::kv_contig_kernel<uint16_t><<<(total + 127) / 128, 128, 0, st>>>(
        (uint16_t*)buf, (const uint16_t*)src, nkv, max_seq, head_dim, offset);
  }
  HB_LAUNCH_CHECK();
  return HB_OK;
}

int hb_kv_assign_paged(void* stream, void* k_cache, void* v_cache, const void* k, const void* v,
                       const int64_t* slot_mapping, int64_t n_tokens, int nkv, int head_dim,
                       int64_t num_blocks, hb_dtype dtype) {
  HB_CHECK_ARG(k_cache && k && slot_mapping, "hb_kv_assign_paged: null pointer");
  HB_CHECK_ARG((v_cache == nullptr) == (v == nullptr), "hb_kv_assign_paged: v and v_cache go together");
  HB_CHECK_ARG(hb::dtype_valid(dtype), "hb_kv_assign_paged: bad dtype");
  HB_CHECK_ARG(nkv > 0 && head_dim > 0 && num_blocks > 0 && n_tokens >= 0,
               "hb_kv_assign_paged: bad shape");
  if (n_tokens == 0) return HB_OK;
  const size_t es = hb::dtype_size(dtype);
  const size_t row_bytes = (size_t)head_dim * es;
  auto st = (cudaStream_t)stream;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = row_bytes % 16 == 0 && al(k_cache) && al(v_cache) && al(k) && al(v);
  if (vec) {
    const int row_v = (int)(row_bytes / 16);
    const int64_t total = n_tokens * nkv * row_v;
    hb::kv_paged_kernel<uint4><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        (uint4*)k_cache, (uint4*)v_cache, (const uint4*)k, (const uint4*)v, slot_mapping, n_tokens,
        nkv, row_v, num_blocks);
  } else if (es == 4) {
    const int64_t total = n_tokens * nkv * head_dim;
    hb::kv_paged_kernel<uint32_t><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        (uint32_t*)k_cache, (uint32_t*)v_cache, (const uint32_t*)k, (const uint32_t*)v,
        slot_mapping, n_tokens, nkv, head_dim, num_blocks);
  } else {
    const int64_t total = n_tokens * nkv * head_dim;
    hb::kv_paged_kernel<uint16_t><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        (uint16_t*)k_cache, (uint16_t*)v_cache, (const uint16_t*)k, (const uint16_t*)v,
        slot_mapping, n_tokens, nkv, head_dim, num_blocks);
  }
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // extern "C"
