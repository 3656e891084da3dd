// Internal launchers shared between the public kernel entry points and the engine.
#pragma once

#include "common.h"

namespace hb {

int paged_attention(cudaStream_t st, void* out, const void* q, int64_t q_stride, const void* k_cache,
                    const void* v_cache, const int32_t* block_tables, const int32_t* ctx_lens,
                    int64_t n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                    int64_t max_blocks_per_seq, int64_t num_blocks, int n_splits, void* workspace,
                    hb_dtype dtype, int* err_flag = nullptr, int window = 0, int fresh_tokens = -1, int q_group = 1);
// q_group > 1 (tensor-core kernel only): the rows are consecutive positions of ONE sequence
// with the same block table (a prefill chunk); q_group of them share a CTA and the K/V stream.
// Must satisfy q_group * (n_q_heads / n_kv_heads) <= 16 and needs n_splits == 1.
// fresh_tokens >= 0: at most that many tokens at the end of every sequence were written by the
// kernels launched right before this one; blocks of older tokens may be fetched before those
// kernels have completed (programmatic launch).  -1: nothing is fetched early.
bool paged_attention_mma_supported(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                                   int nrep, int head_dim, int64_t num_blocks, int hkv, hb_dtype dtype);
// Opts the tensor-core attention kernel in to its shared memory (once per device,
// outside any stream capture).
int paged_attention_mma_prepare();

// dst block := src block for every (src, dst) pair (device array of 2 * n_pairs ids), in the K
// and the V pool of one layer; a block is block_bytes long (kv.cu).
int kv_copy_blocks(cudaStream_t st, void* k_cache, void* v_cache, const int64_t* d_pairs, int64_t n_pairs,
                   int64_t block_bytes, int64_t num_blocks);

// Mixture-of-experts routing (moe.cu): scale[m, e] = renormalised top-k softmax weight of
// expert e for token m, 0 for the others; moe_scale_act multiplies act[m, e*inter + i] by it.
int moe_route(cudaStream_t st, float* scale, const void* x, const void* w_gate, int64_t n_tokens,
              int64_t hidden, int n_experts, int top_k, hb_dtype dtype);
int moe_scale_act(cudaStream_t st, void* act, const float* scale, int64_t n_tokens, int64_t inter,
                  int n_experts, hb_dtype dtype);

// RoPE on the q and k parts of a fused [q | k | v] projection row and the paged KV
// write in one pass: q is rotated in place, rotated k and v go straight to their slot.
int rope_kv_write(cudaStream_t st, void* qkv, void* k_cache, void* v_cache,
                  const int32_t* positions, const int64_t* slot_mapping, const float* inv_freq,
                  int64_t n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                  int64_t num_blocks, hb_dtype dtype);

// table[t * head_dim/2 + i] = (cos, sin) of positions[t] * inv_freq[i], rounded to `dtype`
// as rope_kv_write rounds them (consumed by the GEMM epilogue that rotates q and k).
int rope_table(cudaStream_t st, float2* table, const int32_t* positions, const float* inv_freq,
               int64_t n_tokens, int head_dim, hb_dtype dtype);

// Fill a [rows, cols] slice of a global [g_rows, g_cols] tensor with N(0, std) drawn
// from a counter-based generator keyed by (seed, tensor id, global element index).
int fill_normal(cudaStream_t st, void* dst, hb_dtype dtype, int64_t rows, int64_t cols,
                int64_t row0, int64_t col0, int64_t g_cols, uint64_t seed, uint64_t tensor_id,
                float std, int64_t dst_ld = 0);  // dst_ld: row stride of dst in elements (0 = cols)
int fill_const(cudaStream_t st, void* dst, hb_dtype dtype, int64_t n, float value);
// dst [rows, cols] (row stride dst_ld elements, 0 = cols) := a dense [rows, cols] source of
// another element type, converted on the device (round to nearest even).
int convert_2d(cudaStream_t st, void* dst, hb_dtype dst_dtype, int64_t dst_ld, const void* src, hb_dtype src_dtype,
               int64_t rows, int64_t cols);
// dst (f32) = src (dtype)
// cols / src_ld: the source is [n / cols, cols] with row stride src_ld (0 = contiguous)
int to_f32(cudaStream_t st, float* dst, const void* src, hb_dtype dtype, int64_t n, int64_t cols = 0,
           int64_t src_ld = 0);

}  // namespace hb
