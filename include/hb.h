/*
 * hb.h — C ABI of libhb: the tensor-parallel decode hot path of vllm-hb, written
 * for NVIDIA B200 (sm_100a).
 *
 * Every entry point is what a Rust `extern "C"` block (or any FFI) binds in place of
 * the reference's own item cited beside it.  Citations are paths inside the
 * reference project (avarga1/vllm-hb).
 *
 * Conventions
 *   - plain pointers and sizes only; device pointers are raw CUDA device addresses
 *     (a `cudarc::driver::CudaSlice` device pointer passes straight through);
 *   - `stream` is a `cudaStream_t` passed as `void*` (NULL = the legacy default stream);
 *   - every function returns 0 on success or a negative `HB_ERR_*`; the message of
 *     the last failure on the calling thread is `hb_last_error()`;
 *   - nothing aborts, traps or throws across this boundary;
 *   - there is no CPU fallback: without a CUDA device the compute calls fail with
 *     HB_ERR_CUDA.
 */
#ifndef HB_H_
#define HB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- status codes */
#define HB_OK 0
#define HB_ERR_INVALID_ARG (-1)
#define HB_ERR_UNSUPPORTED_DTYPE (-2)
#define HB_ERR_NOT_DIVISIBLE (-3)
#define HB_ERR_CUDA (-4)
#define HB_ERR_NCCL (-5)
#define HB_ERR_TIMEOUT (-6)
#define HB_ERR_OOM_BLOCKS (-7)
#define HB_ERR_IO (-8)
#define HB_ERR_EMPTY (-9)

/* Element types.  The reference's kernels take F32 and F16 only and send BF16 down a
 * multi-op eager path (src/kernels/rms_norm.rs:24-27, src/kernels/rope.rs:26-29);
 * here all three are first-class. */
typedef enum hb_dtype { HB_F32 = 0, HB_F16 = 1, HB_BF16 = 2 } hb_dtype;

/* All-reduce algorithm selector. */
typedef enum hb_algo {
  HB_ALGO_AUTO = 0,     /* peer memory: one-shot below the crossover size, two-shot above (never MULTIMEM,
                           whose sums differ in the last bf16 digit: it is asked for by name) */
  HB_ALGO_ONE_SHOT = 1, /* every rank reads all partials: (R-1)*bytes inbound, one flag hop */
  HB_ALGO_TWO_SHOT = 2, /* reduce-scatter + all-gather: 2(R-1)/R*bytes, two flag hops */
  HB_ALGO_NCCL = 3,     /* ncclAllReduce: the reference's path, kept as the reported baseline */
  HB_ALGO_MULTIMEM = 4  /* hb_all_reduce_add_rms_norm / hb_fused_rowparallel only: the sum is formed
                           inside the NVLink switch (needs hb_world_attach_multicast) */
} hb_algo;

const char* hb_last_error(void);
const char* hb_version(void);
/* Number of visible CUDA devices (0 without a driver); never fails. */
int hb_device_count(void);

/* ------------------------------------------------------------- kernel surface */

/* y = x * rsqrt(mean(x^2) + eps) * w, fp32 accumulate, one rounding.
 * x,out [rows, hidden] contiguous, w [hidden], all `dtype`, device memory.
 * Replaces rms_norm::apply (src/kernels/rms_norm.rs:23-35) and the kernels
 * rms_norm_{f32,f16}_{256,512} (kernels/rms_norm.cu:117-131). */
int hb_rms_norm(void* stream, void* out, const void* x, const void* w, int64_t rows,
                int64_t hidden, float eps, hb_dtype dtype);

/* resid_out = resid_in + x (rounded to dtype); normed_out = rms_norm(resid_out; w).
 * The residual add and the following norm of the layer loop
 * (src/engine/arch/llama_tp.rs:536-552,566-571,517-522) in one pass.
 * resid_out may alias resid_in. */
int hb_add_rms_norm(void* stream, void* normed_out, void* resid_out, const void* x,
                    const void* resid_in, const void* w, int64_t rows, int64_t hidden,
                    float eps, hb_dtype dtype);

/* inv_freq[i] = 1 / theta^(2i/head_dim) for i in [0, head_dim/2), computed in f32 on
 * the host exactly as apply_rope does (src/engine/arch/llama_tp.rs:119-121).
 * `out` is HOST memory of head_dim/2 floats. */
int hb_rope_inv_freq(float theta, int head_dim, float* out);

/* Rotate-half RoPE in place on q [n_tokens, n_q_heads, head_dim] and
 * k [n_tokens, n_kv_heads, head_dim] (GQA-correct: q and k have their own head
 * counts), token t rotated by angle positions[t] * inv_freq[i].
 * positions: int32 [n_tokens] device; inv_freq: f32 [head_dim/2] device.
 * cos/sin are computed in f32 and rounded to `dtype` before use, as
 * apply_rope does (src/engine/arch/llama_tp.rs:112-152).  k may be NULL. */
int hb_rope(void* stream, void* q, void* k, const int32_t* positions, const float* inv_freq,
            int64_t n_tokens, int n_q_heads, int n_kv_heads, int head_dim, hb_dtype dtype);

/* The reference kernel's own calling convention: x,out [batch*heads, seq_len, head_dim],
 * cos,sin [seq_len, head_dim/2] pre-sliced to the current positions, all `dtype`.
 * Replaces rope::apply (src/kernels/rope.rs:25-49) / rope_single_{f32,f16}
 * (kernels/rope.cu:135-145).  out may alias x. */
int hb_rope_cos_sin(void* stream, void* out, const void* x, const void* cos_table,
                    const void* sin_table, int64_t batch_heads, int64_t seq_len, int head_dim,
                    hb_dtype dtype);

/* buf[head, offset, :] = src[head, :] for every kv head; buf [nkv, max_seq, head_dim],
 * src [nkv, head_dim]; bit-exact copy, in place (the reference clones the whole buffer
 * first: src/kernels/kv_assign.rs:113).  Replaces kv_assign::assign_slot
 * (src/kernels/kv_assign.rs:34-42) / kv_slot_assign_{f16,f32} (kernels/kv_assign.cu:32-44). */
int hb_kv_assign_contig(void* stream, void* buf, const void* src, int nkv, int64_t max_seq,
                        int head_dim, int64_t offset, hb_dtype dtype);

/* Paged KV write.  Pool layout per layer: [num_blocks, nkv, HB_BLOCK_SIZE, head_dim].
 * Token t (k,v rows [n_tokens, nkv, head_dim]) goes to slot slot_mapping[t] =
 * block_id*16 + pos%16, the mapping the block tables of
 * src/scheduler/block_manager.rs:104-110 imply.  slot < 0 skips the token.
 * Bit-exact copy. */
#define HB_BLOCK_SIZE 16
int hb_kv_assign_paged(void* stream, void* k_cache, void* v_cache, const void* k, const void* v,
                       const int64_t* slot_mapping, int64_t n_tokens, int nkv, int head_dim,
                       int64_t num_blocks, hb_dtype dtype);

/* Paged GQA decode attention: one query token per sequence over that sequence's
 * block table.  q,out [n_seqs, n_q_heads, head_dim]; block_tables int32
 * [n_seqs, max_blocks_per_seq]; ctx_lens int32 [n_seqs] (number of keys, including
 * the token just written; an entry above max_blocks_per_seq*16 is cut to that, block ids
 * outside [0, num_blocks) read block 0: nothing outside the tables and the pool is touched).  Query head j reads kv head j / (n_q_heads/n_kv_heads)
 * (src/engine/arch/llama_tp.rs:264-279); scores = q.k/sqrt(d), softmax and the
 * weighted sum accumulate in fp32 (src/engine/arch/llama_tp.rs:304-324).
 * `workspace` holds split-KV partials: hb_attention_workspace_bytes() bytes.
 * Replaces the doc-only stubs of src/attention/ (sdpa.rs:1-11, flash.rs:27-31). */
size_t hb_attention_workspace_bytes(int64_t n_seqs, int n_q_heads, int head_dim, int n_splits);
int hb_paged_decode_attention(void* stream, void* out, const void* q, const void* k_cache,
                              const void* v_cache, const int32_t* block_tables,
                              const int32_t* ctx_lens, int64_t n_seqs, int n_q_heads,
                              int n_kv_heads, int head_dim, int64_t max_blocks_per_seq,
                              int64_t num_blocks, int n_splits, void* workspace, hb_dtype dtype);
/* The same with a sliding window (sliding_causal_mask, src/engine/arch/mixtral.rs:155-176):
 * the query at position ctx-1 attends to the keys ki with ctx-1-ki < sliding_window;
 * 0 = no window.  Blocks wholly outside the window are not read. */
int hb_paged_decode_attention_window(void* stream, void* out, const void* q, const void* k_cache,
                                     const void* v_cache, const int32_t* block_tables,
                                     const int32_t* ctx_lens, int64_t n_seqs, int n_q_heads,
                                     int n_kv_heads, int head_dim, int64_t max_blocks_per_seq,
                                     int64_t num_blocks, int n_splits, void* workspace,
                                     int sliding_window, hb_dtype dtype);

/* Router of the sparse mixture-of-experts block (SparseMoeBlock::forward,
 * src/engine/arch/mixtral.rs:371-412): logits = x . w_gate^T (rounded to dtype), softmax over
 * the experts (rounded to dtype), top_k by descending probability (ties: lower index),
 * weights renormalised by their sum floored at 1e-9.  scale (device f32 [n_tokens,
 * n_experts]) receives the weight of each chosen expert and 0 for the others.
 * x [n_tokens, hidden], w_gate [n_experts, hidden]; n_experts <= 64. */
int hb_moe_route(void* stream, float* scale, const void* x, const void* w_gate, int64_t n_tokens,
                 int64_t hidden, int n_experts, int top_k, hb_dtype dtype);

/* The same split-KV decode attention for callers that must not allocate device memory
 * — a host that runs inside a captured or pre-planned memory budget, an embedding
 * runtime whose allocator the library may not touch, an interrupt-like serving loop
 * that forbids cudaMalloc after start-up.  (No counterpart in the reference: its
 * attention is a doc-only stub and every one of its kernels allocates its output.)
 * The split partials go to an 8 MiB array built into the library image, resident on
 * every GPU that loads the library until the process ends; a request whose partials
 * (hb_attention_workspace_bytes) exceed hb_paged_decode_attention_static_max_bytes()
 * is refused with HB_ERR_INVALID_ARG.  Nothing in the array has to start at zero
 * (every partial is written before it is read), but all calls share it: two calls
 * that overlap on the GPU — different streams, or the same arguments from two
 * threads — race on it.  The first call on each device looks the array's address
 * up; make that first call outside any stream capture.  No cudaMalloc/cudaFree or
 * other allocating routine is called. */
size_t hb_paged_decode_attention_static_max_bytes(void);
int hb_paged_decode_attention_static(void* stream, void* out, const void* q, const void* k_cache,
                                     const void* v_cache, const int32_t* block_tables,
                                     const int32_t* ctx_lens, int64_t n_seqs, int n_q_heads,
                                     int n_kv_heads, int head_dim, int64_t max_blocks_per_seq,
                                     int64_t num_blocks, int n_splits, hb_dtype dtype);

/* Y[M,N] = X[M,K] . W[N,K]^T  (weights stored [out,in] and applied as x.W^T, as every
 * matmul of the path does: src/engine/arch/llama_tp.rs:232-234,327,335-337,354).
 * bf16 with K%64==0 and N%8==0 runs on tcgen05 tensor cores (swap-AB: the weight's
 * output dim fills the 128-row UMMA M, the batch is the UMMA N; split-K fills the
 * SMs); other dtypes/shapes run a SIMT kernel.  `workspace` (may be NULL when
 * hb_gemm_workspace_bytes()==0) holds split-K partials and tile counters; it must be
 * zero-initialised once and is left zeroed by every call. */
size_t hb_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, hb_dtype dtype);
int hb_gemm(void* stream, void* Y, const void* X, const void* W, int64_t M, int64_t N, int64_t K,
            hb_dtype dtype, void* workspace);

/* The same GEMM with the epilogues the decode step fuses into it (bf16, K%64==0 only):
 *   epilogue 0: Y[M,N] = X.W^T, as bf16 or (out_f32 != 0) as fp32 — the logits GEMM;
 *   epilogue 1: W = [gate (N/2 rows) ; up (N/2 rows)], Y[M,N/2] = silu(X.gate^T) * (X.up^T)
 *               — gate, up, SiLU and the product of ffn_partial
 *               (src/engine/arch/llama_tp.rs:333-338) in one kernel.
 * force_splits > 0 overrides the split-K factor.  Workspace:
 * hb_gemm_ex_workspace_bytes(), zero-initialised once. */
size_t hb_gemm_ex_workspace_bytes(int64_t M, int64_t N, int64_t K, int epilogue, int force_splits);
int hb_gemm_ex(void* stream, void* Y, const void* X, const void* W, int64_t M, int64_t N,
               int64_t K, int epilogue, int out_f32, int force_splits, void* workspace);

/* out[m, i] = silu(gate_up[m, i]) * gate_up[m, inter + i]; gate_up [M, 2*inter]
 * (src/engine/arch/llama_tp.rs:333-339). */
int hb_silu_mul(void* stream, void* out, const void* gate_up, int64_t M, int64_t inter,
                hb_dtype dtype);

/* out[t, :] = table[ids[t], :]  (RankState::embed, src/engine/arch/llama_tp.rs:213-216). */
int hb_embed(void* stream, void* out, const void* table, const uint32_t* ids, int64_t n_tokens,
             int64_t hidden, int64_t vocab, hb_dtype dtype);

/* next[t] = index of the first maximum of logits[t, :] (greedy sampling,
 * src/sampling/mod.rs:105-107).  logits [n, vocab] `dtype`; out uint32 [n]. */
int hb_argmax(void* stream, uint32_t* out, const void* logits, int64_t n, int64_t vocab,
              hb_dtype dtype);

/* Sampling on the device (src/sampling/mod.rs:30-113): per row of logits [n, vocab] (fp32,
 * device) the reference's pipeline — presence/frequency penalties from token_counts
 * (uint32 [n, vocab] device, may be NULL: src/sampling/penalty.rs:28-52), division by the
 * temperature, softmax, top-p nucleus filter, renormalisation (src/sampling/nucleus.rs:7-62)
 * — without copying a row to the host.  temperature < 1e-6 is greedy: the delta distribution
 * on the first maximum (mod.rs:79-88).  The nucleus is every token whose probability is at
 * least that of the token at which the descending cumulative mass reaches top_p (tokens tied
 * with it are all kept; the reference's unstable sort keeps an unspecified subset of them).
 * hb_logits_to_probs writes the distribution (what the speculative decoder's acceptance
 * test reads, src/speculative.rs:189-196); hb_sample also draws tokens[i] from row i: the
 * first index whose cumulative probability exceeds u_i, u_i = the top 24 bits of
 * splitmix64(seeds[i]) / 2^24 (the reference draws with rand's SmallRng + WeightedIndex; that
 * stream is not reproduced, only its distribution).  probs_workspace: n * vocab floats. */
int hb_logits_to_probs(void* stream, float* probs, const float* logits, const uint32_t* token_counts, int64_t n,
                       int64_t vocab, float temperature, float top_p, float presence_penalty,
                       float frequency_penalty);
int hb_sample(void* stream, uint32_t* tokens, float* probs_workspace, const float* logits,
              const uint32_t* token_counts, const uint64_t* seeds, int64_t n, int64_t vocab, float temperature,
              float top_p, float presence_penalty, float frequency_penalty);

/* --------------------------------------------------------------- comm surface */

/* One rank's membership of a tensor-parallel group: the replacement of TpWorld
 * (src/parallel/world.rs:95-180).  The reference drives all GPUs from one process;
 * this library supports that (hb_world_create_local: n ranks in this process, peer
 * access enabled between their devices) and one process per GPU
 * (hb_world_create_rank + exchange of the 64-byte IPC handles by any host channel +
 * hb_world_attach). */
typedef struct hb_world hb_world;

#define HB_IPC_HANDLE_BYTES 64
#define HB_MAX_RANKS 8

/* Single-process form of TpWorld::new(n) (src/parallel/world.rs:95-133): worlds_out
 * receives n handles, rank i on device_ids[i] (NULL = 0..n-1).  Fails with a message
 * naming tensor_parallel_size when fewer devices are visible.  An explicit device_ids
 * list may name one device several times (ranks sharing a GPU; their kernels wait for
 * one another, so launch them only where they are known to run concurrently, or use
 * it to exercise the timeout path with hb_world_set_wait_limit). */
int hb_world_create_local(int n, const int* device_ids, size_t staging_bytes,
                          hb_world** worlds_out);
/* One-process-per-GPU form: create this rank's side, export its handle ... */
int hb_world_create_rank(int world_size, int rank, int device, size_t staging_bytes,
                         hb_world** out);
int hb_world_ipc_handle(hb_world* w, void* handle_out /* HB_IPC_HANDLE_BYTES */);
/* ... and attach to all ranks' handles (world_size * HB_IPC_HANDLE_BYTES, rank order). */
int hb_world_attach(hb_world* w, const void* all_handles);
/* Alternative to the IPC pair: hand over peer-mapped staging pointers obtained
 * elsewhere (for example a symmetric-memory allocation); peer_ptrs[rank] is this
 * rank's own buffer of at least hb_world_staging_bytes(). */
int hb_world_attach_ptrs(hb_world* w, void* const* peer_ptrs);
/* Optional window for HB_ALGO_MULTIMEM (reduction inside the NVLink switch, NVLink SHARP).
 * The caller allocates hb_world_multicast_bytes(max_rows, hidden) bytes on every rank, binds
 * the R allocations to ONE multicast object (cuMulticastCreate / cuMulticastAddDevice /
 * cuMulticastBindMem + cuMemMap, or a framework's symmetric-memory allocator that does the
 * same) and passes this rank's ordinary address of its allocation and the multicast address.
 * The library zeroes the window's first 64 KiB; all ranks attach, THEN synchronise on the
 * host, then use it.  The memory stays the caller's: detach (which drains the device) before
 * unbinding or freeing it, on every rank, and end no process while its window is bound.
 * After HB_ERR_TIMEOUT in a call that used the window its counters are out of step: detach
 * and attach again on all ranks.  bf16 rows only, world sizes 2, 4 and 8, hidden a multiple
 * of 8 * world_size, at most 256 rows.  hb_world_multicast_partial: the address inside the
 * window where a row-parallel GEMM should leave its [rows, hidden] partial; hb_all_reduce_add_rms_norm
 * copies a partial that lies elsewhere. */
size_t hb_world_multicast_bytes(int64_t max_rows, int64_t hidden);
int hb_world_attach_multicast(hb_world* w, void* local_ptr, void* multicast_ptr, size_t bytes);
int hb_world_detach_multicast(hb_world* w);
int hb_world_has_multicast(const hb_world* w);
void* hb_world_multicast_partial(const hb_world* w);
/* Optional NCCL communicator for HB_ALGO_NCCL: unique id from hb_nccl_unique_id on
 * rank 0, passed to every rank. */
#define HB_NCCL_ID_BYTES 128
int hb_nccl_unique_id(void* id_out /* HB_NCCL_ID_BYTES */);
int hb_world_init_nccl(hb_world* w, const void* id /* HB_NCCL_ID_BYTES */);
int hb_world_free(hb_world* w);
int hb_world_size(const hb_world* w);   /* TpWorld::world_size, world.rs:135 */
int hb_world_rank(const hb_world* w);
int hb_world_device(const hb_world* w); /* TpWorld::device, world.rs:145 */
int hb_world_is_single(const hb_world* w); /* TpWorld::is_single, world.rs:157 */
size_t hb_world_staging_bytes(const hb_world* w);
void* hb_world_stream(const hb_world* w);
/* Device status word of the collectives on this rank since the last call: 0, or
 * HB_ERR_TIMEOUT when a bounded wait on a peer flag ran out (the kernel then returns
 * instead of hanging, as nccl_all_reduce returns an Err: src/parallel/comm.rs:113-143).
 * Reading a non-zero status clears it.  After a timeout the outputs of that collective
 * are undefined and the sequence counters of the ranks may disagree: free the worlds of
 * the group and create new ones before the next collective. */
int hb_world_status(hb_world* w);
/* Number of polls after which a device-side wait on a peer flag gives up (0 restores
 * the default of 2^22, several hundred milliseconds).  Applies to collectives launched
 * afterwards; a step already captured in a CUDA graph keeps the limit it was captured
 * with.  (No counterpart in the reference: NCCL's own watchdog plays this part there.) */
int hb_world_set_wait_limit(hb_world* w, uint32_t polls);


/* In-place SUM all-reduce of `count` elements at `buf` on this rank; every rank calls
 * it with the same count/dtype.  The result is valid on every rank (a superset of the
 * reference's rank-0 result).  Replaces TpWorld::all_reduce
 * (src/parallel/world.rs:171-180) -> nccl_all_reduce (src/parallel/comm.rs:83-166).
 * Partials are summed in rank order 0,1,... in fp32 (src/parallel/comm.rs:54-58). */
int hb_all_reduce(hb_world* w, void* stream, void* buf, size_t count, hb_dtype dtype,
                  hb_algo algo);

/* All-reduce + residual add + RMSNorm in one kernel per rank:
 *   s = SUM_ranks partial_r (fp32 in rank order, rounded once), resid_out = resid_in + s,
 *   normed_out = rms_norm(resid_out; norm_w, eps)
 * — the exchange and the two elementwise steps between a row-parallel projection and the
 * next layer input (src/engine/arch/llama_tp.rs:533-552 and :563-571,517-522), with the
 * values of hb_all_reduce followed by hb_add_rms_norm bit for bit.  partial, resid_in,
 * resid_out, normed_out are [rows, hidden] on this rank (resid_out may alias resid_in;
 * normed_out may be NULL); rows <= 256, hidden * element size a multiple of 16 bytes and
 * at most 32 KiB; every rank calls it with the same shapes.
 * HB_ALGO_MULTIMEM (world with a multicast window, bf16): the NVLink switch forms the sum —
 * one load per 16 bytes returns the fp32-accumulated sum over all ranks, one store delivers
 * the new residual slice to all ranks.  The switch adds in its own order, so the result
 * agrees with the other algorithms to one bf16 rounding of the sum, not bit for bit; all
 * ranks still hold identical rows.  A partial outside the window is copied into it first. */
int hb_all_reduce_add_rms_norm(hb_world* w, void* stream, void* normed_out, void* resid_out,
                               const void* partial, const void* resid_in, const void* norm_w,
                               int64_t rows, int64_t hidden, float eps, hb_dtype dtype, hb_algo algo);

/* Fused row-parallel projection: normed_out = rms_norm(resid_out),
 * resid_out = resid_in + SUM_ranks( X_r[M,Kl] . W_r[N,Kl]^T ).
 * This is llama_tp.rs steps o_proj/down_proj -> all_reduce -> residual -> next norm
 * (src/engine/arch/llama_tp.rs:327,533-552 and :339,563-571,517-522).  bf16 only.
 * The form depends on the world, the shape and `algo` (hb_fused_rowparallel_form tells
 * which; nothing is substituted silently):
 *   HB_ROWPAR_SINGLE    single-rank world: tcgen05 GEMM, then add + RMSNorm;
 *   HB_ROWPAR_PUSH      the GEMM epilogue writes each 128-feature tile of the partial
 *                       straight into the staging of the rank that reduces that column
 *                       slice (NVLink peer stores + a release flag per tile): the first hop
 *                       of the all-reduce is part of the GEMM kernel; one peer-memory kernel
 *                       then sums, adds the residual, returns the reduced slices and
 *                       normalises.  Taken with HB_ALGO_TWO_SHOT, or HB_ALGO_AUTO above
 *                       (ranks-1) x M x N x 2 bytes >= 4 MiB on 3+ ranks, when N is a multiple of
 *                       128*ranks, M <= 256;
 *   HB_ROWPAR_EXCHANGE  GEMM to a local partial, then hb_all_reduce_add_rms_norm
 *                       (HB_ALGO_ONE_SHOT, small messages, shapes the push form cannot take);
 *   HB_ROWPAR_NCCL      GEMM -> ncclAllReduce -> add + RMSNorm, the reference's own sequence
 *                       (HB_ALGO_NCCL; needs hb_world_init_nccl): the reported baseline;
 *   HB_ROWPAR_MULTIMEM  the GEMM writes its partial into the world's multicast window, one
 *                       kernel per rank lets the NVLink switch form the sum (one load that
 *                       returns the sum over all ranks, one store that reaches all ranks),
 *                       adds the residual and normalises (HB_ALGO_MULTIMEM; needs
 *                       hb_world_attach_multicast).  Sums agree with the other forms to
 *                       bf16 rounding (the switch's order of addition is its own).
 * Shapes none of the forms covers fail with HB_ERR_INVALID_ARG.
 * norm_w may be NULL (then normed_out is not written). */
#define HB_ROWPAR_SINGLE 0
#define HB_ROWPAR_PUSH 1
#define HB_ROWPAR_EXCHANGE 2
#define HB_ROWPAR_NCCL 3
#define HB_ROWPAR_MULTIMEM 4
int hb_fused_rowparallel_form(const hb_world* w, int64_t M, int64_t N, int64_t K_local, hb_algo algo);
size_t hb_fused_rowparallel_workspace_bytes(int64_t M, int64_t N, int64_t K_local);
int hb_fused_rowparallel(hb_world* w, void* stream, void* normed_out, void* resid_out,
                         const void* X, const void* W, const void* resid_in, const void* norm_w,
                         int64_t M, int64_t N, int64_t K_local, float eps, hb_algo algo,
                         void* workspace);

/* ------------------------------------------------------- sharding (load side) */

/* Rows [rank*out/ws, (rank+1)*out/ws) of a [rows, cols] matrix: column_shard
 * (src/parallel/shard.rs:46-54).  Host memory, `elem` bytes per element.
 * Error text contains "divisible" as the reference's does. */
int hb_column_shard(void* dst, const void* src, int64_t rows, int64_t cols, size_t elem,
                    int rank, int world_size);
/* Columns [rank*in/ws, ...) of every row: row_shard (src/parallel/shard.rs:66-74). */
int hb_row_shard(void* dst, const void* src, int64_t rows, int64_t cols, size_t elem, int rank,
                 int world_size);

/* ------------------------------------------------------ block tables (host) */

/* Bit-exact restatement of BlockManager (src/scheduler/block_manager.rs:143-414):
 * FIFO free list initialised 0..n, allocate = pop front, free = push back on
 * refcount 0, FNV-1a prefix cache of 128 entries, append_slot with copy-on-write. */
typedef struct hb_block_manager hb_block_manager;
int hb_bm_create(int64_t num_gpu_blocks, int64_t num_cpu_blocks, hb_block_manager** out);
int hb_bm_free_manager(hb_block_manager* bm);
int64_t hb_bm_num_free_gpu_blocks(const hb_block_manager* bm);
int64_t hb_bm_num_free_cpu_blocks(const hb_block_manager* bm);
int64_t hb_bm_num_prefix_cached_blocks(const hb_block_manager* bm);
/* allocate(): a single-sequence group of prompt_len prompt ids + output_len generated
 * tokens; *hit_blocks receives the number of prefix-cache hits. */
int hb_bm_allocate(hb_block_manager* bm, uint64_t seq_id, const uint32_t* prompt_ids,
                   int64_t prompt_len, int64_t output_len, int64_t* hit_blocks);
int hb_bm_can_allocate(const hb_block_manager* bm, int64_t total_len);
int hb_bm_can_append_slot(const hb_block_manager* bm, uint64_t seq_id, int64_t total_len);
/* append_slot(): total_len = prompt + output tokens so far; cow_pair receives
 * (old,new) or (-1,-1). */
int hb_bm_append_slot(hb_block_manager* bm, uint64_t seq_id, int64_t total_len,
                      int64_t cow_pair[2]);
int hb_bm_free_seq(hb_block_manager* bm, uint64_t seq_id);
/* swap_out/swap_in: mapping_out (capacity 2 * table length, or NULL when the pairs
 * are not wanted) receives (from,to) ids in table order; *n_pairs their number. */
int hb_bm_swap_out(hb_block_manager* bm, uint64_t seq_id, int64_t* mapping_out, int64_t* n_pairs);
int hb_bm_swap_in(hb_block_manager* bm, uint64_t seq_id, int64_t* mapping_out, int64_t* n_pairs);
/* Copies the table into out (capacity cap); returns its length or a negative error. */
int64_t hb_bm_block_table(const hb_block_manager* bm, uint64_t seq_id, int64_t* out, int64_t cap);
/* hash_block (src/scheduler/prefix_cache.rs:40-50). */
uint64_t hb_hash_block(const uint32_t* tokens, int64_t n);
/* Sequence::num_logical_blocks / last_block_num_filled (src/scheduler/sequence.rs:80-92). */
int64_t hb_num_logical_blocks(int64_t len, int64_t block_size);
int64_t hb_last_block_num_filled(int64_t len, int64_t block_size);
/* slot(pos) = table[pos/16]*16 + pos%16. */
int64_t hb_slot_for_position(const int64_t* table, int64_t table_len, int64_t pos);

/* ------------------------------------------------------------ engine surface */

/* Mirrors ModelConfig (src/engine/config.rs:14-26) plus what the C side needs to know
 * that the reference takes from its process: which rank this is and how many KV
 * blocks to reserve (the reference's NUM_GPU_BLOCKS=256 is a compile-time constant,
 * src/worker/mod.rs:68). */
typedef struct hb_model_config {
  const char* model_path; /* directory with config.json + *.safetensors */
  size_t max_seq_len;
  double gpu_memory_utilization;
  int bf16;                 /* 1: BF16, 0: F16 on CUDA (src/engine/dtype.rs:22-28) */
  int tensor_parallel_size;
  /* additions */
  int64_t num_kv_blocks;    /* 0 = derive from max_seq_len * max_batch */
  int max_batch;            /* largest B of hb_decode_batch (0 = 256) */
  int force_f32;            /* 1: keep F32 weights (the reference's CPU dtype) for tight parity */
} hb_model_config;

/* Shape of a model for hb_engine_create_random (no files involved). */
typedef struct hb_model_shape {
  int64_t hidden_size, intermediate_size, num_hidden_layers, num_attention_heads,
      num_key_value_heads, vocab_size;
  double rms_norm_eps, rope_theta;
  /* mixture of experts (src/engine/arch/mixtral.rs:40-57); all 0 for a dense Llama */
  int64_t num_local_experts;    /* experts per layer, each a SwiGLU FFN of intermediate_size */
  int64_t num_experts_per_tok;  /* top-k of the router */
  int64_t sliding_window;       /* attention window in tokens, 0 = none */
} hb_model_shape;

typedef struct hb_engine hb_engine;
typedef struct hb_seq hb_seq;

/* Engine::load (src/engine/loader.rs:66-192) for model_type "llama"/"mistral" and
 * "mixtral" (MixtralBackend::load, src/engine/arch/mixtral.rs:455-516, here also tensor-parallel:
 * every expert's w1/w3 column-parallel and w2 row-parallel over its intermediate size):
 * reads config.json and the sorted *.safetensors, checks the divisibility rules of
 * TpLlamaBackend::load (src/engine/arch/llama_tp.rs:407-427), shards per
 * src/parallel/shard.rs and uploads this rank's slices.  `world` may be NULL for
 * tensor_parallel_size 1. */
int hb_engine_load(const hb_model_config* cfg, hb_world* world, hb_engine** out);
/* Same engine with weights drawn on the device: N(0, std) from a counter-based
 * generator keyed by (seed, tensor, element index of the UNSHARDED tensor), so every
 * rank draws exactly its slice of the same global tensor; norm weights are 1 when
 * norm_ones != 0 else N(0, std). */
int hb_engine_create_random(const hb_model_shape* shape, const hb_model_config* cfg,
                            hb_world* world, uint64_t seed, float std, int norm_ones,
                            hb_engine** out);
int hb_engine_free(hb_engine* e);
int64_t hb_engine_num_layers(const hb_engine* e);  /* loader.rs:331 */
int64_t hb_engine_vocab_size(const hb_engine* e);  /* loader.rs:334 */
int64_t hb_engine_hidden_size(const hb_engine* e); /* loader.rs:337 */
int64_t hb_engine_param_count(const hb_engine* e); /* loader.rs:323-329 */
int64_t hb_engine_num_free_blocks(const hb_engine* e);
/* Bytes of weights + KV the decode step streams from HBM on this rank for the given
 * context lengths (the roofline numerator). */
double hb_engine_step_bytes(const hb_engine* e, const int32_t* ctx_lens, int64_t n_seqs);
/* Copies a named device tensor of this rank (e.g. "model.layers.0.self_attn.q_proj.weight",
 * sharded as loaded) to host as f32; returns element count or negative error. */
int64_t hb_engine_get_tensor(hb_engine* e, const char* name, float* out, int64_t cap);

/* create_kv_cache (src/engine/loader.rs:248): a REAL per-sequence cache (block table
 * over the paged pool), unlike the reference's zero-size LlamaTp marker
 * (src/engine/kv_cache.rs:28-41). */
int hb_seq_create(hb_engine* e, hb_seq** out);
int hb_seq_free(hb_engine* e, hb_seq* s);
int64_t hb_seq_len(const hb_seq* s);
int64_t hb_seq_block_table(const hb_seq* s, int64_t* out, int64_t cap);

/* forward_with_cache (src/engine/loader.rs:256-263): feeds n token ids at absolute
 * position seq_pos and writes the last token's logits [vocab] as f32 to HOST memory
 * logits_out.  Prefill = many ids at seq_pos 0; decode = one id at
 * prompt_len+output_len-1 (src/worker/mod.rs:349-351,404-409).  seq_pos must equal
 * the sequence's current length.  With a multi-rank world every rank calls it with
 * the same arguments. */
int hb_forward(hb_engine* e, hb_seq* s, const uint32_t* ids, size_t n, size_t seq_pos,
               float* logits_out);

/* Additive: one decode step for B sequences at once (the reference decodes them one
 * by one, src/worker/mod.rs:280-293).  last_tokens/next_tokens are HOST uint32 [B];
 * next_tokens = greedy argmax (src/sampling/mod.rs:105-107); logits_opt (HOST f32
 * [B, vocab]) may be NULL.  Copies in and out happen inside the call. */
int hb_decode_batch(hb_engine* e, hb_seq* const* seqs, size_t B, const uint32_t* last_tokens,
                    uint32_t* next_tokens, float* logits_opt);
/* ---- the step driven by a scheduler's block tables.  The reference's scheduler computes
 * block tables, copy-on-write pairs and swap lists every step (SchedulerOutputs,
 * src/scheduler/mod.rs:40-61,203-208; BlockManager::append_slot / swap_in / swap_out,
 * src/scheduler/block_manager.rs:314-406) and its worker drops them
 * (src/worker/mod.rs:250-305).  These entry points consume them: the caller (hb_bm_* or the
 * Rust BlockManager itself) owns the block ids, the engine's KV pool is indexed by them.
 * An engine is driven either through hb_seq handles or through tables, not both at once
 * (the hb_seq allocator hands out ids of the same pool).
 *
 * hb_decode_batch_tables: row b feeds last_tokens[b] at absolute position positions[b]
 * (= prompt_len + output_len - 1, src/worker/mod.rs:404-409) of the sequence whose table is
 * block_tables[b * table_stride ...]; the table must cover that position
 * (entries 0 .. positions[b]/16).  copy_pairs = blocks_to_copy as (src, dst) ids, applied
 * to every layer's K and V before the step.  Outputs as hb_decode_batch.
 * hb_forward_tables: n tokens of ONE sequence at positions seq_pos .. seq_pos+n-1; with
 * seq_pos > 0 the positions below it must already hold this sequence's K/V in the
 * table's blocks — a prefix-cache hit (hit_blocks * 16 tokens are skipped:
 * src/scheduler/block_manager.rs:213-234), or a continued prefill.
 * hb_kv_copy_blocks: dst := src for every pair (all layers, K and V).
 * hb_kv_swap_blocks: swap_out (to_cpu != 0, pairs (gpu, cpu)) / swap_in (pairs (cpu, gpu))
 * between the pool and a pinned host pool of hb_engine_reserve_cpu_blocks() blocks. */
int hb_decode_batch_tables(hb_engine* e, size_t B, const uint32_t* last_tokens, const int64_t* positions,
                           const int64_t* block_tables, size_t table_stride, const int64_t* copy_pairs,
                           size_t n_copies, uint32_t* next_tokens, float* logits_opt);
int hb_forward_tables(hb_engine* e, const uint32_t* ids, size_t n, size_t seq_pos, const int64_t* block_table,
                      size_t table_len, float* logits_out);
int hb_kv_copy_blocks(hb_engine* e, const int64_t* pairs, size_t n_pairs);
/* Speculative verification as ONE forward: the n tokens [last, draft_0 .. draft_{n-2}] are fed
 * at positions seq_pos .. and the logits of EVERY position come back (host f32 [n, vocab]),
 * where the reference runs up to K+1 single-token target forwards (src/speculative.rs:174-212).
 * The caller applies the acceptance rule and then drops the rejected tokens' K/V with
 * hb_seq_truncate(seq, seq_pos + accepted) (the reference stops feeding at the first
 * rejection instead). */
int hb_forward_all_positions(hb_engine* e, hb_seq* s, const uint32_t* ids, size_t n, size_t seq_pos,
                             float* logits_out);
int hb_seq_truncate(hb_engine* e, hb_seq* s, int64_t new_len);
int hb_engine_reserve_cpu_blocks(hb_engine* e, int64_t n_blocks);
int hb_kv_swap_blocks(hb_engine* e, const int64_t* pairs, size_t n_pairs, int to_cpu);

/* One decode step with CUDA events between its kernels — captured into a graph with an
 * event-record node after every kernel and replayed, so the kernels run back to back as in
 * a normal step (HB_NO_GRAPH=1: issued kernel by kernel on the
 * stream): ms_by_kind receives HB_PROFILE_KINDS floats = device time spent in
 * 0 QKV projection, 1 decode attention, 2 RoPE + KV write, 3 (add +) RMSNorm, 4 embedding /
 * argmax / SwiGLU gate, 5 all-reduce, 6 o_proj, 7 gate|up projection, 8 down_proj,
 * 9 lm_head (6 and 8 include the fused all-reduce + residual + norm when that kernel
 * runs).  The step counts like any other decode step. */
#define HB_PROFILE_KINDS 10
int hb_engine_profile_step(hb_engine* e, hb_seq* const* seqs, size_t B,
                           const uint32_t* last_tokens, uint32_t* next_tokens, float* ms_by_kind);
/* Algorithmic bytes all GEMM launches of one decode step move for batch B on this rank
 * (weights + activations in + results out). */
double hb_engine_gemm_bytes(const hb_engine* e, int64_t B);
/* Device-time of the last hb_decode_batch kernels only (ms, CUDA events on the
 * engine's stream); negative if none. */
float hb_engine_last_step_ms(hb_engine* e);
/* Number of kernel launches of this library in the last step. */
int64_t hb_engine_last_step_launches(const hb_engine* e);
void* hb_engine_stream(hb_engine* e);

#ifdef __cplusplus
}
#endif
#endif /* HB_H_ */
