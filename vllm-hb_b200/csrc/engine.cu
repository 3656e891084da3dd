// The decode-step engine behind hb_engine_* / hb_seq_* / hb_forward / hb_decode_batch.
//
// It stands where Engine (src/engine/loader.rs:66-339) -> Backend
// (src/engine/arch/mod.rs:33-118) -> TpLlamaBackend (src/engine/arch/llama_tp.rs) stand
// in the reference, with these differences of structure:
//   - one engine object per rank (the reference loops over ranks inside one process,
//     llama_tp.rs:506-576); with a multi-rank hb_world every rank runs the same step
//     and the row-parallel partials meet in the peer-memory all-reduce;
//   - B sequences per step through batched GEMMs and a paged KV pool, each sequence with
//     a real block table (the reference decodes sequence by sequence over one shared,
//     cat-grown cache: src/worker/mod.rs:280-293, llama_tp.rs:245-259);
//   - no allocation and no host round trip inside a step: all buffers are created at
//     load, the step is captured once per batch size into a CUDA graph and replayed.
#include <cmath>
#include <deque>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "comm.h"
#include "common.h"
#include "gemm.h"
#include "json.h"
#include "ops.h"
#include "rowpar.h"
#include "safetensors.h"

struct hb_seq {
  uint64_t id = 0;
  std::vector<int64_t> blocks;  // physical block ids, table[pos / 16]
  int64_t len = 0;              // tokens whose K/V are in the pool
};

namespace hb {

struct LayerWeights {
  void* wqkv = nullptr;   // [(hq_l + 2*hkv_l) * hd, H]   rows: q | k | v (column-parallel)
  void* wo = nullptr;     // [H, hq_l * hd]               (row-parallel)
  // Dense FFN: E = 1.  Mixture of experts: the experts' weights are concatenated, gate
  // (w1) rows of all experts first, then their up (w3) rows; down (w2) along K.
  void* wgu = nullptr;    // [2 * E * I_l, H]             rows: gate_0..gate_{E-1} | up_0..up_{E-1}
  void* wdown = nullptr;  // [H, E * I_l]                 columns: expert e at [e * I_l, (e+1) * I_l)
  void* wgate = nullptr;  // [E, H] router (replicated), null for a dense FFN
  void* norm_in = nullptr;
  void* norm_post = nullptr;
};

struct NamedTensor {
  void* ptr;
  int64_t rows, cols;
  int64_t ld = 0;  // row stride in elements (0 = cols): expert down-projections are column blocks
};

enum GemmKind { kQkv = 0, kO = 1, kGateUp = 2, kDown = 3, kLmHead = 4 };
constexpr int kPairCap = 1024;  // block pairs per copy launch

struct StepPlans {
  std::vector<TcGemmPlan> layer;  // [L * 4]
  TcGemmPlan lm_head;
  int attn_splits = 1;
  int q_group = 1;          // prefill chunks: consecutive positions that share an attention CTA
  bool defer_norm = false;  // add + norm folded into the GEMM epilogues (TcNormLink)
  bool mm = false;          // exchange through the NVLink switch (multicast window of the world)
  const void* mm_window = nullptr;  // the window the plans (and the captured graph) were made for
  bool rope_epi = false;    // RoPE + KV write folded into the q|k|v GEMM epilogue (TcNormLink)
  bool push = false;        // o_proj / down_proj epilogues push their partials to the reducing ranks (kEpiPush)
  PushGeometry geo_o, geo_down;
  int64_t launches = 0;  // kernels in one step (fixed per batch size)
  cudaGraphExec_t graph = nullptr;
};

}  // namespace hb

struct hb_engine {
  int device = 0;
  cudaStream_t stream = nullptr;
  hb_world* world = nullptr;
  int rank = 0, ws = 1;
  hb_dtype dtype = HB_BF16;
  size_t es = 2;
  // shape
  int64_t H = 0, I = 0, L = 0, hq = 0, hkv = 0, hd = 0, V = 0;
  double eps = 1e-5, theta = 10000.0;
  int64_t hq_l = 0, hkv_l = 0, I_l = 0, qkv_rows = 0;
  // mixture of experts (mixtral.rs:40-57): E experts, top-k routing, sliding window; I_e = E * I_l
  int64_t E = 1, topk = 1, window = 0, I_e = 0;
  bool moe = false;
  float* d_scale = nullptr;  // [max_batch, E] routing weights of the step
  float* d_rowsq = nullptr;  // [max_batch, rowsq_stride] row sums of the deferred norm
  float2* d_rope_cs = nullptr;  // [max_batch, hd/2] (cos, sin) of the step's positions
  int rowsq_stride = 0;
  // weights
  void* embed = nullptr;
  void* lm_head = nullptr;
  void* final_norm = nullptr;
  std::vector<hb::LayerWeights> layers;
  std::map<std::string, hb::NamedTensor> named;
  std::vector<void*> allocations;
  // KV pool
  int64_t num_blocks = 0;
  std::vector<void*> kc, vc;
  std::deque<int64_t> free_blocks;  // FIFO: pop front / push back (block_manager.rs:58,63-83)
  uint64_t next_seq_id = 0;
  // step buffers
  int max_batch = 0;
  int64_t max_blocks_per_seq = 0;
  uint8_t* d_inputs = nullptr;  // [ids | positions | ctx | pad | slots | tables]
  uint8_t* h_inputs = nullptr;  // pinned mirror
  size_t inputs_bytes = 0;
  size_t off_ids = 0, off_pos = 0, off_ctx = 0, off_slots = 0, off_tables = 0;
  void *d_h = nullptr, *d_x = nullptr, *d_qkv = nullptr, *d_attn = nullptr, *d_gu = nullptr,
       *d_act = nullptr, *d_proj = nullptr;
  float* d_logits = nullptr;
  uint32_t* d_next = nullptr;
  uint32_t* h_next = nullptr;  // pinned
  float* d_inv_freq = nullptr;
  void* d_attn_ws = nullptr;
  size_t attn_ws_bytes = 0;
  void* d_gemm_ws = nullptr;
  size_t gemm_ws_bytes = 0;
  int* d_err = nullptr;
  int64_t* d_pairs = nullptr;   // (src, dst) block ids of a copy request, kPairCap pairs at a time
  uint8_t* h_swap = nullptr;    // pinned CPU block pool [cpu_blocks][L][K|V][block bytes] (hb_engine_reserve_cpu_blocks)
  int64_t cpu_blocks = 0;
  bool use_tc = false, use_graph = true, fused_swiglu = true;
  std::map<int, hb::StepPlans> plans;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  float last_ms = -1.f;
  int64_t last_launches = 0;
  // per-kernel-kind timing of one eager step (hb_engine_profile_step)
  bool profiling = false;
  bool prof_capture = false;  // the profiled step is being captured: events become graph nodes
  std::vector<cudaEvent_t> prof_events;
  std::vector<int> prof_cats;
  size_t prof_used = 0;
  float prof_ms[16] = {0};
};

namespace hb {

// ------------------------------------------------------------------ host helpers
static int dev_alloc(hb_engine* e, void** p, size_t bytes) {
  HB_CUDA_CHECK(cudaMalloc(p, bytes ? bytes : 16));
  e->allocations.push_back(*p);
  return HB_OK;
}

static bool same_dtype(const std::string& s, hb_dtype d) {
  return (s == "F32" && d == HB_F32) || (s == "F16" && d == HB_F16) || (s == "BF16" && d == HB_BF16);
}

static hb_dtype st_dtype(const std::string& s) { return s == "F32" ? HB_F32 : s == "F16" ? HB_F16 : HB_BF16; }

// Rows [r0, r0+nr) x cols [c0, c0+nc) of a [rows, cols] tensor of the memory-mapped
// checkpoint go to device memory at dst (row-major [nr, nc], row stride dst_ld elements) in
// the engine dtype — the narrow() of column_shard / row_shard (src/parallel/shard.rs:46-74)
// followed by to_device, without the reference's full CPU copy in the target dtype
// (llama_tp.rs:367-377): only this rank's slice leaves the page cache, as one strided copy
// straight from the mapping, and a checkpoint in another dtype is converted on the device.
// `stage` is a device buffer that grows to the largest slice that needs converting.
struct UploadStage {
  void* buf = nullptr;
  size_t bytes = 0;
  ~UploadStage() { if (buf) cudaFree(buf); }
};

static int upload_slice(hb_engine* e, void* dst, const StTensor& t, int64_t cols, int64_t r0,
                        int64_t nr, int64_t c0, int64_t nc, UploadStage* stage, int64_t dst_ld = 0) {
  const size_t src_es = t.dtype == "F32" ? 4 : 2;
  const uint8_t* src = t.data + ((size_t)r0 * cols + c0) * src_es;
  if (dst_ld <= 0) dst_ld = nc;
  // every copy and conversion is ordered on the engine's stream; hb_engine_load synchronises it
  // before the mapping goes away
  if (same_dtype(t.dtype, e->dtype)) {
    HB_CUDA_CHECK(cudaMemcpy2DAsync(dst, (size_t)dst_ld * e->es, src, (size_t)cols * src_es, (size_t)nc * src_es,
                                    (size_t)nr, cudaMemcpyHostToDevice, e->stream));
    return HB_OK;
  }
  const size_t need = (size_t)nr * nc * src_es;
  if (need > stage->bytes) {
    HB_CUDA_CHECK(cudaStreamSynchronize(e->stream));
    if (stage->buf) cudaFree(stage->buf);
    stage->buf = nullptr;
    stage->bytes = 0;
    HB_CUDA_CHECK(cudaMalloc(&stage->buf, need));
    stage->bytes = need;
  }
  HB_CUDA_CHECK(cudaMemcpy2DAsync(stage->buf, (size_t)nc * src_es, src, (size_t)cols * src_es, (size_t)nc * src_es,
                                  (size_t)nr, cudaMemcpyHostToDevice, e->stream));
  int rc = convert_2d(e->stream, dst, e->dtype, dst_ld, stage->buf, st_dtype(t.dtype), nr, nc);
  if (rc) return rc;
  HB_CUDA_CHECK(cudaStreamSynchronize(e->stream));  // the stage is reused by the next slice
  return HB_OK;
}

static int check_divisibility(const hb_engine* e) {
  // TpLlamaBackend::load (src/engine/arch/llama_tp.rs:407-427)
  const int n = e->ws;
  if (e->hq % n)
    return fail(HB_ERR_NOT_DIVISIBLE,
                "num_attention_heads (%lld) must be divisible by tensor_parallel_size (%d)",
                (long long)e->hq, n);
  if (e->hkv % n)
    return fail(HB_ERR_NOT_DIVISIBLE,
                "num_key_value_heads (%lld) must be divisible by tensor_parallel_size (%d)",
                (long long)e->hkv, n);
  if (e->I % n)
    return fail(HB_ERR_NOT_DIVISIBLE,
                "intermediate_size (%lld) must be divisible by tensor_parallel_size (%d)",
                (long long)e->I, n);
  return HB_OK;
}

static int setup_common(hb_engine* e, const hb_model_config* cfg, hb_world* world) {
  const int tp = cfg->tensor_parallel_size > 0 ? cfg->tensor_parallel_size : 1;
  e->world = world;
  e->ws = world ? world->ws : 1;
  e->rank = world ? world->rank : 0;
  if (tp != e->ws)
    return fail(HB_ERR_INVALID_ARG,
                "tensor_parallel_size=%d but the world handed to the engine has %d rank(s)", tp, e->ws);
  if (world) e->device = world->device;
  else HB_CUDA_CHECK(cudaGetDevice(&e->device));
  HB_CUDA_CHECK(cudaSetDevice(e->device));
  e->dtype = cfg->force_f32 ? HB_F32 : (cfg->bf16 ? HB_BF16 : HB_F16);  // src/engine/dtype.rs:22-28
  e->es = dtype_size(e->dtype);
  HB_CUDA_CHECK(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
  HB_CUDA_CHECK(cudaEventCreate(&e->ev0));
  HB_CUDA_CHECK(cudaEventCreate(&e->ev1));
  const char* g = getenv("HB_NO_GRAPH");
  e->use_graph = !(g && g[0] == '1');
  return HB_OK;
}

static int setup_shape(hb_engine* e, const hb_model_shape& s) {
  e->H = s.hidden_size; e->I = s.intermediate_size; e->L = s.num_hidden_layers;
  e->hq = s.num_attention_heads;
  e->hkv = s.num_key_value_heads == 0 ? s.num_attention_heads : s.num_key_value_heads;  // llama_tp.rs:81-87
  e->V = s.vocab_size;
  e->eps = s.rms_norm_eps; e->theta = s.rope_theta;
  if (e->H <= 0 || e->I <= 0 || e->L <= 0 || e->hq <= 0 || e->V <= 0 || e->H % e->hq)
    return fail(HB_ERR_INVALID_ARG, "bad model shape");
  e->hd = e->H / e->hq;  // llama_tp.rs:77-79
  int rc = check_divisibility(e);
  if (rc) return rc;
  e->hq_l = e->hq / e->ws; e->hkv_l = e->hkv / e->ws; e->I_l = e->I / e->ws;
  e->moe = s.num_local_experts > 0;
  e->E = e->moe ? s.num_local_experts : 1;
  e->topk = e->moe ? (s.num_experts_per_tok > 0 ? s.num_experts_per_tok : 2) : 1;
  e->window = s.sliding_window > 0 ? s.sliding_window : 0;
  if (e->E > 64) return fail(HB_ERR_INVALID_ARG, "num_local_experts %lld unsupported (<= 64)", (long long)e->E);
  e->I_e = e->E * e->I_l;
  e->qkv_rows = (e->hq_l + 2 * e->hkv_l) * e->hd;
  const char* g = getenv("HB_GEMM");
  const bool want_simt = g && std::string(g) == "simt";
  e->use_tc = !want_simt && e->dtype == HB_BF16 && e->H % 64 == 0 && (e->hq_l * e->hd) % 64 == 0 &&
              e->I_l % 64 == 0;
  // expert boundaries must fall on 128-feature tiles of the SwiGLU GEMM
  if (e->moe && e->I_l % 128 != 0) e->use_tc = false;
  return HB_OK;
}

static int alloc_weights(hb_engine* e) {
  const size_t es = e->es;
  int rc;
  if ((rc = dev_alloc(e, &e->embed, (size_t)e->V * e->H * es))) return rc;
  if ((rc = dev_alloc(e, &e->lm_head, (size_t)e->V * e->H * es))) return rc;
  if ((rc = dev_alloc(e, &e->final_norm, (size_t)e->H * es))) return rc;
  e->layers.resize(e->L);
  for (auto& l : e->layers) {
    if ((rc = dev_alloc(e, &l.wqkv, (size_t)e->qkv_rows * e->H * es))) return rc;
    if ((rc = dev_alloc(e, &l.wo, (size_t)e->H * e->hq_l * e->hd * es))) return rc;
    if ((rc = dev_alloc(e, &l.wgu, (size_t)2 * e->I_e * e->H * es))) return rc;
    if ((rc = dev_alloc(e, &l.wdown, (size_t)e->H * e->I_e * es))) return rc;
    if (e->moe && (rc = dev_alloc(e, &l.wgate, (size_t)e->E * e->H * es))) return rc;
    if ((rc = dev_alloc(e, &l.norm_in, (size_t)e->H * es))) return rc;
    if ((rc = dev_alloc(e, &l.norm_post, (size_t)e->H * es))) return rc;
  }
  // names as the reference looks them up (llama_tp.rs:451-462,482-488), sharded shapes
  e->named["model.embed_tokens.weight"] = {e->embed, e->V, e->H};
  e->named["lm_head.weight"] = {e->lm_head, e->V, e->H};
  e->named["model.norm.weight"] = {e->final_norm, 1, e->H};
  for (int64_t i = 0; i < e->L; ++i) {
    const std::string pf = "model.layers." + std::to_string(i);
    auto& l = e->layers[i];
    uint8_t* qkv = (uint8_t*)l.wqkv;
    const size_t rowb = (size_t)e->H * es;
    e->named[pf + ".self_attn.q_proj.weight"] = {qkv, e->hq_l * e->hd, e->H};
    e->named[pf + ".self_attn.k_proj.weight"] = {qkv + (size_t)e->hq_l * e->hd * rowb, e->hkv_l * e->hd, e->H};
    e->named[pf + ".self_attn.v_proj.weight"] = {qkv + (size_t)(e->hq_l + e->hkv_l) * e->hd * rowb, e->hkv_l * e->hd, e->H};
    e->named[pf + ".self_attn.o_proj.weight"] = {l.wo, e->H, e->hq_l * e->hd};
    if (!e->moe) {
      e->named[pf + ".mlp.gate_proj.weight"] = {l.wgu, e->I_l, e->H};
      e->named[pf + ".mlp.up_proj.weight"] = {(uint8_t*)l.wgu + (size_t)e->I_l * rowb, e->I_l, e->H};
      e->named[pf + ".mlp.down_proj.weight"] = {l.wdown, e->H, e->I_l};
    } else {
      // names of mixtral.rs:330-333,354-363
      e->named[pf + ".block_sparse_moe.gate.weight"] = {l.wgate, e->E, e->H};
      for (int64_t x = 0; x < e->E; ++x) {
        const std::string ex = pf + ".block_sparse_moe.experts." + std::to_string(x);
        e->named[ex + ".w1.weight"] = {(uint8_t*)l.wgu + (size_t)(x * e->I_l) * rowb, e->I_l, e->H};
        e->named[ex + ".w3.weight"] = {(uint8_t*)l.wgu + (size_t)(e->I_e + x * e->I_l) * rowb, e->I_l, e->H};
        e->named[ex + ".w2.weight"] = {(uint8_t*)l.wdown + (size_t)(x * e->I_l) * es, e->H, e->I_l, e->I_e};
      }
    }
    e->named[pf + ".input_layernorm.weight"] = {l.norm_in, 1, e->H};
    e->named[pf + ".post_attention_layernorm.weight"] = {l.norm_post, 1, e->H};
  }
  return HB_OK;
}

static int alloc_runtime(hb_engine* e, const hb_model_config* cfg) {
  int rc;
  e->max_batch = cfg->max_batch > 0 ? cfg->max_batch : 256;
  const int64_t max_seq = cfg->max_seq_len > 0 ? (int64_t)cfg->max_seq_len : 2048;
  e->max_blocks_per_seq = (max_seq + HB_BLOCK_SIZE - 1) / HB_BLOCK_SIZE;
  e->num_blocks = cfg->num_kv_blocks > 0 ? cfg->num_kv_blocks : e->max_blocks_per_seq * e->max_batch;
  const size_t blk_bytes = (size_t)e->hkv_l * HB_BLOCK_SIZE * e->hd * e->es;
  e->kc.resize(e->L); e->vc.resize(e->L);
  for (int64_t l = 0; l < e->L; ++l) {
    if ((rc = dev_alloc(e, &e->kc[l], blk_bytes * e->num_blocks))) return rc;
    if ((rc = dev_alloc(e, &e->vc[l], blk_bytes * e->num_blocks))) return rc;
    // unwritten slots are read (and masked) by the attention kernel: keep them finite
    HB_CUDA_CHECK(cudaMemset(e->kc[l], 0, blk_bytes * e->num_blocks));
    HB_CUDA_CHECK(cudaMemset(e->vc[l], 0, blk_bytes * e->num_blocks));
  }
  for (int64_t b = 0; b < e->num_blocks; ++b) e->free_blocks.push_back(b);

  const int B = e->max_batch;
  auto align16 = [](size_t v) { return (v + 15) / 16 * 16; };
  e->off_ids = 0;
  e->off_pos = align16(e->off_ids + (size_t)B * 4);
  e->off_ctx = align16(e->off_pos + (size_t)B * 4);
  e->off_slots = align16(e->off_ctx + (size_t)B * 4);
  e->off_tables = align16(e->off_slots + (size_t)B * 8);
  e->inputs_bytes = align16(e->off_tables + (size_t)B * e->max_blocks_per_seq * 4);
  if ((rc = dev_alloc(e, (void**)&e->d_inputs, e->inputs_bytes))) return rc;
  HB_CUDA_CHECK(cudaMallocHost((void**)&e->h_inputs, e->inputs_bytes));
  HB_CUDA_CHECK(cudaMallocHost((void**)&e->h_next, (size_t)B * 4));
  const size_t es = e->es;
  if ((rc = dev_alloc(e, &e->d_h, (size_t)B * e->H * es))) return rc;
  if ((rc = dev_alloc(e, &e->d_x, (size_t)B * e->H * es))) return rc;
  if ((rc = dev_alloc(e, &e->d_qkv, (size_t)B * e->qkv_rows * es))) return rc;
  if ((rc = dev_alloc(e, &e->d_attn, (size_t)B * e->hq_l * e->hd * es))) return rc;
  if ((rc = dev_alloc(e, &e->d_gu, (size_t)B * 2 * e->I_e * es))) return rc;
  if ((rc = dev_alloc(e, &e->d_act, (size_t)B * e->I_e * es))) return rc;
  if (e->moe && (rc = dev_alloc(e, (void**)&e->d_scale, (size_t)B * e->E * 4))) return rc;
  e->rowsq_stride = (int)(((e->H + 127) / 128 + 3) / 4 * 4);
  if ((rc = dev_alloc(e, (void**)&e->d_rowsq, (size_t)B * e->rowsq_stride * 4))) return rc;
  HB_CUDA_CHECK(cudaMemset(e->d_rowsq, 0, (size_t)B * e->rowsq_stride * 4));
  if ((rc = dev_alloc(e, (void**)&e->d_rope_cs, (size_t)B * (e->hd / 2 + 1) * sizeof(float2)))) return rc;
  if ((rc = dev_alloc(e, &e->d_proj, (size_t)B * e->H * es))) return rc;
  if ((rc = dev_alloc(e, (void**)&e->d_logits, (size_t)B * e->V * 4))) return rc;
  if ((rc = dev_alloc(e, (void**)&e->d_next, (size_t)B * 4))) return rc;
  if ((rc = dev_alloc(e, (void**)&e->d_err, 16))) return rc;
  HB_CUDA_CHECK(cudaMemset(e->d_err, 0, 16));
  if ((rc = dev_alloc(e, (void**)&e->d_pairs, (size_t)kPairCap * 2 * sizeof(int64_t)))) return rc;
  std::vector<float> inv(e->hd / 2);
  if ((rc = hb_rope_inv_freq((float)e->theta, (int)e->hd, inv.data()))) return rc;
  if ((rc = dev_alloc(e, (void**)&e->d_inv_freq, inv.size() * 4))) return rc;
  HB_CUDA_CHECK(cudaMemcpy(e->d_inv_freq, inv.data(), inv.size() * 4, cudaMemcpyHostToDevice));
  if ((rc = paged_attention_mma_prepare())) return rc;
  e->attn_ws_bytes = hb_attention_workspace_bytes(B, (int)e->hq_l, (int)e->hd, 16);
  if ((rc = dev_alloc(e, &e->d_attn_ws, e->attn_ws_bytes))) return rc;
  return HB_OK;
}

// ------------------------------------------------------------------ step
static int pick_attn_splits(const hb_engine* e, int B) {
  DeviceInfo di;
  if (device_info(e->device, &di)) return 1;
  // A split costs a partial write and the merge kernel: only worth it when the
  // (sequence, kv head) units alone leave most SMs idle (measured).
  const int64_t units = (int64_t)B * e->hkv_l;
  if (units * 3 >= 2 * (int64_t)di.sm_count) return 1;
  int s = (int)(((int64_t)di.sm_count + units - 1) / units);
  return std::max(1, std::min(s, 16));
}

// Plans (and the captured graph) of a step of B rows; `chunk`: the rows are consecutive
// positions of one sequence (a prefill chunk), which lets the attention kernel share the K/V
// stream among them.
static int ensure_plans(hb_engine* e, int B, bool chunk, StepPlans** out) {
  const int key = B | (chunk ? 1 << 20 : 0);
  auto it = e->plans.find(key);
  const void* window = e->world ? e->world->mc_base : nullptr;
  if (it != e->plans.end()) {
    if (it->second.mm_window == window) { *out = &it->second; return HB_OK; }
    // the world's multicast window was attached, detached or replaced since: the captured graph
    // addresses the old one
    if (it->second.graph) cudaGraphExecDestroy(it->second.graph);
    e->plans.erase(it);
  }
  StepPlans sp;
  sp.mm_window = window;
  sp.attn_splits = pick_attn_splits(e, B);
  if (chunk && B > 1) {
    const int nrep = (int)(e->hq_l / e->hkv_l);
    const bool tc_attn = !getenv("HB_ATTN") &&
                         paged_attention_mma_supported(e->d_qkv, e->qkv_rows, e->kc[0], e->vc[0], nrep, (int)e->hd,
                                                       e->num_blocks, (int)e->hkv_l, e->dtype);
    if (tc_attn && nrep <= 8) {
      sp.q_group = 16 / nrep;   // 16 MMA rows = q_group positions x nrep heads
      sp.attn_splits = 1;
    }
  }
  size_t ws = 0;
  if (e->use_tc) {
    sp.layer.resize(e->L * 4);
    int rc;
    // Single rank: residual add and RMSNorm ride in the GEMM epilogues (HB_DEFER_NORM=0:
    // separate add+norm kernels) when o_proj and down_proj get cluster plans.
    static const bool no_defer = [] { const char* v = getenv("HB_DEFER_NORM"); return v && v[0] == '0'; }();
    sp.defer_norm = e->ws == 1 && !no_defer && e->H % 128 == 0 && !e->moe;  // the router reads normalised x
    if (sp.defer_norm) {
      TcGemmPlan probe_o, probe_d;
      auto& w0 = e->layers[0];
      if ((rc = gemm_tc_plan(&probe_o, e->d_attn, w0.wo, B, e->H, e->hq_l * e->hd, kEpiResidual, false, e->device))) return rc;
      if ((rc = gemm_tc_plan(&probe_d, e->d_act, w0.wdown, B, e->H, e->I_e, kEpiResidual, false, e->device))) return rc;
      sp.defer_norm = probe_o.cluster && probe_d.cluster && probe_o.m_tiles == 1 && probe_d.m_tiles == 1;
    }
    // Several ranks: the row-parallel GEMMs push their partial tiles straight into the
    // reducing ranks' staging (the first hop of the all-reduce rides in the GEMM epilogue)
    // when the batch is large enough for the two-hop exchange (HB_PUSH=0: GEMM, then the
    // exchange kernel reads the partial back; HB_PUSH=1: push at every batch size).
    // A world with a multicast window lets the switch form the sum instead (HB_MULTIMEM=0: not).
    {
      static const bool mm_off = [] { const char* v = getenv("HB_MULTIMEM"); return v && v[0] == '0'; }();
      sp.mm = e->ws > 1 && !mm_off && mm_ar_add_norm_supported(e->world, B, e->H, e->dtype);
      const char* pe = getenv("HB_PUSH");
      const bool off = pe && pe[0] == '0', always = pe && pe[0] == '1';
      const bool two_hop = exchange_two_hops(e->ws, (size_t)B * e->H * e->es);
      sp.push = e->ws > 1 && !sp.mm && !off && (always || two_hop) && push_exchange_supported(e->world, B, e->H, e->dtype);
      if (sp.push) {
        TcGemmPlan probe_o, probe_d;
        auto& w0 = e->layers[0];
        if ((rc = gemm_tc_plan(&probe_o, e->d_attn, w0.wo, B, e->H, e->hq_l * e->hd, kEpiPush, false, e->device))) return rc;
        if ((rc = gemm_tc_plan(&probe_d, e->d_act, w0.wdown, B, e->H, e->I_e, kEpiPush, false, e->device))) return rc;
        const int tiles = (int)(e->H / 128 / e->ws);
        sp.geo_o = {gemm_tc_push_row_block(probe_o), tiles};
        sp.geo_down = {gemm_tc_push_row_block(probe_d), tiles};
        sp.push = sp.geo_o.row_block > 0 && sp.geo_down.row_block > 0;
      }
    }
    const int row_epi = sp.defer_norm ? kEpiResidual : (sp.push ? kEpiPush : kEpiStore);
    for (int64_t l = 0; l < e->L; ++l) {
      auto& w = e->layers[l];
      if ((rc = gemm_tc_plan(&sp.layer[l * 4 + kQkv], e->d_x, w.wqkv, B, e->qkv_rows, e->H, kEpiStore, false, e->device))) return rc;
      if ((rc = gemm_tc_plan(&sp.layer[l * 4 + kO], e->d_attn, w.wo, B, e->H, e->hq_l * e->hd, row_epi, false, e->device))) return rc;
      if (e->fused_swiglu) {
        if ((rc = gemm_tc_plan(&sp.layer[l * 4 + kGateUp], e->d_x, w.wgu, B, 2 * e->I_e, e->H, kEpiSwiGLU, false, e->device))) return rc;
      } else {
        if ((rc = gemm_tc_plan(&sp.layer[l * 4 + kGateUp], e->d_x, w.wgu, B, 2 * e->I_e, e->H, kEpiStore, false, e->device))) return rc;
      }
      if ((rc = gemm_tc_plan(&sp.layer[l * 4 + kDown], e->d_act, w.wdown, B, e->H, e->I_e, row_epi, false, e->device))) return rc;
      for (int k = 0; k < 4; ++k) ws = std::max(ws, sp.layer[l * 4 + k].workspace_bytes());
    }
    if ((rc = gemm_tc_plan(&sp.lm_head, e->d_x, e->lm_head, B, e->V, e->H, kEpiStore, true, e->device))) return rc;
    ws = std::max(ws, sp.lm_head.workspace_bytes());
    // RoPE and the KV write ride in the q|k|v GEMM epilogue when its output tile is one head
    // (HB_ROPE_EPI=0: the separate kernel)
    const char* re_env = getenv("HB_ROPE_EPI");  // read per plan, so that tests can compare both forms
    const bool no_rope_epi = re_env && re_env[0] == '0';
    sp.rope_epi = !no_rope_epi && e->dtype == HB_BF16 && e->hd == 128 && e->L > 0 &&
                  gemm_tc_rope_epilogue_ok(sp.layer[kQkv]);
    if (sp.defer_norm) {
      auto can_scale = [](const TcGemmPlan& pl) { return pl.tma_store && (pl.cluster || pl.splits == 1) && pl.m_tiles == 1; };
      bool ok = can_scale(sp.lm_head);
      for (int64_t l = 0; l < e->L && ok; ++l)
        ok = can_scale(sp.layer[l * 4 + kQkv]) && can_scale(sp.layer[l * 4 + kGateUp]) && e->fused_swiglu;
      if (!ok) {  // re-plan the row-parallel projections with the plain epilogue
        sp.defer_norm = false;
        for (int64_t l = 0; l < e->L; ++l) {
          auto& w = e->layers[l];
          if ((rc = gemm_tc_plan(&sp.layer[l * 4 + kO], e->d_attn, w.wo, B, e->H, e->hq_l * e->hd, kEpiStore, false, e->device))) return rc;
          if ((rc = gemm_tc_plan(&sp.layer[l * 4 + kDown], e->d_act, w.wdown, B, e->H, e->I_e, kEpiStore, false, e->device))) return rc;
        }
      }
    }
  }
  if (ws > e->gemm_ws_bytes) {
    // grows only when a new batch size needs more; never inside a captured step
    void* p = nullptr;
    HB_CUDA_CHECK(cudaMalloc(&p, ws));
    HB_CUDA_CHECK(cudaMemset(p, 0, ws));
    e->allocations.push_back(p);
    e->d_gemm_ws = p;
    e->gemm_ws_bytes = ws;
    // plans made for other batch sizes keep pointing at buffers that stay allocated
    for (auto& kv : e->plans)
      if (kv.second.graph) { cudaGraphExecDestroy(kv.second.graph); kv.second.graph = nullptr; }
  }
  auto ins = e->plans.emplace(key, std::move(sp));
  *out = &ins.first->second;
  return HB_OK;
}

static int run_gemm(hb_engine* e, StepPlans* sp, int64_t l, int kind, void* Y, const void* X,
                    const void* W, int B, int64_t N, int64_t K, bool out_f32, const TcNormLink* link = nullptr) {
  ++e->last_launches;
  if (e->use_tc) {
    const TcGemmPlan& pl = (kind == kLmHead) ? sp->lm_head : sp->layer[l * 4 + kind];
    return gemm_tc_run(pl, e->stream, Y, pl.N, e->d_gemm_ws, e->d_err, link);
  }
  return gemm_simt(e->stream, Y, X, W, B, N, K, e->dtype, out_f32);
}

// kCatGemm is the QKV projection; the other projections have kinds of their own
enum ProfCat { kCatGemm = 0, kCatAttention = 1, kCatRopeKv = 2, kCatNorm = 3, kCatOther = 4, kCatComm = 5,
               kCatGemmO = 6, kCatGemmGateUp = 7, kCatGemmDown = 8, kCatGemmLmHead = 9, kNumCats = 10 };

// While profiling, every call opens a timed segment of kind `cat` on the stream.
static void prof_mark(hb_engine* e, int cat) {
  if (!e->profiling) return;
  if (e->prof_used == e->prof_events.size()) {
    cudaEvent_t ev = nullptr;
    cudaEventCreate(&ev);
    e->prof_events.push_back(ev);
  }
  if (e->prof_capture) cudaEventRecordWithFlags(e->prof_events[e->prof_used++], e->stream, cudaEventRecordExternal);
  else cudaEventRecord(e->prof_events[e->prof_used++], e->stream);
  e->prof_cats.push_back(cat);
}

// h += SUM_ranks d_proj; x = norm(h; norm_w): one kernel over peer memory when the world has
// several ranks (shapes the kernel does not take: all-reduce kernel, then add+norm), add+norm alone otherwise.
static int reduce_add_norm(hb_engine* e, void* x_out, const void* norm_w, int B, bool mm = false,
                           bool gemm_signals = false) {
  int rc;
  cudaStream_t st = e->stream;
  const float eps = (float)e->eps;
  if (e->ws > 1) {
    prof_mark(e, kCatComm);
    if (mm) {
      // the projection left its partial in the world's multicast window: the switch sums it
      if ((rc = world_mm_ar_add_norm(e->world, st, x_out, e->d_h, mm_partial_ptr(e->world), e->d_h, norm_w, B, e->H, eps,
                                     e->dtype, gemm_signals))) return rc;
      ++e->last_launches;
      return HB_OK;
    }
    if (ar_add_norm_supported(e->world, B, e->H, e->dtype)) {
      if ((rc = world_ar_add_norm(e->world, st, x_out, e->d_h, e->d_proj, e->d_h, norm_w, B, e->H, eps, e->dtype,
                                  HB_ALGO_AUTO))) return rc;
      ++e->last_launches;
      return HB_OK;
    }
    if ((rc = world_all_reduce(e->world, st, e->d_proj, (size_t)B * e->H, e->dtype, HB_ALGO_AUTO))) return rc;
    ++e->last_launches;
  }
  prof_mark(e, kCatNorm);
  if ((rc = hb_add_rms_norm(st, x_out, e->d_h, e->d_proj, e->d_h, norm_w, B, e->H, eps, e->dtype))) return rc;
  ++e->last_launches;
  return HB_OK;
}

// Issues every kernel of one decode step on e->stream (captured or direct).
static int issue_step(hb_engine* e, StepPlans* sp, int B) {
  int rc;
  cudaStream_t st = e->stream;
  const uint32_t* d_ids = (const uint32_t*)(e->d_inputs + e->off_ids);
  const int32_t* d_pos = (const int32_t*)(e->d_inputs + e->off_pos);
  const int32_t* d_ctx = (const int32_t*)(e->d_inputs + e->off_ctx);
  const int64_t* d_slots = (const int64_t*)(e->d_inputs + e->off_slots);
  const int32_t* d_tables = (const int32_t*)(e->d_inputs + e->off_tables);
  const float eps = (float)e->eps;
  e->last_launches = 0;

  // h = embed[ids]; x = norm(h; w_in[0])                       llama_tp.rs:508-522
  prof_mark(e, kCatOther);
  if ((rc = hb_embed(st, e->d_h, e->embed, d_ids, B, e->H, e->V, e->dtype))) return rc;
  prof_mark(e, kCatNorm);
  if ((rc = hb_rms_norm(st, e->d_x, e->d_h, e->layers[0].norm_in, B, e->H, eps, e->dtype))) return rc;
  e->last_launches += 2;
  // deferred norm: the GEMM after a row-parallel projection scales its rows (TcNormLink)
  const bool defer = e->use_tc && sp->defer_norm;
  TcNormLink consume;
  consume.rowsq_in = e->d_rowsq;
  consume.rowsq_tiles = (int)(e->H / 128);
  consume.rowsq_stride = e->rowsq_stride;
  consume.n = (float)e->H;
  consume.eps = eps;
  // Rows of one step are different sequences (decode: one new token each) or consecutive
  // positions of one sequence (prefill chunk): at most B tokens at the end of any context are
  // written by this step, everything older in the pool is final: the attention kernel may
  // fetch it before the q|k|v projection has completed (measured 4.70 -> 4.64 ms per step).
  const int attn_fresh = B;
  const bool rope_epi = e->use_tc && sp->rope_epi;
  TcNormLink push_link;
  if (sp->push) {
    push_link.push_peers = e->world->peer;
    push_link.push_ranks = e->ws;
    push_link.push_rank = e->rank;
    push_link.push_spin = e->world->wait_limit;
  }
  // exchange through the switch: the row-parallel GEMMs announce their completion themselves
  // (HB_MM_SIGNAL=0: the exchange kernel does, with an arrival hop of its own)
  static const bool mm_sig_off = [] { const char* v = getenv("HB_MM_SIGNAL"); return v && v[0] == '0'; }();
  const bool mm_sig = sp->mm && e->use_tc && !mm_sig_off;
  TcNormLink mm_link;
  if (mm_sig) mm_gemm_signal(e->world, &mm_link.ready_mc, &mm_link.ready_calls, &mm_link.ready_ctas);
  if (rope_epi) {
    // the step's (cos, sin) table, shared by the q|k|v epilogues of every layer
    prof_mark(e, kCatRopeKv);
    if ((rc = rope_table(st, e->d_rope_cs, d_pos, e->d_inv_freq, B, (int)e->hd, e->dtype))) return rc;
    ++e->last_launches;
  }
  for (int64_t l = 0; l < e->L; ++l) {
    auto& w = e->layers[l];
    // q|k|v = x . Wqkv^T                                      llama_tp.rs:232-234
    prof_mark(e, kCatGemm);
    TcNormLink qkv_link;
    if (defer && l > 0) qkv_link = consume;
    if (rope_epi) {
      // RoPE + KV append in the epilogue                      llama_tp.rs:242-259
      qkv_link.rope_cs = e->d_rope_cs;
      qkv_link.kv_slots = d_slots;
      qkv_link.k_cache = e->kc[l];
      qkv_link.v_cache = e->vc[l];
      qkv_link.n_q_heads = (int)e->hq_l;
      qkv_link.n_kv_heads = (int)e->hkv_l;
      qkv_link.num_blocks = e->num_blocks;
    }
    if ((rc = run_gemm(e, sp, l, kQkv, e->d_qkv, e->d_x, w.wqkv, B, e->qkv_rows, e->H, false,
                       ((defer && l > 0) || rope_epi) ? &qkv_link : nullptr))) return rc;
    // RoPE + KV append                                        llama_tp.rs:242-259
    if (!rope_epi) {
      prof_mark(e, kCatRopeKv);
      if ((rc = rope_kv_write(st, e->d_qkv, e->kc[l], e->vc[l], d_pos, d_slots, e->d_inv_freq, B,
                              (int)e->hq_l, (int)e->hkv_l, (int)e->hd, e->num_blocks, e->dtype))) return rc;
      ++e->last_launches;
    }
    // softmax(q k^T / sqrt d) v over the block table          llama_tp.rs:264-324
    prof_mark(e, kCatAttention);
    if ((rc = paged_attention(st, e->d_attn, e->d_qkv, e->qkv_rows, e->kc[l], e->vc[l], d_tables,
                              d_ctx, B, (int)e->hq_l, (int)e->hkv_l, (int)e->hd,
                              e->max_blocks_per_seq, e->num_blocks, sp->attn_splits, e->d_attn_ws,
                              e->dtype, e->d_err, (int)e->window, attn_fresh, sp->q_group))) return rc;
    e->last_launches += 1 + (sp->attn_splits > 1 ? 1 : 0);
    // o_proj partial, sum over ranks, residual, post-attention norm   llama_tp.rs:327,533-552
    prof_mark(e, kCatGemmO);
    if (sp->push) {
      // the GEMM epilogue pushes each tile to the rank that reduces its column slice; the
      // exchange kernel starts at the wait                      llama_tp.rs:327,533-552
      if ((rc = run_gemm(e, sp, l, kO, nullptr, e->d_attn, w.wo, B, e->H, e->hq_l * e->hd, false, &push_link))) return rc;
      prof_mark(e, kCatComm);
      if ((rc = world_ar_add_norm(e->world, st, e->d_x, e->d_h, nullptr, e->d_h, w.norm_post, B, e->H, eps, e->dtype,
                                  HB_ALGO_TWO_SHOT, &sp->geo_o))) return rc;
      ++e->last_launches;
    } else if (defer) {
      // h += o_proj(attn); x' = h * w_post; row sums for the gate|up GEMM
      TcNormLink produce;
      produce.resid = e->d_h; produce.norm_w = w.norm_post; produce.rowsq_out = e->d_rowsq;
      produce.rowsq_stride = e->rowsq_stride;
      if ((rc = run_gemm(e, sp, l, kO, e->d_x, e->d_attn, w.wo, B, e->H, e->hq_l * e->hd, false, &produce))) return rc;
    } else {
      void* proj = sp->mm ? mm_partial_ptr(e->world) : e->d_proj;
      if ((rc = run_gemm(e, sp, l, kO, proj, e->d_attn, w.wo, B, e->H, e->hq_l * e->hd, false, mm_sig ? &mm_link : nullptr))) return rc;
      if ((rc = reduce_add_norm(e, e->d_x, w.norm_post, B, sp->mm, mm_sig))) return rc;
    }
    // mixture of experts: routing weights of every token       mixtral.rs:371-412
    if (e->moe) {
      prof_mark(e, kCatOther);
      if ((rc = moe_route(st, e->d_scale, e->d_x, w.wgate, B, e->H, (int)e->E, (int)e->topk, e->dtype))) return rc;
      ++e->last_launches;
    }
    // down( silu(gate x) * up x ) partial                     llama_tp.rs:333-339
    prof_mark(e, kCatGemmGateUp);
    bool moe_scaled = false;
    if (e->use_tc && e->fused_swiglu) {
      TcNormLink moe_link;
      const TcGemmPlan& gpl = sp->layer[l * 4 + kGateUp];
      if (e->moe && gpl.tma_store && (gpl.cluster || gpl.splits == 1) && gpl.m_tiles == 1) {
        // the routing weight of (token, expert) multiplies the expert's activations in the
        // epilogue of the gate|up GEMM (expert = output tile / tiles per expert)
        moe_link.post_scale = e->d_scale;
        moe_link.post_groups = (int)e->E;
        moe_link.post_tiles_per_group = (int)(e->I_l / 128);
        moe_scaled = true;
      }
      if ((rc = run_gemm(e, sp, l, kGateUp, e->d_act, e->d_x, w.wgu, B, 2 * e->I_e, e->H, false,
                         defer ? &consume : (moe_scaled ? &moe_link : nullptr)))) return rc;
    } else {
      if ((rc = run_gemm(e, sp, l, kGateUp, e->d_gu, e->d_x, w.wgu, B, 2 * e->I_e, e->H, false))) return rc;
      prof_mark(e, kCatOther);
      if ((rc = hb_silu_mul(st, e->d_act, e->d_gu, B, e->I_e, e->dtype))) return rc;
      ++e->last_launches;
    }
    if (e->moe && !moe_scaled) {
      // every expert ran on every token; the ones a token did not choose get weight 0,
      // the chosen ones their renormalised probability                 mixtral.rs:404-427
      prof_mark(e, kCatOther);
      if ((rc = moe_scale_act(st, e->d_act, e->d_scale, B, e->I_l, (int)e->E, e->dtype))) return rc;
      ++e->last_launches;
    }
    // residual + the next layer's input norm (or the final norm)   llama_tp.rs:566-571,517-522,349-351
    const void* nw = (l + 1 < e->L) ? e->layers[l + 1].norm_in : e->final_norm;
    prof_mark(e, kCatGemmDown);
    if (sp->push) {
      if ((rc = run_gemm(e, sp, l, kDown, nullptr, e->d_act, w.wdown, B, e->H, e->I_e, false, &push_link))) return rc;
      prof_mark(e, kCatComm);
      if ((rc = world_ar_add_norm(e->world, st, e->d_x, e->d_h, nullptr, e->d_h, nw, B, e->H, eps, e->dtype,
                                  HB_ALGO_TWO_SHOT, &sp->geo_down))) return rc;
      ++e->last_launches;
    } else if (defer) {
      TcNormLink produce;
      produce.resid = e->d_h; produce.norm_w = nw; produce.rowsq_out = e->d_rowsq;
      produce.rowsq_stride = e->rowsq_stride;
      if ((rc = run_gemm(e, sp, l, kDown, e->d_x, e->d_act, w.wdown, B, e->H, e->I_e, false, &produce))) return rc;
    } else {
      void* proj = sp->mm ? mm_partial_ptr(e->world) : e->d_proj;
      if ((rc = run_gemm(e, sp, l, kDown, proj, e->d_act, w.wdown, B, e->H, e->I_e, false, mm_sig ? &mm_link : nullptr))) return rc;
      if ((rc = reduce_add_norm(e, e->d_x, nw, B, sp->mm, mm_sig))) return rc;
    }
  }
  // logits = x . lm_head^T (fp32 out), greedy argmax            llama_tp.rs:352-355, sampling/mod.rs:105-107
  prof_mark(e, kCatGemmLmHead);
  if ((rc = run_gemm(e, sp, 0, kLmHead, e->d_logits, e->d_x, e->lm_head, B, e->V, e->H, true,
                     defer ? &consume : nullptr))) return rc;
  prof_mark(e, kCatOther);
  if ((rc = hb_argmax(st, e->d_next, e->d_logits, B, e->V, HB_F32))) return rc;
  ++e->last_launches;
  prof_mark(e, -1);  // closes the last segment
  return HB_OK;
}

static int seq_ensure_block(hb_engine* e, hb_seq* s, int64_t pos) {
  while ((int64_t)s->blocks.size() * HB_BLOCK_SIZE <= pos) {
    if (e->free_blocks.empty())
      return fail(HB_ERR_OOM_BLOCKS, "no free KV blocks (pool of %lld)", (long long)e->num_blocks);
    if ((int64_t)s->blocks.size() >= e->max_blocks_per_seq)
      return fail(HB_ERR_OOM_BLOCKS, "sequence exceeds max_seq_len (%lld tokens)",
                  (long long)(e->max_blocks_per_seq * HB_BLOCK_SIZE));
    s->blocks.push_back(e->free_blocks.front());
    e->free_blocks.pop_front();
  }
  return HB_OK;
}

// One row of a step: token `tok` of sequence `s` at position `pos`.  A decode step has one
// row per sequence; a prefill chunk has consecutive positions of ONE sequence as its rows
// (row i then attends to the keys of rows 0..i, which the same step wrote before its
// attention kernel runs: causal attention over the growing cache, llama_tp.rs:313-316).
struct StepRow {
  const int64_t* blocks;  // the sequence's block table (ids into the KV pool), table[pos / 16]
  size_t n_blocks;
  int64_t pos;
  uint32_t tok;
};

static int run_rows(hb_engine* e, const StepRow* rows, int B, uint32_t* next_tokens, float* logits_out,
                    int logits_row0, bool chunk = false);

static int decode_step(hb_engine* e, hb_seq* const* seqs, int B, const uint32_t* tokens,
                       uint32_t* next_tokens, float* logits_out /* host [B, V] or null */) {
  if (B <= 0 || B > e->max_batch)
    return fail(HB_ERR_INVALID_ARG, "batch %d outside [1, %d]", B, e->max_batch);
  std::vector<StepRow> rows((size_t)B);
  for (int b = 0; b < B; ++b) {
    hb_seq* s = seqs[b];
    if (!s) return fail(HB_ERR_INVALID_ARG, "null sequence at index %d", b);
    for (int j = 0; j < b; ++j)
      if (seqs[j] == s) return fail(HB_ERR_INVALID_ARG, "sequence repeated in one batch");
  }
  int rc;
  for (int b = 0; b < B; ++b)
    if ((rc = seq_ensure_block(e, seqs[b], seqs[b]->len))) return rc;
  for (int b = 0; b < B; ++b) rows[b] = {seqs[b]->blocks.data(), seqs[b]->blocks.size(), seqs[b]->len, tokens[b]};
  rc = run_rows(e, rows.data(), B, next_tokens, logits_out, 0);
  if (rc) return rc;
  for (int b = 0; b < B; ++b) seqs[b]->len += 1;
  return HB_OK;
}

// Prefill of `n` prompt tokens of one sequence in chunks of up to max_batch rows; the
// logits of the last token go to logits_out (host [V]) when it is not null.
static int prefill(hb_engine* e, hb_seq* s, const uint32_t* ids, size_t n, float* logits_out,
                   bool all_positions = false) {
  std::vector<StepRow> rows;
  size_t done = 0;
  while (done < n) {
    const int c = (int)std::min<size_t>(n - done, (size_t)e->max_batch);
    rows.resize((size_t)c);
    int rc;
    if ((rc = seq_ensure_block(e, s, s->len + c - 1))) return rc;
    for (int i = 0; i < c; ++i) rows[i] = {s->blocks.data(), s->blocks.size(), s->len + i, ids[done + i]};
    const bool last = done + (size_t)c == n;
    if (all_positions) rc = run_rows(e, rows.data(), c, nullptr, logits_out + done * (size_t)e->V, 0, true);
    else rc = run_rows(e, rows.data(), c, nullptr, last ? logits_out : nullptr, c - 1, true);
    if (rc) return rc;
    s->len += c;
    done += (size_t)c;
  }
  return HB_OK;
}

static int run_rows(hb_engine* e, const StepRow* rows, int B, uint32_t* next_tokens, float* logits_out,
                    int logits_row0, bool chunk) {
  HB_CUDA_CHECK(cudaSetDevice(e->device));
  int rc;
  uint32_t* h_ids = (uint32_t*)(e->h_inputs + e->off_ids);
  int32_t* h_pos = (int32_t*)(e->h_inputs + e->off_pos);
  int32_t* h_ctx = (int32_t*)(e->h_inputs + e->off_ctx);
  int64_t* h_slots = (int64_t*)(e->h_inputs + e->off_slots);
  int32_t* h_tables = (int32_t*)(e->h_inputs + e->off_tables);
  for (int b = 0; b < B; ++b) {
    const StepRow& r = rows[b];
    const int64_t pos = r.pos;
    // the reference's embedding lookup fails on an id outside the vocabulary
    // (index_select, llama_tp.rs:213-216); so does this
    if ((int64_t)r.tok >= e->V)
      return fail(HB_ERR_INVALID_ARG, "token id %u at row %d is outside the vocabulary of %lld", r.tok, b,
                  (long long)e->V);
    const int64_t need = pos / HB_BLOCK_SIZE + 1;
    if (pos < 0 || (int64_t)r.n_blocks < need || need > e->max_blocks_per_seq)
      return fail(HB_ERR_INVALID_ARG, "row %d: a block table of %zu block(s) does not cover position %lld", b,
                  r.n_blocks, (long long)pos);
    for (int64_t i = 0; i < need; ++i)
      if (r.blocks[i] < 0 || r.blocks[i] >= e->num_blocks)
        return fail(HB_ERR_INVALID_ARG, "row %d: block id %lld outside the pool of %lld", b, (long long)r.blocks[i],
                    (long long)e->num_blocks);
    h_ids[b] = r.tok;
    h_pos[b] = (int32_t)pos;
    h_ctx[b] = (int32_t)(pos + 1);
    h_slots[b] = r.blocks[pos / HB_BLOCK_SIZE] * HB_BLOCK_SIZE + pos % HB_BLOCK_SIZE;
    int32_t* row = h_tables + (size_t)b * e->max_blocks_per_seq;
    for (int64_t i = 0; i < need; ++i) row[i] = (int32_t)r.blocks[i];
  }
  StepPlans* sp = nullptr;
  if ((rc = ensure_plans(e, B, chunk, &sp))) return rc;
  // only the used prefix of each region matters; one copy of the whole block is simplest
  HB_CUDA_CHECK(cudaMemcpyAsync(e->d_inputs, e->h_inputs, e->inputs_bytes, cudaMemcpyHostToDevice, e->stream));
  if (e->use_graph && !e->profiling) {
    if (!sp->graph) {
      cudaGraph_t g = nullptr;
      HB_CUDA_CHECK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
      rc = issue_step(e, sp, B);
      sp->launches = e->last_launches;
      cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
      if (rc) { if (g) cudaGraphDestroy(g); return rc; }
      if (ce != cudaSuccess) return fail(HB_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(ce));
      ce = cudaGraphInstantiate(&sp->graph, g, 0);
      cudaGraphDestroy(g);
      if (ce != cudaSuccess) return fail(HB_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(ce));
    }
    e->last_launches = sp->launches;
    HB_CUDA_CHECK(cudaEventRecord(e->ev0, e->stream));
    HB_CUDA_CHECK(cudaGraphLaunch(sp->graph, e->stream));
    HB_CUDA_CHECK(cudaEventRecord(e->ev1, e->stream));
  } else {
    // Profiling.  With graphs enabled the step is captured once more with an event-record
    // node between the kernels and replayed, so that the per-kind times are those of the
    // kernels inside a graph (a failed capture: kernel by kernel
    // on the stream, which adds the launch gaps).
    const bool eager_only = false;
    bool done = false;
    if (e->profiling && e->use_graph && !eager_only) {
      cudaGraph_t g = nullptr;
      cudaGraphExec_t ge = nullptr;
      if (cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        e->prof_capture = true;
        rc = issue_step(e, sp, B);
        e->prof_capture = false;
        cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
        if (!rc && ce == cudaSuccess && cudaGraphInstantiate(&ge, g, 0) == cudaSuccess) {
          HB_CUDA_CHECK(cudaEventRecord(e->ev0, e->stream));
          ce = cudaGraphLaunch(ge, e->stream);
          HB_CUDA_CHECK(cudaEventRecord(e->ev1, e->stream));
          HB_CUDA_CHECK(cudaStreamSynchronize(e->stream));
          done = ce == cudaSuccess;
        }
        if (ge) cudaGraphExecDestroy(ge);
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();
      }
      if (!done) { e->prof_used = 0; e->prof_cats.clear(); }
    }
    if (!done) {
      HB_CUDA_CHECK(cudaEventRecord(e->ev0, e->stream));
      if ((rc = issue_step(e, sp, B))) return rc;
      HB_CUDA_CHECK(cudaEventRecord(e->ev1, e->stream));
    }
  }
  HB_CUDA_CHECK(cudaMemcpyAsync(e->h_next, e->d_next, (size_t)B * 4, cudaMemcpyDeviceToHost, e->stream));
  if (logits_out)
    HB_CUDA_CHECK(cudaMemcpyAsync(logits_out, e->d_logits + (size_t)logits_row0 * e->V,
                                  (size_t)(B - logits_row0) * e->V * 4, cudaMemcpyDeviceToHost, e->stream));
  int h_err = 0;
  HB_CUDA_CHECK(cudaMemcpyAsync(&h_err, e->d_err, 4, cudaMemcpyDeviceToHost, e->stream));
  HB_CUDA_CHECK(cudaStreamSynchronize(e->stream));
  HB_CUDA_CHECK(cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1));
  if (e->profiling) {
    for (int c = 0; c < kNumCats; ++c) e->prof_ms[c] = 0.f;
    for (size_t i = 0; i + 1 < e->prof_used; ++i) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e->prof_events[i], e->prof_events[i + 1]);
      if (e->prof_cats[i] >= 0 && e->prof_cats[i] < kNumCats) e->prof_ms[e->prof_cats[i]] += ms;
    }
    e->prof_used = 0;
    e->prof_cats.clear();
  }
  if (h_err) {
    cudaMemsetAsync(e->d_err, 0, 4, e->stream);
    return fail(HB_ERR_TIMEOUT, "a bounded device-side wait ran out during the decode step");
  }
  if (e->world && e->ws > 1) {
    const int stw = hb_world_status(e->world);
    if (stw) return fail(stw, "a peer did not arrive in the all-reduce of the decode step");
  }
  for (int b = 0; b < B; ++b)
    if (next_tokens) next_tokens[b] = e->h_next[b];
  return HB_OK;
}

}  // namespace hb

// ------------------------------------------------------------------------- C ABI
extern "C" {

int hb_engine_free(hb_engine* e) {
  if (!e) return HB_OK;
  cudaSetDevice(e->device);
  if (e->stream) cudaStreamSynchronize(e->stream);
  for (auto& kv : e->plans)
    if (kv.second.graph) cudaGraphExecDestroy(kv.second.graph);
  for (void* p : e->allocations) cudaFree(p);
  if (e->h_swap) cudaFreeHost(e->h_swap);
  if (e->h_inputs) cudaFreeHost(e->h_inputs);
  if (e->h_next) cudaFreeHost(e->h_next);
  if (e->ev0) cudaEventDestroy(e->ev0);
  if (e->ev1) cudaEventDestroy(e->ev1);
  if (e->stream) cudaStreamDestroy(e->stream);
  delete e;
  return HB_OK;
}

int hb_engine_create_random(const hb_model_shape* shape, const hb_model_config* cfg,
                            hb_world* world, uint64_t seed, float std, int norm_ones,
                            hb_engine** out) {
  HB_CHECK_ARG(shape && cfg && out, "hb_engine_create_random: null argument");
  std::unique_ptr<hb_engine, int (*)(hb_engine*)> e(new hb_engine, hb_engine_free);
  int rc;
  if ((rc = hb::setup_common(e.get(), cfg, world))) return rc;
  if ((rc = hb::setup_shape(e.get(), *shape))) return rc;
  if ((rc = hb::alloc_weights(e.get()))) return rc;
  hb_engine* g = e.get();
  cudaStream_t st = g->stream;
  const int r = g->rank;
  // tensor ids: 0 embed, 1 lm_head, 2 final norm, 16 + 16*layer + k for layer tensors.
  // Each rank draws its slice of the global tensor: rows for column-parallel weights,
  // columns for row-parallel ones (src/parallel/shard.rs:46-74).
  if ((rc = hb::fill_normal(st, g->embed, g->dtype, g->V, g->H, 0, 0, g->H, seed, 0, std))) return rc;
  if ((rc = hb::fill_normal(st, g->lm_head, g->dtype, g->V, g->H, 0, 0, g->H, seed, 1, std))) return rc;
  auto fill_norm = [&](void* p, uint64_t tid) {
    return norm_ones ? hb::fill_const(st, p, g->dtype, g->H, 1.0f)
                     : hb::fill_normal(st, p, g->dtype, 1, g->H, 0, 0, g->H, seed, tid, std);
  };
  if ((rc = fill_norm(g->final_norm, 2))) return rc;
  const size_t rowb = (size_t)g->H * g->es;
  for (int64_t l = 0; l < g->L; ++l) {
    auto& w = g->layers[l];
    const uint64_t t0 = 16 + 16 * (uint64_t)l;
    const int64_t qr = g->hq_l * g->hd, kr = g->hkv_l * g->hd;
    uint8_t* qkv = (uint8_t*)w.wqkv;
    if ((rc = hb::fill_normal(st, qkv, g->dtype, qr, g->H, r * qr, 0, g->H, seed, t0 + 0, std))) return rc;
    if ((rc = hb::fill_normal(st, qkv + (size_t)qr * rowb, g->dtype, kr, g->H, r * kr, 0, g->H, seed, t0 + 1, std))) return rc;
    if ((rc = hb::fill_normal(st, qkv + (size_t)(qr + kr) * rowb, g->dtype, kr, g->H, r * kr, 0, g->H, seed, t0 + 2, std))) return rc;
    if ((rc = hb::fill_normal(st, w.wo, g->dtype, g->H, qr, 0, r * qr, g->hq * g->hd, seed, t0 + 3, std))) return rc;
    if (!g->moe) {
      if ((rc = hb::fill_normal(st, w.wgu, g->dtype, g->I_l, g->H, r * g->I_l, 0, g->H, seed, t0 + 4, std))) return rc;
      if ((rc = hb::fill_normal(st, (uint8_t*)w.wgu + (size_t)g->I_l * rowb, g->dtype, g->I_l, g->H, r * g->I_l, 0, g->H, seed, t0 + 5, std))) return rc;
      if ((rc = hb::fill_normal(st, w.wdown, g->dtype, g->H, g->I_l, 0, r * g->I_l, g->I, seed, t0 + 6, std))) return rc;
    } else {
      // tensor ids of expert x: 1024 + 4096*layer + 4*x + {0: w1, 1: w3, 2: w2}; router: t0 + 9
      if ((rc = hb::fill_normal(st, w.wgate, g->dtype, g->E, g->H, 0, 0, g->H, seed, t0 + 9, std))) return rc;
      for (int64_t x = 0; x < g->E; ++x) {
        const uint64_t tx = 1024 + 4096 * (uint64_t)l + 4 * (uint64_t)x;
        uint8_t* w1 = (uint8_t*)w.wgu + (size_t)(x * g->I_l) * rowb;
        uint8_t* w3 = (uint8_t*)w.wgu + (size_t)(g->I_e + x * g->I_l) * rowb;
        uint8_t* w2 = (uint8_t*)w.wdown + (size_t)(x * g->I_l) * g->es;
        if ((rc = hb::fill_normal(st, w1, g->dtype, g->I_l, g->H, r * g->I_l, 0, g->H, seed, tx + 0, std))) return rc;
        if ((rc = hb::fill_normal(st, w3, g->dtype, g->I_l, g->H, r * g->I_l, 0, g->H, seed, tx + 1, std))) return rc;
        if ((rc = hb::fill_normal(st, w2, g->dtype, g->H, g->I_l, 0, r * g->I_l, g->I, seed, tx + 2, std, g->I_e))) return rc;
      }
    }
    if ((rc = fill_norm(w.norm_in, t0 + 7))) return rc;
    if ((rc = fill_norm(w.norm_post, t0 + 8))) return rc;
  }
  HB_CUDA_CHECK(cudaStreamSynchronize(st));
  if ((rc = hb::alloc_runtime(g, cfg))) return rc;
  *out = e.release();
  return HB_OK;
}

int hb_engine_load(const hb_model_config* cfg, hb_world* world, hb_engine** out) {
  HB_CHECK_ARG(cfg && out && cfg->model_path, "hb_engine_load: null argument");
  std::unique_ptr<hb_engine, int (*)(hb_engine*)> e(new hb_engine, hb_engine_free);
  int rc;
  if ((rc = hb::setup_common(e.get(), cfg, world))) return rc;
  const std::string dir = cfg->model_path;
  std::string text;
  if ((rc = hb::read_text_file(dir + "/config.json", &text))) return rc;
  hb::Json root;
  std::string err;
  hb::JsonParser jp(text.data(), text.size());
  if (!jp.parse(&root, &err)) return hb::fail(HB_ERR_IO, "config.json: %s", err.c_str());
  const std::string mt = root.string_or("model_type", "llama");
  if (mt != "llama" && mt != "mistral" && mt != "mixtral")
    return hb::fail(HB_ERR_INVALID_ARG, "model_type '%s' is not served by this path (llama, mistral, mixtral)",
                    mt.c_str());
  const bool mixtral = mt == "mixtral";
  hb_model_shape sh;
  memset(&sh, 0, sizeof(sh));
  sh.hidden_size = (int64_t)root.number_or("hidden_size", 0);
  sh.intermediate_size = (int64_t)root.number_or("intermediate_size", 0);
  sh.num_hidden_layers = (int64_t)root.number_or("num_hidden_layers", 0);
  sh.num_attention_heads = (int64_t)root.number_or("num_attention_heads", 0);
  sh.num_key_value_heads = (int64_t)root.number_or("num_key_value_heads", 0);
  sh.vocab_size = (int64_t)root.number_or("vocab_size", 0);
  sh.rms_norm_eps = root.number_or("rms_norm_eps", 1e-5);     // llama_tp.rs:68-70
  sh.rope_theta = root.number_or("rope_theta", mixtral ? 1000000.0 : 10000.0);  // llama_tp.rs:71-73, mixtral.rs:56-58
  if (mixtral) {  // mixtral.rs:40-57
    sh.num_local_experts = (int64_t)root.number_or("num_local_experts", 0);
    sh.num_experts_per_tok = (int64_t)root.number_or("num_experts_per_tok", 0);
    sh.sliding_window = (int64_t)root.number_or("sliding_window", 4096);
    if (sh.num_local_experts < 1 || sh.num_experts_per_tok < 1)
      return hb::fail(HB_ERR_INVALID_ARG, "mixtral config.json needs num_local_experts and num_experts_per_tok");
  }
  if ((rc = hb::setup_shape(e.get(), sh))) return rc;
  if ((rc = hb::alloc_weights(e.get()))) return rc;

  std::vector<std::string> files;
  if ((rc = hb::list_safetensors(dir, &files))) return rc;
  std::vector<std::unique_ptr<hb::SafetensorsFile>> shards;
  std::map<std::string, const hb::StTensor*> all;
  for (auto& f : files) {
    shards.emplace_back(new hb::SafetensorsFile);
    if ((rc = shards.back()->open(f))) return rc;
    for (auto& kv : shards.back()->tensors()) all[kv.first] = &kv.second;
  }
  hb_engine* g = e.get();
  hb::UploadStage scratch;
  auto get = [&](const std::string& name, int64_t rows, int64_t cols, const hb::StTensor** t) -> int {
    auto it = all.find(name);
    if (it == all.end()) return hb::fail(HB_ERR_IO, "Weight not found: %s", name.c_str());  // llama_tp.rs:380-385
    const hb::StTensor* s = it->second;
    if (s->dtype != "F32" && s->dtype != "F16" && s->dtype != "BF16")
      return hb::fail(HB_ERR_UNSUPPORTED_DTYPE, "%s has dtype %s", name.c_str(), s->dtype.c_str());
    // the shape itself, not only the element count: a transposed matrix must not be sharded
    const bool shape_ok = rows == 1 ? ((s->shape.size() == 1 && s->shape[0] == cols) ||
                                       (s->shape.size() == 2 && s->shape[0] == 1 && s->shape[1] == cols))
                                    : (s->shape.size() == 2 && s->shape[0] == rows && s->shape[1] == cols);
    if (!shape_ok)
      return hb::fail(HB_ERR_IO, "%s has %lld elements in a shape other than the expected [%lld, %lld]", name.c_str(),
                      (long long)s->numel(), (long long)rows, (long long)cols);
    const size_t src_es = s->dtype == "F32" ? 4 : 2;
    if (s->nbytes != (size_t)(rows * cols) * src_es)
      return hb::fail(HB_ERR_IO, "%s holds %zu bytes, [%lld, %lld] of %s needs %zu", name.c_str(), s->nbytes,
                      (long long)rows, (long long)cols, s->dtype.c_str(), (size_t)(rows * cols) * src_es);
    *t = s;
    return HB_OK;
  };
  const int r = g->rank;
  const hb::StTensor* t = nullptr;
  if ((rc = get("model.embed_tokens.weight", g->V, g->H, &t))) return rc;
  if ((rc = hb::upload_slice(g, g->embed, *t, g->H, 0, g->V, 0, g->H, &scratch))) return rc;
  if ((rc = get("lm_head.weight", g->V, g->H, &t))) return rc;  // no tied-embedding fallback (llama_tp.rs:488)
  if ((rc = hb::upload_slice(g, g->lm_head, *t, g->H, 0, g->V, 0, g->H, &scratch))) return rc;
  if ((rc = get("model.norm.weight", 1, g->H, &t))) return rc;
  if ((rc = hb::upload_slice(g, g->final_norm, *t, g->H, 0, 1, 0, g->H, &scratch))) return rc;
  const size_t rowb = (size_t)g->H * g->es;
  for (int64_t l = 0; l < g->L; ++l) {
    const std::string pf = "model.layers." + std::to_string(l);
    auto& w = g->layers[l];
    const int64_t qr = g->hq_l * g->hd, kr = g->hkv_l * g->hd, qd = g->hq * g->hd;
    uint8_t* qkv = (uint8_t*)w.wqkv;
    if ((rc = get(pf + ".self_attn.q_proj.weight", qd, g->H, &t))) return rc;
    if ((rc = hb::upload_slice(g, qkv, *t, g->H, r * qr, qr, 0, g->H, &scratch))) return rc;
    if ((rc = get(pf + ".self_attn.k_proj.weight", g->hkv * g->hd, g->H, &t))) return rc;
    if ((rc = hb::upload_slice(g, qkv + (size_t)qr * rowb, *t, g->H, r * kr, kr, 0, g->H, &scratch))) return rc;
    if ((rc = get(pf + ".self_attn.v_proj.weight", g->hkv * g->hd, g->H, &t))) return rc;
    if ((rc = hb::upload_slice(g, qkv + (size_t)(qr + kr) * rowb, *t, g->H, r * kr, kr, 0, g->H, &scratch))) return rc;
    if ((rc = get(pf + ".self_attn.o_proj.weight", g->H, qd, &t))) return rc;
    if ((rc = hb::upload_slice(g, w.wo, *t, qd, 0, g->H, r * qr, qr, &scratch))) return rc;
    if (!g->moe) {
      if ((rc = get(pf + ".mlp.gate_proj.weight", g->I, g->H, &t))) return rc;
      if ((rc = hb::upload_slice(g, w.wgu, *t, g->H, r * g->I_l, g->I_l, 0, g->H, &scratch))) return rc;
      if ((rc = get(pf + ".mlp.up_proj.weight", g->I, g->H, &t))) return rc;
      if ((rc = hb::upload_slice(g, (uint8_t*)w.wgu + (size_t)g->I_l * rowb, *t, g->H, r * g->I_l, g->I_l, 0, g->H, &scratch))) return rc;
      if ((rc = get(pf + ".mlp.down_proj.weight", g->H, g->I, &t))) return rc;
      if ((rc = hb::upload_slice(g, w.wdown, *t, g->I, 0, g->H, r * g->I_l, g->I_l, &scratch))) return rc;
    } else {
      // mixtral.rs:330-333,354-363: w1 (gate) and w3 (up) column-parallel, w2 (down)
      // row-parallel over the expert's intermediate size; the router is replicated
      if ((rc = get(pf + ".block_sparse_moe.gate.weight", g->E, g->H, &t))) return rc;
      if ((rc = hb::upload_slice(g, w.wgate, *t, g->H, 0, g->E, 0, g->H, &scratch))) return rc;
      for (int64_t x = 0; x < g->E; ++x) {
        const std::string ex = pf + ".block_sparse_moe.experts." + std::to_string(x);
        uint8_t* w1 = (uint8_t*)w.wgu + (size_t)(x * g->I_l) * rowb;
        uint8_t* w3 = (uint8_t*)w.wgu + (size_t)(g->I_e + x * g->I_l) * rowb;
        uint8_t* w2 = (uint8_t*)w.wdown + (size_t)(x * g->I_l) * g->es;
        if ((rc = get(ex + ".w1.weight", g->I, g->H, &t))) return rc;
        if ((rc = hb::upload_slice(g, w1, *t, g->H, r * g->I_l, g->I_l, 0, g->H, &scratch))) return rc;
        if ((rc = get(ex + ".w3.weight", g->I, g->H, &t))) return rc;
        if ((rc = hb::upload_slice(g, w3, *t, g->H, r * g->I_l, g->I_l, 0, g->H, &scratch))) return rc;
        if ((rc = get(ex + ".w2.weight", g->H, g->I, &t))) return rc;
        if ((rc = hb::upload_slice(g, w2, *t, g->I, 0, g->H, r * g->I_l, g->I_l, &scratch, g->I_e))) return rc;
      }
    }
    if ((rc = get(pf + ".input_layernorm.weight", 1, g->H, &t))) return rc;
    if ((rc = hb::upload_slice(g, w.norm_in, *t, g->H, 0, 1, 0, g->H, &scratch))) return rc;
    if ((rc = get(pf + ".post_attention_layernorm.weight", 1, g->H, &t))) return rc;
    if ((rc = hb::upload_slice(g, w.norm_post, *t, g->H, 0, 1, 0, g->H, &scratch))) return rc;
  }
  HB_CUDA_CHECK(cudaStreamSynchronize(g->stream));  // the mapped files are closed when this function returns
  if ((rc = hb::alloc_runtime(g, cfg))) return rc;
  *out = e.release();
  return HB_OK;
}

int64_t hb_engine_num_layers(const hb_engine* e) { return e ? e->L : -1; }
int64_t hb_engine_vocab_size(const hb_engine* e) { return e ? e->V : -1; }
int64_t hb_engine_hidden_size(const hb_engine* e) { return e ? e->H : -1; }
int64_t hb_engine_param_count(const hb_engine* e) {
  if (!e) return -1;
  // Engine::param_count (src/engine/loader.rs:323-329)
  const int64_t attn = 4 * e->H * e->H, ffn = 3 * e->H * e->I;
  return e->V * e->H + e->L * (attn + ffn) + e->V * e->H;
}
int64_t hb_engine_num_free_blocks(const hb_engine* e) { return e ? (int64_t)e->free_blocks.size() : -1; }
void* hb_engine_stream(hb_engine* e) { return e ? (void*)e->stream : nullptr; }
float hb_engine_last_step_ms(hb_engine* e) { return e ? e->last_ms : -1.f; }
int64_t hb_engine_last_step_launches(const hb_engine* e) { return e ? e->last_launches : -1; }

double hb_engine_step_bytes(const hb_engine* e, const int32_t* ctx_lens, int64_t n_seqs) {
  if (!e) return -1.0;
  const double es = (double)e->es;
  double w = 0.0;
  w += (double)e->L * ((double)e->qkv_rows * e->H + (double)e->H * e->hq_l * e->hd +
                       3.0 * (double)e->I_e * e->H + (e->moe ? (double)e->E * e->H : 0.0) + 2.0 * e->H) * es;
  w += ((double)e->V * e->H + e->H) * es;    // lm_head + final norm
  w += (double)n_seqs * e->H * es;            // embedding rows
  double kv = 0.0;
  for (int64_t i = 0; i < n_seqs; ++i)
    kv += (double)(ctx_lens ? ctx_lens[i] : 0) * e->L * 2.0 * e->hkv_l * e->hd * es;  // read
  kv += (double)n_seqs * e->L * 2.0 * e->hkv_l * e->hd * es;                           // write
  return w + kv;
}

int64_t hb_engine_get_tensor(hb_engine* e, const char* name, float* out, int64_t cap) {
  if (!e || !name) return HB_ERR_INVALID_ARG;
  auto it = e->named.find(name);
  if (it == e->named.end()) return hb::fail(HB_ERR_INVALID_ARG, "no tensor named %s", name);
  const int64_t n = it->second.rows * it->second.cols;
  if (!out) return n;
  if (cap < n) return hb::fail(HB_ERR_INVALID_ARG, "buffer of %lld floats too small for %lld", (long long)cap, (long long)n);
  cudaSetDevice(e->device);
  float* tmp = nullptr;
  if (cudaMalloc((void**)&tmp, (size_t)n * 4) != cudaSuccess) return hb::fail(HB_ERR_CUDA, "cudaMalloc failed");
  int rc = hb::to_f32(e->stream, tmp, it->second.ptr, e->dtype, n, it->second.cols, it->second.ld);
  if (!rc && cudaMemcpyAsync(out, tmp, (size_t)n * 4, cudaMemcpyDeviceToHost, e->stream) != cudaSuccess) rc = HB_ERR_CUDA;
  cudaStreamSynchronize(e->stream);
  cudaFree(tmp);
  return rc ? rc : n;
}

int hb_seq_create(hb_engine* e, hb_seq** out) {
  HB_CHECK_ARG(e && out, "hb_seq_create: null argument");
  hb_seq* s = new hb_seq;
  s->id = e->next_seq_id++;
  *out = s;
  return HB_OK;
}

int hb_seq_free(hb_engine* e, hb_seq* s) {
  if (!s) return HB_OK;
  HB_CHECK_ARG(e, "hb_seq_free: null engine");
  for (int64_t b : s->blocks) e->free_blocks.push_back(b);
  delete s;
  return HB_OK;
}

int64_t hb_seq_len(const hb_seq* s) { return s ? s->len : -1; }

int hb_seq_truncate(hb_engine* e, hb_seq* s, int64_t new_len) {
  HB_CHECK_ARG(e && s, "hb_seq_truncate: null argument");
  HB_CHECK_ARG(new_len >= 0 && new_len <= s->len, "hb_seq_truncate: length %lld outside [0, %lld]", (long long)new_len,
               (long long)s->len);
  s->len = new_len;
  // blocks that hold no token any more go back to the free list (FIFO, as freed blocks do)
  const size_t keep = (size_t)((new_len + HB_BLOCK_SIZE - 1) / HB_BLOCK_SIZE);
  while (s->blocks.size() > keep) {
    e->free_blocks.push_back(s->blocks.back());
    s->blocks.pop_back();
  }
  return HB_OK;
}

int hb_forward_all_positions(hb_engine* e, hb_seq* s, const uint32_t* ids, size_t n, size_t seq_pos,
                             float* logits_out) {
  if (n == 0) return hb::fail(HB_ERR_EMPTY, "hb_forward_all_positions: token list is empty");
  HB_CHECK_ARG(e && s && ids && logits_out, "hb_forward_all_positions: null argument");
  if ((int64_t)seq_pos != s->len)
    return hb::fail(HB_ERR_INVALID_ARG, "hb_forward_all_positions: seq_pos %zu but the sequence holds %lld tokens",
                    seq_pos, (long long)s->len);
  return hb::prefill(e, s, ids, n, logits_out, true);
}

int64_t hb_seq_block_table(const hb_seq* s, int64_t* out, int64_t cap) {
  if (!s) return HB_ERR_INVALID_ARG;
  for (size_t i = 0; i < s->blocks.size() && (int64_t)i < cap && out; ++i) out[i] = s->blocks[i];
  return (int64_t)s->blocks.size();
}

int hb_decode_batch(hb_engine* e, hb_seq* const* seqs, size_t B, const uint32_t* last_tokens,
                    uint32_t* next_tokens, float* logits_opt) {
  HB_CHECK_ARG(e && seqs && last_tokens, "hb_decode_batch: null argument");
  return hb::decode_step(e, seqs, (int)B, last_tokens, next_tokens, logits_opt);
}

// ---- the same step driven by a scheduler's own block tables (src/scheduler/mod.rs:40-61,
// 203-208 emits them, with copy-on-write pairs and swap lists; src/worker/mod.rs:250-305
// never consumes them)
int hb_kv_copy_blocks(hb_engine* e, const int64_t* pairs, size_t n_pairs) {
  HB_CHECK_ARG(e && (pairs || n_pairs == 0), "hb_kv_copy_blocks: null argument");
  HB_CUDA_CHECK(cudaSetDevice(e->device));
  const int64_t block_bytes = e->hkv_l * HB_BLOCK_SIZE * e->hd * (int64_t)e->es;
  for (size_t i = 0; i < 2 * n_pairs; ++i)
    if (pairs[i] < 0 || pairs[i] >= e->num_blocks)
      return hb::fail(HB_ERR_INVALID_ARG, "hb_kv_copy_blocks: block id %lld outside the pool of %lld",
                      (long long)pairs[i], (long long)e->num_blocks);
  for (size_t done = 0; done < n_pairs; done += hb::kPairCap) {
    const size_t n = std::min<size_t>(hb::kPairCap, n_pairs - done);
    HB_CUDA_CHECK(cudaMemcpyAsync(e->d_pairs, pairs + 2 * done, n * 2 * sizeof(int64_t), cudaMemcpyHostToDevice, e->stream));
    for (int64_t l = 0; l < e->L; ++l) {
      int rc = hb::kv_copy_blocks(e->stream, e->kc[l], e->vc[l], e->d_pairs, (int64_t)n, block_bytes, e->num_blocks);
      if (rc) return rc;
    }
    HB_CUDA_CHECK(cudaStreamSynchronize(e->stream));  // `pairs` and d_pairs may be reused
  }
  return HB_OK;
}

int hb_engine_reserve_cpu_blocks(hb_engine* e, int64_t n_blocks) {
  HB_CHECK_ARG(e && n_blocks >= 0, "hb_engine_reserve_cpu_blocks: bad argument");
  HB_CUDA_CHECK(cudaSetDevice(e->device));
  if (e->h_swap) { cudaFreeHost(e->h_swap); e->h_swap = nullptr; e->cpu_blocks = 0; }
  if (n_blocks == 0) return HB_OK;
  const size_t block_bytes = (size_t)e->hkv_l * HB_BLOCK_SIZE * e->hd * e->es;
  HB_CUDA_CHECK(cudaMallocHost((void**)&e->h_swap, (size_t)n_blocks * e->L * 2 * block_bytes));
  e->cpu_blocks = n_blocks;
  return HB_OK;
}

int hb_kv_swap_blocks(hb_engine* e, const int64_t* pairs, size_t n_pairs, int to_cpu) {
  HB_CHECK_ARG(e && (pairs || n_pairs == 0), "hb_kv_swap_blocks: null argument");
  HB_CUDA_CHECK(cudaSetDevice(e->device));
  const size_t block_bytes = (size_t)e->hkv_l * HB_BLOCK_SIZE * e->hd * e->es;
  for (size_t i = 0; i < n_pairs; ++i) {
    // swap_out pairs are (gpu, cpu), swap_in pairs (cpu, gpu): block_manager.rs:359-406
    const int64_t g = to_cpu ? pairs[2 * i] : pairs[2 * i + 1], c = to_cpu ? pairs[2 * i + 1] : pairs[2 * i];
    if (g < 0 || g >= e->num_blocks || c < 0 || c >= e->cpu_blocks)
      return hb::fail(HB_ERR_INVALID_ARG, "hb_kv_swap_blocks: pair %zu (gpu %lld, cpu %lld) outside the pools (%lld, %lld)",
                      i, (long long)g, (long long)c, (long long)e->num_blocks, (long long)e->cpu_blocks);
  }
  for (size_t i = 0; i < n_pairs; ++i) {
    const int64_t g = to_cpu ? pairs[2 * i] : pairs[2 * i + 1], c = to_cpu ? pairs[2 * i + 1] : pairs[2 * i];
    for (int64_t l = 0; l < e->L; ++l)
      for (int kv = 0; kv < 2; ++kv) {
        uint8_t* dev = (uint8_t*)(kv ? e->vc[l] : e->kc[l]) + (size_t)g * block_bytes;
        uint8_t* host = e->h_swap + (((size_t)c * e->L + l) * 2 + kv) * block_bytes;
        if (to_cpu) HB_CUDA_CHECK(cudaMemcpyAsync(host, dev, block_bytes, cudaMemcpyDeviceToHost, e->stream));
        else HB_CUDA_CHECK(cudaMemcpyAsync(dev, host, block_bytes, cudaMemcpyHostToDevice, e->stream));
      }
  }
  HB_CUDA_CHECK(cudaStreamSynchronize(e->stream));
  return HB_OK;
}

int hb_decode_batch_tables(hb_engine* e, size_t B, const uint32_t* last_tokens, const int64_t* positions,
                           const int64_t* block_tables, size_t table_stride, const int64_t* copy_pairs,
                           size_t n_copies, uint32_t* next_tokens, float* logits_opt) {
  HB_CHECK_ARG(e && last_tokens && positions && block_tables, "hb_decode_batch_tables: null argument");
  if (B == 0 || (int)B > e->max_batch)
    return hb::fail(HB_ERR_INVALID_ARG, "batch %zu outside [1, %d]", B, e->max_batch);
  int rc;
  // blocks_to_copy first: a sequence that shared its last block writes into its own copy
  if (n_copies && (rc = hb_kv_copy_blocks(e, copy_pairs, n_copies))) return rc;
  std::vector<hb::StepRow> rows(B);
  for (size_t b = 0; b < B; ++b) {
    if (positions[b] < 0) return hb::fail(HB_ERR_INVALID_ARG, "row %zu: negative position", b);
    const size_t covered = std::min<size_t>(table_stride, (size_t)(positions[b] / HB_BLOCK_SIZE + 1));
    rows[b] = {block_tables + b * table_stride, covered, positions[b], last_tokens[b]};
  }
  // two rows of one decode step are two sequences: they never write the same KV slot
  for (size_t b = 0; b < B; ++b) {
    if (rows[b].n_blocks * HB_BLOCK_SIZE <= (size_t)rows[b].pos) continue;  // reported by run_rows
    const int64_t slot = rows[b].blocks[rows[b].pos / HB_BLOCK_SIZE] * HB_BLOCK_SIZE + rows[b].pos % HB_BLOCK_SIZE;
    for (size_t j = 0; j < b; ++j) {
      if (rows[j].n_blocks * HB_BLOCK_SIZE <= (size_t)rows[j].pos) continue;
      if (rows[j].blocks[rows[j].pos / HB_BLOCK_SIZE] * HB_BLOCK_SIZE + rows[j].pos % HB_BLOCK_SIZE == slot)
        return hb::fail(HB_ERR_INVALID_ARG, "rows %zu and %zu write the same KV slot %lld", j, b, (long long)slot);
    }
  }
  return hb::run_rows(e, rows.data(), (int)B, next_tokens, logits_opt, 0);
}

int hb_forward_tables(hb_engine* e, const uint32_t* ids, size_t n, size_t seq_pos, const int64_t* block_table,
                      size_t table_len, float* logits_out) {
  if (n == 0) return hb::fail(HB_ERR_EMPTY, "hb_forward_tables: token list is empty");
  HB_CHECK_ARG(e && ids && block_table && logits_out, "hb_forward_tables: null argument");
  // chunks of consecutive positions, as hb_forward; positions below seq_pos must already hold
  // this sequence's K/V in the table's blocks (a prefix-cache hit: block_manager.rs:213-234)
  std::vector<hb::StepRow> rows;
  size_t done = 0;
  while (done < n) {
    const int c = (int)std::min<size_t>(n - done, (size_t)e->max_batch);
    rows.resize((size_t)c);
    for (int i = 0; i < c; ++i) rows[i] = {block_table, table_len, (int64_t)(seq_pos + done) + i, ids[done + i]};
    const bool last = done + (size_t)c == n;
    int rc = hb::run_rows(e, rows.data(), c, nullptr, last ? logits_out : nullptr, c - 1, true);
    if (rc) return rc;
    done += (size_t)c;
  }
  return HB_OK;
}

int hb_engine_profile_step(hb_engine* e, hb_seq* const* seqs, size_t B, const uint32_t* last_tokens,
                           uint32_t* next_tokens, float* ms_by_kind) {
  HB_CHECK_ARG(e && seqs && last_tokens && ms_by_kind, "hb_engine_profile_step: null argument");
  e->profiling = true;
  int rc = hb::decode_step(e, seqs, (int)B, last_tokens, next_tokens, nullptr);
  e->profiling = false;
  if (rc) return rc;
  for (int c = 0; c < HB_PROFILE_KINDS; ++c) ms_by_kind[c] = e->prof_ms[c];
  return HB_OK;
}

double hb_engine_gemm_bytes(const hb_engine* e, int64_t B) {
  if (!e) return -1.0;
  const double es = (double)e->es, b = (double)B;
  const double qkv = (double)e->qkv_rows, o_in = (double)e->hq_l * e->hd, H = (double)e->H,
               Il = (double)e->I_e, V = (double)e->V;
  double per_layer = (qkv * H + b * H + b * qkv) * es        // q|k|v projection
                     + (H * o_in + b * o_in + b * H) * es    // o_proj
                     + (2 * Il * H + b * H + b * Il) * es    // gate|up with the SwiGLU epilogue
                     + (H * Il + b * Il + b * H) * es;       // down_proj
  return (double)e->L * per_layer + (V * H + b * H) * es + b * V * 4.0;  // + lm_head, fp32 logits
}

int hb_forward(hb_engine* e, hb_seq* s, const uint32_t* ids, size_t n, size_t seq_pos,
               float* logits_out) {
  if (n == 0) return hb::fail(HB_ERR_EMPTY, "hb_forward: token list is empty");
  HB_CHECK_ARG(e && s && ids && logits_out, "hb_forward: null argument");
  if ((int64_t)seq_pos != s->len)
    return hb::fail(HB_ERR_INVALID_ARG, "hb_forward: seq_pos %zu but the sequence holds %lld tokens",
                    seq_pos, (long long)s->len);
  // Prefill runs through the decode kernels in chunks whose rows are consecutive positions
  // of this sequence: causal attention over the growing cache equals the masked prefill of
  // llama_tp.rs:313-316.
  {
    int rc = hb::prefill(e, s, ids, n, logits_out);
    if (rc) return rc;
  }
  return HB_OK;
}

}  // extern "C"
