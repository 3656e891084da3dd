// On-device sampling: penalties -> temperature -> softmax -> top-p nucleus -> renormalise ->
// seeded draw, the pipeline of src/sampling/mod.rs:30-113 (apply_penalties,
// src/sampling/penalty.rs:28-52; apply_temperature / softmax_inplace / nucleus_filter /
// renormalize, src/sampling/nucleus.rs:7-62), for a whole batch of logit rows at once.
// The reference copies every [vocab] logit row to the host and sorts it there; here the
// probabilities never leave the device: one CTA per row, the row streamed from L2, and
// the nucleus found as a probability threshold by bisection instead of a sort.
//
// A row is read a few dozen times (513 KB at the Llama-3 vocabulary: L2-resident), so the
// kernels are latency-, not HBM-bound; all arithmetic is fp32 as in the reference.
#include <cfloat>
#include <climits>

#include "common.h"

namespace hb {

constexpr int kSampleThreads = 1024;

struct SampleParams {
  const float* logits;     // [n, vocab]
  const uint32_t* counts;  // [n, vocab] tokens seen so far per row, or null
  float* probs;            // [n, vocab] out
  uint32_t* tokens;        // [n] out, or null
  const uint64_t* seeds;   // [n] (tokens != null)
  int64_t vocab;
  float temperature, top_p, presence, frequency;
};

__device__ __forceinline__ float block_max(float v, float* smem) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  float t = lane < nw ? smem[lane] : -FLT_MAX;
  return warp_max(t);
}

// splitmix64 of the seed, top 24 bits as a uniform number in [0, 1)
__device__ __forceinline__ float uniform_from_seed(uint64_t seed) {
  uint64_t z = seed + 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const SampleParams p) {
  __shared__ float s_red[33];
  __shared__ unsigned long long s_arg;
  __shared__ int s_found;
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.x, V = p.vocab;
  const float* x = p.logits + row * V;
  const uint32_t* cnt = p.counts ? p.counts + row * V : nullptr;
  float* pr = p.probs + row * V;
  const bool penal = cnt && (fabsf(p.presence) >= 1e-6f || fabsf(p.frequency) >= 1e-6f);
  float total_f = 1.f;
  if (penal) {
    // total tokens seen (exact in fp32 below 2^24, as the reference's u32 sum cast to f32)
    float t = 0.f;
    for (int64_t i = tid; i < V; i += kSampleThreads) t += (float)cnt[i];
    total_f = fmaxf(block_sum(t, s_red), 1.f);
  }
  auto logit = [&](int64_t i) {
    float v = x[i];
    if (penal) {
      const uint32_t c = cnt[i];
      if (c) { v -= p.presence; v -= p.frequency * ((float)c / total_f); }
    }
    return v;
  };
  const bool greedy = p.temperature < 1e-6f;
  const float inv_t = greedy ? 1.f : 1.0f / p.temperature;
  // pass 1: maximum (and, for greedy, the first index that attains it)
  float mx = -FLT_MAX;
  int64_t arg = 0;
  for (int64_t i = tid; i < V; i += kSampleThreads) {
    const float v = logit(i) * inv_t;
    if (v > mx) { mx = v; arg = i; }
  }
  const float gmax = block_max(mx, s_red);
  if (greedy) {
    // delta distribution on the first maximum (logits_to_probs, mod.rs:79-88)
    if (tid == 0) s_arg = ~0ull;
    __syncthreads();
    if (mx == gmax) atomicMin(&s_arg, (unsigned long long)arg);
    __syncthreads();
    const int64_t best = (int64_t)s_arg;
    for (int64_t i = tid; i < V; i += kSampleThreads) pr[i] = i == best ? 1.f : 0.f;
    if (p.tokens && tid == 0) p.tokens[row] = (uint32_t)best;
    return;
  }
  // pass 2: sum of exp, pass 3: probabilities
  float s = 0.f;
  for (int64_t i = tid; i < V; i += kSampleThreads) s += __expf(logit(i) * inv_t - gmax);
  const float inv_sum = 1.0f / block_sum(s, s_red);
  float pmax = 0.f;
  for (int64_t i = tid; i < V; i += kSampleThreads) {
    const float q = __expf(logit(i) * inv_t - gmax) * inv_sum;
    pr[i] = q;
    pmax = fmaxf(pmax, q);
  }
  __syncthreads();
  float kept_mass = 1.f, thr = 0.f;
  if (p.top_p < 1.0f - 1e-6f) {
    // nucleus = the tokens of probability >= thr, where thr is the probability of the token
    // at which the descending cumulative mass first reaches top_p: the largest thr whose
    // mass is still >= top_p, found by bisection (mass is a step function of thr)
    float lo = 0.f, hi = block_max(pmax, s_red);
    for (int it = 0; it < 40 && hi - lo > 1e-12f; ++it) {
      const float mid = 0.5f * (lo + hi);
      float m = 0.f;
      for (int64_t i = tid; i < V; i += kSampleThreads) {
        const float q = pr[i];
        if (q >= mid) m += q;
      }
      m = block_sum(m, s_red);
      if (m >= p.top_p) lo = mid; else hi = mid;
    }
    // snap to an actual probability: the smallest kept one
    float mn = FLT_MAX, m = 0.f;
    for (int64_t i = tid; i < V; i += kSampleThreads) {
      const float q = pr[i];
      if (q >= lo) { mn = fminf(mn, q); m += q; }
    }
    thr = -block_max(-mn, s_red);
    kept_mass = block_sum(m, s_red);
    const float inv = kept_mass > 0.f ? 1.0f / kept_mass : 0.f;
    for (int64_t i = tid; i < V; i += kSampleThreads) {
      const float q = pr[i];
      pr[i] = q >= thr ? q * inv : 0.f;
    }
    __syncthreads();
  }
  if (!p.tokens) return;
  // draw: first index whose inclusive cumulative probability exceeds u * total, in index order
  float tot = 0.f;
  for (int64_t i = tid; i < V; i += kSampleThreads) tot += pr[i];
  tot = block_sum(tot, s_red);
  const float target = uniform_from_seed(p.seeds[row]) * tot;
  if (tid == 0) s_found = INT_MAX;
  __syncthreads();
  float running = 0.f;
  for (int64_t base = 0; base < V; base += kSampleThreads) {
    const int64_t i = base + tid;
    const float q = i < V ? pr[i] : 0.f;
    // inclusive scan of the chunk: warp scan, then the warp totals
    float incl = q;
    const int lane = tid & 31, wid = tid >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) s_red[wid] = incl;
    __syncthreads();
    float warp_off = 0.f;
    for (int w = 0; w < wid; ++w) warp_off += s_red[w];
    float chunk_total = 0.f;
    for (int w = 0; w < kSampleThreads / 32; ++w) chunk_total += s_red[w];
    const float c_incl = running + warp_off + incl;
    if (i < V && q > 0.f && c_incl > target) atomicMin(&s_found, (int)i);  // the first such index wins
    __syncthreads();
    if (s_found != INT_MAX) break;
    running += chunk_total;
  }
  __syncthreads();
  if (tid == 0) {
    int64_t pick = s_found;
    if (s_found == INT_MAX) {
      // rounding left the target at or past the total: the last token with mass
      pick = 0;
      for (int64_t i = V - 1; i >= 0; --i)
        if (pr[i] > 0.f) { pick = i; break; }
    }
    p.tokens[row] = (uint32_t)pick;
  }
}

static int launch_sample(cudaStream_t st, float* probs, uint32_t* tokens, const float* logits, const uint32_t* counts,
                         const uint64_t* seeds, int64_t n, int64_t vocab, float temperature, float top_p,
                         float presence, float frequency) {
  if (n == 0) return HB_OK;
  SampleParams p;
  p.logits = logits; p.counts = counts; p.probs = probs; p.tokens = tokens; p.seeds = seeds;
  p.vocab = vocab; p.temperature = temperature; p.top_p = top_p; p.presence = presence; p.frequency = frequency;
  sample_kernel<<<(unsigned)n, kSampleThreads, 0, st>>>(p);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

}  // namespace hb

extern "C" {

int hb_logits_to_probs(void* stream, float* probs, const float* logits, const uint32_t* token_counts, int64_t n,
                       int64_t vocab, float temperature, float top_p, float presence_penalty,
                       float frequency_penalty) {
  HB_CHECK_ARG(probs && logits, "hb_logits_to_probs: null pointer");
  HB_CHECK_ARG(n >= 0 && vocab > 0 && vocab < (1ll << 31), "hb_logits_to_probs: bad shape");
  HB_CHECK_ARG(temperature >= 0.f && top_p > 0.f, "hb_logits_to_probs: temperature must be >= 0 and top_p > 0");
  return hb::launch_sample((cudaStream_t)stream, probs, nullptr, logits, token_counts, nullptr, n, vocab, temperature,
                           top_p, presence_penalty, frequency_penalty);
}

int hb_sample(void* stream, uint32_t* tokens, float* probs_workspace, const float* logits,
              const uint32_t* token_counts, const uint64_t* seeds, int64_t n, int64_t vocab, float temperature,
              float top_p, float presence_penalty, float frequency_penalty) {
  HB_CHECK_ARG(tokens && probs_workspace && logits, "hb_sample: null pointer");
  HB_CHECK_ARG(seeds || temperature < 1e-6f, "hb_sample: seeds are needed unless the temperature is 0 (greedy)");
  HB_CHECK_ARG(n >= 0 && vocab > 0 && vocab < (1ll << 31), "hb_sample: bad shape");
  HB_CHECK_ARG(temperature >= 0.f && top_p > 0.f, "hb_sample: temperature must be >= 0 and top_p > 0");
  return hb::launch_sample((cudaStream_t)stream, probs_workspace, tokens, logits, token_counts, seeds, n, vocab,
                           temperature, top_p, presence_penalty, frequency_penalty);
}

}  // extern "C"
