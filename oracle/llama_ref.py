"""Oracle (test infrastructure): NumPy restatement of the reference's tensor-parallel
Llama forward pass, src/engine/arch/llama_tp.rs.

``LlamaTpOracle.forward`` follows TpLlamaBackend::forward (llama_tp.rs:506-576) rank by
rank: embed (:213-216), input norm (:517-522), attn_partial (:220-329), all_reduce in
rank order (:533 -> src/parallel/comm.rs:47-62), residual + post-attention norm
(:536-552), ffn_partial (:333-339), all_reduce (:563), residual (:566-571), final norm
and last-token logits (:349-356).  Differences from the reference, on purpose
(its known defects are not copied): every sequence has its own fresh KV cache (the
reference shares one never-reset cache, llama_tp.rs:207); with world_size 1 the same
code runs with one rank (the reference then runs candle-transformers' Llama, whose
source is not in the tree; same architecture: rotate-half RoPE, pre-norm, SwiGLU, GQA).

dtype "f32" does no intermediate rounding; "bf16"/"f16" round wherever the reference
materialises a tensor (after each matmul, RoPE, softmax in dtype per llama_tp.rs:318).
``eager`` selects which of the reference's two arithmetic forms the norm and RoPE take in
a 16-bit dtype:
  eager=True  (default for "bf16")  the multi-op path the reference runs for bf16: RMSNorm as
              candle_fallback, every op rounded (src/kernels/rms_norm.rs:128-132), RoPE with
              every product and sum rounded (llama_tp.rs:135-149);
  eager=False (default for "f32"/"f16") the fused-kernel numerics: fp32 accumulation, one
              rounding (kernels/rms_norm.cu:74-110, kernels/rope.cu:36-39).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

import numpy as np

from . import kernels_ref as K
from . import parallel_ref as P


@dataclass
class LlamaTpConfig:
    """LlamaTpConfig (llama_tp.rs:52-88)."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    vocab_size: int
    num_key_value_heads: int = 0  # 0 -> same as num_attention_heads
    rms_norm_eps: float = 1e-5    # default_eps
    rope_theta: float = 10000.0   # default_rope_theta

    @classmethod
    def from_json(cls, text: str) -> "LlamaTpConfig":
        d = json.loads(text)
        keys = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "vocab_size", "num_key_value_heads", "rms_norm_eps", "rope_theta")
        return cls(**{k: d[k] for k in keys if k in d})

    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def kv_heads(self) -> int:
        return self.num_attention_heads if self.num_key_value_heads == 0 else self.num_key_value_heads


class LlamaTpOracle:
    def __init__(self, cfg: LlamaTpConfig, weights: dict, world_size: int = 1, dtype: str = "f32",
                 reference_reduce: bool = True, softmax_in_dtype: bool = True, eager=None,
                 weights_exact: bool = False):
        n = world_size
        # divisibility rules of TpLlamaBackend::load (llama_tp.rs:407-427)
        if cfg.num_attention_heads % n:
            raise ValueError(f"num_attention_heads ({cfg.num_attention_heads}) must be divisible by "
                             f"tensor_parallel_size ({n})")
        if cfg.kv_heads() % n:
            raise ValueError(f"num_key_value_heads ({cfg.kv_heads()}) must be divisible by "
                             f"tensor_parallel_size ({n})")
        if cfg.intermediate_size % n:
            raise ValueError(f"intermediate_size ({cfg.intermediate_size}) must be divisible by "
                             f"tensor_parallel_size ({n})")
        self.cfg, self.n, self.dtype = cfg, n, dtype
        self.reference_reduce = reference_reduce
        self.softmax_in_dtype = softmax_in_dtype
        self.eager = (dtype == "bf16") if eager is None else bool(eager)
        self.local_heads = cfg.num_attention_heads // n
        self.local_kv_heads = cfg.kv_heads() // n
        # load_all_weights casts to dtype (:367-377); weights_exact: the caller's values already
        # are representable in dtype (read back from a device that holds them in it)
        r = (lambda a: np.asarray(a, dtype=np.float32)) if weights_exact else \
            (lambda a: K.rnd(np.asarray(a, dtype=np.float32), dtype))
        g = lambda name: r(weights[name])
        self.embed = g("model.embed_tokens.weight")
        self.final_norm = g("model.norm.weight")
        self.lm_head = g("lm_head.weight")  # no tied-embedding fallback (:488)
        self.ranks = []
        for rank in range(n):
            layers = []
            for l in range(cfg.num_hidden_layers):
                pf = f"model.layers.{l}"
                layers.append(dict(
                    q=P.column_shard(g(f"{pf}.self_attn.q_proj.weight"), rank, n),
                    k=P.column_shard(g(f"{pf}.self_attn.k_proj.weight"), rank, n),
                    v=P.column_shard(g(f"{pf}.self_attn.v_proj.weight"), rank, n),
                    o=P.row_shard(g(f"{pf}.self_attn.o_proj.weight"), rank, n),
                    gate=P.column_shard(g(f"{pf}.mlp.gate_proj.weight"), rank, n),
                    up=P.column_shard(g(f"{pf}.mlp.up_proj.weight"), rank, n),
                    down=P.row_shard(g(f"{pf}.mlp.down_proj.weight"), rank, n),
                    input_norm=g(f"{pf}.input_layernorm.weight"),
                    post_norm=g(f"{pf}.post_attention_layernorm.weight"),
                ))
            self.ranks.append(layers)

    # ------------------------------------------------------------------ pieces
    def new_cache(self):
        """Per rank, per layer (K, V) each [ctx, local_kv_heads, d]; starts empty."""
        return [[[None, None] for _ in range(self.cfg.num_hidden_layers)] for _ in range(self.n)]

    def _mm(self, x, w):
        return K.rnd(x @ w.T, self.dtype)

    def _norm(self, x, w):
        if self.eager:
            return K.rms_norm_fallback(x, w, self.cfg.rms_norm_eps, self.dtype)
        return K.rms_norm_kernel(x, w, self.cfg.rms_norm_eps, self.dtype)

    def attn_partial(self, rank, x, layer, seq_pos, cache):
        """RankState::attn_partial (llama_tp.rs:220-329)."""
        cfg, w, dt = self.cfg, self.ranks[rank][layer], self.dtype
        seq = x.shape[0]
        d = cfg.head_dim()
        q = self._mm(x, w["q"]).reshape(seq, self.local_heads, d)
        k = self._mm(x, w["k"]).reshape(seq, self.local_kv_heads, d)
        v = self._mm(x, w["v"]).reshape(seq, self.local_kv_heads, d)
        cos, sin = K.rope_tables(np.arange(seq_pos, seq_pos + seq), cfg.rope_theta, d, dt)
        q = K.apply_rope(q, cos, sin, dt, per_op_rounding=self.eager)
        k = K.apply_rope(k, cos, sin, dt, per_op_rounding=self.eager)
        kc, vc = cache[rank][layer]
        k = k if kc is None else np.concatenate([kc, k], axis=0)  # Tensor::cat (:245-259)
        v = v if vc is None else np.concatenate([vc, v], axis=0)
        cache[rank][layer] = [k, v]
        sk = k.shape[0]
        n_rep = self.local_heads // self.local_kv_heads
        ke = np.repeat(k, n_rep, axis=1)  # query head j uses kv head j // n_rep (:264-279)
        ve = np.repeat(v, n_rep, axis=1)
        q_t = q.transpose(1, 0, 2)              # [heads, sq, d]
        k_t = ke.transpose(1, 2, 0)             # [heads, d, sk]
        v_t = ve.transpose(1, 0, 2)             # [heads, sk, d]
        scores = K.rnd(K.rnd(q_t @ k_t, dt) / np.float32(np.sqrt(float(d))), dt)  # (:309-310)
        if seq > 1:
            scores = K.rnd(scores + K.causal_mask(seq, sk, seq_pos)[None], dt)    # (:313-316)
        probs = K.softmax_last(scores.astype(np.float64)).astype(np.float32)
        if self.softmax_in_dtype:
            probs = K.rnd(probs, dt)                                              # (:318)
        out = K.rnd(probs @ v_t, dt).transpose(1, 0, 2).reshape(seq, self.local_heads * d)
        return self._mm(out, w["o"])                                              # (:327)

    def ffn_partial(self, rank, x, layer):
        """RankState::ffn_partial (llama_tp.rs:333-339)."""
        w, dt = self.ranks[rank][layer], self.dtype
        gate = K.rnd(K.silu(self._mm(x, w["gate"]).astype(np.float64)).astype(np.float32), dt)
        up = self._mm(x, w["up"])
        return self._mm(K.rnd(gate * up, dt), w["down"])

    def _reduce(self, partials):
        return (P.all_reduce if self.reference_reduce else P.all_reduce_f32)(partials, self.dtype)

    # ----------------------------------------------------------------- forward
    def final_logits(self, hidden_rows):
        """final_forward (llama_tp.rs:349-356) for a stack of last-token hidden rows [n, H]."""
        normed = self._norm(np.asarray(hidden_rows, dtype=np.float32), self.final_norm)
        return K.rnd(normed @ self.lm_head.T, self.dtype)

    def forward(self, token_ids, seq_pos: int, cache, return_hidden: bool = False, logits: bool = True):
        """TpLlamaBackend::forward (llama_tp.rs:506-576) -> logits [vocab] of the last token.
        logits=False returns the hidden rows only (final_logits() then serves many
        sequences with one lm_head product)."""
        cfg, dt = self.cfg, self.dtype
        ids = np.asarray(token_ids, dtype=np.int64)
        hidden = self.embed[ids]  # identical on every rank (:508-512)
        for layer in range(cfg.num_hidden_layers):
            normed = [self._norm(hidden, self.ranks[r][layer]["input_norm"]) for r in range(self.n)]
            partials = [self.attn_partial(r, normed[r], layer, seq_pos, cache) for r in range(self.n)]
            attn_out = self._reduce(partials)
            after_attn = K.rnd(hidden + attn_out, dt)
            post = self._norm(after_attn, self.ranks[0][layer]["post_norm"])
            ffn = self._reduce([self.ffn_partial(r, post, layer) for r in range(self.n)])
            hidden = K.rnd(after_attn + ffn, dt)
        if not logits:
            return hidden
        normed = self._norm(hidden, self.final_norm)
        logits = K.rnd(normed[-1:] @ self.lm_head.T, dt)[0]  # final_forward (:349-356)
        return (logits, hidden) if return_hidden else logits

    def greedy_generate(self, prompt_ids, n_new: int):
        """Worker-level greedy decode (src/worker/mod.rs:349-358,404-409): prefill the
        prompt at seq_pos 0, sample token 0 from the last logits, then feed
        output_ids.last() at seq_pos = prompt_len + output_len - 1; argmax takes the
        first maximum (src/sampling/mod.rs:105-107)."""
        cache = self.new_cache()
        logits = self.forward(prompt_ids, 0, cache)
        out = [int(np.argmax(logits))]
        all_logits = [logits]
        while len(out) < n_new:
            pos = len(prompt_ids) + len(out) - 1
            logits = self.forward([out[-1]], pos, cache)
            out.append(int(np.argmax(logits)))
            all_logits.append(logits)
        return out, all_logits


# ------------------------------------------------------------- synthetic models
TENSOR_ORDER_NOTE = "tensors are drawn in sorted HF-name order from one PCG64 stream"


def tensor_shapes(cfg: LlamaTpConfig) -> dict:
    """HF tensor names the loader looks up (llama_tp.rs:451-462,482-488) with shapes."""
    H, I, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim()
    hq, hkv = cfg.num_attention_heads, cfg.kv_heads()
    shapes = {
        "model.embed_tokens.weight": (cfg.vocab_size, H),
        "model.norm.weight": (H,),
        "lm_head.weight": (cfg.vocab_size, H),
    }
    for l in range(cfg.num_hidden_layers):
        pf = f"model.layers.{l}"
        shapes.update({
            f"{pf}.self_attn.q_proj.weight": (hq * d, H),
            f"{pf}.self_attn.k_proj.weight": (hkv * d, H),
            f"{pf}.self_attn.v_proj.weight": (hkv * d, H),
            f"{pf}.self_attn.o_proj.weight": (H, hq * d),
            f"{pf}.mlp.gate_proj.weight": (I, H),
            f"{pf}.mlp.up_proj.weight": (I, H),
            f"{pf}.mlp.down_proj.weight": (H, I),
            f"{pf}.input_layernorm.weight": (H,),
            f"{pf}.post_attention_layernorm.weight": (H,),
        })
    return shapes


def random_weights(cfg: LlamaTpConfig, seed: int = 1, std: float = 0.02, norm_ones: bool = False) -> dict:
    """fp32 weights ~N(0, std), seeded; norm weights 1 when norm_ones."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        w = rng.standard_normal(shape, dtype=np.float32) * np.float32(std)
        if norm_ones and name.endswith("norm.weight"):
            w = np.ones(shape, dtype=np.float32)
        out[name] = w
    return out


def write_model(path: str, cfg: LlamaTpConfig, weights: dict, model_type: str = "llama", dtype: str = "F32") -> None:
    """config.json + model.safetensors (F32, or BF16 / F16 as checkpoints ship) as Engine::load
    reads them (src/engine/loader.rs:105-126)."""
    os.makedirs(path, exist_ok=True)
    conf = dict(model_type=model_type, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                num_key_value_heads=cfg.kv_heads(), vocab_size=cfg.vocab_size,
                rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(conf, f)
    write_safetensors(os.path.join(path, "model.safetensors"), weights, dtype)


def write_safetensors(file_path: str, weights: dict, dtype: str = "F32") -> None:
    """One safetensors file: u64 header length, JSON header, raw little-endian data."""
    header, blobs, off = {}, [], 0
    for name in sorted(weights):
        a = np.ascontiguousarray(weights[name], dtype=np.float32)
        if dtype == "BF16":
            raw = K.to_bf16_bits(a).tobytes()
        elif dtype == "F16":
            raw = a.astype(np.float16).tobytes()
        else:
            raw = a.tobytes()
        header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(file_path, "wb") as f:
        f.write(len(hjson).to_bytes(8, "little"))
        f.write(hjson)
        for b in blobs:
            f.write(b)


TINY_CONFIG = LlamaTpConfig(hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, vocab_size=32000,
                            rms_norm_eps=1e-5, rope_theta=10000.0)
