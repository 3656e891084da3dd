"""Oracle (test infrastructure): NumPy restatement of the reference's Mixtral forward pass,
src/engine/arch/mixtral.rs.

``MixtralOracle.forward`` follows MixtralModel::forward (mixtral.rs:455-516): embed,
per layer input norm -> Attention::forward (:234-318: q/k/v projections, RoPE
`x*cos + rotate_half(x)*sin` with full-width cat(freqs, freqs) tables (:106-151),
cache append, repeat_kv (:178-188), sliding-window causal mask (:155-176), softmax, o_proj)
-> residual -> post-attention norm -> SparseMoeBlock::forward (:371-430: router softmax,
top-k by descending probability, renormalised weights floored at 1e-9, Expert::forward
`w2(silu(w1 x) * w3 x)` (:337-341) per chosen expert, weighted sum accumulated in fp32 and
cast back) -> residual; final norm and last-token logits.

The reference runs Mixtral on one device (src/engine/loader.rs:142-144).  ``world_size`` > 1
restates the tensor-parallel form this build adds: attention sharded like llama_tp.rs,
every expert's w1/w3 column-parallel and w2 row-parallel over its intermediate size, the
router replicated, partial sums reduced in rank order.

Ties in the top-k are left open by the reference (sort_unstable_by, :398); this restatement
and the device kernel both take the lower expert index first.

dtype "f32" does no intermediate rounding; "bf16"/"f16" round wherever the reference
materialises a tensor.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

import numpy as np

from . import kernels_ref as K
from . import parallel_ref as P


@dataclass
class MixtralConfig:
    """MixtralConfig (mixtral.rs:40-78)."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_local_experts: int
    num_experts_per_tok: int
    num_key_value_heads: int = 0      # 0 -> num_attention_heads (:64-70)
    rms_norm_eps: float = 1e-5
    rope_theta: float = 1_000_000.0   # default_rope_theta (:56-58)
    sliding_window: int = 4096        # default_sliding_window (:59-61)

    def kv_heads(self) -> int:
        return self.num_attention_heads if self.num_key_value_heads == 0 else self.num_key_value_heads

    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


def sliding_causal_mask(seq_len: int, seq_pos: int, window: int) -> np.ndarray:
    """sliding_causal_mask (mixtral.rs:155-176): 0 where ki <= q_abs and q_abs - ki < window."""
    total = seq_pos + seq_len
    q_abs = seq_pos + np.arange(seq_len)[:, None]
    ki = np.arange(total)[None, :]
    ok = (ki <= q_abs) & (q_abs - ki < window)
    return np.where(ok, np.float32(0.0), np.float32(-np.inf)).astype(np.float32)


def rope_apply(x: np.ndarray, cos: np.ndarray, sin: np.ndarray, dtype: str) -> np.ndarray:
    """rope_apply (mixtral.rs:143-151): x*cos + cat(-x2, x1)*sin; x [seq, heads, d],
    cos/sin [seq, d] (cat(freqs, freqs) tables in dtype)."""
    half = x.shape[-1] // 2
    rotated = np.concatenate([-x[..., half:], x[..., :half]], axis=-1)
    a = K.rnd(x * cos[:, None, :], dtype)
    b = K.rnd(rotated * sin[:, None, :], dtype)
    return K.rnd(a + b, dtype)


def route(probs: np.ndarray, k: int):
    """Top-k of one token's probabilities by descending value, lower index first among
    equals; weights divided by max(sum, 1e-9) (mixtral.rs:396-410)."""
    order = sorted(range(len(probs)), key=lambda e: (-float(probs[e]), e))[: min(k, len(probs))]
    s = np.float32(sum(np.float32(probs[e]) for e in order))
    denom = np.float32(max(float(s), 1e-9))
    return [(e, np.float32(probs[e]) / denom) for e in order]


class MixtralOracle:
    def __init__(self, cfg: MixtralConfig, weights: dict, world_size: int = 1, dtype: str = "f32"):
        n = world_size
        if cfg.num_attention_heads % n or cfg.kv_heads() % n or cfg.intermediate_size % n:
            raise ValueError("heads, kv heads and intermediate_size must be divisible by tensor_parallel_size")
        self.cfg, self.n, self.dtype = cfg, n, dtype
        self.min_route_gap = float("inf")  # reset by the caller between sequences
        self.local_heads = cfg.num_attention_heads // n
        self.local_kv_heads = cfg.kv_heads() // n
        r = lambda a: K.rnd(np.asarray(a, dtype=np.float32), dtype)
        g = lambda name: r(weights[name])
        self.embed = g("model.embed_tokens.weight")
        self.final_norm = g("model.norm.weight")
        self.lm_head = g("lm_head.weight")
        self.ranks = []
        for rank in range(n):
            layers = []
            for l in range(cfg.num_hidden_layers):
                pf = f"model.layers.{l}"
                experts = []
                for x in range(cfg.num_local_experts):
                    ex = f"{pf}.block_sparse_moe.experts.{x}"
                    experts.append(dict(w1=P.column_shard(g(f"{ex}.w1.weight"), rank, n),
                                        w3=P.column_shard(g(f"{ex}.w3.weight"), rank, n),
                                        w2=P.row_shard(g(f"{ex}.w2.weight"), rank, n)))
                layers.append(dict(
                    q=P.column_shard(g(f"{pf}.self_attn.q_proj.weight"), rank, n),
                    k=P.column_shard(g(f"{pf}.self_attn.k_proj.weight"), rank, n),
                    v=P.column_shard(g(f"{pf}.self_attn.v_proj.weight"), rank, n),
                    o=P.row_shard(g(f"{pf}.self_attn.o_proj.weight"), rank, n),
                    gate=g(f"{pf}.block_sparse_moe.gate.weight"),
                    experts=experts,
                    input_norm=g(f"{pf}.input_layernorm.weight"),
                    post_norm=g(f"{pf}.post_attention_layernorm.weight"),
                ))
            self.ranks.append(layers)

    def new_cache(self):
        return [[[None, None] for _ in range(self.cfg.num_hidden_layers)] for _ in range(self.n)]

    def _mm(self, x, w):
        return K.rnd(x @ w.T, self.dtype)

    def _norm(self, x, w):
        return K.rms_norm_kernel(x, w, self.cfg.rms_norm_eps, self.dtype)

    def attn_partial(self, rank, x, layer, seq_pos, cache):
        """Attention::forward (mixtral.rs:234-318), this rank's heads."""
        cfg, w, dt = self.cfg, self.ranks[rank][layer], self.dtype
        seq, d = x.shape[0], cfg.head_dim()
        q = self._mm(x, w["q"]).reshape(seq, self.local_heads, d)
        k = self._mm(x, w["k"]).reshape(seq, self.local_kv_heads, d)
        v = self._mm(x, w["v"]).reshape(seq, self.local_kv_heads, d)
        # RotaryEmbedding::new (:106-131): freqs = pos * inv_freq in f32, emb = cat(freqs, freqs)
        inv = K.rope_inv_freq(cfg.rope_theta, d)
        freqs = np.arange(seq_pos, seq_pos + seq, dtype=np.float32)[:, None] * inv[None, :]
        emb = np.concatenate([freqs, freqs], axis=-1)
        cos, sin = K.rnd(np.cos(emb).astype(np.float32), dt), K.rnd(np.sin(emb).astype(np.float32), dt)
        q, k = rope_apply(q, cos, sin, dt), rope_apply(k, cos, sin, dt)
        kc, vc = cache[rank][layer]
        k = k if kc is None else np.concatenate([kc, k], axis=0)
        v = v if vc is None else np.concatenate([vc, v], axis=0)
        cache[rank][layer] = [k, v]
        n_rep = self.local_heads // self.local_kv_heads
        ke, ve = np.repeat(k, n_rep, axis=1), np.repeat(v, n_rep, axis=1)  # repeat_kv (:178-188)
        q_t, k_t, v_t = q.transpose(1, 0, 2), ke.transpose(1, 2, 0), ve.transpose(1, 0, 2)
        scores = K.rnd(K.rnd(q_t @ k_t, dt) * np.float32(1.0 / np.sqrt(float(d))), dt)      # (:305)
        scores = K.rnd(scores + sliding_causal_mask(seq, seq_pos, cfg.sliding_window)[None], dt)  # (:303-306)
        probs = K.rnd(K.softmax_last(scores.astype(np.float64)).astype(np.float32), dt)
        out = K.rnd(probs @ v_t, dt).transpose(1, 0, 2).reshape(seq, self.local_heads * d)
        return self._mm(out, w["o"])

    def router(self, x, layer):
        """Per token the chosen experts and their renormalised weights (mixtral.rs:378-410)."""
        dt = self.dtype
        logits = self._mm(x, self.ranks[0][layer]["gate"])
        probs = K.rnd(K.softmax_last(logits.astype(np.float64)).astype(np.float32), dt)
        # The reference picks the top-k with an unstable sort (mixtral.rs:395-397): which expert
        # wins a tie, or a gap smaller than the arithmetic noise, is unspecified.  The smallest
        # gap between the last chosen and the first rejected probability of the LAST token
        # (the one whose logits are returned; earlier tokens reach it only through attention)
        # is recorded so that a parity test can tell a different-but-legal choice from an error.
        k = self.cfg.num_experts_per_tok
        if probs.shape[1] > k:
            srt = np.sort(probs[-1])[::-1]
            self.min_route_gap = min(self.min_route_gap, float(srt[k - 1] - srt[k]))
        return [route(probs[t], k) for t in range(x.shape[0])]

    def moe_partial(self, rank, x, layer, routes):
        """SparseMoeBlock::forward (mixtral.rs:371-430) with this rank's slice of every expert:
        out[t] = sum over chosen experts of weight * Expert::forward(x[t]), accumulated in fp32."""
        dt = self.dtype
        out = np.zeros((x.shape[0], self.cfg.hidden_size), dtype=np.float32)
        for t, chosen in enumerate(routes):
            tok = x[t:t + 1]
            for e, wgt in chosen:
                ex = self.ranks[rank][layer]["experts"][e]
                gate = K.rnd(K.silu(self._mm(tok, ex["w1"]).astype(np.float64)).astype(np.float32), dt)  # (:338)
                up = self._mm(tok, ex["w3"])
                y = self._mm(K.rnd(gate * up, dt), ex["w2"])[0]
                out[t] += np.float32(wgt) * y
        return K.rnd(out, dt)

    def forward(self, token_ids, seq_pos: int, cache):
        """MixtralModel::forward (mixtral.rs:491-516) -> logits [vocab] of the last token."""
        cfg, dt = self.cfg, self.dtype
        hidden = self.embed[np.asarray(token_ids, dtype=np.int64)]
        for layer in range(cfg.num_hidden_layers):
            normed = self._norm(hidden, self.ranks[0][layer]["input_norm"])
            attn = P.all_reduce_f32([self.attn_partial(r, normed, layer, seq_pos, cache) for r in range(self.n)], dt)
            hidden = K.rnd(hidden + attn, dt)                                   # (:441-442)
            post = self._norm(hidden, self.ranks[0][layer]["post_norm"])
            routes = self.router(post, layer)
            moe = P.all_reduce_f32([self.moe_partial(r, post, layer, routes) for r in range(self.n)], dt)
            hidden = K.rnd(hidden + moe, dt)                                    # (:444-445)
        normed = self._norm(hidden, self.final_norm)
        return K.rnd(normed[-1:] @ self.lm_head.T, dt)[0]


def tensor_shapes(cfg: MixtralConfig) -> dict:
    """Tensor names of MixtralModel::load (mixtral.rs:330-333,354-363,461-472) with shapes."""
    H, I, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim()
    hq, hkv = cfg.num_attention_heads, cfg.kv_heads()
    shapes = {"model.embed_tokens.weight": (cfg.vocab_size, H), "model.norm.weight": (H,),
              "lm_head.weight": (cfg.vocab_size, H)}
    for l in range(cfg.num_hidden_layers):
        pf = f"model.layers.{l}"
        shapes.update({
            f"{pf}.self_attn.q_proj.weight": (hq * d, H),
            f"{pf}.self_attn.k_proj.weight": (hkv * d, H),
            f"{pf}.self_attn.v_proj.weight": (hkv * d, H),
            f"{pf}.self_attn.o_proj.weight": (H, hq * d),
            f"{pf}.block_sparse_moe.gate.weight": (cfg.num_local_experts, H),
            f"{pf}.input_layernorm.weight": (H,),
            f"{pf}.post_attention_layernorm.weight": (H,),
        })
        for x in range(cfg.num_local_experts):
            ex = f"{pf}.block_sparse_moe.experts.{x}"
            shapes.update({f"{ex}.w1.weight": (I, H), f"{ex}.w3.weight": (I, H), f"{ex}.w2.weight": (H, I)})
    return shapes


def random_weights(cfg: MixtralConfig, seed: int = 1, std: float = 0.02, norm_ones: bool = False) -> dict:
    """fp32 weights ~N(0, std), seeded, drawn in sorted name order; norm weights 1 when norm_ones."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        w = rng.standard_normal(shape, dtype=np.float32) * np.float32(std)
        if norm_ones and name.endswith("norm.weight"):
            w = np.ones(shape, dtype=np.float32)
        out[name] = w
    return out


def write_model(path: str, cfg: MixtralConfig, weights: dict) -> None:
    """config.json (model_type "mixtral") + model.safetensors (F32)."""
    from .llama_ref import write_safetensors

    os.makedirs(path, exist_ok=True)
    conf = dict(model_type="mixtral", hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                num_key_value_heads=cfg.kv_heads(), vocab_size=cfg.vocab_size, rms_norm_eps=cfg.rms_norm_eps,
                rope_theta=cfg.rope_theta, sliding_window=cfg.sliding_window,
                num_local_experts=cfg.num_local_experts, num_experts_per_tok=cfg.num_experts_per_tok)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(conf, f)
    write_safetensors(os.path.join(path, "model.safetensors"), weights)


TINY_MIXTRAL = MixtralConfig(vocab_size=2048, hidden_size=256, intermediate_size=384, num_hidden_layers=2,
                             num_attention_heads=4, num_key_value_heads=2, num_local_experts=4,
                             num_experts_per_tok=2, rms_norm_eps=1e-5, rope_theta=1_000_000.0, sliding_window=24)
