"""The Mixtral restatement (oracle/mixtral_ref.py) against what pins it:
the reference's own known-answer tests for the path (sliding_causal_mask,
src/engine/arch/mixtral.rs:650-673; config defaults :617-634), an independent torch fp32
implementation of the same formulas (the reference's tests never compute router outputs,
expert outputs or logits), and the tensor-parallel decomposition against one rank."""
import numpy as np
import pytest
import torch

from oracle import mixtral_ref as M

torch.set_num_threads(4)

SMALL = M.MixtralConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, num_local_experts=4,
                        num_experts_per_tok=2, rms_norm_eps=1e-5, rope_theta=1e6, sliding_window=5)


def test_sliding_causal_mask_reference_cases():
    # sliding_causal_mask_shape (mixtral.rs:650-654)
    assert M.sliding_causal_mask(3, 0, 4).shape == (3, 3)
    # sliding_causal_mask_blocks_future (:656-662)
    m = M.sliding_causal_mask(2, 0, 16)
    assert np.isneginf(m[0, 1])
    # sliding_causal_mask_blocks_outside_window (:664-673): window 2, position 3
    m = M.sliding_causal_mask(1, 3, 2)
    assert np.isneginf(m[0, 0]) and m[0, 2] == 0.0 and m[0, 3] == 0.0


def test_config_defaults():
    # config_defaults (mixtral.rs:617-634): rope_theta 1e6, sliding_window 4096, kv heads fall back
    c = M.MixtralConfig(vocab_size=8, hidden_size=16, intermediate_size=32, num_hidden_layers=1,
                        num_attention_heads=4, num_local_experts=8, num_experts_per_tok=2)
    assert c.rope_theta == 1_000_000.0 and c.sliding_window == 4096
    assert c.kv_heads() == 4 and c.head_dim() == 4


def test_route_topk_renormalised():
    chosen = M.route(np.array([0.1, 0.4, 0.2, 0.3], dtype=np.float32), 2)
    assert [e for e, _ in chosen] == [1, 3]
    assert abs(sum(w for _, w in chosen) - 1.0) < 1e-6 and abs(chosen[0][1] - 0.4 / 0.7) < 1e-6
    # ties: lower index first
    assert [e for e, _ in M.route(np.array([0.25, 0.25, 0.25, 0.25], dtype=np.float32), 2)] == [0, 1]


def torch_mixtral_logits(cfg, weights, ids):
    """Mixtral block stack in torch fp32 over the whole prompt, written independently of
    oracle/mixtral_ref.py (rotate-half RoPE in its two-term form, dense top-k mask)."""
    W = {k: torch.from_numpy(v) for k, v in weights.items()}
    d, hq, hkv, S = cfg.head_dim(), cfg.num_attention_heads, cfg.kv_heads(), len(ids)
    h = W["model.embed_tokens.weight"][torch.tensor(ids, dtype=torch.long)]

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rope(x):
        x1, x2 = x[..., : d // 2], x[..., d // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    qi, ki = torch.arange(S)[:, None], torch.arange(S)[None, :]
    mask = torch.where((ki <= qi) & (qi - ki < cfg.sliding_window), 0.0, float("-inf"))
    for l in range(cfg.num_hidden_layers):
        pf = f"model.layers.{l}"
        x = norm(h, W[f"{pf}.input_layernorm.weight"])
        q = rope((x @ W[f"{pf}.self_attn.q_proj.weight"].T).view(S, hq, d))
        k = rope((x @ W[f"{pf}.self_attn.k_proj.weight"].T).view(S, hkv, d)).repeat_interleave(hq // hkv, dim=1)
        v = (x @ W[f"{pf}.self_attn.v_proj.weight"].T).view(S, hkv, d).repeat_interleave(hq // hkv, dim=1)
        sc = torch.einsum("qhd,khd->hqk", q, k) / d ** 0.5 + mask
        h = h + torch.einsum("hqk,khd->qhd", sc.softmax(-1), v).reshape(S, hq * d) @ W[f"{pf}.self_attn.o_proj.weight"].T
        x = norm(h, W[f"{pf}.post_attention_layernorm.weight"])
        probs = (x @ W[f"{pf}.block_sparse_moe.gate.weight"].T).softmax(-1)
        top_w, top_e = probs.topk(cfg.num_experts_per_tok, dim=-1)
        top_w = top_w / top_w.sum(-1, keepdim=True)
        out = torch.zeros_like(h)
        for e in range(cfg.num_local_experts):
            ex = f"{pf}.block_sparse_moe.experts.{e}"
            y = (torch.nn.functional.silu(x @ W[f"{ex}.w1.weight"].T) * (x @ W[f"{ex}.w3.weight"].T)) @ W[f"{ex}.w2.weight"].T
            wgt = (top_w * (top_e == e)).sum(-1, keepdim=True)
            out = out + wgt * y
        h = h + out
    return (norm(h, W["model.norm.weight"])[-1] @ W["lm_head.weight"].T).numpy()


@pytest.mark.parametrize("norm_ones", [True, False])
def test_forward_matches_independent_torch(norm_ones):
    w = M.random_weights(SMALL, seed=3, std=0.05, norm_ones=norm_ones)
    ids = np.random.default_rng(1).integers(0, SMALL.vocab_size, size=11).tolist()  # longer than the window
    oracle = M.MixtralOracle(SMALL, w, world_size=1, dtype="f32")
    got = oracle.forward(ids, 0, oracle.new_cache())
    want = torch_mixtral_logits(SMALL, w, ids)
    assert np.max(np.abs(got - want)) <= 2e-4 * max(1.0, float(np.max(np.abs(want))))


def test_incremental_decode_equals_prefill_and_tp_equals_single_rank():
    w = M.random_weights(SMALL, seed=4, std=0.05, norm_ones=True)
    ids = np.random.default_rng(2).integers(0, SMALL.vocab_size, size=9).tolist()
    one = M.MixtralOracle(SMALL, w, world_size=1, dtype="f32")
    full = one.forward(ids, 0, one.new_cache())
    cache = one.new_cache()
    for t, tok in enumerate(ids):
        step = one.forward([tok], t, cache)
    assert np.max(np.abs(step - full)) <= 1e-4 * max(1.0, float(np.max(np.abs(full))))
    two = M.MixtralOracle(SMALL, w, world_size=2, dtype="f32")
    tp = two.forward(ids, 0, two.new_cache())
    assert np.max(np.abs(tp - full)) <= 1e-4 * max(1.0, float(np.max(np.abs(full))))
