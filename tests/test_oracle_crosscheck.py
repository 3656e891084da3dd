"""The reference's own tests do not pin GEMM, attention, SwiGLU or logits, so the NumPy
restatement is cross-checked here against an independent torch fp32 implementation of
the same formulas (different code path, different BLAS entry points), and the
tensor-parallel decomposition against the single-rank model."""
import numpy as np
import pytest
import torch

from oracle import kernels_ref as K
from oracle import llama_ref as R

torch.set_num_threads(4)

SMALL = R.LlamaTpConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=128, rms_norm_eps=1e-5, rope_theta=10000.0)


def torch_llama_logits(cfg, weights, ids):
    """Plain pre-norm Llama block stack in torch fp32 over the whole prompt (masked
    prefill), written independently of oracle/llama_ref.py."""
    W = {k: torch.from_numpy(v) for k, v in weights.items()}
    d, hq, hkv = cfg.head_dim(), cfg.num_attention_heads, cfg.kv_heads()
    S = len(ids)
    h = W["model.embed_tokens.weight"][torch.tensor(ids, dtype=torch.long)]

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    pos = torch.arange(S, dtype=torch.float32)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rope(x):
        x1, x2 = x[..., : d // 2], x[..., d // 2:]
        return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1)

    mask = torch.full((S, S), float("-inf")).triu(1)
    for l in range(cfg.num_hidden_layers):
        pf = f"model.layers.{l}"
        x = norm(h, W[f"{pf}.input_layernorm.weight"])
        q = rope((x @ W[f"{pf}.self_attn.q_proj.weight"].T).view(S, hq, d))
        k = rope((x @ W[f"{pf}.self_attn.k_proj.weight"].T).view(S, hkv, d))
        v = (x @ W[f"{pf}.self_attn.v_proj.weight"].T).view(S, hkv, d)
        k = k.repeat_interleave(hq // hkv, dim=1)
        v = v.repeat_interleave(hq // hkv, dim=1)
        sc = torch.einsum("qhd,khd->hqk", q, k) / d ** 0.5 + mask
        o = torch.einsum("hqk,khd->qhd", sc.softmax(-1), v).reshape(S, hq * d)
        h = h + o @ W[f"{pf}.self_attn.o_proj.weight"].T
        x = norm(h, W[f"{pf}.post_attention_layernorm.weight"])
        g = torch.nn.functional.silu(x @ W[f"{pf}.mlp.gate_proj.weight"].T)
        h = h + (g * (x @ W[f"{pf}.mlp.up_proj.weight"].T)) @ W[f"{pf}.mlp.down_proj.weight"].T
    return (norm(h, W["model.norm.weight"])[-1] @ W["lm_head.weight"].T).numpy()


@pytest.mark.parametrize("norm_ones", [True, False])
def test_forward_matches_independent_torch(norm_ones):
    w = R.random_weights(SMALL, seed=3, std=0.05, norm_ones=norm_ones)
    ids = np.random.default_rng(1).integers(0, SMALL.vocab_size, size=9).tolist()
    oracle = R.LlamaTpOracle(SMALL, w, world_size=1, dtype="f32")
    got = oracle.forward(ids, 0, oracle.new_cache())
    want = torch_llama_logits(SMALL, w, ids)
    assert np.max(np.abs(got - want)) <= 1e-4 * max(np.max(np.abs(want)), 1e-6)


def test_incremental_decode_equals_prefill():
    """Feeding tokens one by one over the growing cache == masked prefill
    (the decode branch skips the mask, llama_tp.rs:313)."""
    w = R.random_weights(SMALL, seed=4, std=0.05, norm_ones=True)
    ids = np.random.default_rng(2).integers(0, SMALL.vocab_size, size=7).tolist()
    oracle = R.LlamaTpOracle(SMALL, w, dtype="f32")
    full = oracle.forward(ids, 0, oracle.new_cache())
    cache = oracle.new_cache()
    for i, t in enumerate(ids):
        step = oracle.forward([t], i, cache)
    assert np.max(np.abs(step - full)) <= 1e-4 * np.max(np.abs(full))


@pytest.mark.parametrize("world", [2])
def test_tensor_parallel_equals_single_rank(world):
    """Column/row sharding + rank-order sum reproduces the unsharded model
    (src/parallel/shard.rs, src/engine/arch/llama_tp.rs:464-471,533,563)."""
    w = R.random_weights(SMALL, seed=5, std=0.05, norm_ones=True)
    ids = np.random.default_rng(3).integers(0, SMALL.vocab_size, size=6).tolist()
    one = R.LlamaTpOracle(SMALL, w, world_size=1, dtype="f32")
    tp = R.LlamaTpOracle(SMALL, w, world_size=world, dtype="f32")
    a = one.forward(ids, 0, one.new_cache())
    b = tp.forward(ids, 0, tp.new_cache())
    assert np.max(np.abs(a - b)) <= 1e-4 * np.max(np.abs(a))


def test_divisibility_rules():
    w = R.random_weights(SMALL, seed=1)
    for ws, word in [(3, "num_attention_heads"), (4, "num_key_value_heads")]:
        with pytest.raises(ValueError) as ei:
            R.LlamaTpOracle(SMALL, w, world_size=ws)
        assert word in str(ei.value) and "tensor_parallel_size" in str(ei.value)


def test_bf16_rounding_helpers_match_torch():
    x = np.random.default_rng(0).standard_normal(10000).astype(np.float32) * 100
    want = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(K.round_bf16(x), want)
    assert np.array_equal(K.from_bf16_bits(K.to_bf16_bits(x)), want)
    assert np.array_equal(K.rnd(x, "f16"), torch.from_numpy(x).to(torch.float16).float().numpy())


def test_rms_norm_forms_agree():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 256)).astype(np.float32)
    w = rng.standard_normal(256).astype(np.float32)
    a, b = K.rms_norm_kernel(x, w, 1e-5), K.rms_norm_fallback(x, w, 1e-5)
    assert np.max(np.abs(a - b)) < 1e-5
    t = torch.from_numpy(x)
    c = (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5) * torch.from_numpy(w)).numpy()
    assert np.max(np.abs(a - c)) < 1e-5


def test_model_file_round_trip(tmp_path):
    """write_model produces a safetensors file the `safetensors` package reads back."""
    from safetensors.numpy import load_file

    w = R.random_weights(SMALL, seed=9)
    R.write_model(str(tmp_path), SMALL, w)
    back = load_file(str(tmp_path / "model.safetensors"))
    assert set(back) == set(w)
    for k in w:
        assert np.array_equal(back[k], w[k])
    cfg = R.LlamaTpConfig.from_json((tmp_path / "config.json").read_text())
    assert cfg == SMALL
