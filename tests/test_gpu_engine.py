"""End-to-end parity of the decode engine with the CPU oracle on identical seeded
weights and prompts: last-token logits within 1e-3 (fp32) / 2e-2 (bf16) of the largest
|logit|, greedy next-token agreement >= 99 %, block tables as the FIFO allocator
dictates."""
import numpy as np
import pytest

from oracle import llama_ref as R

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    return float(np.max(np.abs(got - want))) / max(float(np.max(np.abs(want))), 1e-30)


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    cfg = R.TINY_CONFIG
    weights = R.random_weights(cfg, seed=1, std=0.02, norm_ones=True)
    path = tmp_path_factory.mktemp("tiny_llama")
    R.write_model(str(path), cfg, weights)
    return cfg, weights, str(path)


def test_tiny_fp32_logits_and_greedy(hb, cuda, tiny):
    """Config 1 of the baseline: tiny fp32 Llama, 8 prompts x 32 ids (seed 0), greedy."""
    cfg, weights, path = tiny
    eng = hb.Engine.load(path, max_seq_len=128, bf16=False, force_f32=True, max_batch=8)
    assert eng.num_layers() == 2 and eng.vocab_size() == 32000 and eng.hidden_size() == 256
    oracle = R.LlamaTpOracle(cfg, weights, world_size=1, dtype="f32")
    prompts = np.random.default_rng(0).integers(0, cfg.vocab_size, size=(8, 32)).astype(np.uint32)
    n_new, agree, total = 8, 0, 0
    for p in prompts[:3]:
        want_tokens, want_logits = oracle.greedy_generate(p.tolist(), n_new)
        seq = eng.create_kv_cache()
        logits = eng.forward_with_cache(p, 0, seq)
        got_tokens = [int(np.argmax(logits))]
        assert rel_err(logits, want_logits[0]) <= 1e-3
        while len(got_tokens) < n_new:
            pos = len(p) + len(got_tokens) - 1
            # teacher-forced on the oracle's token so that one early flip cannot cascade
            logits = eng.forward_with_cache([want_tokens[len(got_tokens) - 1]], pos, seq)
            assert rel_err(logits, want_logits[len(got_tokens)]) <= 1e-3
            got_tokens.append(int(np.argmax(logits)))
        agree += sum(int(a == b) for a, b in zip(got_tokens, want_tokens))
        total += n_new
        seq.free()
    assert agree / total >= 0.99
    eng.close()


def test_tiny_batched_decode_matches_per_sequence(hb, cuda, tiny):
    """hb_decode_batch over ragged sequences == the per-sequence path of the reference
    (src/worker/mod.rs:280-293), and the block tables follow the FIFO allocator."""
    cfg, weights, path = tiny
    eng = hb.Engine.load(path, max_seq_len=128, bf16=False, force_f32=True, max_batch=8, num_kv_blocks=64)
    oracle = R.LlamaTpOracle(cfg, weights, world_size=1, dtype="f32")
    rng = np.random.default_rng(3)
    lens = [1, 15, 16, 17, 33]
    prompts = [rng.integers(0, cfg.vocab_size, size=n).astype(np.uint32) for n in lens]
    seqs, caches, last = [], [], []
    for p in prompts:
        s = eng.create_kv_cache()
        logits = eng.forward_with_cache(p, 0, s)
        c = oracle.new_cache()
        want = oracle.forward(p.tolist(), 0, c)
        assert rel_err(logits, want) <= 1e-3
        seqs.append(s); caches.append(c); last.append(int(np.argmax(want)))
    # FIFO block ids: sequences were prefilled one after another from a fresh pool
    nxt = 0
    for s, n in zip(seqs, lens):
        nb = -(-n // 16)
        assert s.block_table() == list(range(nxt, nxt + nb))
        nxt += nb
    for step in range(4):
        logits = np.empty((len(seqs), cfg.vocab_size), dtype=np.float32)
        got = eng.decode_batch(seqs, np.array(last, dtype=np.uint32), logits=logits)
        new_last = []
        for i, (c, n) in enumerate(zip(caches, lens)):
            want = oracle.forward([last[i]], n + step, c)
            assert rel_err(logits[i], want) <= 1e-3
            assert int(got[i]) == int(np.argmax(logits[i]))  # device argmax = first maximum
            new_last.append(int(np.argmax(want)))
        last = new_last
    assert all(len(s) == n + 4 for s, n in zip(seqs, lens))
    free_before = eng.num_free_blocks()
    for s in seqs:
        s.free()
    assert eng.num_free_blocks() > free_before
    eng.close()


def test_tiny_bf16_logits(hb, cuda, tiny):
    cfg, weights, path = tiny
    eng = hb.Engine.load(path, max_seq_len=64, bf16=True, max_batch=4)
    oracle = R.LlamaTpOracle(cfg, weights, world_size=1, dtype="bf16")
    p = np.random.default_rng(5).integers(0, cfg.vocab_size, size=12).astype(np.uint32)
    seq = eng.create_kv_cache()
    got = eng.forward_with_cache(p, 0, seq)
    want = oracle.forward(p.tolist(), 0, oracle.new_cache())
    assert rel_err(got, want) <= 2e-2
    eng.close()


def test_engine_errors(hb, cuda, tiny, tmp_path):
    cfg, weights, path = tiny
    with pytest.raises(hb.HbError) as ei:
        hb.Engine.load(str(tmp_path / "missing"), bf16=True)
    assert ei.value.code == hb.ERR_IO
    eng = hb.Engine.load(path, max_seq_len=32, bf16=False, force_f32=True, max_batch=2, num_kv_blocks=2)
    seq = eng.create_kv_cache()
    with pytest.raises(hb.HbError):
        eng.forward_with_cache([1, 2, 3], 5, seq)       # seq_pos must equal the cached length
    with pytest.raises(hb.HbError) as ei:
        eng.forward_with_cache([], 0, seq)
    assert "empty" in ei.value.msg
    with pytest.raises(hb.HbError) as ei:
        eng.forward_with_cache(list(range(40)), 0, seq)  # needs 3 blocks, pool has 2
    assert ei.value.code == hb.ERR_OOM_BLOCKS
    eng.close()


SHAPE_TC = dict(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                num_key_value_heads=2, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=500000.0)
# head_dim 128: the tensor-core attention kernel (head_dim 64 above runs the CUDA-core one)
SHAPE_TC128 = dict(hidden_size=1024, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                   num_key_value_heads=2, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=500000.0)


def fetch_weights(eng, cfg):
    out = {}
    for name, shape in R.tensor_shapes(cfg).items():
        out[name] = eng.get_tensor(name).reshape(shape)
    return out


@pytest.mark.parametrize("fused", ["0", "1", "rope"])
@pytest.mark.parametrize("norm_ones", [True, False])
def test_random_init_bf16_tensor_core_path(hb, cuda, norm_ones, fused, monkeypatch):
    """Device-initialised bf16 model on the tcgen05 GEMM path; the oracle runs on the
    very weights read back from the device.  fused=1 routes o_proj / down_proj through
    the one-kernel GEMM + reduce + residual + norm (the engine reads HB_FUSED when it is
    created), fused=0 through the default path, "rope" additionally with RoPE and the KV
    append fused into the attention kernel."""
    if fused == "rope":  # RoPE and the KV append inside the attention kernel
        monkeypatch.setenv("HB_FUSE_ROPE", "1")
    else:
        monkeypatch.setenv("HB_FUSED", fused)
    shape = SHAPE_TC128 if fused == "rope" or not norm_ones else SHAPE_TC
    eng = hb.Engine.create_random(shape, seed=1, std=0.02, norm_ones=norm_ones, max_seq_len=128,
                                  bf16=True, max_batch=16)
    cfg = R.LlamaTpConfig(**shape)
    weights = fetch_weights(eng, cfg)
    w = weights["model.layers.0.mlp.down_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 2e-3 and abs(float(w.mean())) < 1e-3
    oracle = R.LlamaTpOracle(cfg, weights, world_size=1, dtype="bf16")
    rng = np.random.default_rng(0)
    B, plen = 16, 20
    prompts = rng.integers(0, cfg.vocab_size, size=(B, plen)).astype(np.uint32)
    seqs = [eng.create_kv_cache() for _ in range(B)]
    caches = [oracle.new_cache() for _ in range(B)]
    # lock-step prefill through the batched decode step
    logits = np.empty((B, cfg.vocab_size), dtype=np.float32)
    for t in range(plen):
        eng.decode_batch(seqs, prompts[:, t], logits=logits)
    want = np.stack([oracle.forward(prompts[i].tolist(), 0, caches[i]) for i in range(B)])
    assert rel_err(logits, want) <= 2e-2
    agree = np.mean(np.argmax(logits, 1) == np.argmax(want, 1))
    last = np.argmax(want, 1).astype(np.uint32)
    for step in range(3):
        got = eng.decode_batch(seqs, last, logits=logits)
        want = np.stack([oracle.forward([int(last[i])], plen + step, caches[i]) for i in range(B)])
        assert rel_err(logits, want) <= 2e-2
        assert np.array_equal(got, np.argmax(logits, 1).astype(np.uint32))
        last = np.argmax(want, 1).astype(np.uint32)
    if norm_ones:
        assert agree >= 0.9  # bf16 logits of a random model are near-tied; fp32 parity is the tight gate
    assert eng.last_step_ms() > 0 and eng.last_step_launches() > 0
    eng.close()


@pytest.mark.parametrize("B", [1, 16, 48])
def test_rope_epilogue_matches_separate_kernel(hb, cuda, B, monkeypatch):
    """RoPE and the paged KV write in the epilogue of the q|k|v GEMM (the default when a
    head is one output tile) against the separate RoPE + KV kernel (HB_ROPE_EPI=0): the
    roundings fall in the same places, so logits and tokens are identical bit for bit."""
    outs = []
    for mode in ("1", "0"):
        monkeypatch.setenv("HB_ROPE_EPI", mode)
        eng = hb.Engine.create_random(SHAPE_TC128, seed=3, std=0.02, norm_ones=False, max_seq_len=64,
                                      bf16=True, max_batch=B)
        rng = np.random.default_rng(1)
        prompts = rng.integers(0, SHAPE_TC128["vocab_size"], size=(B, 24)).astype(np.uint32)
        seqs = [eng.create_kv_cache() for _ in range(B)]
        logits = np.empty((B, SHAPE_TC128["vocab_size"]), dtype=np.float32)
        got = []
        for t in range(24):
            tok = eng.decode_batch(seqs, prompts[:, t], logits=logits)
            got.append((tok.copy(), logits.copy()))
        launches = eng.last_step_launches()
        # a prompt through the chunked prefill path as well
        seq2 = eng.create_kv_cache()
        pre = eng.forward_with_cache(prompts[0].tolist(), 0, seq2)
        outs.append((got, launches, np.asarray(pre).copy()))
        eng.close()
    (a, la, pa), (b, lb, pb) = outs
    assert la < lb  # one launch per layer less, one table kernel more
    for (ta, xa), (tb, xb) in zip(a, b):
        assert np.array_equal(ta, tb)
        assert np.array_equal(xa, xb)
    assert np.array_equal(pa, pb)


def test_step_bytes_formula(hb, cuda):
    eng = hb.Engine.create_random(SHAPE_TC, max_seq_len=64, bf16=True, max_batch=4)
    H, I, L, V, hd, hq, hkv = 512, 1024, 2, 2048, 64, 8, 2
    ctx = [10, 20]
    w = L * ((hq + 2 * hkv) * hd * H + H * hq * hd + 3 * I * H + 2 * H) * 2 + (V * H + H) * 2 + len(ctx) * H * 2
    kv = sum(ctx) * L * 2 * hkv * hd * 2 + len(ctx) * L * 2 * hkv * hd * 2
    assert eng.step_bytes(ctx) == pytest.approx(w + kv)
    assert eng.param_count() == 2 * V * H + L * (4 * H * H + 3 * H * I)
    eng.close()
