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


def greedy_report(got, want, band=2e-2):
    """Greedy agreement between two [n, vocab] logit stacks: over all rows, and over the rows
    the oracle itself decides clearly (top-1 margin above twice the logit tolerance `band`,
    relative to the largest |logit|: inside that band a flip is a tie-break that both logit
    vectors satisfy within tolerance).  Also the oracle margins of the rows that flipped."""
    got, want = np.asarray(got), np.asarray(want)
    a, b = np.argmax(got, -1), np.argmax(want, -1)
    scale = float(np.max(np.abs(want)))
    top2 = np.partition(want, -2, axis=-1)[:, -2:]
    margin = (top2[:, 1] - top2[:, 0]) / scale
    clear = margin > 2 * band
    agree_clear = float(np.mean(a[clear] == b[clear])) if clear.any() else 1.0
    return float(np.mean(a == b)), agree_clear, int(clear.sum()), [float(m) for m in margin[a != b]]


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
    n_new, agree, total = 32, 0, 0   # 1 prefill + 31 decode forwards (src/worker/mod.rs:349-358,404-409)
    for p in prompts:
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


@pytest.mark.parametrize("file_dtype,engine", [("BF16", "bf16"), ("F16", "bf16"), ("F32", "bf16"), ("BF16", "f32")])
def test_checkpoint_dtypes(hb, cuda, tiny, tmp_path, file_dtype, engine):
    """Checkpoints in bf16 (native: the slices go from the mapped file to the device as they
    are) and in other dtypes (converted on the device): the tensors on the device equal the
    file's values rounded to the engine dtype, bit for bit."""
    from oracle import kernels_ref as K

    cfg, weights, _ = tiny
    R.write_model(str(tmp_path), cfg, weights, dtype=file_dtype)
    eng = hb.Engine.load(str(tmp_path), max_seq_len=32, bf16=engine == "bf16", force_f32=engine == "f32", max_batch=2)
    for name in ("model.layers.1.mlp.down_proj.weight", "model.layers.0.self_attn.k_proj.weight", "model.norm.weight",
                 "lm_head.weight"):
        in_file = K.rnd(weights[name], {"BF16": "bf16", "F16": "f16", "F32": "f32"}[file_dtype])
        want = K.rnd(in_file, engine)
        assert np.array_equal(eng.get_tensor(name).reshape(want.shape), want), name
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


def rewrite_header(src_dir, dst_dir, edit):
    """Copy a model directory, passing the safetensors JSON header through `edit`."""
    import json
    import os
    import shutil

    os.makedirs(dst_dir, exist_ok=True)
    shutil.copy(os.path.join(src_dir, "config.json"), dst_dir)
    raw = open(os.path.join(src_dir, "model.safetensors"), "rb").read()
    hlen = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + hlen])
    edit(header)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(os.path.join(dst_dir, "model.safetensors"), "wb") as f:
        f.write(len(h).to_bytes(8, "little") + h + raw[8 + hlen:])
    return str(dst_dir)


def test_malformed_checkpoints_are_refused(hb, cuda, tiny, tmp_path):
    """A header whose offsets, shapes or sizes do not add up ends in HB_ERR_IO, never in a read
    past the mapping or a silently mis-sharded tensor."""
    cfg, weights, path = tiny
    name = "model.layers.0.self_attn.q_proj.weight"

    def truncated(h):        # fewer bytes than shape x dtype
        b, e = h[name]["data_offsets"]
        h[name]["data_offsets"] = [b, e - 64]

    def transposed(h):       # right element count, wrong shape: must not be sharded as if it were right
        name2 = "model.layers.0.mlp.down_proj.weight"
        h[name2]["shape"] = h[name2]["shape"][::-1]

    def negative(h):
        h[name]["shape"] = [-256, -256]

    def fractional(h):
        b, e = h[name]["data_offsets"]
        h[name]["data_offsets"] = [b + 0.5, e]

    def past_the_end(h):
        b, e = h[name]["data_offsets"]
        h[name]["data_offsets"] = [b + 10 ** 12, e + 10 ** 12]

    def mislabelled(h):      # same bytes declared as a 2-byte type
        h[name]["dtype"] = "BF16"

    for i, edit in enumerate((truncated, transposed, negative, fractional, past_the_end, mislabelled)):
        bad = rewrite_header(path, tmp_path / f"bad{i}", edit)
        with pytest.raises(hb.HbError) as ei:
            hb.Engine.load(bad, max_seq_len=32, bf16=False, force_f32=True, max_batch=2)
        assert ei.value.code == hb.ERR_IO, (edit.__name__, ei.value.msg)


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


@pytest.mark.parametrize("shape", [SHAPE_TC, SHAPE_TC128], ids=["hd64", "hd128"])
@pytest.mark.parametrize("norm_ones", [True, False])
@pytest.mark.parametrize("eager", [True, False], ids=["eager-oracle", "kernel-oracle"])
def test_random_init_bf16_tensor_core_path(hb, cuda, norm_ones, shape, eager):
    """Device-initialised bf16 model on the tcgen05 GEMM path; the oracle runs on the
    very weights read back from the device, once with the reference's multi-op bf16 norm and
    RoPE (src/kernels/rms_norm.rs:128-132, llama_tp.rs:135-149) and once with its fused-kernel
    numerics (kernels/rms_norm.cu:74-110)."""
    eng = hb.Engine.create_random(shape, seed=1, std=0.02, norm_ones=norm_ones, max_seq_len=128,
                                  bf16=True, max_batch=16)
    cfg = R.LlamaTpConfig(**shape)
    weights = fetch_weights(eng, cfg)
    w = weights["model.layers.0.mlp.down_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 2e-3 and abs(float(w.mean())) < 1e-3
    oracle = R.LlamaTpOracle(cfg, weights, world_size=1, dtype="bf16", eager=eager, weights_exact=True)
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
    all_got, all_want = [logits.copy()], [want]
    last = np.argmax(want, 1).astype(np.uint32)
    for step in range(3):
        got = eng.decode_batch(seqs, last, logits=logits)
        want = np.stack([oracle.forward([int(last[i])], plen + step, caches[i]) for i in range(B)])
        assert rel_err(logits, want) <= 2e-2
        assert np.array_equal(got, np.argmax(logits, 1).astype(np.uint32))
        all_got.append(logits.copy()); all_want.append(want)
        last = np.argmax(want, 1).astype(np.uint32)
    # greedy agreement over the 64 teacher-forced tokens: every flip must be a near-tie of the
    # oracle itself (top-1 margin inside the logit tolerance); with unit norm weights the
    # logits are spread enough for >= 99 % agreement outright
    agree, agree_clear, n_clear, margins = greedy_report(np.concatenate(all_got), np.concatenate(all_want))
    print(f"greedy agreement {agree:.4f} over 64 tokens, {agree_clear:.4f} over the {n_clear} the oracle decides "
          f"clearly; oracle top-1 margins of the flips {margins}")
    assert agree_clear >= 0.99, (agree_clear, margins)    # the north-star gate, on decidable tokens
    assert all(m <= 2 * 2e-2 for m in margins), margins   # every flip is a tie inside the tolerance band
    if norm_ones:
        assert agree >= 0.95, (agree, margins)
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


def test_8b_widths_two_layers(hb, cuda):
    """Two layers at the Llama-3.1-8B widths (hidden 4096, FFN 14336, 32/8 heads of 128, vocabulary
    128256) with B = 64: the plans the benchmark runs (deferred norm over 32 row-sum tiles,
    RoPE + KV write in the q|k|v epilogue, 8-way cluster split-K, fp32 logits GEMM over the full
    vocabulary) against the oracle on the weights read back from the device."""
    shape = dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=2, num_attention_heads=32,
                 num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)
    B, plen, n_check = 64, 5, 16
    eng = hb.Engine.create_random(shape, seed=7, std=0.02, norm_ones=True, max_seq_len=32, bf16=True, max_batch=B)
    cfg = R.LlamaTpConfig(**shape)
    oracle = R.LlamaTpOracle(cfg, fetch_weights(eng, cfg), world_size=1, dtype="bf16", weights_exact=True)
    prompts = np.random.default_rng(0).integers(0, cfg.vocab_size, size=(B, plen)).astype(np.uint32)
    seqs = [eng.create_kv_cache() for _ in range(B)]
    logits = np.empty((B, cfg.vocab_size), dtype=np.float32)
    for t in range(plen):
        tok = eng.decode_batch(seqs, prompts[:, t], logits=logits)
    assert np.array_equal(tok, np.argmax(logits, 1).astype(np.uint32))   # device argmax over 128256 entries
    # the oracle on a sample of the sequences (one lm_head product for all of them)
    rows = np.linspace(0, B - 1, n_check).astype(int)
    hidden = np.stack([oracle.forward(prompts[i].tolist(), 0, oracle.new_cache(), logits=False)[-1] for i in rows])
    want = oracle.final_logits(hidden)
    assert rel_err(logits[rows], want) <= 2e-2
    agree, agree_clear, n_clear, margins = greedy_report(logits[rows], want)
    print(f"8B widths: greedy agreement {agree:.4f}, {agree_clear:.4f} over {n_clear} clearly decided; flips {margins}")
    assert agree_clear >= 0.99 and all(m <= 2 * 2e-2 for m in margins), (agree_clear, margins)
    eng.close()


@pytest.mark.parametrize("heads,kv_heads", [(8, 2), (8, 1), (4, 4)], ids=["nrep4", "nrep8", "nrep1"])
def test_prefill_chunks_share_the_kv_stream(hb, cuda, heads, kv_heads):
    """A multi-token forward runs as chunks of consecutive positions; on the tensor-core
    attention path 16 / n_rep of them share a CTA (each MMA row with its own causal limit,
    src/engine/arch/llama_tp.rs:313-316).  The logits must equal those of feeding the same
    tokens one at a time, and match the oracle's masked prefill."""
    shape = dict(hidden_size=128 * heads, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=heads,
                 num_key_value_heads=kv_heads, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=500000.0)
    eng = hb.Engine.create_random(shape, seed=9, std=0.02, norm_ones=True, max_seq_len=128, bf16=True, max_batch=16)
    cfg = R.LlamaTpConfig(**shape)
    oracle = R.LlamaTpOracle(cfg, fetch_weights(eng, cfg), world_size=1, dtype="bf16", weights_exact=True)
    prompt = np.random.default_rng(4).integers(0, cfg.vocab_size, size=45).astype(np.uint32)   # chunks of 16, 16, 13
    chunked = eng.create_kv_cache()
    got = eng.forward_with_cache(prompt, 0, chunked)
    one_by_one = eng.create_kv_cache()
    for i, tok in enumerate(prompt):
        ref = eng.forward_with_cache([int(tok)], i, one_by_one)
    assert rel_err(got, ref) <= 2e-3          # same kernels, same order of the blocks per warp
    want = oracle.forward(prompt.tolist(), 0, oracle.new_cache())
    assert rel_err(got, want) <= 2e-2
    # and the cache the chunks wrote serves a following decode step
    tok = int(np.argmax(want))
    assert rel_err(eng.forward_with_cache([tok], len(prompt), chunked),
                   eng.forward_with_cache([tok], len(prompt), one_by_one)) <= 2e-3
    # every position's logits (speculative verification) through the grouped kernel as well
    seq3 = eng.create_kv_cache()
    allpos = eng.forward_all_positions(prompt[:20], 0, seq3)
    seq4 = eng.create_kv_cache()
    for i in range(20):
        ref_i = eng.forward_with_cache([int(prompt[i])], i, seq4)
        assert rel_err(allpos[i], ref_i) <= 2e-3, i
    eng.close()


def test_step_bytes_formula(hb, cuda):
    eng = hb.Engine.create_random(SHAPE_TC, max_seq_len=64, bf16=True, max_batch=4)
    H, I, L, V, hd, hq, hkv = 512, 1024, 2, 2048, 64, 8, 2
    ctx = [10, 20]
    w = L * ((hq + 2 * hkv) * hd * H + H * hq * hd + 3 * I * H + 2 * H) * 2 + (V * H + H) * 2 + len(ctx) * H * 2
    kv = sum(ctx) * L * 2 * hkv * hd * 2 + len(ctx) * L * 2 * hkv * hd * 2
    assert eng.step_bytes(ctx) == pytest.approx(w + kv)
    assert eng.param_count() == 2 * V * H + L * (4 * H * H + 3 * H * I)
    eng.close()
