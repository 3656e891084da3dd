"""On-device sampling against the oracle's restatement of src/sampling/ (penalties,
temperature, softmax, top-p, renormalisation: within 1e-3 relative in fp32; the draw: the same
token for the same uniform number), and speculative verification as one forward
(src/speculative.rs:174-212) against token-by-token forwards."""
import numpy as np
import pytest
import torch

from oracle import llama_ref as R
from oracle import sampling_ref as S

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("vocab", [50, 4096, 128256])
@pytest.mark.parametrize("temperature,top_p", [(1.0, 1.0), (0.7, 0.9), (1.3, 0.5), (0.0, 1.0), (0.5, 0.05)])
def test_probabilities_match_the_oracle(hb, cuda, vocab, temperature, top_p):
    rng = np.random.default_rng(vocab)
    n = 5
    logits = (rng.standard_normal((n, vocab)) * 2.5).astype(np.float32)
    counts = np.zeros((n, vocab), dtype=np.uint32)
    for i in range(n):
        seen = rng.integers(0, vocab, size=40)
        np.add.at(counts[i], seen, 1)
    for presence, frequency in ((0.0, 0.0), (0.6, 0.4)):
        got = hb.logits_to_probs(torch.from_numpy(logits).to(cuda), temperature, top_p,
                                 torch.from_numpy(counts.view(np.int32)).to(cuda), presence, frequency).cpu().numpy()
        for i in range(n):
            want = S.logits_to_probs(logits[i], temperature, top_p, counts[i], presence, frequency)
            assert abs(float(got[i].sum()) - 1.0) < 1e-4
            # the kept sets agree, except for tokens sitting exactly on the nucleus boundary
            diff = np.nonzero((got[i] > 0) != (want > 0))[0]
            assert len(diff) <= 1, (i, diff)
            same = (got[i] > 0) & (want > 0)
            assert np.max(np.abs(got[i][same] - want[same])) <= 1e-3 * float(want.max()) + (0.0 if len(diff) == 0 else 1e-2)


def test_known_answers_on_the_device(hb, cuda, kats):
    case = kats["sampling"]["nucleus_filter_keeps_top_mass"]
    logits = np.log(np.array([case["probs"]], dtype=np.float32))
    p = hb.logits_to_probs(torch.from_numpy(logits).to(cuda), 1.0, case["top_p"]).cpu().numpy()[0]
    assert all(p[i] == 0.0 for i in case["zero"]) and all(p[i] > 0.0 for i in case["positive"])
    for pc in kats["sampling"]["penalties"]:
        lg = np.array([pc["logits"]], dtype=np.float32)
        ct = np.array([pc["counts"]], dtype=np.int32)
        got = hb.logits_to_probs(torch.from_numpy(lg).to(cuda), 1.0, 1.0, torch.from_numpy(ct).to(cuda), pc["presence"],
                                 pc["frequency"]).cpu().numpy()[0]
        want = S.softmax(np.array(pc["expect"], dtype=np.float32))
        assert np.allclose(got, want, atol=1e-5), pc


def test_seeded_draw(hb, cuda):
    rng = np.random.default_rng(3)
    n, vocab = 64, 32000
    logits = (rng.standard_normal((n, vocab)) * 3).astype(np.float32)
    seeds = rng.integers(0, 2 ** 62, size=n).astype(np.int64)
    toks, probs = hb.sample(torch.from_numpy(logits).to(cuda), torch.from_numpy(seeds).to(cuda), 0.8, 0.95)
    toks2, _ = hb.sample(torch.from_numpy(logits).to(cuda), torch.from_numpy(seeds).to(cuda), 0.8, 0.95)
    assert torch.equal(toks, toks2)                                  # same seed, same token
    toks, probs = toks.cpu().numpy(), probs.cpu().numpy()
    for i in range(n):
        u = S.uniform_from_seed(int(seeds[i]))
        c = np.cumsum(probs[i].astype(np.float64))
        want = S.draw(probs[i], u)
        # the device sums in fp32: a target within rounding of a boundary may fall one token aside
        near = abs(c[want] - u * c[-1]) < 1e-5 or (want > 0 and abs(c[want - 1] - u * c[-1]) < 1e-5)
        assert toks[i] == want or (near and probs[i][toks[i]] > 0), (i, toks[i], want)
        assert probs[i][toks[i]] > 0
    # greedy needs no seeds
    g, _ = hb.sample(torch.from_numpy(logits).to(cuda), None, 0.0)
    assert np.array_equal(g.cpu().numpy(), np.argmax(logits, 1))
    # the draws follow the distribution: chi-square over the five most likely tokens of one row
    row = np.tile(logits[:1], (4096, 1))
    s2 = np.arange(4096, dtype=np.int64) * 7919 + 11
    t4, p4 = hb.sample(torch.from_numpy(row).to(cuda), torch.from_numpy(s2).to(cuda), 1.0, 1.0)
    p0 = p4[0].cpu().numpy()
    top = np.argsort(-p0)[:5]
    freq = np.array([(t4.cpu().numpy() == t).mean() for t in top])
    assert np.all(np.abs(freq - p0[top]) < 4 * np.sqrt(p0[top] * (1 - p0[top]) / 4096) + 1e-3)


def test_speculative_verify_is_one_forward(hb, cuda, tmp_path):
    cfg = R.TINY_CONFIG
    weights = R.random_weights(cfg, seed=1, std=0.02, norm_ones=True)
    R.write_model(str(tmp_path), cfg, weights)
    eng = hb.Engine.load(str(tmp_path), max_seq_len=128, bf16=False, force_f32=True, max_batch=8)
    oracle = R.LlamaTpOracle(cfg, weights, world_size=1, dtype="f32")
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, cfg.vocab_size, size=21).astype(np.uint32)
    seq = eng.create_kv_cache()
    eng.forward_with_cache(prompt[:-1], 0, seq)
    cache = oracle.new_cache()
    oracle.forward(prompt[:-1].tolist(), 0, cache)
    draft = rng.integers(0, cfg.vocab_size, size=4).astype(np.uint32)      # K = 4 draft tokens
    feed = np.concatenate([prompt[-1:], draft])                           # [last, d0..d3]: K+1 target positions
    got = eng.forward_all_positions(feed, len(prompt) - 1, seq)
    assert got.shape == (5, cfg.vocab_size) and len(seq) == len(prompt) + 4
    for i, tok in enumerate(feed):
        want = oracle.forward([int(tok)], len(prompt) - 1 + i, cache)      # what K+1 sequential forwards give
        assert float(np.max(np.abs(got[i] - want))) <= 1e-3 * float(np.max(np.abs(want)))
    # two drafts accepted: the rejected tokens' K/V are dropped and decoding continues from there
    eng.truncate(seq, len(prompt) + 2)
    assert len(seq) == len(prompt) + 2
    cache2 = oracle.new_cache()
    oracle.forward(np.concatenate([prompt, draft[:2]]).tolist(), 0, cache2)
    nxt = 777
    want = oracle.forward([nxt], len(prompt) + 2, cache2)
    got2 = eng.forward_with_cache([nxt], len(prompt) + 2, seq)
    assert float(np.max(np.abs(got2 - want))) <= 1e-3 * float(np.max(np.abs(want)))
    with pytest.raises(hb.HbError):
        eng.truncate(seq, 10 ** 6)
    eng.close()
