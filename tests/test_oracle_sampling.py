"""The sampling oracle against the reference's own known answers
(src/sampling/nucleus.rs:69-86, src/sampling/penalty.rs:72-139), transcribed in
tests/golden/reference_kats.json."""
import numpy as np

from oracle import sampling_ref as S


def test_softmax_sums_to_one(kats):
    case = kats["sampling"]["softmax_sums_to_one"]
    p = S.softmax(np.array(case["logits"], dtype=np.float32))
    assert abs(float(p.sum()) - 1.0) < case["tol"]


def test_nucleus_filter_keeps_top_mass(kats):
    case = kats["sampling"]["nucleus_filter_keeps_top_mass"]
    p = S.nucleus_filter(np.array(case["probs"], dtype=np.float32), case["top_p"])
    assert all(p[i] == 0.0 for i in case["zero"]) and all(p[i] > 0.0 for i in case["positive"])


def test_penalties(kats):
    for case in kats["sampling"]["penalties"]:
        got = S.apply_penalties(np.array(case["logits"], dtype=np.float32), np.array(case["counts"], dtype=np.uint32),
                                case["presence"], case["frequency"])
        assert np.allclose(got, case["expect"], atol=1e-5), case


def test_count_tokens(kats):
    for case in kats["sampling"]["count_tokens"]:
        assert S.count_tokens(case["ids"], case["vocab"]).tolist() == case["expect"]


def test_pipeline_properties():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(1000).astype(np.float32) * 3
    greedy = S.logits_to_probs(x, 0.0, 1.0)
    assert greedy[int(np.argmax(x))] == 1.0 and greedy.sum() == 1.0
    p = S.logits_to_probs(x, 0.7, 0.9)
    assert abs(float(p.sum()) - 1.0) < 1e-5
    kept = np.sort(S.softmax(x / np.float32(0.7)))[::-1]
    n_kept = int(np.count_nonzero(p))
    assert kept[:n_kept].sum() >= 0.9 - 1e-6 and kept[:n_kept - 1].sum() < 0.9 + 1e-6
    # the draw is the inverse CDF: u = 0 gives the first token with mass, u -> 1 the last
    assert S.draw(p, 0.0) == int(np.nonzero(p)[0][0])
    assert S.draw(p, 0.999999) == int(np.nonzero(p)[0][-1])
    assert 0.0 <= S.uniform_from_seed(123) < 1.0 and S.uniform_from_seed(123) == S.uniform_from_seed(123)
