"""The CPU oracle against every known-answer test the reference holds for the path
(tests/golden/reference_kats.json; each entry cites its reference test)."""
import json

import numpy as np
import pytest

from oracle import block_manager_ref as BM
from oracle import kernels_ref as K
from oracle import llama_ref as R
from oracle import parallel_ref as P


def test_all_reduce_kats(kats):
    for case in kats["all_reduce"]:
        shards = [np.array(s, dtype=np.float32).reshape(case["shape"]) for s in case["shards"]]
        out = P.all_reduce(shards)
        assert out.dtype == np.float32  # all_reduce_preserves_dtype
        assert out.reshape(-1).tolist() == case["expect"], case["cite"]
        assert P.all_reduce_f32(shards).reshape(-1).tolist() == case["expect"]


def test_all_reduce_empty(kats):
    with pytest.raises(ValueError, match=kats["all_reduce_empty_error_contains"]["word"]):
        P.all_reduce([])
    with pytest.raises(ValueError, match="empty"):
        P.all_gather([], 0)


def test_all_gather_kats(kats):
    for case in kats["all_gather"]:
        out = P.all_gather([np.array(s, dtype=np.float32) for s in case["shards"]], case["dim"])
        assert out.tolist() == case["expect"], case["cite"]


def test_shard_kats(kats):
    for case in kats["column_shard"]:
        w = np.array(case["w"], dtype=np.float32)
        for rank, exp in enumerate(case["expect"]):
            assert P.column_shard(w, rank, case["world"]).tolist() == exp, case["cite"]
    for case in kats["row_shard"]:
        w = np.array(case["w"], dtype=np.float32)
        for rank, exp in enumerate(case["expect"]):
            assert P.row_shard(w, rank, case["world"]).tolist() == exp, case["cite"]
    for case in kats["column_shard_shapes"]:
        w = np.zeros(case["shape"], dtype=np.float32)
        for rank in range(case["world"]):
            assert list(P.column_shard(w, rank, case["world"]).shape) == case["expect_shape"]
    for case in kats["row_shard_shapes"]:
        w = np.zeros(case["shape"], dtype=np.float32)
        for rank in range(case["world"]):
            assert list(P.row_shard(w, rank, case["world"]).shape) == case["expect_shape"]
    nd = kats["shard_not_divisible"]
    w = np.zeros(nd["shape"], dtype=np.float32)
    with pytest.raises(ValueError, match=nd["word"]):
        P.column_shard(w, 0, nd["world"])
    with pytest.raises(ValueError, match=nd["word"]):
        P.row_shard(w, 0, nd["world"])
    b = kats["bias_shard"]
    for rank, exp in enumerate(b["expect"]):
        assert P.bias_shard(np.array(b["b"], dtype=np.float32), rank, b["world"]).tolist() == exp
    for o, n, e in kats["chunk_sizes"]["column"]:
        assert P.column_chunk_size(o, n) == e
    for o, n, e in kats["chunk_sizes"]["row"]:
        assert P.row_chunk_size(o, n) == e
    rt = kats["shard_round_trip"]
    w = np.arange(12, dtype=np.float32).reshape(rt["column_shape"])
    assert np.array_equal(np.concatenate([P.column_shard(w, r, 2) for r in range(2)], 0), w)
    w = np.arange(12, dtype=np.float32).reshape(rt["row_shape"])
    assert np.array_equal(np.concatenate([P.row_shard(w, r, 2) for r in range(2)], 1), w)


def test_world_size_rules(kats):
    P.world_size_check(1, 0)
    with pytest.raises(ValueError) as ei:
        P.world_size_check(kats["world"]["too_large"], 8)
    assert any(w in str(ei.value) for w in kats["world"]["error_mentions_any_of"])


def test_rms_norm_kats(kats):
    for case in kats["rms_norm"]:
        x = np.array(case["x"], dtype=np.float32)
        w = np.array(case["w"], dtype=np.float32)
        for fn in (K.rms_norm_kernel, K.rms_norm_fallback):
            out = fn(x, w, case["eps"])
            if "expect_mean_square" in case:
                assert abs(float(np.mean(out ** 2)) - case["expect_mean_square"]) < case["tol"], case["cite"]
            else:
                assert np.all(np.abs(out) < case["expect_all_abs_below"]), case["cite"]


def test_rope_kats(kats):
    c = kats["rope"]["preserves_shape"]
    q = np.random.default_rng(0).standard_normal(c["shape"]).astype(np.float32)
    cos, sin = K.rope_tables(np.arange(c["seq_pos"], c["seq_pos"] + c["shape"][0]), c["theta"], c["shape"][2])
    assert K.apply_rope(q, cos, sin).shape == q.shape
    c = kats["rope"]["pos0_pos1_differ"]
    q = np.full(c["shape"], c["fill"], dtype=np.float32)
    outs = []
    for pos in (0, 1):
        cos, sin = K.rope_tables(np.array([pos]), c["theta"], c["shape"][2])
        outs.append(K.apply_rope(q, cos, sin))
    assert not np.array_equal(outs[0], outs[1])
    # position 0 is the identity rotation
    assert np.array_equal(outs[0], q)


def test_causal_mask_kats(kats):
    a, b, c = kats["causal_mask"]
    assert list(K.causal_mask(a["sq"], a["sk"], a["seq_pos"]).shape) == a["expect_shape"]
    m = K.causal_mask(b["sq"], b["sk"], b["seq_pos"])
    for i in range(4):
        for j in range(4):
            assert (m[i, j] == 0.0) if j <= i else (np.isinf(m[i, j]) and m[i, j] < 0)
    assert np.all(K.causal_mask(c["sq"], c["sk"], c["seq_pos"]) == 0.0)


def test_config_kats(kats):
    a, b = kats["config"]
    assert R.LlamaTpConfig.from_json(a["json"]).kv_heads() == a["kv_heads"]
    assert R.LlamaTpConfig.from_json(b["json"]).head_dim() == b["head_dim"]
    cfg = R.LlamaTpConfig.from_json(a["json"])
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0  # serde defaults


def test_sequence_kats(kats):
    for n, e in kats["sequence"]["num_logical_blocks"]:
        assert BM.num_logical_blocks(n) == e
    for n, e in kats["sequence"]["last_block_num_filled"]:
        assert BM.last_block_num_filled(n) == e


def run_bm_case(make, case):
    bm = make(case["gpu"], case["cpu"])
    for n, e in case.get("can_allocate", []):
        assert bm.can_allocate(n) == e, case["cite"]
    for op in case.get("ops", []):
        if op[0] == "allocate":
            bm.allocate(op[1], [0] * op[2])
        elif op[0] == "allocate_fails":
            with pytest.raises(Exception):
                bm.allocate(op[1], [0] * op[2])
        elif op[0] == "free":
            bm.free(op[1])
        elif op[0] == "expect_free_gpu":
            assert bm.num_free_gpu_blocks() == op[1], case["cite"]
        elif op[0] == "expect_table_len":
            assert len(bm.get_block_table(op[1])) == op[2], case["cite"]
        elif op[0] == "swap_out":
            assert len(bm.swap_out(op[1])) == op[2], case["cite"]
        elif op[0] == "swap_in":
            assert len(bm.swap_in(op[1])) == op[2], case["cite"]
    if "free_gpu" in case:
        assert bm.num_free_gpu_blocks() == case["free_gpu"], case["cite"]
    if "free_cpu" in case:
        assert bm.num_free_cpu_blocks() == case["free_cpu"], case["cite"]


def test_block_manager_kats(kats):
    for case in kats["block_manager"]:
        run_bm_case(BM.BlockManager, case)


def test_prefix_cache_kats(kats):
    pc = kats["prefix_cache"]
    t = pc["hash_deterministic_tokens"]
    assert BM.hash_block(t) == BM.hash_block(list(t))
    a, b = pc["hash_differs"]
    assert BM.hash_block(a) != BM.hash_block(b)
    sw = list(t)
    i, j = pc["hash_order_sensitive_swap"]
    sw[i], sw[j] = sw[j], sw[i]
    assert BM.hash_block(sw) != BM.hash_block(t)
    assert BM.hash_block([]) == int(kats["fnv1a"]["empty_hash"], 16)
    ev = pc["evicts_oldest"]
    c = BM.PrefixCache(ev["capacity"])
    for h, i in ev["inserts"]:
        c.insert(h, i)
    for h in ev["missing"]:
        assert c.lookup(h) is None
    for h, i in ev["present"]:
        assert c.lookup(h) == i
    up = pc["insert_same_hash_updates"]
    c = BM.PrefixCache(up["capacity"])
    for h, i in up["inserts"]:
        c.insert(h, i)
    assert c.lookup(up["lookup"][0]) == up["lookup"][1] and len(c) == up["len"]
    rm = pc["remove_by_block_id"]
    c = BM.PrefixCache(rm["capacity"])
    c.insert(*rm["insert"])
    c.remove_by_block_id(rm["remove"])
    assert c.lookup(rm["insert"][0]) is None
    assert BM.PrefixCache(8).lookup(42) is None


def test_kv_slot_assign_formula():
    """kernels/kv_assign.cu:26 index formula on a small buffer."""
    nkv, max_seq, hd = 3, 5, 4
    buf = np.arange(nkv * max_seq * hd, dtype=np.float32).reshape(nkv, max_seq, hd)
    src = -np.arange(1, nkv * hd + 1, dtype=np.float32).reshape(nkv, hd)
    out = K.kv_slot_assign(buf, src, 2)
    exp = buf.copy()
    exp[:, 2, :] = src
    assert np.array_equal(out, exp)
    assert BM.BLOCK_SIZE == 16 and K.slot_for_position([7, 3], 17) == 3 * 16 + 1
