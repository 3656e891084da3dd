"""CPU-side checks of the C ABI: the library loads, exports every symbol the header
declares, and its host logic (sharding, block tables, RoPE table, error reporting)
agrees with the oracle and with the reference's known-answer tests.  No compute call
needs a GPU here."""
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import block_manager_ref as BM
from oracle import kernels_ref as K
from oracle import parallel_ref as P
from tests.test_oracle_kats import run_bm_case

ROOT = Path(__file__).resolve().parent.parent


def header_symbols():
    text = (ROOT / "include" / "hb.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(hb):
    syms = header_symbols()
    assert len(syms) > 60
    for s in syms:
        assert hasattr(hb.lib, s), f"libhb.so does not export {s}"
    # the binding declares a signature for each of them too
    assert set(syms) == set(hb.DECLARED_SYMBOLS)


def test_version_and_device_count(hb):
    assert b"sm_100a" in hb.lib.hb_version()
    assert hb.device_count() >= 0


def test_shard_kats_through_cabi(hb, kats):
    for case in kats["column_shard"]:
        w = np.array(case["w"], dtype=np.float32)
        for rank, exp in enumerate(case["expect"]):
            assert hb.column_shard(w, rank, case["world"]).tolist() == exp
    for case in kats["row_shard"]:
        w = np.array(case["w"], dtype=np.float32)
        for rank, exp in enumerate(case["expect"]):
            assert hb.row_shard(w, rank, case["world"]).tolist() == exp
    nd = kats["shard_not_divisible"]
    w = np.zeros(nd["shape"], dtype=np.float32)
    for fn in (hb.column_shard, hb.row_shard):
        with pytest.raises(hb.HbError) as ei:
            fn(w, 0, nd["world"])
        assert nd["word"] in ei.value.msg and ei.value.code == hb.ERR_NOT_DIVISIBLE


@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.uint16])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shard_matches_oracle_and_round_trips(hb, dtype, world):
    rng = np.random.default_rng(world)
    w = rng.integers(0, 60000, size=(16, 24)).astype(dtype)
    cols = [hb.column_shard(w, r, world) for r in range(world)]
    rows = [hb.row_shard(w, r, world) for r in range(world)]
    for r in range(world):
        assert np.array_equal(cols[r], P.column_shard(w, r, world))
        assert np.array_equal(rows[r], P.row_shard(w, r, world))
    assert np.array_equal(np.concatenate(cols, 0), w)
    assert np.array_equal(np.concatenate(rows, 1), w)


def test_sequence_arithmetic(hb, kats):
    for n, e in kats["sequence"]["num_logical_blocks"]:
        assert hb.lib.hb_num_logical_blocks(n, 16) == e
    for n, e in kats["sequence"]["last_block_num_filled"]:
        assert hb.lib.hb_last_block_num_filled(n, 16) == e
    for n in range(0, 100):
        assert hb.lib.hb_num_logical_blocks(n, 16) == BM.num_logical_blocks(n)
        assert hb.lib.hb_last_block_num_filled(n, 16) == BM.last_block_num_filled(n)


def test_hash_block_bit_exact(hb, kats):
    rng = np.random.default_rng(0)
    assert hb.hash_block([]) == int(kats["fnv1a"]["empty_hash"], 16)
    for _ in range(50):
        t = rng.integers(0, 2 ** 32, size=16, dtype=np.uint64).astype(np.uint32)
        assert hb.hash_block(t) == BM.hash_block(t.tolist())


def test_block_manager_kats_through_cabi(hb, kats):
    for case in kats["block_manager"]:
        run_bm_case(hb.BlockManager, case)


def test_block_manager_bit_exact_random_walk(hb):
    """Same calls on the C++ manager and on the Python restatement of
    src/scheduler/block_manager.rs: every table, free count, copy-on-write pair and
    swap pair must be identical (prefix-cache hits included: prompts share blocks)."""
    rng = np.random.default_rng(42)
    a, b = hb.BlockManager(48, 24), BM.BlockManager(48, 24)
    vocab_blocks = [rng.integers(0, 1000, size=16).astype(np.uint32) for _ in range(6)]
    live, lens, swapped, next_id = [], {}, set(), 0
    for step in range(600):
        op = rng.integers(0, 6)
        if op == 0 or not live:
            nb = int(rng.integers(0, 4))
            tail = rng.integers(0, 1000, size=int(rng.integers(0, 16))).astype(np.uint32)
            prompt = np.concatenate([vocab_blocks[int(rng.integers(0, 6))] for _ in range(nb)] + [tail]).astype(np.uint32)
            if len(prompt) == 0:
                prompt = np.array([1], dtype=np.uint32)
            try:
                hb_hits = a.allocate(next_id, prompt)
                ok_a = True
            except hb.HbError:
                ok_a = False
            try:
                py_hits = b.allocate(next_id, prompt.tolist())
                ok_b = True
            except RuntimeError:
                ok_b = False
            assert ok_a == ok_b
            if ok_a:
                assert hb_hits == py_hits
                live.append(next_id)
                lens[next_id] = len(prompt)
            next_id += 1
        elif op in (1, 2):
            sid = live[int(rng.integers(0, len(live)))]
            if sid in swapped:
                continue
            assert a.can_append_slot(sid, lens[sid]) == b.can_append_slot(sid, lens[sid])
            if b.can_append_slot(sid, lens[sid]):
                assert a.append_slot(sid, lens[sid]) == b.append_slot(sid, lens[sid])
                lens[sid] += 1
        elif op == 3:
            sid = live.pop(int(rng.integers(0, len(live))))
            swapped.discard(sid)
            a.free(sid)
            b.free(sid)
        elif op == 4:
            sid = live[int(rng.integers(0, len(live)))]
            if sid not in swapped and b.num_free_cpu_blocks() >= len(b.get_block_table(sid)):
                assert a.swap_out(sid) == b.swap_out(sid)
                swapped.add(sid)
        else:
            sid = live[int(rng.integers(0, len(live)))]
            if sid in swapped and b.num_free_gpu_blocks() >= len(b.get_block_table(sid)):
                assert a.swap_in(sid) == b.swap_in(sid)
                swapped.discard(sid)
        assert a.num_free_gpu_blocks() == b.num_free_gpu_blocks()
        assert a.num_free_cpu_blocks() == b.num_free_cpu_blocks()
        assert a.num_prefix_cached_blocks() == b.num_prefix_cached_blocks()
        for sid in live:
            assert a.get_block_table(sid) == b.get_block_table(sid)
    assert a.get_block_table(10 ** 9) is None


def test_slot_mapping(hb):
    table = np.array([7, 3, 11], dtype=np.int64)
    for pos in range(48):
        assert hb.lib.hb_slot_for_position(table.ctypes.data, 3, pos) == K.slot_for_position(table.tolist(), pos)
    assert hb.lib.hb_slot_for_position(table.ctypes.data, 3, 48) == -1


@pytest.mark.parametrize("theta,hd", [(10000.0, 64), (500000.0, 128), (1e6, 128), (10000.0, 8)])
def test_rope_inv_freq_table(hb, theta, hd):
    got = hb.kernels.rope.inv_freq(theta, hd)
    want = K.rope_inv_freq(theta, hd)
    assert got.shape == (hd // 2,) and got[0] == 1.0
    assert np.max(np.abs(got - want) / want) < 1e-6  # f32 powf: within an ulp or two


def test_errors_are_reported_not_thrown(hb):
    with pytest.raises(hb.HbError) as ei:
        hb.kernels.rope.inv_freq(10000.0, 7)
    assert ei.value.code == hb.ERR_INVALID_ARG and "head_dim" in ei.value.msg
    assert hb.lib.hb_bm_create(-1, 0, None) == hb.ERR_INVALID_ARG
    assert hb.lib.hb_world_size(None) == hb.ERR_INVALID_ARG
    # TpWorld::new(64): the message names tensor_parallel_size or CUDA (world.rs:243-252)
    with pytest.raises(hb.HbError) as ei:
        hb.TpWorld.new_local(64)
    assert "tensor_parallel_size" in ei.value.msg or "CUDA" in ei.value.msg


def test_no_fallback_without_gpu(hb):
    if hb.device_count() > 0:
        pytest.skip("a GPU is present")
    x = np.zeros((2, 8), dtype=np.float32)
    rc = hb.lib.hb_rms_norm(None, x.ctypes.data, x.ctypes.data, x.ctypes.data, 2, 8, 1e-5, hb.F32)
    assert rc == hb.ERR_CUDA  # fails loudly; host memory is never computed on
    with pytest.raises(hb.HbError):
        hb.Engine.create_random(dict(hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                                     num_attention_heads=2, vocab_size=64))


def test_missing_library_fails_the_import(tmp_path):
    """There is no fallback path: without the built library (here: HB_LIBRARY pointing at a
    file that does not exist) importing the package raises instead of degrading."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    code = ("import sys; sys.path.insert(0, %r); import __graft_entry__ as e\n"
            "try:\n    e.load_package()\nexcept ImportError as ex:\n    print('IMPORT-ERROR', ex); sys.exit(7)\n"
            "sys.exit(0)\n") % str(root)
    env = dict(**__import__("os").environ, HB_LIBRARY=str(tmp_path / "libhb_absent.so"))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert res.returncode == 7, res.stdout + res.stderr
    assert "IMPORT-ERROR" in res.stdout and "libhb_absent.so" in res.stdout
