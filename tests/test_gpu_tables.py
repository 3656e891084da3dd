"""The decode step fed by the scheduler's own block tables.  The reference's scheduler
emits block tables, copy-on-write pairs and swap lists every step (src/scheduler/mod.rs:40-61,
203-208, src/scheduler/block_manager.rs:194-406) and its worker drops them
(src/worker/mod.rs:250-305); here the bit-exact BlockManager of the C ABI makes the
decisions in the scheduler's order and the engine consumes them.  Logits are checked
against the per-sequence oracle; prefix-cache hits skip their tokens' prefill."""
import numpy as np
import pytest

from oracle import llama_ref as R

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    return float(np.max(np.abs(got - want))) / max(float(np.max(np.abs(want))), 1e-30)


@pytest.fixture(scope="module")
def model(hb, cuda, tmp_path_factory):
    cfg = R.TINY_CONFIG
    weights = R.random_weights(cfg, seed=1, std=0.02, norm_ones=True)
    path = tmp_path_factory.mktemp("tiny_llama_tables")
    R.write_model(str(path), cfg, weights)
    eng = hb.Engine.load(str(path), max_seq_len=128, bf16=False, force_f32=True, max_batch=8, num_kv_blocks=64)
    oracle = R.LlamaTpOracle(cfg, weights, world_size=1, dtype="f32")
    yield hb, eng, oracle, cfg
    eng.close()


def test_scheduler_driven_decode(model):
    """Admission (allocate), then per step append_slot for every running sequence before the
    forward, as Scheduler::schedule orders them (src/scheduler/mod.rs:203-208); sequences
    finish and free their blocks; a late arrival reuses freed ids."""
    hb, eng, oracle, cfg = model
    bm = hb.BlockManager(64, 0)
    rng = np.random.default_rng(11)
    lens = [5, 20, 31, 47]   # block-boundary crossings happen at different steps
    prompts = [rng.integers(0, cfg.vocab_size, size=n).astype(np.uint32) for n in lens]
    seqs = {}                # seq_id -> dict(tokens so far, oracle cache, last token)
    for sid, p in enumerate(prompts):
        assert bm.can_allocate(len(p))
        bm.allocate(sid, p.tolist())
        table = bm.get_block_table(sid)
        got = eng.forward_tables(p, 0, table)
        cache = oracle.new_cache()
        want = oracle.forward(p.tolist(), 0, cache)
        assert rel_err(got, want) <= 1e-3
        seqs[sid] = dict(n=len(p), cache=cache, last=int(np.argmax(want)))
    next_id = len(prompts)
    for step in range(20):
        if step == 6:        # sequence 1 finishes: its blocks go back to the FIFO free list
            bm.free(1)
            del seqs[1]
        if step == 9:        # a new request is admitted into the freed ids
            p = rng.integers(0, cfg.vocab_size, size=18).astype(np.uint32)
            bm.allocate(next_id, p.tolist())
            cache = oracle.new_cache()
            want = oracle.forward(p.tolist(), 0, cache)
            got = eng.forward_tables(p, 0, bm.get_block_table(next_id))
            assert rel_err(got, want) <= 1e-3
            seqs[next_id] = dict(n=len(p), cache=cache, last=int(np.argmax(want)))
            next_id += 1
        ids = sorted(seqs)
        copies = []
        for sid in ids:      # append_slot sees total_len = prompt + output tokens so far
            total = seqs[sid]["n"] + 1
            assert bm.can_append_slot(sid, total)
            copies += bm.append_slot(sid, total)
        tables = [bm.get_block_table(sid) for sid in ids]
        # the scheduler's table must cover the position this step writes
        pos = [seqs[sid]["n"] for sid in ids]
        assert all(len(t) * 16 > p_ for t, p_ in zip(tables, pos))
        width = max(len(t) for t in tables)
        tab = np.zeros((len(ids), width), dtype=np.int64)
        for i, t in enumerate(tables):
            tab[i, :len(t)] = t
        logits = np.empty((len(ids), cfg.vocab_size), dtype=np.float32)
        nxt = eng.decode_batch_tables([seqs[s]["last"] for s in ids], pos, tab, copy_pairs=copies, logits=logits)
        for i, sid in enumerate(ids):
            st = seqs[sid]
            want = oracle.forward([st["last"]], st["n"], st["cache"])
            assert rel_err(logits[i], want) <= 1e-3, (step, sid)
            assert int(nxt[i]) == int(np.argmax(logits[i]))
            st["n"] += 1
            st["last"] = int(np.argmax(want))


def test_prefix_cache_hit_skips_prefill_and_copy_on_write(model):
    """A freed sequence leaves its complete prompt blocks in the prefix cache
    (block_manager.rs:264-276); the next prompt with the same first 32 tokens gets those ids
    back (hit_blocks = 2, :213-234) and only its tail is prefilled.  Then the shared block is
    copied (copy-on-write pair) and the table switched to the copy: same logits."""
    hb, eng, oracle, cfg = model
    bm = hb.BlockManager(64, 0)
    rng = np.random.default_rng(5)
    head = rng.integers(0, cfg.vocab_size, size=32).astype(np.uint32)
    a = np.concatenate([head, rng.integers(0, cfg.vocab_size, size=8).astype(np.uint32)])
    b = np.concatenate([head, rng.integers(0, cfg.vocab_size, size=5).astype(np.uint32)])
    assert bm.allocate(100, a.tolist()) == 0
    ta = bm.get_block_table(100)
    eng.forward_tables(a, 0, ta)
    bm.free(100)
    hits = bm.allocate(101, b.tolist())
    tb = bm.get_block_table(101)
    assert hits == 2 and tb[:2] == ta[:2]
    got = eng.forward_tables(b[hits * 16:], hits * 16, tb)       # 32 of 37 tokens are not recomputed
    want = oracle.forward(b.tolist(), 0, oracle.new_cache())
    assert rel_err(got, want) <= 1e-3
    # copy-on-write of the second shared block into a block nobody uses
    spare = 60
    assert spare not in tb
    eng.kv_copy_blocks([(tb[1], spare)])
    tb2 = [tb[0], spare, tb[2]]
    cache = oracle.new_cache()
    oracle.forward(b.tolist(), 0, cache)
    tok = int(np.argmax(want))
    logits = np.empty((1, cfg.vocab_size), dtype=np.float32)
    eng.decode_batch_tables([tok], [len(b)], np.array([tb2], dtype=np.int64), logits=logits)
    want2 = oracle.forward([tok], len(b), cache)
    assert rel_err(logits[0], want2) <= 1e-3


def test_swap_out_and_in_round_trip(model):
    """swap_out moves a sequence's blocks to the CPU pool and swap_in brings them back under
    new ids (block_manager.rs:359-406): decoding continues with identical logits."""
    hb, eng, oracle, cfg = model
    bm = hb.BlockManager(64, 8)
    eng.reserve_cpu_blocks(8)
    p = np.random.default_rng(9).integers(0, cfg.vocab_size, size=40).astype(np.uint32)
    bm.allocate(7, p.tolist())
    t0 = bm.get_block_table(7)
    cache = oracle.new_cache()
    want = oracle.forward(p.tolist(), 0, cache)
    assert rel_err(eng.forward_tables(p, 0, t0), want) <= 1e-3
    out_pairs = bm.swap_out(7)
    eng.kv_swap_blocks(out_pairs, to_cpu=True)
    # somebody else takes (and dirties) GPU blocks in the meantime
    bm.allocate(8, list(range(1, 49)))
    eng.forward_tables(np.arange(1, 49, dtype=np.uint32), 0, bm.get_block_table(8))
    in_pairs = bm.swap_in(7)
    eng.kv_swap_blocks(in_pairs, to_cpu=False)
    t1 = bm.get_block_table(7)
    assert t1 != t0
    tok = int(np.argmax(want))
    logits = np.empty((1, cfg.vocab_size), dtype=np.float32)
    eng.decode_batch_tables([tok], [len(p)], np.array([t1], dtype=np.int64), logits=logits)
    assert rel_err(logits[0], oracle.forward([tok], len(p), cache)) <= 1e-3


def test_table_errors(model):
    hb, eng, oracle, cfg = model
    with pytest.raises(hb.HbError):       # the table does not cover the position
        eng.decode_batch_tables([1], [40], np.array([[0, 1]], dtype=np.int64))
    with pytest.raises(hb.HbError):       # block id outside the pool
        eng.decode_batch_tables([1], [3], np.array([[64]], dtype=np.int64))
    with pytest.raises(hb.HbError):       # two rows writing one slot
        eng.decode_batch_tables([1, 2], [3, 3], np.array([[5], [5]], dtype=np.int64))
    with pytest.raises(hb.HbError) as ei:  # token id outside the vocabulary
        eng.decode_batch_tables([cfg.vocab_size], [3], np.array([[5]], dtype=np.int64))
    assert "vocabulary" in ei.value.msg
    with pytest.raises(hb.HbError):
        eng.kv_swap_blocks([(0, 99)], to_cpu=True)
