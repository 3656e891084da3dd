"""The multi-rank host logic on CPU: two `gloo` ranks shard the same seeded model with
the C ABI's column/row sharding, compute their row-parallel partials with the oracle,
sum them with a real collective and must reproduce the single-rank result — the
decomposition of src/engine/arch/llama_tp.rs:464-471,533,563 without a GPU.  Also the
rank plumbing of bench.py (env parsing, rank-0-only output of the reference arm)."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent

WORKER = r"""
import os, sys, json
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["HB_ROOT"])
import __graft_entry__ as entry
from oracle import llama_ref as R, kernels_ref as K
hb = entry.load_package()
dist.init_process_group("gloo")
rank, ws = dist.get_rank(), dist.get_world_size()
cfg = R.LlamaTpConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=64)
w = R.random_weights(cfg, seed=7, std=0.05, norm_ones=True)
x = np.random.default_rng(1).standard_normal((3, 64)).astype(np.float32)
# row-parallel down projection: column-sharded gate/up feed a row-sharded down (C ABI sharding)
gate = hb.column_shard(w["model.layers.0.mlp.gate_proj.weight"], rank, ws)
up = hb.column_shard(w["model.layers.0.mlp.up_proj.weight"], rank, ws)
down = hb.row_shard(w["model.layers.0.mlp.down_proj.weight"], rank, ws)
act = K.silu(x @ gate.T) * (x @ up.T)
partial = torch.from_numpy((act @ down.T).astype(np.float32))
dist.all_reduce(partial)  # SUM over ranks
full = (K.silu(x @ w["model.layers.0.mlp.gate_proj.weight"].T) * (x @ w["model.layers.0.mlp.up_proj.weight"].T)) \
       @ w["model.layers.0.mlp.down_proj.weight"].T
err = float(np.max(np.abs(partial.numpy() - full)) / np.max(np.abs(full)))
# the IPC-handle exchange pattern of TpWorld.from_torch_distributed, with stand-in handles
handles = [None] * ws
dist.all_gather_object(handles, bytes([rank]) * hb.IPC_HANDLE_BYTES)
ok_handles = all(h == bytes([r]) * hb.IPC_HANDLE_BYTES for r, h in enumerate(handles))
# engines refuse shapes the world size does not divide (llama_tp.rs:407-427)
try:
    R.LlamaTpOracle(R.LlamaTpConfig(hidden_size=60, intermediate_size=96, num_hidden_layers=1,
                                    num_attention_heads=3, vocab_size=8), {}, world_size=ws)
    div = "no error"
except ValueError as e:
    div = str(e)
out = dict(rank=rank, err=err, ok_handles=ok_handles, div=div)
gathered = [None] * ws
dist.all_gather_object(gathered, out)
if rank == 0:
    print("RESULT " + json.dumps(gathered), flush=True)
dist.destroy_process_group()
"""


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def torchrun(script_args, nproc=2, timeout=600, env_extra=None):
    env = dict(os.environ, HB_ROOT=str(ROOT), OMP_NUM_THREADS="2")
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port())] + script_args
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=str(ROOT))


def test_two_rank_row_parallel_decomposition(hb, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    res = torchrun([str(script)])
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    ranks = json.loads(line[len("RESULT "):])
    assert [r["rank"] for r in ranks] == [0, 1]
    for r in ranks:
        assert r["err"] < 1e-5
        assert r["ok_handles"]
        assert "divisible" in r["div"] and "tensor_parallel_size" in r["div"]


def test_bench_reference_arm_prints_on_rank0_only(hb):
    """Under torchrun the reference arm runs on rank 0 alone; the other rank exits 0
    without output.  A tiny layer count keeps the CPU work bounded."""
    res = torchrun(["bench.py", "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0",
                    "--layers", "1", "--shape-scale", "16"], timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["value"] > 0
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["cpu_baseline"]["kind"] == "port"
