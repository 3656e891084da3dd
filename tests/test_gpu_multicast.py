"""The all-reduce + residual + RMSNorm whose sum is formed inside the NVLink switch
(hb_world_attach_multicast, HB_ALGO_MULTIMEM): one process per GPU, because the multicast
window comes from a collective allocation.  The worker (tests/multicast_worker.py) compares
every case with the oracle's rank-order sum (src/parallel/comm.rs:47-62 followed by
llama_tp.rs:533-552), with hb_rms_norm on its own output, across ranks, and with the
peer-memory kernel; it detaches and frees the window on every rank before any process ends.
Skipped on a single-GPU box and where the fabric offers no multicast."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = Path(__file__).resolve().parent.parent


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_switch_reduction_matches_oracle_and_peer_kernel(hb):
    n = min(hb.device_count(), int(os.environ.get("HB_TEST_MAX_RANKS", "2")))
    if n < 2:
        pytest.skip("needs at least two GPUs")
    n = 1 << (n.bit_length() - 1)
    env = dict(os.environ, HB_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0")  # NCCL itself stays off the switch here
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), str(ROOT / "tests" / "multicast_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    out = json.loads(line[len("RESULT "):])
    print(json.dumps(out, indent=1))
    if "unavailable" in out:
        pytest.skip("no switch reduction on this box: " + out["unavailable"])
    assert out["errors"] == []
    assert len(out["cases"]) == 6 and out["rowparallel"]["form"] == "multimem"
    assert max(out["prefill_vs_stepwise"].values()) <= 2e-2   # calls of 16, 16 and 5 rows, then single rows
    assert out["tp_parity"]["ok"] and out["tp_parity"]["max_rel_err"] <= 2e-2 and out["tp_parity"]["ranks_identical"]
    for c in out["cases"]:
        assert c["max_rel_vs_oracle"] <= 2e-2 and c["max_rel_vs_peer_kernel"] <= 2e-2
