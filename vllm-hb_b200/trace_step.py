"""Where one replayed decode step spends its time, one GPU:

    python vllm-hb_b200/build.py --variant trace        # libhb_trace.so, -DHB_TC_TRACE
    python vllm-hb_b200/trace_step.py [--batch 64] [--prompt-len 512] [--steps 8]

The trace variant of the library stamps every GEMM launch with the global nanosecond timer:
entry of CTA (0,0), the moment its producer thread passes the dependency wait (the previous
kernel of the stream has completed; the kernels are launched programmatically, so a GEMM is
resident and prefetching weights long before that), and the latest exit of any CTA.  The
launches of a captured graph keep their slots, so after a few replays the ring holds the
timeline of the last step.  The step of the 8B shape is  [qkv GEMM] attention [o_proj GEMM]
[gate|up GEMM] [down_proj GEMM]  per layer and the lm_head GEMM at the end.  Printed per GEMM
kind, in microseconds: how long before its dependency resolved the kernel was resident
(early), dependency resolved -> last CTA exit (exclusive), and last exit -> the next GEMM's
dependency resolved (handover; after the qkv GEMM this is the attention kernel with its two
boundaries).  exclusive + handover sum to the step.  The product library carries none of this.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
os.environ["HB_LIBRARY"] = str(HERE / "libhb_trace.so")

import torch  # noqa: E402

import __graft_entry__ as entry  # noqa: E402

SHAPE_8B = dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)
RING = 1024


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--steps", type=int, default=8)
    a = ap.parse_args()
    if not Path(os.environ["HB_LIBRARY"]).exists():
        raise SystemExit("build the trace variant first: python vllm-hb_b200/build.py --variant trace")
    hb = entry.load_package()
    torch.cuda.set_device(0)
    shape, B, P = dict(SHAPE_8B), a.batch, a.prompt_len
    eng = hb.Engine.create_random(shape, seed=1, std=0.02, norm_ones=True, max_seq_len=P + a.steps + 16, bf16=True,
                                  max_batch=B)
    prompts = np.random.default_rng(0).integers(0, shape["vocab_size"], size=(B, P)).astype(np.uint32)
    seqs = [eng.create_kv_cache() for _ in range(B)]
    nxt = np.empty(B, dtype=np.uint32)
    for t in range(P):
        eng.decode_batch(seqs, prompts[:, t], next_tokens=nxt)
    ms = []
    for _ in range(a.steps):
        eng.decode_batch(seqs, nxt.copy(), next_tokens=nxt)
        ms.append(eng.last_step_ms())
    torch.cuda.synchronize()

    buf = np.zeros(RING * 4, dtype=np.uint64)
    hb.lib.hb_debug_tc_launches.argtypes = [C.c_void_p, C.c_int]
    if hb.lib.hb_debug_tc_launches(buf.ctypes.data, RING):
        raise SystemExit("reading the trace failed")
    rec = buf.reshape(RING, 4)
    rec = rec[rec[:, 1] > 0]
    rec = rec[np.argsort(rec[:, 0])]
    L = shape["num_hidden_layers"]
    n_step = 4 * L + 1
    rec = rec[-n_step:]  # the GEMM launches of the last replay
    start, end, dep = rec[:, 0].astype(np.int64), rec[:, 1].astype(np.int64), rec[:, 3].astype(np.int64)
    n_feat, k_dim = (rec[:, 2] >> np.uint64(32)).astype(np.int64), (rec[:, 2] & np.uint64(0xFFFFFFFF)).astype(np.int64)
    names = ["qkv", "o_proj", "gate|up", "down_proj"]
    early = (dep - start) / 1e3
    excl = (end - dep) / 1e3
    hand = np.append((dep[1:] - end[:-1]) / 1e3, 0.0)
    out = {"ms_per_step_events": round(float(np.mean(ms[-4:])), 4),
           "first_dependency_to_last_exit_ms": round(float(end[-1] - dep[0]) / 1e6, 4), "kinds": {}}
    for k, name in enumerate(names):
        idx = np.arange(k, 4 * L, 4)
        out["kinds"][name] = {"N": int(n_feat[idx[0]]), "K": int(k_dim[idx[0]]),
                              "early_us": round(float(early[idx].mean()), 2),
                              "exclusive_us": round(float(excl[idx].mean()), 2),
                              "handover_us": round(float(hand[idx].mean()), 2),
                              "sum_exclusive_ms": round(float(excl[idx].sum()) / 1e3, 3),
                              "sum_handover_ms": round(float(hand[idx].sum()) / 1e3, 3)}
    out["kinds"]["lm_head"] = {"N": int(n_feat[-1]), "K": int(k_dim[-1]), "early_us": round(float(early[-1]), 2),
                               "exclusive_us": round(float(excl[-1]), 2)}
    print(json.dumps(out))
    for s in seqs:
        s.free()
    eng.close()


if __name__ == "__main__":
    main()
