"""Phase timeline of the exchange + residual + RMSNorm kernel inside the decode graph, N GPUs:

    python vllm-hb_b200/build.py --variant trace        # libhb_trace.so, -DHB_TC_TRACE
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        vllm-hb_b200/trace_exchange.py [--layers 40] [--batch 128] [--prompt-len 32] [--steps 24]

The trace variant of the library records the global nanosecond timer at six points of
ar_add_norm_kernel, for the CTA of one row the rank reduces and of one row it only
receives, in a ring indexed by the call number.  This script runs a 70B-shape
tensor-parallel engine (random weights) for a few decode steps through the captured
graph, i.e. exactly as the product runs it, then prints per rank the mean duration of every
phase in microseconds, the span of the kernel, and the time between the end of one call
and the start of the next (the GEMMs, RoPE and attention of half a layer).  Timers of
different GPUs are not compared.  The product library carries none of this.
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
import torch.distributed as dist  # noqa: E402

import __graft_entry__ as entry  # noqa: E402

SHAPE_70B = dict(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                 num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)
RING, SLOTS = 2048, 8


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=32)
    ap.add_argument("--steps", type=int, default=24)
    a = ap.parse_args()
    if not Path(os.environ["HB_LIBRARY"]).exists():
        raise SystemExit("build the trace variant first: python vllm-hb_b200/build.py --variant trace")
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    hb = entry.load_package()
    torch.cuda.set_device(lr)
    dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
    shape = dict(SHAPE_70B, num_hidden_layers=a.layers)
    B, P = a.batch, a.prompt_len
    tpw = hb.TpWorld.from_torch_distributed(lr, staging_bytes=64 << 20, nccl=False)
    eng = hb.Engine.create_random(shape, seed=1, std=0.02, norm_ones=True, max_seq_len=P + a.steps + 16, bf16=True,
                                  tensor_parallel_size=world, world=tpw, max_batch=B)
    prompts = np.random.default_rng(0).integers(0, shape["vocab_size"], size=(B, P)).astype(np.uint32)
    seqs = [eng.create_kv_cache() for _ in range(B)]
    nxt = np.empty(B, dtype=np.uint32)
    for t in range(P):
        eng.decode_batch(seqs, prompts[:, t], next_tokens=nxt)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    ms = 0.0
    for _ in range(a.steps):
        eng.decode_batch(seqs, nxt.copy(), next_tokens=nxt)
        ms += eng.last_step_ms()
    torch.cuda.synchronize()

    buf = np.zeros(RING * 2 * SLOTS, dtype=np.uint64)
    hb.lib.hb_debug_an_trace.argtypes = [C.c_void_p, C.c_int]
    if hb.lib.hb_debug_an_trace(buf.ctypes.data, RING):
        raise SystemExit("reading the trace failed")
    tr = buf.reshape(RING, 2, SLOTS).astype(np.int64)
    tr = tr[np.argsort(tr[:, 0, 0])]
    tr = tr[tr[:, 0, 0] > 0]
    per_step = 2 * a.layers
    tr = tr[-min(len(tr), (a.steps - 2) * per_step):]  # the calls of the last decode steps

    def us(x) -> float:
        return round(float(np.mean(x)) / 1e3, 2)

    def phases(which: int) -> dict:
        t = tr[:, which, :]
        out = {"wait for peers' done flags": us(t[:, 1] - t[:, 0]), "push + release": us(t[:, 2] - t[:, 1]),
               "wait for the row": us(t[:, 3] - t[:, 2])}
        if which == 0:
            out["reduce + gather push + release"] = us(t[:, 4] - t[:, 3])
            out["norm + exit"] = us(t[:, 5] - t[:, 4])
        else:
            out["read + norm + exit"] = us(t[:, 5] - t[:, 3])
        out["total"] = us(t[:, 5] - t[:, 0])
        return out

    start = np.minimum(tr[:, 0, 0], tr[:, 1, 0])
    end = np.maximum(tr[:, 0, 5], tr[:, 1, 5])
    gap = (start[1:] - end[:-1]) / 1e3
    gap = gap[gap < 2000]  # drop the step boundaries
    res = {"rank": rank, "ms_per_step": round(ms / a.steps, 3), "calls": int(len(tr)),
           "row this rank reduces": phases(0), "row it receives": phases(1),
           "kernel_span_us": us(end - start),
           "between_calls_us": {"mean": round(float(gap.mean()), 2), "after_even": round(float(gap[0::2].mean()), 2),
                                "after_odd": round(float(gap[1::2].mean()), 2)},
           "span_percentiles_us": {f"p{q}": round(float(np.percentile(end - start, q)) / 1e3, 2) for q in (50, 90, 99)}}
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        for r in gathered:
            print(json.dumps(r))
    for s in seqs:
        s.free()
    eng.close()
    torch.cuda.synchronize()
    dist.barrier()
    tpw.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
