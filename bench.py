"""Decode throughput of the tensor-parallel hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (N>1: under torchrun, one rank per GPU)
    python bench.py --impl reference ...                     (CPU arm: the reference's per-sequence path)

A step is one greedy decode step of the whole batch.  N=1 runs the Llama-3.1-8B shape
(64 sequences, 512-token prompts); N>1 runs the Llama-3.1-70B shape at TP=N
(128 sequences, 1024-token prompts).  Weights are random-initialised on the device,
prompts are seeded uniform token ids; prompts are prefilled through the same decode
kernels before the timed region.  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA_8B = dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)
LLAMA_70B = dict(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                 num_key_value_heads=8, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)

MIXTRAL_8X7B = dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                    num_key_value_heads=8, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=1000000.0,
                    num_local_experts=8, num_experts_per_tok=2, sliding_window=4096)

METRIC = "decode_tokens_per_s"
UNIT = "tok/s"


def workload_for(n_gpus: int, args) -> dict:
    if n_gpus == 1:
        w = dict(name="llama-3.1-8b-shape tp1 b64 prompt512 greedy-decode", shape=dict(LLAMA_8B),
                 batch=64, prompt_len=512, norm_ones=True)
    else:
        w = dict(name=f"llama-3.1-70b-shape tp{n_gpus} b128 prompt1024 greedy-decode", shape=dict(LLAMA_70B),
                 batch=128, prompt_len=1024, norm_ones=True)
    if args.workload == "mixtral":  # the sparse-MoE configuration: 64 sequences, 512-token prompts
        w = dict(name=f"mixtral-8x7b-shape tp{n_gpus} b64 prompt512 greedy-decode", shape=dict(MIXTRAL_8X7B),
                 batch=64, prompt_len=512, norm_ones=True)
    if args.layers:
        w["shape"]["num_hidden_layers"] = args.layers
        w["name"] += f" layers{args.layers}"
    if args.shape_scale > 1:  # debugging / CPU tests only: a proportionally smaller model
        for k in ("hidden_size", "intermediate_size", "vocab_size"):
            w["shape"][k] //= args.shape_scale
        w["name"] += f" scaled-1/{args.shape_scale}"
    if args.batch:
        w["batch"] = args.batch
    if args.prompt_len:
        w["prompt_len"] = args.prompt_len
    return w


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.rows, self.proc, self.t_begin = gpu_index, [], None, 0.0

    def begin_region(self):
        """Samples that arrive from now on count (nvidia-smi is started earlier: its own
        start-up takes longer than a short timed region)."""
        self.t_begin = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t_arrival, r in self.rows:
            if len(r) < 9 or t_arrival < self.t_begin:
                continue
            try:
                sm.append(float(r[1])); smax.append(float(r[2])); power.append(float(r[3]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ CPU reference arm
def cpu_reference_tok_s(shape: dict, ctx: int, n_tokens: int, threads: int) -> dict:
    """The reference's CPU path (`--no-default-features`): F32 weights
    (src/engine/dtype.rs:22-28) and ONE forward per sequence per step
    (src/worker/mod.rs:280-293), timed with the NumPy restatement of llama_tp.rs on a
    bounded sample: `n_tokens` single-token forwards at context `ctx` through 1 and
    through 3 layers of the model's shape (the same layer weights reused, KV pre-filled
    with random values), extrapolated linearly to the full depth plus the lm_head."""
    ref = CpuReference(shape, ctx)
    return ref.sample(n_tokens, threads)


class CpuReference:
    """Weights and pre-filled caches are built once; sample() times forwards only."""

    def __init__(self, shape: dict, ctx: int):
        from oracle import llama_ref as R

        self.full_layers = shape["num_hidden_layers"]
        self.ctx = ctx
        rng = np.random.default_rng(0)

        def uniform(*s):
            return (rng.random(s, dtype=np.float32) - np.float32(0.5)) * np.float32(0.07)

        base = {}
        self.models = {}
        for n_layers in (1, 3):
            cfg = R.LlamaTpConfig(**{**shape, "num_hidden_layers": n_layers})
            if not base:
                for name, s in R.tensor_shapes(cfg).items():
                    if name.startswith("model.layers.0.") or not name.startswith("model.layers."):
                        base[name] = np.ones(s, dtype=np.float32) if name.endswith("norm.weight") else uniform(*s)
                base["lm_head.weight"] = base["model.embed_tokens.weight"]  # same size, saves a copy
            weights = {name: base[name if not name.startswith("model.layers.") else
                                  "model.layers.0." + name.split(".", 3)[3]] for name in R.tensor_shapes(cfg)}
            oracle = R.LlamaTpOracle(cfg, weights, world_size=1, dtype="f32")
            cache = oracle.new_cache()
            for l in range(n_layers):
                cache[0][l] = [uniform(ctx, cfg.kv_heads(), cfg.head_dim()), uniform(ctx, cfg.kv_heads(), cfg.head_dim())]
            oracle.forward([1], ctx, [[list(kv) for kv in cache[0]]])  # warm-up
            self.models[n_layers] = (oracle, cache, cfg.vocab_size)

    def sample(self, n_tokens: int, threads: int) -> dict:
        times = {}
        for n_layers, (oracle, cache, vocab) in self.models.items():
            t0 = time.perf_counter()
            for i in range(n_tokens):
                c = [[list(kv) for kv in cache[0]]]  # every sequence decodes over its own cache
                oracle.forward([int(i) % vocab], self.ctx, c)
            times[n_layers] = (time.perf_counter() - t0) / n_tokens
        per_layer = (times[3] - times[1]) / 2.0
        head = max(times[1] - per_layer, 0.0)
        per_token = per_layer * self.full_layers + head
        return {"value": 1.0 / per_token, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"{n_tokens} single-sequence decode forwards (fp32, ctx {self.ctx}) through 1 and 3 layers "
                          f"of the shape, extrapolated to {self.full_layers} layers + lm_head; per-sequence M=1 as "
                          "the reference decodes",
                "s_per_token": per_token}


def run_reference_arm(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    w = workload_for(args.gpus, args)
    threads = os.cpu_count() or 1
    ref = CpuReference(w["shape"], w["prompt_len"])
    vals = []
    for _ in range(args.warmup):
        ref.sample(1, threads)
    t0 = time.perf_counter()
    budget_s = 150.0  # the whole run must end within a few minutes whatever K is
    for i in range(args.steps):
        vals.append(ref.sample(2, threads))
        if time.perf_counter() - t0 > budget_s and i + 1 < args.steps:
            args.steps = i + 1
            break
    wall = time.perf_counter() - t0
    v = statistics.median(x["value"] for x in vals)
    base = dict(vals[-1]); base["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": w["name"], "batch": w["batch"],
                                            "prompt_len": w["prompt_len"], "parallelism": "cpu"},
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args, rank: int, world: int, local_rank: int) -> None:
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    hb = entry.load_package()  # raises if libhb.so is missing: there is no fallback path
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    w = workload_for(world, args)
    shape, B, P = w["shape"], w["batch"], w["prompt_len"]
    K, W = args.steps, args.warmup
    max_seq = P + W + K + args.profile_steps + 8

    tp_world = None
    if world > 1:
        staging = 64 << 20
        tp_world = hb.TpWorld.from_torch_distributed(local_rank, staging_bytes=staging, nccl=False)
    eng = hb.Engine.create_random(shape, seed=1, std=0.02, norm_ones=w["norm_ones"], max_seq_len=max_seq,
                                  bf16=True, tensor_parallel_size=world, world=tp_world, max_batch=B)
    prompts = np.random.default_rng(0).integers(0, shape["vocab_size"], size=(B, P)).astype(np.uint32)
    seqs = [eng.create_kv_cache() for _ in range(B)]

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # prefill: the prompts go through the same decode step in lock-step (untimed)
    nxt = np.empty(B, dtype=np.uint32)
    for t in range(P):
        eng.decode_batch(seqs, prompts[:, t], next_tokens=nxt)
    for _ in range(W):
        eng.decode_batch(seqs, nxt.copy(), next_tokens=nxt)

    barrier()
    sampler.begin_region()
    dev_ms = 0.0
    ctx_sum = 0
    t0 = time.perf_counter()
    for step in range(K):
        ctx_sum += sum(len(s) + 1 for s in seqs) if step in (0, K - 1) else 0
        eng.decode_batch(seqs, nxt.copy(), next_tokens=nxt)  # H2D ids/tables in, D2H tokens out, inside
        dev_ms += eng.last_step_ms()
    barrier()
    wall_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    launches = eng.last_step_launches() * K

    # per-kernel-kind device time of a few profile steps (CUDA events between the kernels on the engine's stream)
    prof = {}
    for _ in range(args.profile_steps):
        barrier()  # ranks enter together: a rank that arrives early books the wait as exchange time
        nxt2, ms = eng.profile_step(seqs, nxt.copy())
        nxt = nxt2
        for k, v in ms.items():
            prof[k] = prof.get(k, 0.0) + v / args.profile_steps

    # the exchange kernels also hold a rank until its slowest peer arrives: keep every rank's share
    prof_ranks = None
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, {k: round(v, 4) for k, v in prof.items()})
        prof_ranks = {k: [g.get(k, 0.0) for g in gathered] for k in ("all_reduce", "gemm", "attention")}

    ctx_mid = [P + W + K // 2 + 1] * B
    step_bytes = eng.step_bytes(ctx_mid)
    gemm_bytes = eng.gemm_bytes(B)

    # max over ranks of the device time and of the wall time
    stats = torch.tensor([dev_ms, wall_s * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = float(stats[0]), float(stats[1])

    if rank == 0:
        peak, peak_kind = measured_peaks()
        tokens = B * K
        value = tokens / (dev_ms / 1e3)
        e2e = tokens / (wall_ms / 1e3)
        gemm_ms = prof.get("gemm", 0.0)
        achieved = gemm_bytes / (gemm_ms / 1e3) / 1e9 if gemm_ms > 0 else None
        # DRAM bytes (read + write) of the GEMM launches of one step, from the ncu captures
        # (summaries are committed under profiles/): per layer qkv 50.96 MB,
        # o_proj 34.15, gate|up 239.4, down_proj 123.1, plus lm_head 1085.8.  Only the
        # full-size single-GPU workload was captured.
        traffic = None
        if world == 1 and B == 64 and shape["num_hidden_layers"] == 32 and shape["hidden_size"] == 4096 \
                and shape["intermediate_size"] == 14336 and shape["vocab_size"] == 128256:
            traffic = (32 * (50.96 + 34.15 + 239.4 + 123.1) + 1085.8) * 1e6
        h2d = 4 * B * 3 + 8 * B + 4 * B * ((max_seq + 15) // 16)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "batch": B, "prompt_len": P, "decode_steps": K,
                       "layers": shape["num_hidden_layers"], "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2 (weights + KV read once per step)",
                       "timing": "value: CUDA events around each step's kernels on the engine stream, summed; "
                                 "e2e: wall clock around the K hb_decode_batch calls; max over ranks"},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B + 4},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "gemm_tc_kernel (all GEMM launches of a step)",
                         "achieved": achieved, "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                         "frac": (achieved / peak) if achieved else None, "traffic": traffic,
                         "algorithmic_bytes_per_step": gemm_bytes, "ms_per_step": gemm_ms,
                         "timing": "CUDA events recorded between the kernels of profile steps on the engine stream (graph with event nodes)"},
            "step_roofline": {"bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (dev_ms / K / 1e3) / 1e9,
                              "frac": step_bytes / (dev_ms / K / 1e3) / 1e9 / peak},
            "kernel_ms_per_step": prof,
            "kernel_ms_per_step_by_rank": prof_ranks,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline and args.workload == "auto":
            threads = os.cpu_count() or 1
            line["cpu_baseline"] = cpu_reference_tok_s(shape, P, 4, threads)
        print(json.dumps(line), flush=True)
    for s in seqs:
        s.free()
    eng.close()
    if tp_world is not None:
        barrier()
        tp_world.close()
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only)")
    ap.add_argument("--shape-scale", type=int, default=1, help="shrink the model (debugging only)")
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--prompt-len", type=int, default=0)
    ap.add_argument("--profile-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="auto", choices=["auto", "mixtral"],
                    help="auto: Llama-3.1-8B shape on one GPU, 70B shape on several; mixtral: Mixtral-8x7B shape")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world != args.gpus:
        if args.gpus != 1 or world != 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    args.warmup = max(args.warmup, 3)
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
