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

# The CPU arm uses every host core through the BLAS behind NumPy.  torch.distributed.run
# exports OMP_NUM_THREADS=1 to its workers; that must be undone BEFORE NumPy loads its BLAS.
if "--impl" in sys.argv and "reference" in sys.argv:
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)

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


def blas_threads() -> int:
    """Threads the BLAS behind NumPy really uses (not the core count of the box)."""
    try:
        from threadpoolctl import threadpool_info

        n = [int(i.get("num_threads", 0)) for i in threadpool_info() if i.get("user_api") == "blas"]
        if n:
            return max(n)
    except Exception:
        pass
    try:
        return int(os.environ.get("OMP_NUM_THREADS", "") or (os.cpu_count() or 1))
    except ValueError:
        return os.cpu_count() or 1


def cpu_config1() -> dict:
    """The reference's own CPU-runnable configuration timed on the port, whole: tiny fp32
    Llama (2 layers, hidden 256, 4/2 heads, FFN 688, vocabulary 32000), 8 prompts of 32
    uniform token ids (seed 0), 32 greedy tokens each = 1 prefill + 31 decode forwards per
    sequence, one sequence at a time (src/worker/mod.rs:280-293,349-358,404-409)."""
    from oracle import llama_ref as R

    cfg = R.TINY_CONFIG
    oracle = R.LlamaTpOracle(cfg, R.random_weights(cfg, seed=1, std=0.02, norm_ones=True), world_size=1, dtype="f32")
    prompts = np.random.default_rng(0).integers(0, cfg.vocab_size, size=(8, 32))
    oracle.greedy_generate(prompts[0].tolist(), 2)  # warm-up
    t0 = time.perf_counter()
    n = 0
    for p in prompts:
        toks, _ = oracle.greedy_generate(p.tolist(), 32)
        n += len(toks)
    dt = time.perf_counter() - t0
    return {"workload": "tiny fp32 llama, 8 prompts x 32 ids, 32 greedy tokens each, per sequence", "tokens": n,
            "seconds": dt, "tok_s": n / dt, "threads": blas_threads()}


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
    ref = CpuReference(w["shape"], w["prompt_len"])
    threads = blas_threads()
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
    base["config1"] = cpu_config1()
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": gpu_config(w, args.gpus, args.steps),
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def gpu_config(w: dict, world: int, steps: int) -> dict:
    """The `config` object of both arms: the workload, not how an arm runs it."""
    return {"workload": w["name"], "batch": w["batch"], "prompt_len": w["prompt_len"], "decode_steps": steps,
            "layers": w["shape"]["num_hidden_layers"], "parallelism": f"tp{world}",
            "l2": "inputs larger than L2 (weights + KV read once per step)",
            "timing": "value: CUDA events around each step's kernels on the engine stream, summed; "
                      "e2e: wall clock around the K hb_decode_batch calls; max over ranks"}


# ------------------------------------------------------------ parity at N > 1 (untimed)
def tp_parity(hb, tp_world, rank: int, world: int, dev) -> dict:
    """Checks made on all N ranks before anything is timed, with the CPU oracle as the
    checker: (1) a small bf16 tensor-parallel model (2 layers, hidden 2048, 16/8 heads of
    128), 48 sequences, 6 lock-step steps: every rank's logits against LlamaTpOracle with
    world_size N and against rank 0 bit for bit; (2) hb_all_reduce_add_rms_norm one-shot and
    two-shot against the rank-order fp32 sum + residual + RMSNorm of the oracle; (3) the
    row-parallel projection whose GEMM epilogue pushes the first hop, against the same."""
    import torch
    import torch.distributed as dist
    from oracle import kernels_ref as K
    from oracle import llama_ref as R
    from oracle import parallel_ref as P

    out = {}
    shape = dict(hidden_size=2048, intermediate_size=2048, num_hidden_layers=2, num_attention_heads=16,
                 num_key_value_heads=8, vocab_size=4096, rms_norm_eps=1e-5, rope_theta=500000.0)
    B, steps, n_check = 48, 6, 8
    eng = hb.Engine.create_random(shape, seed=11, std=0.02, norm_ones=True, max_seq_len=32, bf16=True,
                                  tensor_parallel_size=world, world=tp_world, max_batch=B)
    cfg = R.LlamaTpConfig(**shape)
    prompts = np.random.default_rng(0).integers(0, cfg.vocab_size, size=(B, steps)).astype(np.uint32)
    seqs = [eng.create_kv_cache() for _ in range(B)]
    logits = np.empty((B, cfg.vocab_size), dtype=np.float32)
    for t in range(steps):
        eng.decode_batch(seqs, prompts[:, t], logits=logits)
    local = {name: eng.get_tensor(name) for name in R.tensor_shapes(cfg)}
    all_w = [None] * world
    all_l = [None] * world
    dist.gather_object(local, all_w if rank == 0 else None, dst=0)
    dist.gather_object(logits, all_l if rank == 0 else None, dst=0)
    if rank == 0:
        weights = {}
        for name, shp in R.tensor_shapes(cfg).items():
            pieces = [all_w[r][name] for r in range(world)]
            if name.endswith(("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate_proj.weight", "up_proj.weight")):
                weights[name] = np.concatenate([p.reshape(shp[0] // world, shp[1]) for p in pieces], 0)
            elif name.endswith(("o_proj.weight", "down_proj.weight")):
                weights[name] = np.concatenate([p.reshape(shp[0], shp[1] // world) for p in pieces], 1)
            else:
                weights[name] = pieces[0].reshape(shp)
        oracle = R.LlamaTpOracle(cfg, weights, world_size=world, dtype="bf16", reference_reduce=False, weights_exact=True)
        rows = np.linspace(0, B - 1, n_check).astype(int)
        want = np.stack([oracle.forward(prompts[i].tolist(), 0, oracle.new_cache()) for i in rows])
        scale = float(np.max(np.abs(want)))
        out["max_rel_err"] = max(float(np.max(np.abs(all_l[r][rows] - want))) / scale for r in range(world))
        out["ranks_identical"] = all(np.array_equal(all_l[r], all_l[0]) for r in range(world))
        out["greedy_agreement"] = float(np.mean(np.argmax(all_l[0][rows], 1) == np.argmax(want, 1)))
        out["model"] = "2 layers, hidden 2048, 16/8 heads, FFN 2048, vocab 4096, bf16, B=48, 6 steps"
    for s_ in seqs:
        s_.free()
    eng.close()

    # (2) exchange + residual + norm kernel, both algorithms, M=64 x N=8192 bf16
    M, N = 64, 8192
    parts = [K.round_bf16(np.random.default_rng(10 + r).standard_normal((M, N)).astype(np.float32)) for r in range(world)]
    resid = K.round_bf16(np.random.default_rng(4).standard_normal((M, N)).astype(np.float32))
    nw = K.round_bf16((1.0 + 0.1 * np.random.default_rng(5).standard_normal(N)).astype(np.float32))
    acc = np.zeros((M, N), dtype=np.float32)
    for p_ in parts:
        acc = acc + p_                                   # rank order, fp32 (src/parallel/comm.rs:54-58)
    want_h = K.round_bf16(resid + K.round_bf16(acc))
    want_n = K.rms_norm_kernel(want_h, nw, 1e-5, "bf16")
    put = lambda a: torch.from_numpy(a).to(dev, torch.bfloat16)
    exact, nerr = True, 0.0
    for algo in (hb.ALGO_ONE_SHOT, hb.ALGO_TWO_SHOT):
        for _ in range(2):                               # the second call reuses the staging area
            normed, res = tp_world.all_reduce_add_rms_norm(put(parts[rank]), put(resid), put(nw), 1e-5, algo)
            torch.cuda.synchronize()
            exact = exact and bool(np.array_equal(res.float().cpu().numpy(), want_h))
            nerr = max(nerr, float(np.max(np.abs(normed.float().cpu().numpy() - want_n))) / float(np.max(np.abs(want_n))))
    # (3) GEMM with the push epilogue + the same kernel starting at its wait
    Kl = 1024
    xs = [K.round_bf16(np.random.default_rng(20 + r).standard_normal((M, Kl)).astype(np.float32)) for r in range(world)]
    wts = [K.round_bf16((0.02 * np.random.default_rng(30 + r).standard_normal((N, Kl))).astype(np.float32)) for r in range(world)]
    form = hb.fused_rowparallel_form(tp_world, M, N, Kl, hb.ALGO_TWO_SHOT)
    normed, res = hb.fused_rowparallel(tp_world, put(xs[rank]), put(wts[rank]), put(resid), put(nw), 1e-5, hb.ALGO_TWO_SHOT)
    torch.cuda.synchronize()
    acc = resid.copy()
    for r in range(world):
        acc = acc + K.round_bf16((xs[r].astype(np.float64) @ wts[r].astype(np.float64).T).astype(np.float32))
    want_h2 = K.round_bf16(acc)
    perr = float(np.max(np.abs(res.float().cpu().numpy() - want_h2))) / float(np.max(np.abs(want_h2)))
    digest = int(np.frombuffer(res.view(torch.int16).cpu().numpy().tobytes(), dtype=np.uint32).sum(dtype=np.uint64))
    stats = torch.tensor([0.0 if exact else 1.0, nerr, perr, float(tp_world.status() != 0)], dtype=torch.float64, device=dev)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    digests = [None] * world
    dist.all_gather_object(digests, digest)
    out.update({"engine_exchange": "switch reduction" if tp_world.has_multicast() else "peer memory",
                "ar_resid_bit_exact": bool(stats[0] == 0.0), "ar_norm_max_rel_err": float(stats[1]),
                "push_form": form, "push_max_rel_err": float(stats[2]), "push_ranks_identical": len(set(digests)) == 1,
                "world_status_clean": bool(stats[3] == 0.0)})
    ok = (out.get("max_rel_err", 0.0) <= 2e-2 and out.get("ranks_identical", True) and out["ar_resid_bit_exact"]
          and out["ar_norm_max_rel_err"] <= 2e-2 and out["push_max_rel_err"] <= 2e-2 and out["push_ranks_identical"]
          and out["world_status_clean"])
    out["ok"] = bool(ok)
    return out


def tp1_same_shape(hb, shape: dict, B: int, P: int, layers: int, steps: int) -> dict:
    """The N > 1 workload's shape on ONE GPU with `layers` layers (the full depth does not fit
    180 GB): per-layer time from the per-kind profile, scaled to the full depth plus the
    lm_head and the small kernels, so that the TP=1/2/4/8 curve has its base on one workload."""
    full = shape["num_hidden_layers"]
    sh = dict(shape, num_hidden_layers=layers)
    eng = hb.Engine.create_random(sh, seed=1, std=0.02, norm_ones=True, max_seq_len=P + steps + 16, bf16=True,
                                  tensor_parallel_size=1, world=None, max_batch=B)
    prompts = np.random.default_rng(0).integers(0, sh["vocab_size"], size=(B, P)).astype(np.uint32)
    seqs = [eng.create_kv_cache() for _ in range(B)]
    nxt = np.empty(B, dtype=np.uint32)
    for t in range(P):
        eng.decode_batch(seqs, prompts[:, t], next_tokens=nxt)
    for _ in range(3):
        eng.decode_batch(seqs, nxt.copy(), next_tokens=nxt)
    ms = 0.0
    for _ in range(steps):
        eng.decode_batch(seqs, nxt.copy(), next_tokens=nxt)
        ms += eng.last_step_ms()
    ms /= steps
    _, prof = eng.profile_step(seqs, nxt.copy())
    fixed = prof.get("gemm_lm_head", 0.0) + prof.get("other", 0.0)
    fixed = min(fixed, 0.5 * ms)
    full_ms = (ms - fixed) * full / layers + fixed
    for s_ in seqs:
        s_.free()
    eng.close()
    return {"layers_run": layers, "ms_per_step_run": ms, "ms_per_step_full_depth": full_ms,
            "value": B / (full_ms / 1e3), "unit": UNIT,
            "how": f"{layers} of {full} layers on one GPU, B={B}, prompt {P}; (step - lm_head - small kernels) "
                   f"x {full}/{layers} + lm_head + small kernels"}


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
    parity = same_shape = None
    dev = torch.device("cuda", local_rank)
    if world > 1:
        staging = 64 << 20
        tp_world = hb.TpWorld.from_torch_distributed(local_rank, staging_bytes=staging, nccl=True)
        # the exchange after o_proj / down_proj: sum formed inside the NVLink switch where the
        # fabric offers multicast, else the peer-memory kernel
        exchange = "peer memory (--exchange peer)"
        if args.exchange == "auto":
            why = tp_world.enable_multicast(256, max(8192, shape["hidden_size"]))
            exchange = "switch reduction (multimem)" if not why else f"peer memory ({why})"
        if args.workload == "auto" and not args.skip_checks:
            # correctness on all N ranks first (untimed); a failure ends the run non-zero
            parity = tp_parity(hb, tp_world, rank, world, dev)
            if rank == 0:
                same_shape = tp1_same_shape(hb, shape, B, P, args.tp1_layers, 8)
            dist.barrier()
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

    rowpar = None
    if world > 1 and args.workload == "auto" and not args.skip_checks:
        import vllm_hb_b200.bench_rowparallel as brp

        peak0, _ = measured_peaks()
        rowpar = brp.run_points(hb, tp_world, rank, world, dev, peak0)

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
            "config": dict(gpu_config(w, world, K), **({"exchange": exchange} if world > 1 else {})),
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B + 4},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "gemm_tc_kernel (all GEMM launches of a step)",
                         "achieved": achieved, "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                         "frac": (achieved / peak) if achieved else None, "traffic": traffic,
                         "traffic_source": "DRAM read+write bytes of the ncu captures summarised in "
                                           "profiles/gemm_tc_kernel_decode_shapes.md (not measured by this run)",
                         "algorithmic_bytes_per_step": gemm_bytes, "ms_per_step": gemm_ms,
                         "timing": "CUDA events recorded between the kernels of profile steps on the engine stream (graph with event nodes)"},
            "step_roofline": {"bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (dev_ms / K / 1e3) / 1e9,
                              "frac": step_bytes / (dev_ms / K / 1e3) / 1e9 / peak},
            "kernel_ms_per_step": prof,
            "kernel_ms_per_step_by_rank": prof_ranks,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline and args.workload == "auto":
            line["cpu_baseline"] = cpu_reference_tok_s(shape, P, 4, blas_threads())
            line["cpu_baseline"]["config1"] = cpu_config1()
        if parity is not None:
            line["tp_parity"] = parity
        if same_shape is not None:
            line["tp1_same_shape"] = same_shape
        if rowpar is not None:
            line["rowparallel"] = rowpar
        print(json.dumps(line), flush=True)
    for s in seqs:
        s.free()
    eng.close()
    if tp_world is not None:
        barrier()
        tp_world.disable_multicast()  # collective; before the window's memory and the process group go away
        tp_world.close()
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity.get("ok", True):
        raise SystemExit("tensor-parallel parity check failed: " + json.dumps(parity))


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
    ap.add_argument("--exchange", choices=["auto", "peer"], default="auto",
                    help="N > 1: 'auto' reduces inside the NVLink switch when multicast memory is available, 'peer' "
                         "always takes the peer-memory kernel")
    ap.add_argument("--skip-checks", action="store_true",
                    help="N > 1: skip the untimed parity checks, the single-GPU base point and the row-parallel points")
    ap.add_argument("--tp1-layers", type=int, default=8, help="layers of the single-GPU base point of the N > 1 shape")
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
