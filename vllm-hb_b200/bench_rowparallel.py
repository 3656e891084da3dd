"""Micro-benchmark of the fused row-parallel projection (GEMM + all-reduce + residual +
RMSNorm) against the unfused sequences, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node TP --master-addr 127.0.0.1 \
        --master-port 29500 vllm-hb_b200/bench_rowparallel.py [--iters 100] [--out FILE]

Shapes: X [M, K/TP] ~N(0,1), W [N, K/TP] ~N(0,0.02) per rank, residual [M, N] ~N(0,1),
norm weight ones, eps 1e-5; M in {1, 8, 64, 256}; (K, N) = (28672, 8192) (down_proj) and
(8192, 8192) (o_proj).  Variants timed per point:
    fused      hb_fused_rowparallel (auto / one-shot / two-shot)
    gemm_arn   hb_gemm -> hb_all_reduce_add_rms_norm (one peer-memory kernel: what the engine runs)
    unfused    hb_gemm -> hb_all_reduce (peer memory) -> hb_add_rms_norm
    baseline   torch.matmul (cuBLAS) -> NCCL all_reduce -> hb_add_rms_norm: the
               reference's sequence (src/engine/arch/llama_tp.rs:327,533-552)
    baseline_eager  the same with the add and the norm as the reference ships them for bf16:
               six eager elementwise launches (src/kernels/rms_norm.rs:128-132)
Device time with CUDA events on the launching stream, max over ranks, weights rotated
over 4 buffers so that they come from HBM, not L2.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--out", default="")
    ap.add_argument("--ms", default="1,8,64,256")
    args = ap.parse_args()
    hb = entry.load_package()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tp = hb.TpWorld.from_torch_distributed(local, staging_bytes=96 << 20) if world > 1 else None
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    nvl = 770.0  # measured peer copy GB/s per direction on this pool (nominal 900)
    results = []

    def timed(fn, nbuf):
        for i in range(args.warmup):
            fn(i % nbuf)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.iters):
            fn(i % nbuf)
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) * 1e3 / args.iters], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    for K, N in ((28672, 8192), (8192, 8192)):
        Kl = K // world
        g = torch.Generator(device=dev).manual_seed(3 + rank)
        ws = [(torch.randn(N, Kl, generator=g, device=dev) * 0.02).to(torch.bfloat16) for _ in range(4)]
        nw = torch.ones(N, device=dev, dtype=torch.bfloat16)
        for M in [int(m) for m in args.ms.split(",")]:
            gx = torch.Generator(device=dev).manual_seed(2)
            x = torch.randn(M, Kl, generator=gx, device=dev).to(torch.bfloat16)
            resid = torch.randn(M, N, generator=torch.Generator(device=dev).manual_seed(4), device=dev).to(torch.bfloat16)
            fws = hb.fused_rowparallel_workspace(x, ws[0])
            out = (torch.empty(M, N, device=dev, dtype=torch.bfloat16), torch.empty(M, N, device=dev, dtype=torch.bfloat16))
            part = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            gws = torch.zeros(max(hb.lib.hb_gemm_workspace_bytes(M, N, Kl, hb.BF16), 16), dtype=torch.uint8, device=dev)
            st = torch.cuda.current_stream().cuda_stream

            def fused(algo):
                return lambda i: hb.fused_rowparallel(tp, x, ws[i], resid, nw, 1e-5, algo, workspace=fws, out=out)

            def unfused(i):
                hb.check(hb.lib.hb_gemm(st, part.data_ptr(), x.data_ptr(), ws[i].data_ptr(), M, N, Kl, hb.BF16, gws.data_ptr()))
                if tp is not None:
                    tp.all_reduce(part)
                hb.check(hb.lib.hb_add_rms_norm(st, out[0].data_ptr(), out[1].data_ptr(), part.data_ptr(), resid.data_ptr(),
                                                nw.data_ptr(), M, N, 1e-5, hb.BF16))

            def gemm_arn(i):
                hb.check(hb.lib.hb_gemm(st, part.data_ptr(), x.data_ptr(), ws[i].data_ptr(), M, N, Kl, hb.BF16, gws.data_ptr()))
                hb.check(hb.lib.hb_all_reduce_add_rms_norm(tp.handle, st, out[0].data_ptr(), out[1].data_ptr(), part.data_ptr(),
                                                           resid.data_ptr(), nw.data_ptr(), M, N, 1e-5, hb.BF16, hb.ALGO_AUTO))

            def baseline(i):
                p2 = torch.matmul(x, ws[i].t())
                if world > 1:
                    dist.all_reduce(p2)
                hb.check(hb.lib.hb_add_rms_norm(st, out[0].data_ptr(), out[1].data_ptr(), p2.data_ptr(), resid.data_ptr(),
                                                nw.data_ptr(), M, N, 1e-5, hb.BF16))

            def baseline_eager(i):
                p2 = torch.matmul(x, ws[i].t())
                if world > 1:
                    dist.all_reduce(p2)
                h = resid + p2
                var = h.pow(2).mean(-1, keepdim=True) + 1e-5
                out[0].copy_(h / var.sqrt() * nw)

            row = {"K": K, "N": N, "M": M, "tp": world}
            row["fused_auto_us"] = timed(fused(hb.ALGO_AUTO), 4)
            if world > 1:
                row["fused_one_shot_us"] = timed(fused(hb.ALGO_ONE_SHOT), 4)
                row["fused_two_shot_us"] = timed(fused(hb.ALGO_TWO_SHOT), 4)
            if world > 1:
                row["gemm_arn_us"] = timed(gemm_arn, 4)
            row["unfused_us"] = timed(unfused, 4)
            row["baseline_cublas_nccl_us"] = timed(baseline, 4)
            row["baseline_eager_norm_us"] = timed(baseline_eager, 4)
            hbm_bytes = 2 * (Kl * N + M * Kl + 3 * M * N + N)
            nvl_bytes = 2 * (world - 1) / world * 2 * M * N if world > 1 else 0
            row["hbm_bytes"], row["nvlink_bytes_per_dir"] = hbm_bytes, nvl_bytes
            roof_us = max(hbm_bytes / hbm / 1e3, nvl_bytes / nvl / 1e3)
            row["roofline_us"] = roof_us
            best = min(v for k, v in row.items() if k.startswith("fused_") or k == "gemm_arn_us")
            row["best_frac_of_roofline"] = roof_us / best
            row["speedup_vs_baseline"] = row["baseline_cublas_nccl_us"] / best
            row["speedup_vs_unfused"] = row["unfused_us"] / best
            if tp is not None and tp.status() != 0:
                row["status"] = tp.status()
            results.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        Path(args.out).write_text(json.dumps(results, indent=1))
    if tp is not None:
        torch.cuda.synchronize()
        dist.barrier()
        tp.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
