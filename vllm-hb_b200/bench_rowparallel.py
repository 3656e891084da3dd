"""Micro-benchmark of the row-parallel projection + all-reduce + residual + RMSNorm against
the reference's sequence of library calls, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node TP --master-addr 127.0.0.1 \
        --master-port 29500 vllm-hb_b200/bench_rowparallel.py [--out FILE]

Shapes: X [M, K/TP] ~N(0,1), W [N, K/TP] ~N(0,0.02) per rank, residual [M, N] ~N(0,1),
norm weight ones, eps 1e-5; M in {1, 8, 64, 256}; (K, N) = (28672, 8192) (down_proj) and
(8192, 8192) (o_proj).  Arms, each CAPTURED IN A CUDA GRAPH of at least 24 calls that
rotate over enough weight buffers to exceed L2, so that neither arm pays host dispatch
per call and the weights come from HBM:
    fused     hb_fused_rowparallel (HB_ALGO_AUTO: the form hb_fused_rowparallel_form names)
    baseline  cuBLAS GEMM (torch.matmul) -> hb_all_reduce(HB_ALGO_NCCL) -> hb_add_rms_norm:
              the reference's sequence (src/engine/arch/llama_tp.rs:327,533-552,
              src/parallel/comm.rs:83-166)
Device time with CUDA events around the graph replays, max over ranks; roofline =
max(HBM bytes / measured peak, NVLink bytes per direction / 770 GB/s).
`run_points` is also what bench.py calls at N > 1.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
NVLINK_GBS = 770.0  # measured peer copy per direction on this pool (nominal 900)
L2_BYTES = 126 << 20


def run_points(hb, tp, rank: int, world: int, dev, hbm_gbs: float, ms=(1, 8, 64, 256),
               shapes=((28672, 8192), (8192, 8192)), replays: int = 4, check: bool = True) -> list:
    """One row per (K, N, M).  `tp` is this rank's TpWorld with its NCCL communicator
    initialised (world > 1) or None."""
    import torch
    import torch.distributed as dist

    rows = []
    side = torch.cuda.Stream(device=dev)
    # the fused arm takes the switch reduction where the world has a multicast window
    algo = hb.ALGO_MULTIMEM if tp is not None and tp.has_multicast() else hb.ALGO_AUTO
    for K, N in shapes:
        Kl = K // world
        w_bytes = N * Kl * 2
        n_sets = max(4, -(-int(1.25 * L2_BYTES) // w_bytes))
        calls = max(24, 3 * n_sets)
        g = torch.Generator(device=dev).manual_seed(3 + rank)
        ws = [(torch.randn(N, Kl, generator=g, device=dev) * 0.02).to(torch.bfloat16) for _ in range(n_sets)]
        nw = torch.ones(N, device=dev, dtype=torch.bfloat16)
        for M in ms:
            x = torch.randn(M, Kl, generator=torch.Generator(device=dev).manual_seed(2), device=dev).to(torch.bfloat16)
            resid = torch.randn(M, N, generator=torch.Generator(device=dev).manual_seed(4), device=dev).to(torch.bfloat16)
            fws = hb.fused_rowparallel_workspace(x, ws[0])
            out_f = (torch.empty(M, N, device=dev, dtype=torch.bfloat16), torch.empty(M, N, device=dev, dtype=torch.bfloat16))
            out_b = (torch.empty(M, N, device=dev, dtype=torch.bfloat16), torch.empty(M, N, device=dev, dtype=torch.bfloat16))
            part = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

            def fused(i):
                hb.fused_rowparallel(tp, x, ws[i], resid, nw, 1e-5, algo, workspace=fws, out=out_f)

            def baseline(i):
                st = torch.cuda.current_stream().cuda_stream
                torch.matmul(x, ws[i].t(), out=part)
                if tp is not None:
                    hb.check(hb.lib.hb_all_reduce(tp.handle, st, part.data_ptr(), part.numel(), hb.BF16, hb.ALGO_NCCL))
                hb.check(hb.lib.hb_add_rms_norm(st, out_b[0].data_ptr(), out_b[1].data_ptr(), part.data_ptr(),
                                                resid.data_ptr(), nw.data_ptr(), M, N, 1e-5, hb.BF16))

            def graph_time(fn):
                # eager warm-up (one-time attribute and library set-up must not fall into the capture)
                with torch.cuda.stream(side):
                    for i in range(3):
                        fn(i % n_sets)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(calls):
                        fn(i % n_sets)
                with torch.cuda.stream(side):
                    graph.replay()
                    side.synchronize()
                    if world > 1:
                        dist.barrier()
                    torch.cuda.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(side)
                    for _ in range(replays):
                        graph.replay()
                    b.record(side)
                    side.synchronize()
                t = torch.tensor([a.elapsed_time(b) * 1e3 / (replays * calls)], device=dev, dtype=torch.float64)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                del graph
                return float(t)

            row = {"M": M, "K": K, "N": N, "tp": world, "form": hb.fused_rowparallel_form(tp, M, N, Kl, algo),
                   "weight_sets": n_sets, "calls_per_graph": calls}
            row["fused_us"] = graph_time(fused)
            row["baseline_us"] = graph_time(baseline)
            row["ratio"] = row["baseline_us"] / row["fused_us"]
            hbm_bytes = 2 * (Kl * N + M * Kl + 3 * M * N + N)
            nvl_bytes = 2 * (world - 1) / world * 2 * M * N if world > 1 else 0
            row["roofline_us"] = max(hbm_bytes / hbm_gbs / 1e3, nvl_bytes / NVLINK_GBS / 1e3)
            row["frac_of_roofline"] = row["roofline_us"] / row["fused_us"]
            if check:
                # both arms ran the same inputs last (weight set (calls-1) % n_sets): same sums up to
                # the order of the additions and one bf16 rounding of the partials
                diff = (out_f[1].float() - out_b[1].float()).abs().max() / out_b[1].float().abs().max()
                t = torch.tensor([float(diff)], device=dev, dtype=torch.float64)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                row["max_rel_diff_resid"] = float(t)
            if tp is not None:
                row["status"] = tp.status()
            rows.append(row)
    return rows


def main() -> None:
    import torch
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry

    ap = argparse.ArgumentParser()
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
    tp = hb.TpWorld.from_torch_distributed(local, staging_bytes=96 << 20, nccl=True) if world > 1 else None
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    rows = run_points(hb, tp, rank, world, dev, float(peaks.get("hbm_gbs", 6650.0)), ms=[int(m) for m in args.ms.split(",")])
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if args.out:
            Path(args.out).write_text(json.dumps(rows, indent=1))
    if tp is not None:
        torch.cuda.synchronize()
        dist.barrier()
        tp.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
