"""Micro-benchmarks of the two HBM-bound kernels of the decode step, one GPU:

    python vllm-hb_b200/bench_kernels.py gemm      [--cublas] [--iters 24] [--out FILE]
    python vllm-hb_b200/bench_kernels.py attention [--iters 24] [--out FILE]
    python vllm-hb_b200/bench_kernels.py gemm --only qkv8b --plain     # one shape, no graph: for ncu
    python vllm-hb_b200/bench_kernels.py gemm --cublas --buffers 1     # weights resident in L2 where they fit

gemm       Y = X W^T (hb_gemm_ex) on the projection shapes of the Llama-3.1-8B (TP=1) and
           70B (TP=2/4/8) decode steps, optionally next to torch.matmul (cuBLAS).
attention  hb_paged_decode_attention on the KV shapes of the same configurations.

Every point is a CUDA graph of `iters` launches that rotate over several weight / KV
buffers (together larger than the 126 MB L2), replayed four times and timed with CUDA
events; GB/s = algorithmic bytes (weights, or K and V rows) / time.  Inputs: X ~N(0,1),
W ~N(0,0.02), KV ~N(0,1), block tables a random permutation of the pool.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

GEMM_SHAPES = [
    # name, M (batch), N (weight rows), K, epilogue (1 = SwiGLU over [gate|up] rows), fp32 out
    ("qkv8b", 64, 6144, 4096, 0, False),
    ("o8b", 64, 4096, 4096, 0, False),
    ("gate_up8b", 64, 28672, 4096, 1, False),
    ("down8b", 64, 4096, 14336, 0, False),
    ("lm_head8b", 64, 128256, 4096, 0, True),
    ("o70b-tp2", 64, 8192, 4096, 0, False),
    ("down70b-tp2", 64, 8192, 14336, 0, False),
    ("gate_up70b-tp4", 128, 14336, 8192, 1, False),
    ("down70b-tp4", 128, 8192, 7168, 0, False),
    ("qkv70b-tp8", 128, 1280, 8192, 0, False),
    ("o70b-tp8", 128, 8192, 1024, 0, False),
    ("gate_up70b-tp8", 128, 7168, 8192, 1, False),
    ("down70b-tp8", 128, 8192, 3584, 0, False),
]

ATTN_SHAPES = [
    # name, sequences, query heads, kv heads, context tokens
    ("8b", 64, 32, 8, 576),
    ("8b-long", 64, 32, 8, 2048),
    ("70b-tp2", 128, 32, 4, 1100),
    ("70b-tp8", 128, 8, 1, 1100),
]


def time_graph(run, iters: int, plain: bool) -> float:
    """Microseconds per launch of run(i, stream)."""
    st0 = torch.cuda.current_stream().cuda_stream
    for i in range(3):
        run(i, st0)
    torch.cuda.synchronize()
    if plain:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters):
            run(i, st0)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / iters
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for i in range(iters):
                run(i, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(4):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (4 * iters)


def bench_gemm(hb, args) -> list[dict]:
    dev = torch.device("cuda", 0)
    rows = []
    for name, M, N, K, epi, f32 in GEMM_SHAPES:
        if args.only and name not in args.only.split(","):
            continue
        nbuf = args.buffers or (3 if N * K * 2 > (256 << 20) else 6)
        iters = max(6, args.iters // 4) if N * K * 2 > (256 << 20) else args.iters
        g = torch.Generator(device=dev).manual_seed(1)
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        ws = [(torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(nbuf)]
        n_out = N // 2 if epi == 1 else N
        y = torch.empty(M, n_out, device=dev, dtype=torch.float32 if f32 else torch.bfloat16)
        wk = torch.zeros(max(hb.lib.hb_gemm_ex_workspace_bytes(M, N, K, epi, 0), 16), dtype=torch.uint8, device=dev)

        def run(i, st):
            hb.check(hb.lib.hb_gemm_ex(st, y.data_ptr(), x.data_ptr(), ws[i % nbuf].data_ptr(), M, N, K, epi, int(f32), 0,
                                       wk.data_ptr()))

        us = time_graph(run, iters, args.plain)
        row = {"kernel": "gemm", "shape": name, "M": M, "N": N, "K": K, "swiglu": bool(epi), "us": us,
               "weight_gbs": N * K * 2 / us / 1e3}
        if args.cublas and not f32:
            y2 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

            def run_ref(i, st):
                torch.matmul(x, ws[i % nbuf].t(), out=y2)

            row["cublas_us"] = time_graph(run_ref, iters, args.plain)
        rows.append(row)
        print(json.dumps(row), flush=True)
        del ws
    return rows


def bench_attention(hb, args) -> list[dict]:
    dev = torch.device("cuda", 0)
    rows = []
    hd, nbuf = 128, 6
    for name, B, hq, hkv, ctx in ATTN_SHAPES:
        if args.only and name not in args.only.split(","):
            continue
        nblk = (ctx + 15) // 16
        num_blocks = B * nblk + 8
        g = torch.Generator(device=dev).manual_seed(1)
        q = torch.randn(B, hq, hd, device=dev, generator=g).to(torch.bfloat16)
        pools = [(torch.randn(num_blocks, hkv, 16, hd, device=dev, generator=g).to(torch.bfloat16),
                  torch.randn(num_blocks, hkv, 16, hd, device=dev, generator=g).to(torch.bfloat16)) for _ in range(nbuf)]
        tables = torch.randperm(num_blocks - 8, device=dev, generator=g)[: B * nblk].reshape(B, nblk).to(torch.int32)
        ctxs = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        out = torch.empty_like(q)
        for splits in ([1] if args.plain else [1, 2, 4]):
            wsb = torch.zeros(max(hb.lib.hb_attention_workspace_bytes(B, hq, hd, splits), 16), dtype=torch.uint8, device=dev)

            def run(i, st):
                kc, vc = pools[i % nbuf]
                hb.check(hb.lib.hb_paged_decode_attention(st, out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                          tables.data_ptr(), ctxs.data_ptr(), B, hq, hkv, hd, nblk,
                                                          num_blocks, splits, wsb.data_ptr(), hb.BF16))

            us = time_graph(run, args.iters, args.plain)
            row = {"kernel": "attention", "shape": name, "seqs": B, "q_heads": hq, "kv_heads": hkv, "ctx": ctx,
                   "splits": splits, "us": us, "kv_gbs": B * ctx * hkv * hd * 2 * 2 / us / 1e3}
            rows.append(row)
            print(json.dumps(row), flush=True)
        del pools
    return rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attention"])
    ap.add_argument("--iters", type=int, default=24)
    ap.add_argument("--only", default="", help="comma-separated shape names")
    ap.add_argument("--cublas", action="store_true", help="gemm: also time torch.matmul on the same inputs")
    ap.add_argument("--plain", action="store_true", help="stream launches instead of a CUDA graph (for profilers)")
    ap.add_argument("--buffers", type=int, default=0,
                    help="gemm: weight buffers to rotate over (default 6, 3 for the largest; 1 keeps a matrix that "
                         "fits in L2 resident there: the time that is left is the part of the kernel that is not HBM)")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    hb = entry.load_package()
    if not torch.cuda.is_available():
        raise SystemExit("bench_kernels.py needs a GPU")
    torch.cuda.set_device(0)
    rows = bench_gemm(hb, args) if args.what == "gemm" else bench_attention(hb, args)
    if args.out:
        Path(args.out).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
