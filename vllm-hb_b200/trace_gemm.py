"""Phase timeline of the tcgen05 GEMM kernel, one GPU:

    python vllm-hb_b200/build.py --variant trace        # libhb_trace.so, -DHB_TC_TRACE
    python vllm-hb_b200/trace_gemm.py [--only qkv8b,down8b]

The trace variant of the library records the global nanosecond timer at fixed points of
every CTA's life (kernel entry, setup done, first stage landed, last MMA issued,
accumulator complete, the two cluster barriers of the split-K exchange, output staged,
bulk store read, exit) into a device array.  This script launches each shape a few times
back to back (rotating weights), reads the array of the last launch and prints, per
point, the min / median / max over the CTAs relative to the earliest CTA start, plus the
SM clock seen by the CTAs.  The product library carries none of this.
"""
from __future__ import annotations

import argparse
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
from bench_kernels import GEMM_SHAPES  # noqa: E402  (same shapes as the micro-benchmark)

POINTS = ["start", "setup done", "first stage landed", "last MMA issued", "accumulator complete",
          "cluster barrier 1", "cluster barrier 2", "exit"]
EPILOGUE = [(10, "output staged"), (11, "CTA barrier"), (12, "bulk store read")]
SLOTS = 16


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    path = HERE / "libhb_trace.so"
    if not path.exists():
        raise SystemExit("build the trace variant first: python vllm-hb_b200/build.py --variant trace")
    lib = C.CDLL(str(path))
    vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int
    lib.hb_gemm_ex.argtypes = [vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, vp]
    lib.hb_gemm_ex_workspace_bytes.restype = C.c_size_t
    lib.hb_gemm_ex_workspace_bytes.argtypes = [i64, i64, i64, i32, i32]
    lib.hb_debug_tc_trace.argtypes = [vp, i32]
    lib.hb_last_error.restype = C.c_char_p
    dev = torch.device("cuda", 0)
    for name, M, N, K, epi, f32 in GEMM_SHAPES:
        if args.only and name not in args.only.split(","):
            continue
        nbuf = 3 if N * K * 2 > (256 << 20) else 6
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        ws = [(torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(nbuf)]
        y = torch.empty(M, N // 2 if epi else N, device=dev, dtype=torch.float32 if f32 else torch.bfloat16)
        wk = torch.zeros(max(lib.hb_gemm_ex_workspace_bytes(M, N, K, epi, 0), 16), dtype=torch.uint8, device=dev)
        st = torch.cuda.current_stream().cuda_stream
        for i in range(nbuf + 1):
            rc = lib.hb_gemm_ex(st, y.data_ptr(), x.data_ptr(), ws[i % nbuf].data_ptr(), M, N, K, epi, int(f32), 0,
                                wk.data_ptr())
            if rc:
                raise SystemExit(lib.hb_last_error().decode())
        torch.cuda.synchronize()
        buf = np.zeros((4096, SLOTS), dtype=np.uint64)
        if lib.hb_debug_tc_trace(buf.ctypes.data, 4096):
            raise SystemExit("reading the trace failed")
        t0 = buf[:, 0].astype(np.int64)
        b = buf[t0 > t0.max() - 2_000_000].astype(np.int64)   # the CTAs of the last launch
        base = b[:, 0].min()
        per_sm = np.bincount(b[:, 9], minlength=148)
        mhz = np.median((b[:, 15] - b[:, 8]) / ((b[:, 7] - b[:, 0]) / 1e3))
        print(f"--- {name} M={M} N={N} K={K}: {len(b)} CTAs on {np.count_nonzero(per_sm)} SMs "
              f"(max {per_sm.max()} per SM), SM clock {mhz:.0f} MHz")
        for s, nm in list(enumerate(POINTS))[:5] + [(s, n) for s, n in enumerate(POINTS)][5:7] + EPILOGUE + [(7, "exit")]:
            v = (b[:, s] - base) / 1e3
            v = v[(b[:, s] > 0) & (v > -1e3) & (v < 1e4)]
            if len(v):
                print(f"   {nm:22s} min {v.min():7.1f}  median {np.median(v):7.1f}  max {v.max():7.1f} us")
        del ws


if __name__ == "__main__":
    main()
