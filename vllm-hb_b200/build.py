"""Build libhb.so in-tree with nvcc for sm_100a.

    python vllm-hb_b200/build.py [--force] [--verbose]

Every translation unit under csrc/ is compiled to an object file under build/ and
linked into vllm-hb_b200/libhb.so (static cudart, no other link-time dependency; NCCL
is opened lazily at run time).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ_DIR = HERE / "build"
LIB = HERE / "libhb.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function,-Wno-parentheses",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found")
    return cand


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cc")))


def _headers_mtime() -> float:
    hs = list(CSRC.glob("*.h")) + list((HERE.parent / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def _compile(src: Path, force: bool, verbose: bool, obj_dir: Path = OBJ_DIR, defines: tuple = ()) -> Path:
    obj = obj_dir / (src.name + ".o")
    newest_dep = max(src.stat().st_mtime, _headers_mtime())
    if not force and obj.exists() and obj.stat().st_mtime >= newest_dep:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cc":
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose or res.stderr.strip():
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, variant: str = "") -> Path:
    """variant "trace": the library with -DHB_TC_TRACE (phase timestamps inside the GEMM
    kernel, read by trace_gemm.py), built beside the product as libhb_trace.so."""
    obj_dir = OBJ_DIR if not variant else HERE / f"build_{variant}"
    lib = LIB if not variant else HERE / f"libhb_{variant}.so"
    defines = {"": (), "trace": ("HB_TC_TRACE",)}[variant]
    obj_dir.mkdir(exist_ok=True)
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose, obj_dir, defines), srcs))
    if force or not lib.exists() or any(o.stat().st_mtime > lib.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-shared", "-o", str(lib), *map(str, objs), "-ldl", "-lpthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--variant", default="", choices=["", "trace"])
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.variant))
