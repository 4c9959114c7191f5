"""Build ``libmoe_b200.so`` in-tree with nvcc for sm_100a.

    python -m tilelang_moe_b200.build [--force] [--verbose]

The shared library carries the CUDA kernels and the C ABI declared in
``include/moe_b200.h``.  It is built next to this file so that it travels with
the source tree; nothing is installed into site-packages and nothing is JIT
compiled at import time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libmoe_b200.so"
SOURCES = ["common.cu", "topk_softmax.cu", "route.cu", "gemm_sm100.cu", "mhc.cu", "layer.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def sources():
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def needs_build(lib: Path = None) -> bool:
    lib = LIB if lib is None else lib
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "moe_b200.h"]
    return any(d.stat().st_mtime > t for d in deps if d.exists())


TRACE_LIB = PKG / "libmoe_b200_trace.so"   # --trace: same sources with -DMOE_GEMM_TRACE (tile timeline tool only)
CHECK_LIB = PKG / "libmoe_b200_check.so"   # --check: same sources with -DMOE_BOUNDS_CHECK (index-checked accesses)


def build(force: bool = False, verbose: bool = False, trace: bool = False, check: bool = False) -> Path:
    if check and not force and CHECK_LIB.exists() and not needs_build(CHECK_LIB):
        return CHECK_LIB
    if not trace and not check and not force and not needs_build():
        return LIB
    objs = []
    obj_dir = PKG / ("build_trace" if trace else ("build_check" if check else "build"))
    obj_dir.mkdir(exist_ok=True)
    procs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if trace:
            cmd.insert(1, "-DMOE_GEMM_TRACE")
        if check:
            cmd.insert(1, "-DMOE_BOUNDS_CHECK")
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src.name}:\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc compilation failed")
    target = TRACE_LIB if trace else (CHECK_LIB if check else LIB)
    link = [_nvcc(), "-shared", "-o", str(target), *[str(o) for o in objs], "-gencode",
            "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout)
    return target


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv,
                 check="--check" in sys.argv)
    print(path)
