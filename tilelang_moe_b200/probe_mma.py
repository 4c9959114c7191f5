"""Build and run the tcgen05.mma measurement tool (``csrc/probe_mma.cu``) on the current GPU.

    python -m tilelang_moe_b200.probe_mma            # clocks per K=16 step of the instruction shapes the GEMM kernels use
    python -m tilelang_moe_b200.probe_mma layout     # where cta_group::2 M=128 accumulators sit in tensor memory

It is a stand-alone executable (no part of ``libmoe_b200.so``): nvcc compiles it next to the library's objects on
first use.  The tile shapes of the grouped GEMM follow from its output; the summary of a run on a B200 is kept with
the other measurement summaries of this repository.
"""
from __future__ import annotations

import subprocess
import sys

from .build import CSRC, PKG, _nvcc

SRC = CSRC / "probe_mma.cu"
EXE = PKG / "build" / "probe_mma"


def build(force: bool = False):
    EXE.parent.mkdir(exist_ok=True)
    if force or not EXE.exists() or EXE.stat().st_mtime < SRC.stat().st_mtime:
        subprocess.run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", str(EXE), str(SRC)],
                       check=True)
    return EXE


if __name__ == "__main__":
    exe = build()
    sys.exit(subprocess.run([str(exe), *sys.argv[1:]]).returncode)
