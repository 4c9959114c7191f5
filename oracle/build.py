"""Compile the C restatement of the routing oracle (test infrastructure) with gcc.

    python oracle/build.py        ->  oracle/libroute_oracle.so
"""
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "route_oracle.c"
LIB = HERE / "libroute_oracle.so"


def build(force: bool = False) -> Path:
    if LIB.exists() and not force and LIB.stat().st_mtime >= SRC.stat().st_mtime:
        return LIB
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        raise RuntimeError("no C compiler found for the oracle")
    subprocess.run([cc, "-O2", "-std=c99", "-shared", "-fPIC", "-o", str(LIB), str(SRC), "-lm"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
