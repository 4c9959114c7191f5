"""Build the checker side (test infrastructure): the C restatement of the routing oracle, compiled with gcc, and -
where the reference checkout is present - a copy of the reference's own CPU baseline files under ``oracle/_ref/``
(git-ignored output, like the compiled library) so that the benchmark's reference arm can time the reference's
unmodified Python on a machine where the checkout itself is absent.

    python oracle/build.py        ->  oracle/libroute_oracle.so  [+ oracle/_ref/*_baseline.py]
"""
import os
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


REF_DIR = HERE / "_ref"
REF_FILES = ("topk_softmax_baseline.py", "grouped_gemm_baseline.py", "fusedmoe_baseline.py")


def fetch_reference(reference_root=None):
    """Copy the reference's PyTorch baseline files (they import nothing but torch) into ``oracle/_ref/``.
    Returns the directory, or None where no reference checkout is reachable."""
    root = Path(reference_root or os.environ.get("MOE_REFERENCE_DIR", "/root/reference"))
    src = root / "kernels"
    if not all((src / f).exists() for f in REF_FILES):
        return None
    REF_DIR.mkdir(exist_ok=True)
    for f in REF_FILES:
        shutil.copyfile(src / f, REF_DIR / f)
    return REF_DIR


if __name__ == "__main__":
    print(build(force=True))
    print(fetch_reference())
