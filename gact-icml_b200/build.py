"""Builds libgact_b200.so (the C-ABI library, sm_100a only) next to the ``gact`` Python package.

    python gact-icml_b200/build.py [--force] [--verbose]

The shared object is built in-tree so that it travels with a snapshot of the repository; it is git-ignored.
"""
from __future__ import annotations

import argparse
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
INCLUDE = HERE.parent / "include"
OUT = HERE / "gact" / "libgact_b200.so"
OBJ = HERE / "build"

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", f"-I{INCLUDE}", f"-I{CSRC}"]


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    OBJ.mkdir(exist_ok=True)
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = ["nvcc", "-c", str(src), "-o", str(obj)] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=4) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode:
                print(" ".join(cmd))
                print(r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError("nvcc failed")
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if force or jobs or _stale(OUT, objs):
        cmd = ["nvcc", "-shared", "-o", str(OUT)] + [str(o) for o in objs] + ["-gencode", "arch=compute_100a,code=sm_100a"]
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
