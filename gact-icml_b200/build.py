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
    build_fastcall(force)
    build_hooks(force)
    return OUT


FASTCALL = HERE / "gact" / "_fastcall.so"


def build_fastcall(force: bool = False):
    """The CPython entry points for the two hot calls (csrc/fastcall.c), linked against libgact_b200.so beside it.
    Optional: without it the binding goes through ctypes.  Returns the path, or None when the compile failed."""
    src = CSRC / "fastcall.c"
    if not (force or _stale(FASTCALL, [src, OUT] + sorted(INCLUDE.glob("*.h")))):
        return FASTCALL
    import sysconfig
    cmd = ["gcc", "-O2", "-shared", "-fPIC", f"-I{sysconfig.get_paths()['include']}", f"-I{INCLUDE}", str(src), "-o", str(FASTCALL),
           f"-L{OUT.parent}", "-l:" + OUT.name, "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        print("fastcall module not built:", r.stderr.strip().splitlines()[-1] if r.stderr.strip() else r.returncode)
        return None
    return FASTCALL


HOOKS = HERE / "gact" / "_hooks.so"


def build_hooks(force: bool = False):
    """The native fast path of the saved-tensor hooks (csrc/hooks.cpp): host C++ against libtorch, calling
    libgact_b200.so beside it through the C ABI.  Optional: without it the hooks run their Python implementation.
    Returns the path, or None when the compile failed."""
    src = CSRC / "hooks.cpp"
    if not (force or _stale(HOOKS, [src, OUT] + sorted(INCLUDE.glob("*.h")))):
        return HOOKS
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce
    incs = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}", f"-I{INCLUDE}"]
    libs = [f"-L{p}" for p in ce.library_paths("cuda")] + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"] + incs + [str(src), "-o", str(HOOKS)] + libs + \
          [f"-L{OUT.parent}", "-l:" + OUT.name, "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        print("hooks module not built:", r.stderr.strip().splitlines()[-1] if r.stderr.strip() else r.returncode)
        return None
    return HOOKS


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
