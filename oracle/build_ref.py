"""Build the UNMODIFIED reference extensions into ``oracle/_ref/`` (test infrastructure only).

The reference ships three torch extensions (its ``gact/setup.py``): ``calc_precision`` (host C++),
``minimax`` and ``quantization`` (CUDA).  This recipe compiles them from the sources where they lie
in a read-only checkout of the reference, for sm_100a, against the installed torch.  Nothing is
copied: the only additions are two forwarding headers under ``oracle/ref_shim/`` for include paths
that moved in current PyTorch (``ATen/CUDAGeneratorImpl.h``, ``THC/THCAtomics.cuh``).

The outputs (``oracle/_ref/ref_*.so``) are git-ignored.  They are used only by tests and by the
benchmark's reference arm, as the checker: the greedy bit allocator runs on the CPU anywhere; the CUDA
kernels run only where a GPU exists.  The product never loads them.

``install_package`` additionally lays the reference out as an importable package under
``oracle/_ref/pkg/gact`` - what ``pip install --target`` of the reference would produce: its seven Python
files as they are, and the same three extensions linked under the names the package imports
(``gact.cpp_extension.{calc_precision,minimax,quantization}``).  Only the benchmark's reference TRAINING arm
imports it (``bench.py --impl reference --workload ...``), in a process that never imports the product's
``gact``.  Git-ignored like the rest of ``oracle/_ref``.

Usage:  python oracle/build_ref.py [--ref /path/to/reference] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
SHIM = HERE / "ref_shim"
# checkout of the reference: $GACT_REFERENCE_DIR, else a folder named "reference" beside this repository
DEFAULT_REF = Path(os.environ.get("GACT_REFERENCE_DIR", str(HERE.parent.parent / "reference")))

EXTENSIONS = {
    # name -> (sources relative to <ref>/gact/gact/cpp_extension, needs nvcc)
    "ref_calc_precision": (["calc_precision.cc"], False),
    "ref_minimax": (["minimax.cc", "minimax_cuda_kernel.cu"], True),
    "ref_quantization": (["quantization.cc", "quantization_cuda_kernel.cu"], True),
}


def _torch_paths():
    import torch  # noqa: F401
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    lib = ce.library_paths("cuda")
    return inc, lib


def _run(cmd):
    print(" ".join(str(c) for c in cmd), flush=True)
    subprocess.check_call([str(c) for c in cmd])


def build(ref: Path = DEFAULT_REF, force: bool = False) -> dict:
    """Compile every extension; returns {name: path or None}.  Missing reference => all None."""
    src_dir = ref / "gact" / "gact" / "cpp_extension"
    result = {}
    if not src_dir.is_dir():
        for name in EXTENSIONS:
            so = OUT / f"{name}.so"
            result[name] = so if so.exists() else None
        return result
    OUT.mkdir(exist_ok=True)
    inc, lib = _torch_paths()
    common = ["-O2", "-std=c++17", "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1"]
    incs = [f"-I{SHIM}", f"-I{src_dir}"] + [f"-I{p}" for p in inc]
    libs = [f"-L{p}" for p in lib] + ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    for name, (srcs, cuda) in EXTENSIONS.items():
        so = OUT / f"{name}.so"
        result[name] = so
        if so.exists() and not force:
            continue
        objs = []
        for s in srcs:
            obj = OUT / f"{name}.{Path(s).stem}.o"
            objs.append(obj)
            defs = [f"-DTORCH_EXTENSION_NAME={name}"]
            if s.endswith(".cu"):
                # nvcc's defaults on purpose (in particular -fmad=true), as the reference's setup.py
                # passes no flags of its own.
                _run(["nvcc", "-c", src_dir / s, "-o", obj, "-gencode", "arch=compute_100a,code=sm_100a",
                      "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
                      "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                      "-D__CUDA_NO_HALF2_OPERATORS__", "-D__CUDA_NO_BFLOAT16_CONVERSIONS__"]
                     + common + defs + incs)
            else:
                _run(["g++", "-c", src_dir / s, "-o", obj, "-fPIC"] + common + defs + incs)
        link = ["g++", "-shared", "-o", so] + objs + libs
        if cuda:
            link += ["-lc10_cuda", "-ltorch_cuda", "-lcudart"]
        _run(link)
        for o in objs:
            os.remove(o)
    return result


def install_package(ref: Path = DEFAULT_REF, force: bool = False):
    """The reference as an importable package under oracle/_ref/pkg (see the module docstring).  Returns the
    package root, or None when neither a checkout of the reference nor an earlier install is there."""
    import shutil
    pkg = OUT / "pkg"
    src_py = ref / "gact" / "gact"
    src_dir = src_py / "cpp_extension"
    if not src_dir.is_dir():
        return pkg if (pkg / "gact" / "__init__.py").exists() else None
    dst = pkg / "gact" / "cpp_extension"
    dst.mkdir(parents=True, exist_ok=True)
    for f in sorted(src_py.glob("*.py")):
        shutil.copyfile(f, pkg / "gact" / f.name)
    inc, lib = _torch_paths()
    common = ["-O2", "-std=c++17", "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1"]
    incs = [f"-I{SHIM}", f"-I{src_dir}"] + [f"-I{p}" for p in inc]
    libs = [f"-L{p}" for p in lib] + ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    for ref_name, (srcs, cuda) in EXTENSIONS.items():
        name = ref_name[len("ref_"):]
        so = dst / f"{name}.so"
        if so.exists() and not force:
            continue
        objs = []
        for s in srcs:
            obj = dst / f"{name}.{Path(s).stem}.o"
            objs.append(obj)
            defs = [f"-DTORCH_EXTENSION_NAME={name}"]
            if s.endswith(".cu"):
                _run(["nvcc", "-c", src_dir / s, "-o", obj, "-gencode", "arch=compute_100a,code=sm_100a",
                      "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
                      "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                      "-D__CUDA_NO_HALF2_OPERATORS__", "-D__CUDA_NO_BFLOAT16_CONVERSIONS__"]
                     + common + defs + incs)
            else:
                _run(["g++", "-c", src_dir / s, "-o", obj, "-fPIC"] + common + defs + incs)
        link = ["g++", "-shared", "-o", so] + objs + libs
        if cuda:
            link += ["-lc10_cuda", "-ltorch_cuda", "-lcudart"]
        _run(link)
        for o in objs:
            os.remove(o)
    return pkg


def load(name: str):
    """Import a built reference extension (``ref_calc_precision`` / ``ref_minimax`` / ``ref_quantization``)
    or return None when it was never built."""
    so = OUT / f"{name}.so"
    if not so.exists():
        return None
    import importlib.util

    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location(name, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=str(DEFAULT_REF))
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = build(Path(a.ref), a.force)
    for k, v in out.items():
        print(k, "->", v)
    print("package ->", install_package(Path(a.ref), a.force))
    sys.exit(0)
