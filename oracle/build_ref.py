"""Build recipe for the compiled reference (test infrastructure, not product code).

Compiles the reference project's own CPU operator sources
(sparse_transformers/csrc/sparse_mlp_op.cpp, which includes weight_cache.h and
approx_topk.h) *where they lie*, unmodified, into ``oracle/_ref/sparse_mlp_ref.so``.
Nothing is copied out of the reference tree; only the built shared object lands in
``oracle/_ref/`` (git-ignored).

The one deviation from a stock build is ``-Dsparse_mlp=sparse_mlp_ref``: the token
``sparse_mlp`` occurs in the source only as the TORCH_LIBRARY namespace argument
(sparse_mlp_op.cpp:195), so this registers the reference class/op under
``torch.classes.sparse_mlp_ref.WeightCache`` / ``torch.ops.sparse_mlp_ref.forward``
and lets the compiled reference be loaded in the same process as this repository's own
``sparse_mlp`` library.  ``-march=x86-64-v3`` (not ``native``) is used so the object
built on one machine runs on another x86-64 host; the matmuls live in libtorch anyway.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--force]
"""
from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_SO = os.path.join(OUT_DIR, "sparse_mlp_ref.so")
# where the reference project's checkout lies: $STX_REFERENCE_DIR, else a directory named "reference" beside
# this repository (absent on machines that only run the prebuilt oracle/_ref)
DEFAULT_REFERENCE = os.environ.get("STX_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def ref_so_path() -> str:
    return OUT_SO


def build(reference: str = DEFAULT_REFERENCE, force: bool = False, verbose: bool = True) -> str | None:
    """Compile the reference op. Returns the .so path, or None if the sources are absent."""
    src = os.path.join(reference, "sparse_transformers", "csrc", "sparse_mlp_op.cpp")
    if not os.path.isfile(src):
        return OUT_SO if os.path.isfile(OUT_SO) else None
    if os.path.isfile(OUT_SO) and not force and os.path.getmtime(OUT_SO) >= os.path.getmtime(src):
        return OUT_SO
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT_DIR, exist_ok=True)
    incs = ce.include_paths() + [sysconfig.get_paths()["include"]]
    try:
        import pybind11

        incs.append(pybind11.get_include())
    except Exception:
        pass
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    gcc_lib = "/usr/lib/gcc/x86_64-linux-gnu/13"
    cmd = [
        "g++", "-std=c++17", "-O3", "-fopenmp", "-fPIC", "-shared", "-march=x86-64-v3",
        "-DCPU_ONLY", "-Dsparse_mlp=sparse_mlp_ref",
        "-DTORCH_EXTENSION_NAME=sparse_mlp_ref", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        "-w",
    ]
    cmd += [f"-I{p}" for p in incs]
    cmd += [src, "-o", OUT_SO, f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}",
            "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python"]
    # `-fopenmp` at link time needs libgomp.spec through the compiler driver; linking
    # libgomp explicitly avoids depending on it.
    if os.path.isdir(gcc_lib):
        cmd += [f"-L{gcc_lib}"]
    cmd += ["-lgomp"]
    # compile and link in one step would pass -fopenmp to the link; split it.
    obj = os.path.join(OUT_DIR, "sparse_mlp_op.o")
    compile_cmd = [c for c in cmd if not c.startswith("-l") and not c.startswith("-L")
                   and not c.startswith("-Wl,") and c != "-shared"]
    compile_cmd[compile_cmd.index("-o") + 1] = obj
    compile_cmd.insert(1, "-c")
    link_cmd = ["g++", "-shared", obj, "-o", OUT_SO] + [c for c in cmd if c.startswith(("-l", "-L", "-Wl,"))]
    for c in (compile_cmd, link_cmd):
        if verbose:
            print(" ".join(shlex.quote(x) for x in c), flush=True)
        subprocess.check_call(c)
    os.remove(obj)
    return OUT_SO


def load():
    """Load the compiled reference into this process; returns (WeightCache class, forward op, approx_topk op)."""
    import torch

    if not os.path.isfile(OUT_SO):
        raise FileNotFoundError(OUT_SO)
    torch.classes.load_library(OUT_SO)
    return (torch.classes.sparse_mlp_ref.WeightCache,
            torch.ops.sparse_mlp_ref.forward,
            torch.ops.sparse_mlp_ref.approx_topk_threshold)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = build(a.reference, a.force)
    print("built:" if out else "reference sources not found; nothing built", out or "")
    sys.exit(0)
