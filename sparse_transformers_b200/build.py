"""In-tree build of the native libraries (run as ``python -m sparse_transformers_b200.build``).

  libstx.so        CUDA kernels + C ABI (include/stx.h); nvcc, sm_100a only, no torch
  libstx_torch.so  TORCH_LIBRARY(sparse_mlp) shim over the C ABI; g++, links libtorch

Both land next to this file so they travel with the source tree.
"""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIBSTX = os.path.join(HERE, "libstx.so")
LIBSHIM = os.path.join(HERE, "libstx_torch.so")

CU_SOURCES = ["stx_api.cu", "stx_cache.cu", "stx_predictor.cu", "stx_select.cu", "stx_mlp.cu", "stx_mlp_tma.cu", "stx_mlp_batch.cu", "stx_mlp_row.cu", "stx_stack_b1.cu", "stx_stack_flow.cu", "stx_prefill.cu", "stx_peer.cu", "stx_attn.cu", "stx_layer.cu"]

def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.isfile(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str], verbose: bool) -> str:
    if verbose:
        print(" ".join(shlex.quote(c) for c in cmd), flush=True)
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        sys.stderr.write(p.stdout)
        raise RuntimeError(f"build step failed ({p.returncode}): {cmd[0]}")
    return p.stdout


def cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build_libstx(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in os.listdir(CSRC) if h.endswith(".cuh")] + [os.path.join(INCLUDE, "stx.h")]
    if not force and _newer(LIBSTX, deps):
        return LIBSTX
    nvcc = os.path.join(cuda_home(), "bin", "nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xcompiler", "-fPIC", "-shared", f"-I{INCLUDE}", f"-I{CSRC}", "-Xptxas", "-v"] + shlex.split(os.environ.get("STX_NVCC_FLAGS", "")) + srcs + ["-o", LIBSTX]
    out = _run(cmd, verbose)
    with open(os.path.join(HERE, "ptxas_libstx.log"), "w") as f:  # registers / spills / shared memory per kernel
        f.write(out)
    return LIBSTX


def build_shim(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "torch_shim.cpp")
    if not force and _newer(LIBSHIM, [src, os.path.join(INCLUDE, "stx.h"), LIBSTX]):
        return LIBSHIM
    import torch
    from torch.utils import cpp_extension as ce

    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    incs = ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home(), "include"), INCLUDE]
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in incs]
    cmd += [src, "-o", LIBSHIM, f"-L{HERE}", "-lstx", "-Wl,-rpath,$ORIGIN",
            f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            f"-L{os.path.join(cuda_home(), 'lib64')}", "-lcudart"]
    _run(cmd, verbose)
    return LIBSHIM


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_libstx(force, verbose)
    build_shim(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built", LIBSTX, LIBSHIM)
