"""B200 (sm_100a) implementation of the contextual-sparsity MLP path of
NimbleEdge/sparse_transformers, behind that project's own operator API.

Exports, with the names the reference exposes (sparse_transformers/__init__.py:24-33 and
README "sparse_mlp_forward(x, concat_w, active_down_w, down_buf, combined_buf, act)"):

  WeightCache            torch.classes.sparse_mlp.WeightCache
  sparse_mlp_forward     6-argument wrapper over torch.ops.sparse_mlp.forward (has_gate=True)
  approx_topk_threshold  torch.ops.sparse_mlp.approx_topk_threshold

plus the host-side mirror of the three hot functions of src/modeling_skip.py
(FastLoRAProjection, SkipMLP, compute_binary_mask) and the fused layer/stack objects.

Everything runs through libstx.so (hand-written CUDA behind the C ABI of include/stx.h).
Importing this package fails if the native libraries are missing: there is no CPU path.
Unlike the reference's package, importing it does not touch thread-count settings.
"""
from __future__ import annotations

import os
import sys

if any(a == "sparse_transformers_b200.build" for a in getattr(sys, "orig_argv", [])):
    # `python -m sparse_transformers_b200.build`: the libraries may not exist yet
    raise SystemExit(__import__("runpy").run_path(os.path.join(os.path.dirname(__file__), "build.py"), run_name="__main__") and 0)

import torch

from . import _capi  # noqa: F401  (raises ImportError when libstx.so is absent)

_HERE = os.path.dirname(os.path.abspath(__file__))
_SHIM = os.path.join(_HERE, "libstx_torch.so")
if not os.path.isfile(_SHIM):
    raise ImportError(f"{_SHIM} is missing: build it with `python -m sparse_transformers_b200.build`")
torch.classes.load_library(_SHIM)

WeightCache = torch.classes.sparse_mlp.WeightCache
approx_topk_threshold = torch.ops.sparse_mlp.approx_topk_threshold


def sparse_mlp_forward(x, concat_weight, active_down_weight, down_buf, combined_buf, act="silu", has_gate=True):
    """README-documented call of the reference (README.md:108-117); the registered op takes a
    seventh positional ``has_gate`` (sparse_mlp_op.cpp:53-60) which defaults to True here.
    Returns an alias of ``down_buf`` (sparse_mlp_op.cpp:191)."""
    return torch.ops.sparse_mlp.forward(x, concat_weight, active_down_weight, down_buf, combined_buf, act, has_gate)


from .layer import SparseLayer, SparseStack  # noqa: E402
from .skip import FastLoRAProjection, SkipMLP, compute_binary_mask  # noqa: E402

__all__ = [
    "WeightCache", "sparse_mlp_forward", "approx_topk_threshold",
    "SparseLayer", "SparseStack", "FastLoRAProjection", "SkipMLP", "compute_binary_mask",
]
