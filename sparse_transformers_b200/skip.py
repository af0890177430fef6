"""Host-side mirror of the three hot pieces of the reference's src/modeling_skip.py, wired to
the native operators: FastLoRAProjection (:32-53), SkipMLP (:55-128) and
SkipDecoderLayer._compute_binary_mask (:204-219).  Same constructor arguments and method
names, so a LlamaSkip-style decoder layer can use them unchanged.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

_ACT_FN = {
    "relu": torch.relu,
    "silu": torch.nn.functional.silu,
    "gelu_pytorch_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
    "gelu": torch.nn.functional.gelu,
    "sigmoid": torch.sigmoid,
}


class FastLoRAProjection(nn.Module):
    """Low-rank importance predictor; forward = up(down(x)) (modeling_skip.py:52-53)."""

    def __init__(self, hidden_size: int, intermediate_size: int, lora_size: int):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.lora_size = lora_size
        self.down = nn.Linear(hidden_size, lora_size, bias=False)
        self.up = nn.Linear(lora_size, intermediate_size, bias=False)

    def _init_weights(self):
        with torch.no_grad():
            nn.init.xavier_normal_(self.down.weight)
            nn.init.xavier_normal_(self.up.weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.up(self.down(x))


def compute_binary_mask(hidden_states: torch.Tensor, lora: FastLoRAProjection, sparsity_method: str = "naive",
                        *, threshold: float = 0.0, k: Optional[int] = None, std_multiplier: Optional[float] = None,
                        weight_cache=None) -> torch.Tensor:
    """_compute_binary_mask (modeling_skip.py:204-219) in one native call: predictor, per-row
    rule, OR over the batch; if ``weight_cache`` is given it is updated like :216-217.

    ``naive`` is ``scores >= threshold`` (the reference fixes threshold = 0); ``topk`` takes
    ``k``; ``statistical_topk`` takes ``std_multiplier`` = Phi^-1(sparsity) (:141-142)."""
    if sparsity_method in ("naive", "threshold"):
        param = float(threshold)
    elif sparsity_method == "topk":
        param = float(k)
    elif sparsity_method == "statistical_topk":
        param = float(std_multiplier)
    else:
        raise ValueError(f"unknown sparsity_method {sparsity_method!r}")
    x = hidden_states.reshape(-1, hidden_states.shape[-1])
    mask = torch.ops.sparse_mlp.predict_mask(x, lora.down.weight, lora.up.weight, sparsity_method, param)
    if weight_cache is not None:
        weight_cache.update_active_weights(mask)
    return mask


class SkipMLP(nn.Module):
    """Gated MLP whose decode path runs on the active neurons only (modeling_skip.py:55-128)."""

    def __init__(self, hidden_size: int, intermediate_size: int, sparsity: float, bias: bool = False,
                 act_fn: str = "silu", use_weight_cache: bool = True):
        super().__init__()
        if bias:
            raise NotImplementedError("the sparse path has no bias terms (the reference's WeightCache ignores them too)")
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)
        self.sparsity = sparsity
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.act_fn_name = act_fn
        self.act_fn = _ACT_FN[act_fn]
        self.use_weight_cache = use_weight_cache
        self.fused_getters = True  # False: the reference's literal call sequence (getters + sparse_mlp_forward)
        self.register_buffer("init_mask", torch.ones(intermediate_size, dtype=torch.bool))
        self.weight_cache = None
        self.register_buffer("down_proj_buffer", torch.zeros(1, hidden_size), persistent=False)
        self.register_buffer("combined_proj_buffer", torch.zeros(1, 2 * int(intermediate_size * sparsity)), persistent=False)

    def initialize_weight_cache(self):
        """Build the device-resident cache from the current weights (modeling_skip.py:81-92)."""
        if self.weight_cache is None and self.use_weight_cache:
            from . import WeightCache

            self.weight_cache = WeightCache(self.init_mask, self.hidden_size, self.gate_proj.weight,
                                            self.up_proj.weight, self.down_proj.weight, True)

    def reset_cache(self):
        self.weight_cache = None
        self.initialize_weight_cache()

    def forward(self, x: torch.Tensor, use_sparse: bool = True) -> torch.Tensor:
        if use_sparse:
            return self._forward_sparse_weight_cache(x)
        return self._forward_dense(x)

    def _forward_sparse_weight_cache(self, x: torch.Tensor) -> torch.Tensor:
        # modeling_skip.py:114-117, as one fused native op instead of two matmuls
        from . import sparse_mlp_forward

        if self.down_proj_buffer.dtype != x.dtype:
            self.down_proj_buffer = self.down_proj_buffer.to(x.dtype)
            self.combined_proj_buffer = self.combined_proj_buffer.to(x.dtype)
        if self.fused_getters:
            # same result without the two getters (each reads K back from the device): nothing synchronises,
            # the decode step stays capturable in a CUDA graph
            out = self.weight_cache.sparse_forward(x, self.down_proj_buffer, self.act_fn_name)
        else:
            out = sparse_mlp_forward(x, self.weight_cache.get_concat_weight(), self.weight_cache.get_active_down_weight(),
                                     self.down_proj_buffer, self.combined_proj_buffer, self.act_fn_name)
        return out.clone()  # the op returns an alias of the persistent buffer

    def _forward_dense(self, x: torch.Tensor) -> torch.Tensor:
        # prefill path (modeling_skip.py:127-128)
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))
