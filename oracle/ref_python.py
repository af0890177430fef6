"""Torch (CPU) restatement of the Python half of the reference path, and a driver that feeds
it to the reference's own compiled WeightCache / op.  TEST INFRASTRUCTURE ONLY.

The reference's src/ package does not import against the installed transformers release, so
the ~25 hot lines are restated here, each citing src/modeling_skip.py.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)
import build_ref  # noqa: E402

ACT2FN = {
    "relu": torch.relu,
    "silu": F.silu,
    "gelu_pytorch_tanh": lambda t: F.gelu(t, approximate="tanh"),
    "gelu": F.gelu,
    "sigmoid": torch.sigmoid,
}


def lora_scores(x: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor) -> torch.Tensor:
    """FastLoRAProjection.forward: up(down(x)), bias-free (modeling_skip.py:39-40,52-53)."""
    return F.linear(F.linear(x, A), Bm)


def gaussian_topk(scores: torch.Tensor, sparsity: float) -> torch.Tensor:
    """_gaussian_topk (modeling_skip.py:197-202) with std_multiplier = icdf(sparsity) (:141-142)."""
    std_multiplier = torch.distributions.normal.Normal(0, 1).icdf(torch.tensor(sparsity)).type(scores.dtype)
    mean = torch.mean(scores, dim=-1, keepdim=True)
    std = torch.std(scores, dim=-1, keepdim=True, unbiased=False)
    return (scores > mean + std * std_multiplier).bool()


def compute_binary_mask(scores: torch.Tensor, method: str, *, tau: float = 0.0, k: int | None = None,
                        sparsity: float | None = None) -> torch.Tensor:
    """_compute_binary_mask (modeling_skip.py:204-214) on precomputed scores [B,I] -> bool [I].
    "naive" with tau = 0 is the reference rule; tau != 0 is the benchmark's generalisation."""
    if method in ("naive", "threshold"):
        m = (scores >= tau).bool()
    elif method == "topk":
        idx = scores.topk(k, sorted=False)[1]
        m = torch.zeros_like(scores, dtype=torch.bool)
        m.scatter_(-1, idx, True)
    elif method == "statistical_topk":
        m = gaussian_topk(scores, sparsity)
    else:
        raise ValueError(method)
    return m.any(dim=0)


def skip_mlp_sparse(x, concat_w, down_w, act: str, has_gate: bool = True):
    """SkipMLP._forward_sparse_weight_cache (modeling_skip.py:114-117); OPT's no-gate form
    (src/models/opt/modelling_opt_skip.py:116-119) when has_gate is False."""
    if has_gate:
        gate, up = x.matmul(concat_w.t()).chunk(2, dim=-1)
        return (ACT2FN[act](gate) * up).matmul(down_w.t())
    return ACT2FN[act](x.matmul(concat_w.t())).matmul(down_w.t())


_REF = None


def reference():
    """(WeightCache class, forward op, approx_topk op) of the compiled, unmodified reference."""
    global _REF
    if _REF is None:
        if not os.path.isfile(build_ref.ref_so_path()):
            build_ref.build(verbose=False)
        _REF = build_ref.load()
    return _REF


def have_reference() -> bool:
    try:
        reference()
        return True
    except Exception:
        return False


def ref_active_indices(wc, K_hint: int | None = None) -> list[int]:
    """Order of the reference cache, read through its public getters: requires the cache to
    have been built from weights with up[n,0] == n (weight tagging)."""
    c = wc.get_concat_weight()
    K = c.shape[0] // 2 if K_hint is None else K_hint
    return c[c.shape[0] - K:, 0].round().long().tolist()


class RefLayer:
    """One sparse layer on the reference's CPU implementation (fp32 only, like the reference
    cache: weight_cache.h:29-31): restated predictor/mask + compiled WeightCache + op."""

    def __init__(self, gate, up, down, A, Bm, *, act="silu", method="threshold", tau=0.0, k=None, sparsity=None,
                 has_gate=True):
        WC, self.fwd, _ = reference()
        f = lambda t: t.detach().float().cpu().contiguous()
        self.gate, self.up, self.down, self.A, self.Bm = map(f, (gate, up, down, A, Bm))
        self.I, self.H = self.up.shape
        self.act, self.method, self.tau, self.k, self.sparsity, self.has_gate = act, method, tau, k, sparsity, has_gate
        self.wc = WC(torch.ones(self.I, dtype=torch.bool), self.H,
                     self.gate if has_gate else torch.empty(0), self.up, self.down, has_gate)
        self.down_buf = torch.zeros(1, self.H)
        self.comb_buf = torch.zeros(1, 2)

    def mask(self, x: torch.Tensor) -> torch.Tensor:
        s = lora_scores(x.float().cpu().view(-1, self.H), self.A, self.Bm)
        return compute_binary_mask(s, self.method, tau=self.tau, k=self.k, sparsity=self.sparsity)

    def step(self, x_pred, x_mlp=None, op: bool = False):
        """mask -> update_active_weights -> MLP.  op=True runs the compiled op (ReLU whatever
        ``act`` says); op=False runs the expression the models run, honouring ``act``."""
        x_mlp = x_pred if x_mlp is None else x_mlp
        m = self.mask(x_pred)
        self.wc.update_active_weights(m)
        xm = x_mlp.float().cpu().view(-1, self.H)
        cw, dw = self.wc.get_concat_weight(), self.wc.get_active_down_weight()
        if op:
            out = self.fwd(xm, cw, dw, self.down_buf, self.comb_buf, self.act, self.has_gate).clone()
        else:
            out = skip_mlp_sparse(xm, cw, dw, self.act, self.has_gate)
        return m, out
