"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations (they stand in for real checkpoints and prompts, which are not available
offline).

Weights ~ N(0, 0.02); hidden states follow the AR(1) process x_t = 0.9 x_{t-1} + 0.436 n_t
(stationary unit variance), so consecutive masks overlap and the differential cache is
exercised.  For B > 1 the streams share a fraction ``alpha`` of their variance
(x = sqrt(1-alpha) x_private + sqrt(alpha) x_shared) so that the union of the per-row masks
lands in the intended density range.  The threshold that yields a per-row density d is
tau = 0.02^2 sqrt(H r) Phi^-1(1 - d) (scores are ~N(0, 0.02^4 H r) for unit-variance x).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from statistics import NormalDist

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    H: int
    I: int
    r: int
    B: int
    dtype: torch.dtype
    density: float
    layers: int = 1
    steps: int = 128
    alpha: float = 0.0
    act: str = "silu"
    has_gate: bool = True
    rho: float = 0.9
    sigma: float = 0.436
    wstd: float = 0.02

    @property
    def tau(self) -> float:
        return self.wstd ** 2 * math.sqrt(self.H * self.r) * NormalDist().inv_cdf(1.0 - self.density)

    def scaled(self, **kw) -> "Workload":
        return replace(self, **kw)


WORKLOADS = {
    # Llama-3.2-1B-shaped single layer, fp32 (runnable on the reference CPU op as is)
    "C1": Workload("C1-llama1b-layer-fp32", H=2048, I=8192, r=64, B=1, dtype=torch.float32, density=0.20, layers=1, steps=128),
    # Llama-3.2-3B-shaped 28-layer sparse-MLP stack, fp16, batch 1
    "C2": Workload("C2-llama3b-mlp-stack-fp16", H=3072, I=8192, r=64, B=1, dtype=torch.float16, density=0.20, layers=28, steps=128),
    # Mistral-7B-shaped 32-layer stack, bf16, 8 streams, union of masks ~40-60 %
    "C3": Workload("C3-mistral7b-mlp-stack-bf16-b8", H=4096, I=14336, r=128, B=8, dtype=torch.bfloat16, density=0.15, layers=32, steps=256, alpha=0.7),
    # ReluLLaMA-7B-shaped sparse MLP on the prefill path: 4 x 2048 rows, ReLU gated, fp16
    "C4": Workload("C4-relullama7b-prefill-fp16", H=4096, I=11008, r=128, B=8192, dtype=torch.float16, density=0.10, layers=1, steps=16, act="relu"),
    # same shapes, 64 streams, intermediate dimension sharded over the GPUs
    "C5": Workload("C5-mistral7b-mlp-stack-bf16-b64-sharded", H=4096, I=14336, r=128, B=64, dtype=torch.bfloat16, density=0.15, layers=32, steps=512, alpha=0.7),
}


def layer_weights(w: Workload, gen: torch.Generator, device: str | torch.device = "cpu"):
    """gate [I,H], up [I,H], down [H,I], A [r,H], Bm [I,r] in fp32 drawn in this order from
    ``gen`` (whose device must match ``device``), then cast to the workload dtype."""
    def rn(*shape):
        return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * w.wstd).to(w.dtype)

    gate, up, down = rn(w.I, w.H), rn(w.I, w.H), rn(w.H, w.I)
    A, Bm = rn(w.r, w.H), rn(w.I, w.r)
    return gate, up, down, A, Bm


class HiddenStream:
    """AR(1) hidden states [B,H], generated in fp32 on the CPU and cast to the workload dtype."""

    def __init__(self, w: Workload, gen: torch.Generator):
        self.w, self.gen = w, gen
        self.priv = torch.randn(w.B, w.H, generator=gen)
        self.shared = torch.randn(1, w.H, generator=gen) if w.alpha > 0 else None

    def _mix(self) -> torch.Tensor:
        if self.shared is None:
            return self.priv
        a = self.w.alpha
        return math.sqrt(1.0 - a) * self.priv + math.sqrt(a) * self.shared

    def next(self) -> torch.Tensor:
        w = self.w
        x = self._mix().to(w.dtype)
        self.priv = w.rho * self.priv + w.sigma * torch.randn(w.B, w.H, generator=self.gen)
        if self.shared is not None:
            self.shared = w.rho * self.shared + w.sigma * torch.randn(1, w.H, generator=self.gen)
        return x

    def take(self, n: int) -> torch.Tensor:
        return torch.stack([self.next() for _ in range(n)])  # [n,B,H]
