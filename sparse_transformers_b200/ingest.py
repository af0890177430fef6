"""On-disk formats either side of the sparse-MLP path.

  predictor   `final_predictor_layer_{i}_lora_{pct:.1f}pct.pt`: the state dict of a
              FastLoRAProjection, keys `down.weight` [r,H] and `up.weight` [I,r], as the reference
              trainer writes it (src/trainer.py:570-587) and its benchmark loads it
              (benchmark.py:460-468; there the size is formatted by the caller).
  MLP weights Hugging Face state-dict names per architecture: `gate_proj/up_proj/down_proj`
              (Llama, Mistral, Qwen2, Gemma), Phi-3's fused `gate_up_proj` whose halves are gate
              and up (src/models/phi3/modelling_phi_skip.py:36-41), OPT's `fc1/fc2` without a gate
              (src/models/opt/modelling_opt_skip.py:87-94).

Everything here is host-side plumbing (tensor views and file names); building the device-side
layer (pools, transposed down, cache) is SparseLayer's job.
"""
from __future__ import annotations

import os
from typing import Mapping

import torch

# architecture -> (prefix template, gate, up, down); gate None: no gate; fused: one tensor holds gate then up
MLP_LAYOUTS = {
    "llama": ("model.layers.{i}.mlp.", "gate_proj.weight", "up_proj.weight", "down_proj.weight"),
    "mistral": ("model.layers.{i}.mlp.", "gate_proj.weight", "up_proj.weight", "down_proj.weight"),
    "qwen2": ("model.layers.{i}.mlp.", "gate_proj.weight", "up_proj.weight", "down_proj.weight"),
    "gemma": ("model.layers.{i}.mlp.", "gate_proj.weight", "up_proj.weight", "down_proj.weight"),
    "phi3": ("model.layers.{i}.mlp.", "gate_up_proj.weight", None, "down_proj.weight"),
    "opt": ("model.decoder.layers.{i}.", None, "fc1.weight", "fc2.weight"),
}


def predictor_filename(layer_idx: int, lora_pct: float) -> str:
    """File name the reference trainer gives a layer's final predictor."""
    return f"final_predictor_layer_{layer_idx}_lora_{lora_pct:.1f}pct.pt"


def predictor_rank(intermediate: int, lora_pct: float) -> int:
    """r = int(I * pct / 100) (src/modeling_skip.py:157-158 with pct in percent)."""
    return int(intermediate * lora_pct / 100.0)


def load_predictor(src: str | os.PathLike | Mapping[str, torch.Tensor], hidden: int | None = None,
                   intermediate: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """-> (A = down.weight [r,H], Bm = up.weight [I,r]).  `src`: a .pt path or a loaded state dict.
    Raises KeyError / ValueError on anything that is not a FastLoRAProjection state dict."""
    sd = torch.load(os.fspath(src), map_location="cpu", weights_only=True) if not isinstance(src, Mapping) else src
    missing = [k for k in ("down.weight", "up.weight") if k not in sd]
    if missing:
        raise KeyError(f"not a predictor state dict: missing {missing}; has {sorted(sd)[:6]}")
    extra = [k for k in sd if k not in ("down.weight", "up.weight")]
    if extra:
        raise ValueError(f"unexpected keys in predictor state dict: {extra[:6]}")
    A, Bm = sd["down.weight"], sd["up.weight"]
    if A.dim() != 2 or Bm.dim() != 2 or A.shape[0] != Bm.shape[1]:
        raise ValueError(f"predictor shapes do not chain: down {tuple(A.shape)}, up {tuple(Bm.shape)}")
    if hidden is not None and A.shape[1] != hidden:
        raise ValueError(f"predictor was trained for hidden size {A.shape[1]}, model has {hidden}")
    if intermediate is not None and Bm.shape[0] != intermediate:
        raise ValueError(f"predictor was trained for intermediate size {Bm.shape[0]}, model has {intermediate}")
    return A, Bm


def load_predictor_dir(sp_dir: str | os.PathLike, layers: range | list[int], lora_pct: float, **kw):
    """{layer: (A, Bm)} for the given layers; FileNotFoundError names the first missing file
    (the reference aborts the run in that case, benchmark.py:463-465)."""
    out = {}
    for i in layers:
        path = os.path.join(os.fspath(sp_dir), predictor_filename(i, lora_pct))
        if not os.path.exists(path):
            raise FileNotFoundError(f"pretrained predictor for layer {i} does not exist: {path}")
        out[i] = load_predictor(path, **kw)
    return out


def save_predictor(path: str | os.PathLike, A: torch.Tensor, Bm: torch.Tensor) -> None:
    """Writes the same two-key state dict the reference trainer writes."""
    torch.save({"down.weight": A.detach().cpu().contiguous(), "up.weight": Bm.detach().cpu().contiguous()}, os.fspath(path))


def mlp_weights(sd: Mapping[str, torch.Tensor], layer_idx: int, arch: str = "llama"):
    """-> (gate [I,H] or None, up [I,H], down [H,I]) views into the state dict `sd`.
    Phi-3: the fused [2I,H] tensor's first half is gate, second half up (torch.chunk(2, dim=0))."""
    if arch not in MLP_LAYOUTS:
        raise ValueError(f"unknown architecture '{arch}' (known: {sorted(MLP_LAYOUTS)})")
    prefix, g, u, d = MLP_LAYOUTS[arch]
    prefix = prefix.format(i=layer_idx)

    def get(name):
        key = prefix + name
        if key not in sd:
            raise KeyError(f"state dict has no '{key}'")
        return sd[key]

    down = get(d)
    if arch == "phi3":
        fused = get(g)
        if fused.shape[0] % 2:
            raise ValueError(f"fused gate_up_proj has an odd number of rows: {tuple(fused.shape)}")
        gate, up = fused.chunk(2, dim=0)
    else:
        gate = get(g) if g is not None else None
        up = get(u)
    I, H = up.shape
    if tuple(down.shape) != (H, I) or (gate is not None and tuple(gate.shape) != (I, H)):
        raise ValueError(f"layer {layer_idx}: MLP shapes do not agree: up {tuple(up.shape)}, down {tuple(down.shape)}, "
                         f"gate {None if gate is None else tuple(gate.shape)}")
    return gate, up, down


def sparse_layer_from_state(sd: Mapping[str, torch.Tensor], layer_idx: int, predictor, *, arch: str = "llama",
                            device="cuda", dtype: torch.dtype | None = None, **layer_kw):
    """SparseLayer for one decoder layer: MLP weights from a model state dict, predictor from
    load_predictor (or a path).  OPT-style layers get has_gate=False and need act='relu'."""
    from .layer import SparseLayer

    gate, up, down = mlp_weights(sd, layer_idx, arch)
    A, Bm = predictor if isinstance(predictor, tuple) else load_predictor(predictor, hidden=up.shape[1], intermediate=up.shape[0])
    dt = dtype or up.dtype
    mv = lambda t: None if t is None else t.to(device=device, dtype=dt).contiguous()
    return SparseLayer(mv(gate), mv(up), mv(down), mv(A), mv(Bm), has_gate=gate is not None, **layer_kw)
