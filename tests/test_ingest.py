"""Predictor / MLP-weight ingestion (host-side formats): file names and state-dict layouts the
reference writes and reads (src/trainer.py:570-587, benchmark.py:460-468,
src/models/phi3/modelling_phi_skip.py:36-41, src/models/opt/modelling_opt_skip.py:87-94)."""
import os

import pytest
import torch

from sparse_transformers_b200 import ingest


def test_predictor_file_name_and_rank():
    assert ingest.predictor_filename(3, 4.0) == "final_predictor_layer_3_lora_4.0pct.pt"
    assert ingest.predictor_filename(27, 12.5) == "final_predictor_layer_27_lora_12.5pct.pt"
    assert ingest.predictor_rank(8192, 4.0) == 327  # int(I * 0.04), src/modeling_skip.py:157-158


def test_predictor_round_trip_and_reference_module_state_dict(tmp_path):
    H, I, r = 48, 160, 6
    # the reference's FastLoRAProjection is two bias-free nn.Linear called down and up (src/modeling_skip.py:39-40)
    m = torch.nn.ModuleDict({"down": torch.nn.Linear(H, r, bias=False), "up": torch.nn.Linear(r, I, bias=False)})
    p = tmp_path / ingest.predictor_filename(0, 4.0)
    torch.save(m.state_dict(), p)
    A, Bm = ingest.load_predictor(p, hidden=H, intermediate=I)
    assert torch.equal(A, m["down"].weight.detach()) and torch.equal(Bm, m["up"].weight.detach())
    x = torch.randn(3, H)
    assert torch.allclose((x @ A.t()) @ Bm.t(), m["up"](m["down"](x)), atol=1e-6)
    q = tmp_path / "again.pt"
    ingest.save_predictor(q, A, Bm)
    m2 = torch.nn.ModuleDict({"down": torch.nn.Linear(H, r, bias=False), "up": torch.nn.Linear(r, I, bias=False)})
    m2.load_state_dict(torch.load(q, weights_only=True))  # what benchmark.py:467-468 does
    assert torch.equal(m2["up"].weight, Bm)


def test_predictor_errors(tmp_path):
    with pytest.raises(KeyError):
        ingest.load_predictor({"down.weight": torch.zeros(2, 4)})
    with pytest.raises(ValueError):
        ingest.load_predictor({"down.weight": torch.zeros(2, 4), "up.weight": torch.zeros(8, 3)})
    with pytest.raises(ValueError):
        ingest.load_predictor({"down.weight": torch.zeros(2, 4), "up.weight": torch.zeros(8, 2)}, hidden=5)
    with pytest.raises(ValueError):
        ingest.load_predictor({"down.weight": torch.zeros(2, 4), "up.weight": torch.zeros(8, 2), "bias": torch.zeros(1)})
    ingest.save_predictor(tmp_path / ingest.predictor_filename(0, 4.0), torch.zeros(2, 4), torch.zeros(8, 2))
    with pytest.raises(FileNotFoundError) as e:
        ingest.load_predictor_dir(tmp_path, range(2), 4.0)
    assert "layer 1" in str(e.value)
    assert set(ingest.load_predictor_dir(tmp_path, [0], 4.0)) == {0}


def test_mlp_weight_layouts():
    H, I = 8, 24
    g, u, d = torch.randn(I, H), torch.randn(I, H), torch.randn(H, I)
    for arch in ("llama", "mistral", "qwen2", "gemma"):
        sd = {"model.layers.2.mlp.gate_proj.weight": g, "model.layers.2.mlp.up_proj.weight": u, "model.layers.2.mlp.down_proj.weight": d}
        gg, uu, dd = ingest.mlp_weights(sd, 2, arch)
        assert gg is g and uu is u and dd is d
    fused = torch.cat([g, u], 0)
    gg, uu, dd = ingest.mlp_weights({"model.layers.0.mlp.gate_up_proj.weight": fused, "model.layers.0.mlp.down_proj.weight": d}, 0, "phi3")
    assert torch.equal(gg, g) and torch.equal(uu, u) and dd is d
    gg, uu, dd = ingest.mlp_weights({"model.decoder.layers.1.fc1.weight": u, "model.decoder.layers.1.fc2.weight": d}, 1, "opt")
    assert gg is None and uu is u and dd is d
    with pytest.raises(KeyError):
        ingest.mlp_weights({}, 0, "llama")
    with pytest.raises(ValueError):
        ingest.mlp_weights({"model.decoder.layers.1.fc1.weight": u, "model.decoder.layers.1.fc2.weight": d.t()}, 1, "opt")
    with pytest.raises(ValueError):
        ingest.mlp_weights({}, 0, "nope")
