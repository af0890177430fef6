"""A SparseLayer built from on-disk formats (Phi-3 fused gate_up_proj, OPT fc1/fc2 without a gate,
predictor .pt file) steps exactly like one built from the tensors directly."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("arch", ["phi3", "opt", "llama"])
def test_layer_from_state_dict(tmp_path, arch):
    from sparse_transformers_b200 import SparseLayer, ingest
    from sparse_transformers_b200.synth import HiddenStream, Workload, layer_weights

    has_gate = arch != "opt"
    w = Workload("ing", H=512, I=1024, r=32, B=2, dtype=torch.float16, density=0.3, alpha=0.5,
                 act="silu" if has_gate else "relu", has_gate=has_gate)
    gen = torch.Generator().manual_seed(0)
    gate, up, down, A, Bm = layer_weights(w, gen)
    if arch == "phi3":
        sd = {"model.layers.4.mlp.gate_up_proj.weight": torch.cat([gate, up], 0), "model.layers.4.mlp.down_proj.weight": down}
    elif arch == "opt":
        sd = {"model.decoder.layers.4.fc1.weight": up, "model.decoder.layers.4.fc2.weight": down}
    else:
        sd = {f"model.layers.4.mlp.{n}_proj.weight": t for n, t in (("gate", gate), ("up", up), ("down", down))}
    path = tmp_path / ingest.predictor_filename(4, 3.1)
    ingest.save_predictor(path, A, Bm)
    a = ingest.sparse_layer_from_state(sd, 4, path, arch=arch, device="cuda:0", act=w.act, param=w.tau, max_batch=w.B)
    dev = lambda t: t.to("cuda:0")
    b = SparseLayer(dev(gate) if has_gate else None, dev(up), dev(down), dev(A), dev(Bm), act=w.act, param=w.tau, max_batch=w.B,
                    has_gate=has_gate)
    xs = HiddenStream(w, gen)
    for _ in range(4):
        x = dev(xs.next())
        oa, ob = a.step(x), b.step(x)
        torch.cuda.synchronize()
        assert torch.equal(oa, ob)
        assert torch.equal(a.mask(), b.mask())
        assert a.active_indices().tolist() == b.active_indices().tolist()
    a.close()
    b.close()
