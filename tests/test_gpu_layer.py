"""Fused layer step / graph stack on the GPU vs the oracle pipeline on the same seeded inputs:
masks and cache indices bit-exact, outputs within tolerance (1e-5 fp32, 2e-2 fp16/bf16,
as max|a-b|/max|b|)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.float16: 2e-2, torch.bfloat16: 2e-2}
ODT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


class OracleLayer:
    def __init__(self, w, gate, up, down, A, Bm):
        f = lambda t: t.float().numpy()
        self.w = w
        self.gate, self.up, self.downT = f(gate), f(up), np.ascontiguousarray(f(down).T)
        self.A, self.Bm = f(A), f(Bm)
        self.cache = orc.OracleCache(w.I)
        self.cache.update(np.ones(w.I, bool))

    def step(self, x):
        w = self.w
        _, s = orc.predictor(x.float().numpy(), self.A, self.Bm, ODT[w.dtype])
        _, mask = orc.mask_threshold(s, ODT[w.dtype], w.tau)
        self.cache.update(mask)
        wcat = np.concatenate([self.cache.gather(self.gate), self.cache.gather(self.up)]) if w.has_gate else self.cache.gather(self.up)
        out, _ = orc.sparse_mlp(x.float().numpy(), wcat, self.cache.gather(self.downT), w.act, w.has_gate)
        return mask, out


def _run(w, steps, seed=0):
    from sparse_transformers_b200 import SparseLayer
    from sparse_transformers_b200.synth import HiddenStream, layer_weights
    from stxgpu import DEV, rel_err

    gen = torch.Generator().manual_seed(seed)
    gate, up, down, A, Bm = layer_weights(w, gen)
    xs = HiddenStream(w, gen)
    layer = SparseLayer(gate.to(DEV), up.to(DEV), down.to(DEV), A.to(DEV), Bm.to(DEV), act=w.act, method="threshold",
                        param=w.tau, max_batch=w.B, has_gate=w.has_gate)
    ol = OracleLayer(w, gate, up, down, A, Bm)
    ks, worst = [], 0.0
    for t in range(steps):
        x = xs.next()
        out = layer.step(x.to(DEV))
        torch.cuda.synchronize()
        mask, ref = ol.step(x)
        assert np.array_equal(layer.mask().cpu().numpy(), mask), f"mask differs at step {t}"
        assert layer.active_indices().tolist() == ol.cache.active.tolist(), f"cache order differs at step {t}"
        worst = max(worst, rel_err(out.float().cpu().numpy(), ref))
        ks.append(layer.num_active())
    assert worst <= TOL[w.dtype], worst
    layer.close()
    return ks


def test_c1_llama1b_layer_fp32():
    """Llama-3.2-1B-shaped layer, fp32, batch 1, AR(1) hidden states (the reference's own
    CPU-runnable configuration), 24 steps."""
    from sparse_transformers_b200.synth import WORKLOADS

    ks = _run(WORKLOADS["C1"], steps=24)
    assert 0.15 * 8192 < np.mean(ks[2:]) < 0.25 * 8192


@pytest.mark.parametrize("name,scale", [("C2", dict(I=4096)), ("C3", dict(I=2048, H=1024))])
def test_half_precision_shapes(name, scale):
    from sparse_transformers_b200.synth import WORKLOADS

    _run(WORKLOADS[name].scaled(layers=1, **scale), steps=8)


@pytest.mark.parametrize("dtype,has_gate,density", [(torch.float32, True, 0.9), (torch.float16, True, 0.97),
                                                    (torch.bfloat16, False, 0.9), (torch.float16, True, 0.4)])
def test_one_row_with_more_neurons_per_cta_than_row_spaces(dtype, has_gate, density):
    """Dense masks at one row: a CTA of the one-kernel path owns 20 to 55 neurons, more than the
    36 (fp32: 27) rows its shared memory holds, so row spaces are re-used within the launch, over
    one block of neurons and over several."""
    from sparse_transformers_b200.synth import Workload

    w = Workload("dense-b1", H=2048, I=8192, r=64, B=1, dtype=dtype, density=density, has_gate=has_gate,
                 act="silu" if has_gate else "relu")
    ks = _run(w, steps=4)
    assert np.mean(ks) > 0.3 * 8192


def test_no_gate_relu_ragged():
    from sparse_transformers_b200.synth import Workload

    w = Workload("ragged", H=72, I=333, r=20, B=3, dtype=torch.float32, density=0.3, act="relu", has_gate=False, alpha=0.5)
    _run(w, steps=10)


def test_stack_graph_matches_eager_layers():
    """The CUDA-graph replay of L layers equals stepping the layers one by one."""
    from sparse_transformers_b200 import SparseLayer, SparseStack
    from sparse_transformers_b200.synth import HiddenStream, WORKLOADS, layer_weights
    from stxgpu import DEV

    w = WORKLOADS["C2"].scaled(I=2048, H=512, layers=3)
    gen = torch.Generator().manual_seed(1)
    ws = [layer_weights(w, gen) for _ in range(w.layers)]
    mk = lambda: [SparseLayer(*[t.to(DEV) for t in lw], act=w.act, param=w.tau, max_batch=w.B) for lw in ws]
    eager, graphed = mk(), mk()
    stack = SparseStack(graphed, w.B)
    assert stack.launches_per_step >= 2  # persistent kernel (+ plan and row copies per layer where it does not run them itself) + status collector
    xs = HiddenStream(w, gen)
    out = torch.empty(w.layers, w.B, w.H, dtype=w.dtype, device=DEV)
    xh = torch.empty(w.B, w.H, dtype=w.dtype).pin_memory()
    oh = torch.empty(w.layers, w.B, w.H, dtype=w.dtype).pin_memory()
    for t in range(6):
        x = xs.next()
        if t % 2 == 0:
            stack.step(x.to(DEV), out)
            torch.cuda.synchronize()
            got = out.cpu()
        else:
            xh.copy_(x)
            stack.step_host(xh, oh)
            got = oh.clone()
        for l in range(w.layers):
            ref = eager[l].step(x.to(DEV))
            torch.cuda.synchronize()
            assert eager[l].active_indices().tolist() == graphed[l].active_indices().tolist()
            assert torch.allclose(got[l].float(), ref.float().cpu(), rtol=2e-2, atol=2e-3)
    stack.close()


def test_step_host_equals_device_step():
    from sparse_transformers_b200 import SparseLayer
    from sparse_transformers_b200.synth import WORKLOADS, layer_weights
    from stxgpu import DEV

    w = WORKLOADS["C1"].scaled(I=1024, H=256)
    gen = torch.Generator().manual_seed(2)
    lw = layer_weights(w, gen)
    a = SparseLayer(*[t.to(DEV) for t in lw], param=w.tau)
    b = SparseLayer(*[t.to(DEV) for t in lw], param=w.tau)
    x = torch.randn(1, w.H, generator=gen)
    oh = torch.empty(1, w.H)
    b.step_host(x, oh)
    od = a.step(x.to(DEV)).cpu()
    assert torch.allclose(od, oh, rtol=1e-5, atol=1e-6)
    assert a.active_indices().tolist() == b.active_indices().tolist()


@pytest.mark.parametrize("lazy", [False, True])
def test_packed_cache_current_after_fused_steps(lazy):
    """The fused step's MLP gathers from the full pools; the packed cache must still be what
    WeightCache would hold — immediately (eager) or when it is read (lazy row copies)."""
    from sparse_transformers_b200 import SparseLayer
    from sparse_transformers_b200.synth import HiddenStream, WORKLOADS, layer_weights
    from stxgpu import DEV

    w = WORKLOADS["C2"].scaled(I=2048, H=512, layers=1)
    gen = torch.Generator().manual_seed(5)
    gate, up, down, A, Bm = layer_weights(w, gen)
    layer = SparseLayer(gate.to(DEV), up.to(DEV), down.to(DEV), A.to(DEV), Bm.to(DEV), param=w.tau, lazy_cache=lazy)
    eager = SparseLayer(gate.to(DEV), up.to(DEV), down.to(DEV), A.to(DEV), Bm.to(DEV), param=w.tau)
    oc = orc.OracleCache(w.I)
    oc.update(np.ones(w.I, bool))
    xs = HiddenStream(w, gen)
    for t in range(7):
        x = xs.next().to(DEV)
        out = layer.step(x)
        ref = eager.step(x)
        assert torch.equal(out, ref)  # same kernels, same order: identical bits
        oc.update(layer.mask().cpu().numpy())
        if t in (2, 6):  # read the cache after a few steps in a row
            idx = torch.from_numpy(oc.active.astype(np.int64))
            assert layer.active_indices().tolist() == oc.active.tolist()
            cw = layer.concat_weight().cpu()
            K = len(idx)
            assert torch.equal(cw[:K], gate[idx]) and torch.equal(cw[K:], up[idx])
            assert torch.equal(layer.active_down_weight().cpu(), down[:, idx])


@pytest.mark.parametrize("rows", [9, 24, 40])
def test_row_blocks_from_nine_rows_up_take_the_tensor_core_path(rows):
    """Any row count above the 8 of the streaming kernels runs as GEMMs over the packed cache (rows beyond the
    batch are out-of-bounds zeros of the TMA box)."""
    from sparse_transformers_b200.synth import Workload

    w = Workload("b%d" % rows, H=1024, I=2048, r=32, B=rows, dtype=torch.bfloat16, density=0.08, alpha=0.7)
    _run(w, steps=5, seed=rows)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_row_block_of_64_runs_on_the_packed_cache(dtype):
    """64 rows: the layer step brings the packed cache up to date first and runs the two tensor-core
    GEMMs over it, following the device-side K (the union of 64 masks leaves a changing K)."""
    from sparse_transformers_b200.synth import Workload

    w = Workload("b64", H=1024, I=2048, r=32, B=64, dtype=dtype, density=0.05, alpha=0.8)
    ks = _run(w, steps=6, seed=3)
    assert 64 < min(ks) and max(ks) < 2048 and len(set(ks)) > 1


@pytest.mark.parametrize("B,dtype,act,H,I", [(2, torch.float16, "silu", 512, 1024), (3, torch.bfloat16, "relu", 1024, 2048),
                                             (5, torch.float16, "gelu_pytorch_tanh", 512, 4096), (7, torch.bfloat16, "silu", 1536, 1000)])
def test_two_to_eight_rows_one_kernel_path(B, dtype, act, H, I):
    """Ragged row counts and every activation through the 2..8-row kernel (k_mlp_bn); I = 1000 leaves a
    partial mask byte and CTAs without neurons, density 0.3 with shared streams makes some CTAs hand
    neurons to others."""
    from sparse_transformers_b200 import SparseLayer
    from sparse_transformers_b200.synth import Workload, layer_weights

    w = Workload("bn", H=H, I=I, r=32, B=B, dtype=dtype, density=0.3, alpha=0.6, act=act)
    g = torch.Generator().manual_seed(1)
    probe = SparseLayer(*[t.to("cuda:0") for t in layer_weights(w, g)], act=act, param=w.tau, max_batch=B)
    assert probe.single_row_fused(B)
    probe.close()
    _run(w, steps=6, seed=11)
