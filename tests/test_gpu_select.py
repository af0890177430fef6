"""Per-row selection rules (statistical_topk, topk) and approx_topk_threshold on the GPU
(C ABI) vs the oracle: bit-exact masks and thresholds."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu
ODT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _case(B, H, r, I, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, H, generator=g).to(dtype)
    A = (torch.randn(r, H, generator=g) * 0.02).to(dtype)
    Bm = (torch.randn(I, r, generator=g) * 0.02).to(dtype)
    return x, A, Bm


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,r,I", [(1, 512, 32, 8192), (4, 256, 16, 1000), (3, 128, 8, 14336), (2, 64, 8, 37)])
def test_statistical_and_topk_bit_exact(dtype, B, H, r, I):
    from sparse_transformers_b200 import _capi as C
    from stxgpu import DEV, predict_mask

    x, A, Bm = _case(B, H, r, I, dtype, seed=I + B)
    f = lambda t: t.float().numpy()
    _, s_ref = orc.predictor(f(x), f(A), f(Bm), ODT[dtype])
    z = 0.8416
    mask, scores, _ = predict_mask(x.to(DEV), A.to(DEV), Bm.to(DEV), method=C.MASK_STATISTICAL, param=z)
    assert np.array_equal(scores.float().cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    _, uni, _ = orc.mask_statistical(s_ref, ODT[dtype], z)
    assert np.array_equal(mask.cpu().numpy(), uni)
    for k in (1, max(1, I // 5), I):
        mask, _, _ = predict_mask(x.to(DEV), A.to(DEV), Bm.to(DEV), method=C.MASK_TOPK, param=float(k))
        rows, uni = orc.mask_topk(s_ref, k)
        assert np.array_equal(mask.cpu().numpy(), uni), k
        assert (rows.sum(axis=1) == k).all()   # exactly k per row, ties included


def test_rules_against_golden_reference_masks(golden):
    """The reference's own masks (torch on its own scores) for the three rules."""
    from sparse_transformers_b200 import _capi as C
    from stxgpu import DEV, predict_mask

    g = golden
    x, A, Bm = (torch.from_numpy(g[k]).to(DEV) for k in ("pred_x", "pred_A", "pred_Bm"))
    mask, scores, _ = predict_mask(x, A, Bm, method=C.MASK_TOPK, param=float(g["pred_topk_k"]))
    ref = g["pred_scores"]
    assert np.abs(scores.cpu().numpy() - ref).max() <= 2e-6 * np.abs(ref).max()
    # identical unless accumulation-order noise reorders two scores at the k-th place
    assert (mask.cpu().numpy() != g["pred_mask_topk"]).sum() <= 2
    mask, _, _ = predict_mask(x, A, Bm, method=C.MASK_STATISTICAL, param=float(g["pred_stat_z"]))
    assert (mask.cpu().numpy() != g["pred_mask_stat"]).sum() <= 2


@pytest.mark.parametrize("name", ["tk_a", "tk_b", "tk_c", "tk_d"])
def test_approx_topk_threshold_golden(golden, name):
    from sparse_transformers_b200 import _capi as C
    from stxgpu import DEV, stream

    s = torch.from_numpy(golden[f"{name}_scores"]).to(DEV)
    B, I = s.shape
    thr = torch.zeros(B, device=DEV)
    n = ctypes.c_size_t()
    C.check(C.lib.stx_approx_topk_scratch_bytes(B, I, ctypes.byref(n)))
    scratch = torch.zeros(n.value, dtype=torch.uint8, device=DEV)
    C.check(C.lib.stx_approx_topk_threshold(s.data_ptr(), B, I, int(golden[f"{name}_k"]), C.F32, thr.data_ptr(),
                                            scratch.data_ptr(), stream()))
    torch.cuda.synchronize()
    assert np.array_equal(thr.cpu().numpy(), golden[f"{name}_thr"])   # the compiled reference's output, bit for bit


def test_approx_topk_op_and_errors():
    import sparse_transformers_b200 as stb
    from stxgpu import DEV

    s = torch.randn(3, 4096, generator=torch.Generator().manual_seed(1))
    thr = stb.approx_topk_threshold(s.to(DEV), 400)
    assert thr.shape == (3, 1)
    assert np.array_equal(thr.cpu().numpy().reshape(-1), orc.approx_topk_threshold(s.numpy(), 400))
    with pytest.raises(RuntimeError, match="k must be positive"):
        stb.approx_topk_threshold(s.to(DEV), 0)
    with pytest.raises(RuntimeError, match="larger than feature size"):
        stb.approx_topk_threshold(s.to(DEV), 5000)


def test_layer_with_statistical_rule():
    """A fused layer step under the statistical rule: mask and cache order vs the oracle."""
    from sparse_transformers_b200 import SparseLayer
    from sparse_transformers_b200.synth import HiddenStream, Workload, layer_weights
    from stxgpu import DEV

    w = Workload("stat", H=256, I=1024, r=16, B=2, dtype=torch.float16, density=0.2, alpha=0.5)
    gen = torch.Generator().manual_seed(3)
    gate, up, down, A, Bm = layer_weights(w, gen)
    z = 0.8416
    layer = SparseLayer(gate.to(DEV), up.to(DEV), down.to(DEV), A.to(DEV), Bm.to(DEV), method="statistical_topk", param=z, max_batch=w.B)
    oc = orc.OracleCache(w.I)
    oc.update(np.ones(w.I, bool))
    xs = HiddenStream(w, gen)
    f = lambda t: t.float().numpy()
    for _ in range(5):
        x = xs.next()
        out = layer.step(x.to(DEV))
        torch.cuda.synchronize()
        _, s = orc.predictor(f(x), f(A), f(Bm), orc.F16)
        _, mask, _ = orc.mask_statistical(s, orc.F16, z)
        oc.update(mask)
        assert np.array_equal(layer.mask().cpu().numpy(), mask)
        assert layer.active_indices().tolist() == oc.active.tolist()
        wcat = np.concatenate([oc.gather(f(gate)), oc.gather(f(up))])
        ref, _ = orc.sparse_mlp(f(x), wcat, oc.gather(np.ascontiguousarray(f(down).T)), "silu", True)
        assert np.abs(f(out.cpu()) - ref).max() <= 2e-2 * np.abs(ref).max()
