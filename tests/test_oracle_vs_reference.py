"""The CPU oracle against the reference's own CPU operator, compiled unmodified and executed
here (differential testing; the reference has no tests of its own to borrow vectors from).
Skipped where the compiled reference is not available."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from oracle import oracle as orc


def _tagged(I, H, seed):
    g = torch.Generator().manual_seed(seed)
    gate, up, down = torch.randn(I, H, generator=g), torch.randn(I, H, generator=g), torch.randn(H, I, generator=g)
    up[:, 0] = torch.arange(I, dtype=torch.float32)
    return gate, up, down


def _ref_order(wc):
    c = wc.get_concat_weight()
    K = c.shape[0] // 2
    return c[K:, 0].round().long().tolist()


@settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(data=st.data())
def test_cache_order_property(refmod, data):
    I = data.draw(st.integers(2, 90))
    steps = data.draw(st.integers(1, 8))
    WC, _, _ = refmod.reference()
    gate, up, down = _tagged(I, 8, 7)
    wc = WC(torch.ones(I, dtype=torch.bool), 8, gate, up, down, True)
    c = orc.OracleCache(I)
    c.update(np.ones(I, bool))
    for _ in range(steps):
        bits = data.draw(st.lists(st.booleans(), min_size=I, max_size=I))
        m = torch.tensor(bits)
        if not m.any():
            with pytest.raises(RuntimeError, match="No active weights"):
                wc.update_active_weights(m)
            with pytest.raises(orc.NoActiveWeights):
                c.update(m.numpy())
            return  # the reference object is unusable after the throw
        wc.update_active_weights(m)
        k = c.update(m.numpy())
        assert _ref_order(wc) == c.active.tolist() and k == len(c.active)


def test_cache_order_config_shape(refmod):
    # Llama-3.2-1B-sized index space, AR(1)-like churn, 12 steps
    I = 8192
    WC, _, _ = refmod.reference()
    gate, up, down = _tagged(I, 8, 3)
    wc = WC(torch.ones(I, dtype=torch.bool), 8, gate, up, down, True)
    c = orc.OracleCache(I)
    c.update(np.ones(I, bool))
    g = torch.Generator().manual_seed(5)
    z = torch.randn(I, generator=g)
    for _ in range(12):
        z = 0.9 * z + 0.436 * torch.randn(I, generator=g)
        m = z > 0.84
        wc.update_active_weights(m)
        c.update(m.numpy())
        assert _ref_order(wc) == c.active.tolist()


@pytest.mark.parametrize("has_gate", [True, False])
def test_mlp_matches_reference_op(refmod, has_gate):
    _, fwd, _ = refmod.reference()
    g = torch.Generator().manual_seed(11)
    B, H, K = 5, 96, 70
    x = torch.randn(B, H, generator=g)
    cw = torch.randn(2 * K if has_gate else K, H, generator=g) * 0.2
    packed = torch.randn(K, H, generator=g) * 0.2
    dw = packed.t()  # [H,K] strides (1,H), as the reference cache returns it
    db, cb = torch.zeros(1, H), torch.zeros(1, 2)
    ref = fwd(x, cw, dw, db, cb, "relu", has_gate).clone()
    out, comb = orc.sparse_mlp(x.numpy(), cw.numpy(), packed.numpy(), "relu", has_gate)
    np.testing.assert_allclose(out, ref.numpy(), rtol=1e-5, atol=1e-5 * ref.abs().max().item())
    np.testing.assert_allclose(comb, cb.numpy(), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("act", ["relu", "silu", "gelu_pytorch_tanh"])
def test_mlp_matches_model_expression(refmod, act):
    g = torch.Generator().manual_seed(13)
    B, H, K = 3, 64, 40
    x = torch.randn(B, H, generator=g)
    cw = torch.randn(2 * K, H, generator=g) * 0.2
    packed = torch.randn(K, H, generator=g) * 0.2
    ref = refmod.skip_mlp_sparse(x, cw, packed.t(), act, True)
    out, _ = orc.sparse_mlp(x.numpy(), cw.numpy(), packed.numpy(), act, True)
    np.testing.assert_allclose(out, ref.numpy(), rtol=1e-5, atol=1e-5 * ref.abs().max().item())


@pytest.mark.parametrize("B,I,k", [(4, 256, 32), (2, 8192, 1638), (1, 14336, 2150), (3, 100, 1)])
def test_approx_topk_bit_exact(refmod, B, I, k):
    _, _, topk = refmod.reference()
    s = torch.randn(B, I, generator=torch.Generator().manual_seed(B * I + k))
    assert np.array_equal(orc.approx_topk_threshold(s.numpy(), k), topk(s, k).numpy().reshape(-1))


@pytest.mark.parametrize("dtype,tdt", [(orc.F32, torch.float32), (orc.F16, torch.float16), (orc.BF16, torch.bfloat16)])
def test_predictor_vs_torch_linear(refmod, dtype, tdt):
    """Scores of the fixed-order restatement vs torch's nn.Linear pair in the same dtype:
    equal up to accumulation-order noise; masks may differ only where a score sits within
    that noise of the cut, and such flips are counted."""
    g = torch.Generator().manual_seed(17)
    B, H, r, I = 2, 512, 64, 1024
    x = torch.randn(B, H, generator=g).to(tdt)
    A = (torch.randn(r, H, generator=g) * 0.02).to(tdt)
    Bm = (torch.randn(I, r, generator=g) * 0.02).to(tdt)
    ref = refmod.lora_scores(x, A, Bm).float()
    _, s = orc.predictor(x.float().numpy(), A.float().numpy(), Bm.float().numpy(), dtype)
    scale = ref.abs().max().item()
    tol = {orc.F32: 3e-6, orc.F16: 2e-3, orc.BF16: 2e-2}[dtype]
    assert np.abs(s - ref.numpy()).max() <= tol * scale
    tau = 0.5 * ref.std().item()
    _, uni = orc.mask_threshold(s, dtype, tau)
    ref_mask = refmod.compute_binary_mask(refmod.lora_scores(x, A, Bm), "threshold", tau=tau).numpy()
    flips = int((uni != ref_mask).sum())
    near = int((np.abs(ref.numpy() - tau) <= tol * scale).any(axis=0).sum())
    assert flips <= near


def test_threshold_compare_rounds_tau_to_dtype():
    # comparing a half tensor with a Python float compares in half precision
    s = torch.tensor([[0.1499, 0.14990234375, 0.1501]], dtype=torch.float16)
    tau = 0.1493
    _, uni = orc.mask_threshold(s.float().numpy(), orc.F16, tau)
    assert np.array_equal(uni, (s >= tau).any(dim=0).numpy())
    edge = torch.tensor([[tau]], dtype=torch.float16)  # exactly the rounded threshold
    _, uni = orc.mask_threshold(edge.float().numpy(), orc.F16, tau)
    assert bool(uni[0]) == bool((edge >= tau).item())


@pytest.mark.parametrize("tdt,dtype", [(torch.float32, orc.F32), (torch.float16, orc.F16)])
def test_statistical_rule_vs_torch(refmod, tdt, dtype):
    g = torch.Generator().manual_seed(19)
    s = (torch.randn(3, 4096, generator=g) * 0.15).to(tdt)
    ref = refmod.compute_binary_mask(s, "statistical_topk", sparsity=0.8).numpy()
    z = torch.distributions.normal.Normal(0, 1).icdf(torch.tensor(0.8)).item()
    _, uni, cut = orc.mask_statistical(s.float().numpy(), dtype, z)
    # identical unless a score ties with the cutoff's last bit
    assert (uni != ref).sum() <= 2
