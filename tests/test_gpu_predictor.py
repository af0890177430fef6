"""Predictor -> threshold -> bit mask -> batch union on the GPU (C ABI) vs the oracle:
scores and masks must be BIT-EXACT (same fixed summation order, same rounding points)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _case(B, H, r, I, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, H, generator=g).to(dtype)
    A = (torch.randn(r, H, generator=g) * 0.02).to(dtype)
    Bm = (torch.randn(I, r, generator=g) * 0.02).to(dtype)
    return x, A, Bm


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,r,I", [(1, 2048, 64, 8192), (1, 3072, 64, 8192), (8, 4096, 128, 14336), (3, 256, 24, 1000),
                                     (2, 64, 327, 333), (9, 128, 7, 70), (1, 64, 8, 31), (20, 512, 32, 1030), (64, 1024, 128, 2048)])
def test_scores_and_mask_bit_exact(dtype, B, H, r, I):
    from stxgpu import DEV, ODT, predict_mask

    x, A, Bm = _case(B, H, r, I, dtype, seed=B + H + r + I)
    tau = 0.02 ** 2 * np.sqrt(H * r) * 0.8416  # ~20 % per-row density
    mask, scores, bits = predict_mask(x.to(DEV), A.to(DEV), Bm.to(DEV), param=tau)
    t_ref, s_ref = orc.predictor(x.float().numpy(), A.float().numpy(), Bm.float().numpy(), ODT[dtype])
    s_gpu = scores.float().cpu().numpy()
    assert np.array_equal(s_gpu.view(np.uint32), s_ref.view(np.uint32)), f"scores differ: max {np.abs(s_gpu - s_ref).max()}"
    _, uni = orc.mask_threshold(s_ref, ODT[dtype], tau)
    assert np.array_equal(mask.cpu().numpy(), uni)
    # packed bits: neuron n is bit n&31 of word n>>5, padding bits zero
    w = bits.cpu().numpy().view(np.uint32)
    unpacked = ((w[:, None] >> np.arange(32, dtype=np.uint32)) & 1).astype(bool).reshape(-1)
    assert np.array_equal(unpacked[:I], uni) and not unpacked[I:].any()


def test_naive_rule_is_scores_ge_zero():
    from stxgpu import DEV, ODT, predict_mask

    x, A, Bm = _case(2, 128, 16, 500, torch.float16, seed=1)
    mask, scores, _ = predict_mask(x.to(DEV), A.to(DEV), Bm.to(DEV), param=0.0)
    assert np.array_equal(mask.cpu().numpy(), (scores.float().cpu().numpy() >= 0).any(axis=0))


def test_mask_without_scores_buffer():
    from stxgpu import DEV, predict_mask

    x, A, Bm = _case(1, 256, 32, 777, torch.bfloat16, seed=2)
    m1, _, _ = predict_mask(x.to(DEV), A.to(DEV), Bm.to(DEV), param=0.01, want_scores=True)
    m2, s2, _ = predict_mask(x.to(DEV), A.to(DEV), Bm.to(DEV), param=0.01, want_scores=False)
    assert s2 is None and torch.equal(m1, m2)


def test_vs_torch_linear_flip_report():
    """Against torch's own nn.Linear pair on the same device and dtype (what the reference
    model would run): differences are accumulation-order noise; flips only next to the cut."""
    from stxgpu import DEV, predict_mask

    for dtype, tol in ((torch.float32, 3e-6), (torch.float16, 2e-3)):
        x, A, Bm = _case(1, 3072, 64, 8192, dtype, seed=3)
        x, A, Bm = x.to(DEV), A.to(DEV), Bm.to(DEV)
        tau = 0.1493
        mask, scores, _ = predict_mask(x, A, Bm, param=tau)
        ref = torch.nn.functional.linear(torch.nn.functional.linear(x, A), Bm)
        scale = float(ref.float().abs().max())
        assert float((scores.float() - ref.float()).abs().max()) <= tol * scale
        flips = int((mask != (ref >= tau).any(dim=0)).sum())
        near = int(((ref.float() - tau).abs() <= tol * scale).any(dim=0).sum())
        assert flips <= near


def test_mask_byte_bit_round_trip():
    import ctypes
    from sparse_transformers_b200 import _capi as C
    from stxgpu import DEV, stream

    for I in (1, 31, 32, 33, 8192, 14336, 1001):
        m = (torch.rand(I, generator=torch.Generator().manual_seed(I)) < 0.3).to(DEV)
        bits = torch.zeros((I + 31) // 32, dtype=torch.int32, device=DEV)
        back = torch.zeros(I, dtype=torch.bool, device=DEV)
        C.check(C.lib.stx_mask_bytes_to_bits(m.data_ptr(), I, bits.data_ptr(), stream()))
        C.check(C.lib.stx_mask_bits_to_bytes(bits.data_ptr(), I, back.data_ptr(), stream()))
        torch.cuda.synchronize()
        assert torch.equal(m, back)
        assert int(sum(bin(int(v) & 0xFFFFFFFF).count("1") for v in bits.cpu().tolist())) == int(m.sum())
