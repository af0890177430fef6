"""Sparse MLP forward on the GPU (C ABI) vs the oracle and the golden reference outputs.
Tolerance: max|a-b| / max|b| <= 1e-5 in fp32, <= 2e-2 in fp16/bf16."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.float16: 2e-2, torch.bfloat16: 2e-2}


def _case(B, H, K, dtype, seed, has_gate=True, scale=None):
    g = torch.Generator().manual_seed(seed)
    scale = scale or (1.0 / np.sqrt(H))
    x = torch.randn(B, H, generator=g).to(dtype)
    cw = (torch.randn(2 * K if has_gate else K, H, generator=g) * scale).to(dtype)
    dp = (torch.randn(K, H, generator=g) * scale).to(dtype)
    return x, cw, dp


def test_golden_reference_outputs(golden):
    from stxgpu import DEV, mlp_forward, rel_err

    g = golden
    x = torch.from_numpy(g["mlp_x"]).to(DEV)
    cw = torch.from_numpy(g["mlp_concat"]).to(DEV)
    dp = torch.from_numpy(np.ascontiguousarray(g["mlp_down_active"].T)).to(DEV)
    out, comb = mlp_forward(x, cw, dp, "relu")
    assert rel_err(out.cpu().numpy(), g["mlp_out_op_gated"]) <= 1e-5      # the compiled reference op
    assert rel_err(comb.cpu().numpy(), g["mlp_combined_op_gated"]) <= 1e-5
    for act in ("relu", "silu", "gelu_pytorch_tanh"):                     # the expression the models run
        out, _ = mlp_forward(x, cw, dp, act)
        assert rel_err(out.cpu().numpy(), g[f"mlp_out_expr_{act}"]) <= 1e-5
    x3 = torch.from_numpy(g["mlp_x3"]).to(DEV)
    out, _ = mlp_forward(x3.view(-1, x3.shape[-1]), cw, dp, "relu")
    assert rel_err(out.cpu().numpy().reshape(g["mlp_x3"].shape), g["mlp_out3_op_gated"]) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("act", ["relu", "silu", "gelu_pytorch_tanh"])
@pytest.mark.parametrize("B,H,K", [(1, 2048, 1556), (1, 3072, 400), (8, 4096, 300), (3, 512, 77), (2, 64, 1), (5, 128, 1000)])
def test_vs_oracle(dtype, act, B, H, K):
    from stxgpu import DEV, mlp_forward, rel_err

    x, cw, dp = _case(B, H, K, dtype, seed=B * 1000 + K)
    out, comb = mlp_forward(x.to(DEV), cw.to(DEV), dp.to(DEV), act)
    ref, rcomb = orc.sparse_mlp(x.float().numpy(), cw.float().numpy(), dp.float().numpy(), act, True)
    assert rel_err(out.float().cpu().numpy(), ref) <= TOL[dtype]
    assert rel_err(comb.float().cpu().numpy(), rcomb) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_no_gate(dtype):
    from stxgpu import DEV, mlp_forward, rel_err

    x, cw, dp = _case(4, 256, 130, dtype, seed=5, has_gate=False)
    for act in ("relu", "gelu"):
        out, comb = mlp_forward(x.to(DEV), cw.to(DEV), dp.to(DEV), act, has_gate=False)
        ref, rcomb = orc.sparse_mlp(x.float().numpy(), cw.float().numpy(), dp.float().numpy(), act, False)
        assert rel_err(out.float().cpu().numpy(), ref) <= TOL[dtype]
        assert rel_err(comb.float().cpu().numpy(), rcomb) <= TOL[dtype]


def test_zero_active_gives_zero_output():
    from stxgpu import DEV, mlp_forward

    x = torch.randn(2, 64).to(DEV)
    cw = torch.zeros(0, 64, device=DEV)
    dp = torch.zeros(0, 64, device=DEV)
    # K == 0: empty weights still need valid (non-null) pointers
    cw_buf, dp_buf = torch.zeros(16, device=DEV), torch.zeros(16, device=DEV)
    import ctypes
    from sparse_transformers_b200 import _capi as C
    from stxgpu import stream
    out = torch.full((2, 64), 7.0, device=DEV)
    n = ctypes.c_size_t(); C.lib.stx_mlp_scratch_bytes(2, 64, 0, ctypes.byref(n))
    scratch = torch.zeros(n.value, dtype=torch.uint8, device=DEV)
    C.check(C.lib.stx_sparse_mlp_forward(x.data_ptr(), 2, 64, cw_buf.data_ptr(), dp_buf.data_ptr(), 0, out.data_ptr(), None,
                                         C.ACT_SILU, 1, C.F32, scratch.data_ptr(), stream()))
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0


def test_linearity_and_repeatability_full_size():
    """Size-independent properties at the Llama-3.2-3B shape: the op is linear in the down
    weights, and repeated calls on the same scratch agree to fp32-summation noise."""
    from stxgpu import DEV, mlp_forward, rel_err

    B, H, K = 1, 3072, 1583
    x, cw, dp = _case(B, H, K, torch.float16, seed=21)
    x, cw, dp = x.to(DEV), cw.to(DEV), dp.to(DEV)
    o1, _ = mlp_forward(x, cw, dp, "silu")
    o2, _ = mlp_forward(x, cw, dp, "silu")
    assert rel_err(o1.float().cpu().numpy(), o2.float().cpu().numpy()) <= 2e-3
    oh, _ = mlp_forward(x, cw, (dp.float() * 0.5).half(), "silu")
    assert rel_err((oh.float() * 2).cpu().numpy(), o1.float().cpu().numpy()) <= 2e-3


def test_argument_errors():
    import ctypes
    from sparse_transformers_b200 import _capi as C
    from stxgpu import DEV, stream

    x = torch.zeros(1, 64, device=DEV)
    assert C.lib.stx_sparse_mlp_forward(x.data_ptr(), 1, 64, None, x.data_ptr(), 1, x.data_ptr(), None, 0, 1, 0, x.data_ptr(), stream()) == C.ERR_INVALID_ARG
    assert C.lib.stx_sparse_mlp_forward(x.data_ptr(), 1, 64, x.data_ptr(), x.data_ptr(), 1, x.data_ptr(), None, 99, 1, 0, x.data_ptr(), stream()) == C.ERR_INVALID_ARG
    # H*elem not a multiple of 16 bytes
    assert C.lib.stx_sparse_mlp_forward(x.data_ptr(), 1, 6, x.data_ptr(), x.data_ptr(), 1, x.data_ptr(), None, 0, 1, 0, x.data_ptr(), stream()) == C.ERR_UNSUPPORTED
