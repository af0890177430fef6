"""Prefill-sized row blocks (tcgen05 tensor-core path of stx_sparse_mlp_forward) vs the oracle
(small cases) and a torch fp32 evaluation of the same expression on the same device (large
cases, where the scalar oracle would take minutes).  Tolerance 2e-2 (fp16/bf16), as
max|a-b| / max|b|."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu
ACTS = {"relu": torch.relu, "silu": torch.nn.functional.silu,
        "gelu_pytorch_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}


def _case(B, H, K, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, H, generator=g).to(dtype)
    cw = (torch.randn(2 * K, H, generator=g) / np.sqrt(H)).to(dtype)
    dp = (torch.randn(K, H, generator=g) / np.sqrt(K)).to(dtype)
    return x, cw, dp


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,K,act", [(128, 256, 128, "relu"), (256, 512, 300, "silu"), (70, 64, 77, "gelu_pytorch_tanh")])
def test_small_vs_oracle(dtype, B, H, K, act):
    from stxgpu import DEV, mlp_forward, rel_err

    x, cw, dp = _case(B, H, K, dtype, seed=B + K)
    out, comb = mlp_forward(x.to(DEV), cw.to(DEV), dp.to(DEV), act)
    ref, rcomb = orc.sparse_mlp(x.float().numpy(), cw.float().numpy(), dp.float().numpy(), act, True)
    assert rel_err(comb.float().cpu().numpy(), rcomb) <= 2e-2
    assert rel_err(out.float().cpu().numpy(), ref) <= 2e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,K", [(1000, 4096, 1100), (2048, 1024, 4103), (8192, 4096, 1101)])
def test_large_vs_torch_fp32(dtype, B, H, K):
    """ReluLLaMA-7B-like widths; ragged K (not a multiple of 8 or 128) and ragged row counts."""
    from stxgpu import DEV, mlp_forward

    x, cw, dp = _case(B, H, K, dtype, seed=K)
    x, cw, dp = x.to(DEV), cw.to(DEV), dp.to(DEV)
    out, comb = mlp_forward(x, cw, dp, "relu")
    g, u = (x.float() @ cw.float().t()).chunk(2, dim=-1)
    a = torch.relu(g) * u
    ref = a.to(dtype).float() @ dp.float()   # the path rounds the activations to the model dtype between the GEMMs
    assert float((comb[:, :K].float() - a).abs().max() / a.abs().max()) <= 2e-2
    assert float((comb[:, K:].float() - u).abs().max() / u.abs().max()) <= 2e-2
    assert float((out.float() - ref).abs().max() / ref.abs().max()) <= 2e-2


def test_prefill_equals_decode_kernels_on_same_rows():
    """Linearity across the dispatch boundary: 64 rows through the tensor-core path give the
    rows that the decode kernels give one batch of 8 at a time."""
    from stxgpu import DEV, mlp_forward, rel_err

    x, cw, dp = _case(64, 512, 256, torch.float16, seed=9)
    x, cw, dp = x.to(DEV), cw.to(DEV), dp.to(DEV)
    big, _ = mlp_forward(x, cw, dp, "silu")
    for i in range(0, 64, 8):
        small, _ = mlp_forward(x[i:i + 8].contiguous(), cw, dp, "silu")
        assert rel_err(big[i:i + 8].float().cpu().numpy(), small.float().cpu().numpy()) <= 2e-2
