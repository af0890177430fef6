"""The allocation-free MLP entry point (stx_sparse_mlp_forward_noalloc), for callers that
cannot hand the library a scratch buffer because they are not allowed to allocate device
memory.  It must give the same result as the regular entry point, call after call, although
all calls share one built-in scratch array.  This file sorts last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.float16: 2e-2}


def _noalloc(x, concat, down_packed, act, has_gate=True):
    from sparse_transformers_b200 import _capi as C
    from stxgpu import ACT, DEV, DT, stream

    B, H = x.shape
    K = down_packed.shape[0]
    out = torch.full((B, H), float("nan"), dtype=x.dtype, device=DEV)
    comb = torch.full((B, concat.shape[0]), float("nan"), dtype=x.dtype, device=DEV)
    C.check(C.lib.stx_sparse_mlp_forward_noalloc(x.data_ptr(), B, H, concat.data_ptr(), down_packed.data_ptr(), K,
                                                 out.data_ptr(), comb.data_ptr(), ACT[act], int(has_gate), DT[x.dtype], stream()))
    torch.cuda.synchronize()
    return out, comb


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_noalloc_matches_regular_entry_point_twice(dtype):
    from stxgpu import DEV, mlp_forward, rel_err

    g = torch.Generator().manual_seed(123)
    # two different calls in a row: the second one must not see the first one's leftovers
    for (B, H, K, act) in [(2, 1024, 300, "silu"), (1, 3072, 777, "relu"), (12, 512, 200, "silu")]:  # 12 rows: streaming kernels here
        x = torch.randn(B, H, generator=g).to(dtype).to(DEV)
        cw = (torch.randn(2 * K, H, generator=g) / H ** 0.5).to(dtype).to(DEV)
        dp = (torch.randn(K, H, generator=g) / H ** 0.5).to(dtype).to(DEV)
        ref, rcomb = mlp_forward(x, cw, dp, act)
        out, comb = _noalloc(x, cw, dp, act)
        assert rel_err(out.float().cpu().numpy(), ref.float().cpu().numpy()) <= TOL[dtype]
        assert rel_err(comb.float().cpu().numpy(), rcomb.float().cpu().numpy()) <= TOL[dtype]
        out2, _ = _noalloc(x, cw, dp, act)   # same call again
        assert rel_err(out2.float().cpu().numpy(), ref.float().cpu().numpy()) <= TOL[dtype]


def test_noalloc_clears_what_the_fallback_kernel_accumulates_into():
    """Rows narrower than 512 bytes take the kernel that accumulates into the head of the scratch and
    expects it zero.  A streaming-kernel call first leaves activations right where the next, narrower
    call keeps its accumulator: only the per-call clear makes the second result right.  Checked
    against the regular entry point (fresh scratch) and against the CPU oracle; also K = 0."""
    from oracle import oracle as orc
    from stxgpu import DEV, mlp_forward, rel_err

    g = torch.Generator().manual_seed(7)
    dtype = torch.float32
    for (B, H, K) in [(1, 128, 200), (8, 64, 150), (1, 128, 90), (3, 32, 40)]:
        x = torch.randn(B, H, generator=g).to(dtype).to(DEV)
        cw = (torch.randn(2 * K, H, generator=g) / H ** 0.5).to(dtype).to(DEV)
        dp = (torch.randn(K, H, generator=g) / H ** 0.5).to(dtype).to(DEV)
        ref, _ = mlp_forward(x, cw, dp, "silu")
        out, _ = _noalloc(x, cw, dp, "silu")
        assert rel_err(out.cpu().numpy(), ref.cpu().numpy()) <= 1e-5
        want, _ = orc.sparse_mlp(x.cpu().numpy(), cw.cpu().numpy(), dp.cpu().numpy(), "silu", True)
        assert rel_err(out.cpu().numpy(), want) <= 1e-5
        again, _ = _noalloc(x, cw, dp, "silu")
        assert torch.equal(out, again)  # the blocks' partial outputs are added in block order: same bits every time
    # no active neuron: the output is zero, as the regular entry point gives
    x = torch.randn(2, 64, generator=g).to(DEV)
    cw = torch.zeros(0, 64, device=DEV)
    dp = torch.zeros(0, 64, device=DEV)
    pad = torch.zeros(16, device=DEV)  # a valid, aligned address for the empty operands
    from sparse_transformers_b200 import _capi as C
    from stxgpu import ACT, DT, stream

    out = torch.full((2, 64), float("nan"), device=DEV)
    C.check(C.lib.stx_sparse_mlp_forward_noalloc(x.data_ptr(), 2, 64, pad.data_ptr(), pad.data_ptr(), 0, out.data_ptr(),
                                                 pad.data_ptr(), ACT["silu"], 1, DT[torch.float32], stream()))
    torch.cuda.synchronize()
    assert torch.count_nonzero(out) == 0


def test_noalloc_refused_call_enqueues_nothing():
    """A call with a bad argument is refused before the shared array is touched."""
    from sparse_transformers_b200 import _capi as C
    from stxgpu import DEV, stream

    x = torch.zeros(64, device=DEV)
    rc = C.lib.stx_sparse_mlp_forward_noalloc(x.data_ptr(), 1, 64, x.data_ptr(), x.data_ptr(), 1, x.data_ptr(), None,
                                              99, 1, C.F32, stream())
    assert rc == C.ERR_INVALID_ARG and "bad activation" in C.last_error()


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    from sparse_transformers_b200 import _capi as C
    from stxgpu import DEV, stream

    x = torch.zeros(16, device=DEV)
    rc = C.lib.stx_sparse_mlp_forward_noalloc(x.data_ptr(), 64, 4096, x.data_ptr(), x.data_ptr(), 1, x.data_ptr(), None,
                                              0, 1, C.F32, stream())
    assert rc == C.ERR_TOO_LARGE and "exceeds the built-in scratch" in C.last_error()
