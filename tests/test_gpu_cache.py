"""Differential weight cache on the GPU (through the C ABI) vs the oracle: index order and
packed contents must be bit-exact."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _weights(I, H, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    w = [(torch.randn(I, H, generator=g)).to(dtype), (torch.randn(I, H, generator=g)).to(dtype),
         (torch.randn(H, I, generator=g)).to(dtype)]
    return w


def _check_state(cache, oc, gate, up, down, has_gate=True):
    act = cache.active()
    assert act.tolist() == oc.active.tolist()
    K = len(act)
    idx = torch.from_numpy(act.astype(np.int64))
    cw = cache.concat().cpu()
    if has_gate:
        assert cw.shape[0] == 2 * K
        assert torch.equal(cw[:K].view(torch.uint8), gate[idx].contiguous().view(torch.uint8))
        assert torch.equal(cw[K:].view(torch.uint8), up[idx].contiguous().view(torch.uint8))
    else:
        assert cw.shape[0] == K
        assert torch.equal(cw.view(torch.uint8), up[idx].contiguous().view(torch.uint8))
    dp = cache.down_packed().cpu()
    assert torch.equal(dp.view(torch.uint8), down.t()[idx].contiguous().view(torch.uint8))


@pytest.mark.parametrize("name", ["kat", "seq_a", "seq_b", "seq_c"])
def test_golden_sequences(golden, name):
    from stxgpu import DEV, Cache

    masks, orders, ks = golden[f"{name}_masks"], golden[f"{name}_orders"], golden[f"{name}_k"]
    I = masks.shape[1]
    gate, up, down = _weights(I, 8, torch.float32)
    c = Cache(gate.to(DEV), up.to(DEV), down.to(DEV))
    oc = orc.OracleCache(I)
    oc.update(np.ones(I, bool))
    _check_state(c, oc, gate, up, down)
    for m, o, k in zip(masks, orders, ks):
        c.update(torch.from_numpy(m))
        oc.update(m)
        assert c.active().tolist() == o[:k].tolist()
        _check_state(c, oc, gate, up, down)


def test_golden_no_gate(golden):
    from stxgpu import DEV, Cache

    masks, orders, ks = golden["seq_nogate_masks"], golden["seq_nogate_orders"], golden["seq_nogate_k"]
    I = masks.shape[1]
    gate, up, down = _weights(I, 8, torch.float32)
    c = Cache(None, up.to(DEV), down.to(DEV), has_gate=False)
    oc = orc.OracleCache(I)
    oc.update(np.ones(I, bool))
    for m, o, k in zip(masks, orders, ks):
        c.update(torch.from_numpy(m))
        oc.update(m)
        assert c.active().tolist() == o[:k].tolist()
        _check_state(c, oc, gate, up, down, has_gate=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("I,H", [(8192, 256), (14336, 64), (1000, 40), (33, 8)])
def test_ar1_churn(dtype, I, H):
    from stxgpu import DEV, Cache

    if dtype != torch.float32 and H % 8:
        pytest.skip("16-bit rows need H % 8 == 0")
    gate, up, down = _weights(I, H, dtype, seed=I)
    c = Cache(gate.to(DEV), up.to(DEV), down.to(DEV))
    oc = orc.OracleCache(I)
    oc.update(np.ones(I, bool))
    g = torch.Generator().manual_seed(3)
    z = torch.randn(I, generator=g)
    for step in range(10):
        z = 0.9 * z + 0.436 * torch.randn(I, generator=g)
        m = z > 0.84
        c.update(m)
        oc.update(m.numpy())
        a, r, copied = c.stats()
        assert (a, r) == (oc.last_added, oc.last_removed)
        if step in (0, 1, 5, 9):
            _check_state(c, oc, gate, up, down)
        else:
            assert c.active().tolist() == oc.active.tolist()


def test_edge_cases():
    from sparse_transformers_b200 import _capi as C
    from stxgpu import DEV, Cache

    I, H = 100, 16
    gate, up, down = _weights(I, H, torch.float32)
    c = Cache(gate.to(DEV), up.to(DEV), down.to(DEV))
    oc = orc.OracleCache(I)
    oc.update(np.ones(I, bool))
    seq = []
    m = torch.zeros(I, dtype=torch.bool); m[99] = True; seq.append(m)            # single survivor = last element
    seq.append(m.clone())                                                          # unchanged: no-op
    m2 = m.clone(); m2[:50] = True; seq.append(m2)                                 # additions only
    m3 = m2.clone(); m3[10:40] = False; seq.append(m3)                             # removals only
    m4 = torch.ones(I, dtype=torch.bool); seq.append(m4)                           # all true
    m5 = torch.zeros(I, dtype=torch.bool); m5[0] = True; seq.append(m5)            # remove all but the first
    for m in seq:
        c.update(m)
        oc.update(m.numpy())
        _check_state(c, oc, gate, up, down)
    a, r, copied = c.stats()
    c.update(seq[-1])  # unchanged again
    assert c.stats() == (0, 0, 0)
    # all-false: the reference throws "No active weights"
    c.update(torch.zeros(I, dtype=torch.bool))
    rc, k = c.num_active_status()
    assert rc == C.ERR_NO_ACTIVE and k == 0 and "No active weights" in C.last_error()


def test_cache_without_initial_mask_is_invalid():
    from sparse_transformers_b200 import _capi as C
    from stxgpu import DEV, Cache

    gate, up, down = _weights(64, 8, torch.float32)
    c = Cache(gate.to(DEV), up.to(DEV), down.to(DEV), init_mask=None)
    rc, k = c.num_active_status()
    assert rc == C.ERR_CACHE_INVALID and k == 0
    m = torch.zeros(64, dtype=torch.bool); m[[3, 5, 60]] = True
    c.update(m)
    assert c.active().tolist() == [3, 5, 60]


def test_large_removal_uses_generic_path():
    """More surplus removals than the shared-memory fast path holds (first step after the
    all-ones initial mask at a large I)."""
    from stxgpu import DEV, Cache

    I, H = 16384, 8
    gate, up, down = _weights(I, H, torch.float32, seed=9)
    c = Cache(gate.to(DEV), up.to(DEV), down.to(DEV))
    oc = orc.OracleCache(I)
    oc.update(np.ones(I, bool))
    g = torch.Generator().manual_seed(4)
    m = torch.rand(I, generator=g) < 0.2   # ~13k removals at once
    c.update(m); oc.update(m.numpy())
    _check_state(c, oc, gate, up, down)
    m = torch.rand(I, generator=g) < 0.7   # mostly additions
    c.update(m); oc.update(m.numpy())
    m = torch.rand(I, generator=g) < 0.6   # ~1.6k surplus removals: fast path with tail interplay
    c.update(m); oc.update(m.numpy())
    _check_state(c, oc, gate, up, down)
