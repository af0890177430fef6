"""A single row through a stack of layers as ONE persistent kernel (stx_stack_step on a batch-1
stack) vs the oracle pipeline run layer by layer on the same seeded inputs: masks and cache orders
bit-exact, outputs within tolerance (1e-5 fp32, 2e-2 fp16/bf16 as max|a-b|/max|b|).  Also the same
stack on the per-layer kernels (STX_STACK_KERNEL=layers) and with the strict layer order
(STX_STACK_STRICT=1): identical masks, outputs within tolerance of each other."""
import numpy as np
import pytest
import torch

from test_gpu_layer import ODT, TOL, OracleLayer

pytestmark = pytest.mark.gpu


def _stack_vs_oracle(w, steps, seed=0, check_every=1, lazy=False):
    from sparse_transformers_b200 import SparseLayer, SparseStack
    from sparse_transformers_b200.synth import HiddenStream, layer_weights
    from stxgpu import DEV, rel_err

    gen = torch.Generator().manual_seed(seed)
    ws = [layer_weights(w, gen) for _ in range(w.layers)]
    xs = HiddenStream(w, gen)
    layers = [SparseLayer(*[t.to(DEV) for t in lw], act=w.act, method="threshold", param=w.tau, max_batch=1,
                          has_gate=w.has_gate, lazy_cache=lazy) for lw in ws]
    ols = [OracleLayer(w, *lw) for lw in ws]
    stack = SparseStack(layers, 1)
    out = torch.empty(w.layers, 1, w.H, dtype=w.dtype, device=DEV)
    worst, ks = 0.0, []
    for t in range(steps):
        x = xs.next()
        stack.step(x.to(DEV), out)
        torch.cuda.synchronize()
        got = out.float().cpu().numpy()
        for li, (l, ol) in enumerate(zip(layers, ols)):
            mask, ref = ol.step(x)
            if t % check_every:
                continue
            assert np.array_equal(l.mask().cpu().numpy(), mask), f"mask differs at step {t} layer {li}"
            assert l.active_indices().tolist() == ol.cache.active.tolist(), f"cache order differs at step {t} layer {li}"
            if t in (1, steps - 1):  # the packed rows themselves
                idx = torch.from_numpy(ol.cache.active.astype(np.int64))
                gate, up, down = ws[li][0], ws[li][1], ws[li][2]
                cw = l.concat_weight().cpu()
                want = torch.cat([gate[idx], up[idx]]) if w.has_gate else up[idx]
                assert torch.equal(cw, want), f"packed gate/up rows differ at step {t} layer {li}"
                assert torch.equal(l.active_down_weight().cpu(), down[:, idx]), f"packed down rows differ at step {t} layer {li}"
            worst = max(worst, rel_err(got[li], ref))
            ks.append(l.num_active())
    assert worst <= TOL[w.dtype], worst
    n_launch = stack.launches_per_step
    stack.close()
    for l in layers:
        l.close()
    return ks, n_launch


@pytest.mark.parametrize("dtype,H,I,r,has_gate,act,density,layers", [
    (torch.float16, 512, 2048, 64, True, "silu", 0.2, 3),
    (torch.bfloat16, 1024, 4096, 32, True, "gelu_pytorch_tanh", 0.2, 5),
    (torch.float32, 512, 2048, 16, True, "relu", 0.2, 2),
    (torch.float16, 1024, 3000, 128, False, "relu", 0.3, 4),      # no gate, ragged I (partial mask byte, CTAs without neurons)
    (torch.float16, 2048, 8192, 64, True, "silu", 0.9, 2),        # dense mask: several rounds of row spaces per pair
    (torch.bfloat16, 512, 1024, 64, True, "silu", 0.02, 3),       # nearly empty: pairs without neurons
    (torch.float16, 4096, 4096, 64, True, "silu", 0.2, 3),        # two groups of slots
    (torch.bfloat16, 4096, 14336, 128, True, "silu", 0.15, 2),    # Mistral-7B shape: two score passes per CTA and layer
])
def test_persistent_stack_matches_oracle(dtype, H, I, r, has_gate, act, density, layers):
    from sparse_transformers_b200.synth import Workload

    w = Workload("stack", H=H, I=I, r=r, B=1, dtype=dtype, density=density, layers=layers, act=act, has_gate=has_gate)
    ks, n_launch = _stack_vs_oracle(w, steps=6, seed=layers)
    # the persistent kernel + the status collector; where the kernel's CTAs lack the shared memory to run the index plans
    # themselves, also an index plan and a row-copy kernel per layer
    assert n_launch in (2, 2 + 2 * layers)


def test_c2_full_shape_16_steps():
    """Llama-3.2-3B shape (H 3072, I 8192, r 64, fp16), 4 layers, 16 steps of AR(1) hidden states."""
    from sparse_transformers_b200.synth import WORKLOADS

    w = WORKLOADS["C2"].scaled(layers=4)
    ks, _ = _stack_vs_oracle(w, steps=16, check_every=3)
    assert 0.15 * w.I < np.mean(ks[4:]) < 0.25 * w.I


@pytest.mark.parametrize("env", [{"STX_STACK_STRICT": "1"}, {"STX_STACK_ORDER": "layerwise"}, {"STX_STACK_UPKEEP": "kernels"},
                                 {"STX_STACK_KERNEL": "layers"}, {"STX_STACK_GROUP": "2"}])
def test_stack_variants_agree(monkeypatch, env):
    """Every documented switch of the stack - strict layer order, layer by layer in the overlapped order, cache
    upkeep in kernels of their own, the per-layer kernels, groups of two layers per launch - gives the same masks,
    cache orders and packed rows as the oracle, outputs within tolerance."""
    from sparse_transformers_b200.synth import WORKLOADS

    for k, v in env.items():
        monkeypatch.setenv(k, v)
    w = WORKLOADS["C2"].scaled(I=4096, H=1024, layers=5)
    _, n_launch = _stack_vs_oracle(w, steps=5, seed=9)
    if "STX_STACK_KERNEL" in env:
        assert n_launch == 5 * w.layers + 1
    elif "STX_STACK_GROUP" in env:
        assert n_launch in (3 + 1, 3 + 2 * w.layers + 1)  # three launches of the persistent kernel


def test_stack_with_lazy_cache_rows():
    """Lazy cache rows: the stack's kernel runs the index plans itself and leaves the rewritten slots in the stale
    bitmap; reading the cache (every check of the packed rows) brings the rows up to date."""
    from sparse_transformers_b200.synth import WORKLOADS

    w = WORKLOADS["C2"].scaled(I=4096, H=1024, layers=4)
    _stack_vs_oracle(w, steps=6, seed=11, lazy=True)


def test_stack_replay_is_deterministic():
    """Two stacks over the same weights fed the same inputs produce identical bits (fixed summation
    order: pair partials are added in ascending pair order)."""
    from sparse_transformers_b200 import SparseLayer, SparseStack
    from sparse_transformers_b200.synth import HiddenStream, WORKLOADS, layer_weights
    from stxgpu import DEV

    w = WORKLOADS["C2"].scaled(I=4096, H=1024, layers=3)
    gen = torch.Generator().manual_seed(4)
    ws = [layer_weights(w, gen) for _ in range(w.layers)]
    mk = lambda: [SparseLayer(*[t.to(DEV) for t in lw], act=w.act, param=w.tau, max_batch=1) for lw in ws]
    a, b = mk(), mk()
    sa, sb = SparseStack(a, 1), SparseStack(b, 1)
    xs = HiddenStream(w, gen)
    oa = torch.empty(w.layers, 1, w.H, dtype=w.dtype, device=DEV)
    ob = torch.empty_like(oa)
    for _ in range(5):
        x = xs.next().to(DEV)
        sa.step(x, oa)
        sb.step(x, ob)
        torch.cuda.synchronize()
        assert torch.equal(oa, ob)
    sa.close(); sb.close()


@pytest.mark.parametrize("room_for_layers", [1, 2])
def test_expired_wait_makes_the_next_step_fail(monkeypatch, room_for_layers):
    """A wait that runs out inside a step must not pass silently.  World of two whose second rank does not
    exist (its exchange buffer is a second buffer on this GPU that nobody writes): the stack kernel's wait for
    the peer's partial sums expires after its poll limit, the step finishes (the context stays usable), the
    error bits reach pinned host memory with the step's last node, and the next step call is refused.  With
    room for one layer's sums in the exchange buffer the layer-by-layer kernel runs, with room for both layers
    the flow kernel (all layers exchanged at once)."""
    import ctypes

    from sparse_transformers_b200 import SparseLayer, SparseStack
    from sparse_transformers_b200 import _capi as C
    from sparse_transformers_b200.synth import HiddenStream, WORKLOADS, layer_weights
    from stxgpu import DEV

    monkeypatch.setenv("STX_PEER_WAIT_ITERS", "500")
    w = WORKLOADS["C2"].scaled(I=2048, H=512, layers=2)
    a, b = ctypes.c_void_p(), ctypes.c_void_p()
    C.check(C.lib.stx_peer_create(ctypes.byref(a), 0, 2, room_for_layers * w.H))
    C.check(C.lib.stx_peer_create(ctypes.byref(b), 1, 2, room_for_layers * w.H))  # only its buffer is used
    pa, pb = ctypes.c_void_p(), ctypes.c_void_p()
    C.check(C.lib.stx_peer_local_buffer(a, ctypes.byref(pa)))
    C.check(C.lib.stx_peer_local_buffer(b, ctypes.byref(pb)))
    C.check(C.lib.stx_peer_connect_ptrs(a, (ctypes.c_void_p * 2)(pa.value, pb.value)))

    class _Peer:
        handle = a

    gen = torch.Generator().manual_seed(3)
    layers = [SparseLayer(*[t.to(DEV) for t in layer_weights(w, gen)], act=w.act, param=w.tau, max_batch=1) for _ in range(w.layers)]
    for l in layers:
        l.set_peer(_Peer)
    stack = SparseStack(layers, 1)
    try:
        assert stack.launches_per_step in (2, 2 + 2 * w.layers)  # the persistent kernel carries the exchange
        xs = HiddenStream(w, gen).take(2).to(DEV)
        stack.step(xs[0])          # finishes: every wait for the absent peer gives up after 500 polls
        torch.cuda.synchronize()
        assert float((torch.ones(8, device=DEV) * 2).sum()) == 16.0  # context alive
        with pytest.raises(C.StxError) as ei:
            stack.step(xs[1])
        assert ei.value.status == C.ERR_TIMEOUT and "bounded wait expired" in str(ei.value)
    finally:
        stack.close()
        for l in layers:
            l.close()
        C.lib.stx_peer_destroy(a)
        C.lib.stx_peer_destroy(b)
