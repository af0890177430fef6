"""The reference-named torch interface (torch.classes.sparse_mlp.WeightCache,
torch.ops.sparse_mlp.forward) on the GPU: same observable behaviour as the reference's
(signatures, shapes, strides, aliasing, error texts), checked against the golden vectors
and, where it is available, the compiled reference itself."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tagged(I, H, seed=0):
    g = torch.Generator().manual_seed(seed)
    gate, up, down = torch.randn(I, H, generator=g), torch.randn(I, H, generator=g), torch.randn(H, I, generator=g)
    up[:, 0] = torch.arange(I, dtype=torch.float32)
    return gate, up, down


def test_weight_cache_drop_in_trace(golden):
    import sparse_transformers_b200 as stb

    I, H = 12, 8
    gate, up, down = _tagged(I, H)
    wc = stb.WeightCache(torch.ones(I, dtype=torch.bool), H, gate.to(DEV), up.to(DEV), down.to(DEV), True)
    for m, o, k in zip(golden["kat_masks"], golden["kat_orders"], golden["kat_k"]):
        wc.update_active_weights(torch.from_numpy(m))          # CPU mask, as the reference is fed
        cw, dw = wc.get_concat_weight(), wc.get_active_down_weight()
        assert cw.shape == (2 * k, H) and cw.is_contiguous()
        assert dw.shape == (H, k) and (k == 1 or dw.stride() == (1, H))   # like the reference: packed.t()
        order = cw[k:, 0].round().long().cpu()
        assert order.tolist() == o[:k].tolist() == wc.get_active_indices().tolist()
        assert torch.equal(cw[:k].cpu(), gate[order]) and torch.equal(cw[k:].cpu(), up[order])
        assert torch.equal(dw.cpu(), down[:, order])
        assert wc.get_num_active() == k
    wc.update_active_weights(torch.from_numpy(golden["kat_masks"][0]).to(DEV))  # CUDA mask works too
    assert wc.get_num_active() == 5


def test_weight_cache_errors_like_reference():
    import sparse_transformers_b200 as stb

    gate, up, down = _tagged(8, 8)
    wc = stb.WeightCache(torch.ones(8, dtype=torch.bool), 8, gate.to(DEV), up.to(DEV), down.to(DEV), True)
    wc.update_active_weights(torch.zeros(8, dtype=torch.bool))
    with pytest.raises(RuntimeError, match="No active weights"):
        wc.get_concat_weight()
    wc2 = stb.WeightCache(torch.zeros(8, dtype=torch.bool), 8, gate.to(DEV), up.to(DEV), down.to(DEV), True)
    with pytest.raises(RuntimeError, match="Cache is not valid"):
        wc2.get_active_down_weight()


def test_forward_op_semantics(golden):
    import sparse_transformers_b200 as stb

    g = golden
    x = torch.from_numpy(g["mlp_x"]).to(DEV)
    gate, up, down = (torch.from_numpy(g[k]).to(DEV) for k in ("mlp_gate", "mlp_up", "mlp_down"))
    I, H = up.shape
    wc = stb.WeightCache(torch.ones(I, dtype=torch.bool), H, gate, up, down, True)
    wc.update_active_weights(torch.from_numpy(g["mlp_mask"]))
    cw, dw = wc.get_concat_weight(), wc.get_active_down_weight()
    assert torch.equal(cw.cpu(), torch.from_numpy(g["mlp_concat"]))
    assert torch.equal(dw.cpu(), torch.from_numpy(g["mlp_down_active"]))
    db, cb = torch.zeros(1, H, device=DEV), torch.zeros(1, 2, device=DEV)   # wrongly sized: the op resizes them
    out = torch.ops.sparse_mlp.forward(x, cw, dw, db, cb, "relu", True)
    assert out.data_ptr() == db.data_ptr() and db.shape == (3, H) and cb.shape == (3, cw.shape[0])
    ref = torch.from_numpy(g["mlp_out_op_gated"])
    assert (out.cpu() - ref).abs().max() <= 1e-5 * ref.abs().max()
    assert (cb.cpu() - torch.from_numpy(g["mlp_combined_op_gated"])).abs().max() <= 1e-5
    # the 6-argument form of the README, honouring the activation name
    out = stb.sparse_mlp_forward(x, cw, dw, db, cb, "silu")
    ref = torch.from_numpy(g["mlp_out_expr_silu"])
    assert (out.cpu() - ref).abs().max() <= 1e-5 * ref.abs().max()
    # 3-D input keeps its shape
    x3 = torch.from_numpy(g["mlp_x3"]).to(DEV)
    out3 = stb.sparse_mlp_forward(x3, cw, dw, db, cb, "relu")
    assert out3.shape == x3.shape
    ref3 = torch.from_numpy(g["mlp_out3_op_gated"])
    assert (out3.cpu() - ref3).abs().max() <= 1e-5 * ref3.abs().max()
    # a contiguous [H,K] down weight (not the cache's strided view) is accepted too
    out = stb.sparse_mlp_forward(x, cw, dw.contiguous(), db, cb, "silu")
    assert (out.cpu() - ref).abs().max() <= 1e-5 * ref.abs().max()
    with pytest.raises(RuntimeError, match="unknown activation"):
        stb.sparse_mlp_forward(x, cw, dw, db, cb, "tanhshrink")


def test_skip_mlp_module_and_mask_helper():
    """SkipMLP / FastLoRAProjection / compute_binary_mask as a LlamaSkip-style layer uses them."""
    import sparse_transformers_b200 as stb

    torch.manual_seed(0)
    H, I, r = 256, 1024, 32
    for dtype, tol in ((torch.float32, 1e-5), (torch.float16, 2e-2)):
        mlp = stb.SkipMLP(H, I, sparsity=0.8, act_fn="silu").to(DEV, dtype)
        lora = stb.FastLoRAProjection(H, I, r).to(DEV, dtype)
        mlp.initialize_weight_cache()
        x = torch.randn(1, 1, H, device=DEV, dtype=dtype)
        mask = stb.compute_binary_mask(x, lora, "naive", weight_cache=mlp.weight_cache)
        ref_mask = (lora(x.view(-1, H)) >= 0).any(dim=0)
        assert (mask != ref_mask).sum() <= 2   # accumulation-order ties at the cut only
        y = mlp(x, use_sparse=True)
        # dense MLP restricted to the same mask
        a = (mlp.act_fn(mlp.gate_proj(x)) * mlp.up_proj(x)) * mask
        ref = mlp.down_proj(a)
        assert y.shape == x.shape
        assert (y.float() - ref.float()).abs().max() <= tol * ref.float().abs().max() + 1e-6
        assert torch.equal(mlp(x, use_sparse=False), mlp._forward_dense(x))


def test_against_live_reference(refmod):
    """Same mask sequence through the compiled reference (CPU) and this library (GPU)."""
    import sparse_transformers_b200 as stb

    WC, fwd, _ = refmod.reference()
    I, H = 300, 64
    gate, up, down = _tagged(I, H, seed=4)
    ref = WC(torch.ones(I, dtype=torch.bool), H, gate, up, down, True)
    mine = stb.WeightCache(torch.ones(I, dtype=torch.bool), H, gate.to(DEV), up.to(DEV), down.to(DEV), True)
    g = torch.Generator().manual_seed(8)
    db, cb = torch.zeros(1, H), torch.zeros(1, 2)
    dbg, cbg = torch.zeros(1, H, device=DEV), torch.zeros(1, 2, device=DEV)
    for _ in range(15):
        m = torch.rand(I, generator=g) < 0.3
        ref.update_active_weights(m)
        mine.update_active_weights(m)
        assert torch.equal(ref.get_concat_weight(), mine.get_concat_weight().cpu())
        assert torch.equal(ref.get_active_down_weight(), mine.get_active_down_weight().cpu())
        x = torch.randn(2, H, generator=g)
        r = fwd(x, ref.get_concat_weight(), ref.get_active_down_weight(), db, cb, "relu", True)
        o = torch.ops.sparse_mlp.forward(x.to(DEV), mine.get_concat_weight(), mine.get_active_down_weight(), dbg, cbg, "relu", True)
        assert (o.cpu() - r).abs().max() <= 1e-5 * r.abs().max()


@pytest.mark.parametrize("dtype,rows,H,I", [(torch.float16, 1, 1024, 2048), (torch.float32, 3, 256, 512), (torch.bfloat16, 12, 512, 1024),
                                            (torch.float16, 1, 64, 256)])
def test_sparse_forward_equals_getters_plus_forward(dtype, rows, H, I):
    """WeightCache.sparse_forward (no getters, K stays on the device) gives what the reference's call
    sequence get_concat_weight / get_active_down_weight / sparse_mlp_forward gives, update after
    update and for changing row counts; a scratch-path shape (64-element rows) is among the cases,
    and the MLP calls of a SkipMLP agree between the two forms."""
    import sparse_transformers_b200 as stb

    g = torch.Generator().manual_seed(rows + H)
    gate, up, down = (torch.randn(I, H, generator=g) / H ** 0.5).to(dtype), (torch.randn(I, H, generator=g) / H ** 0.5).to(dtype), \
        (torch.randn(H, I, generator=g) / I ** 0.5).to(dtype)
    wc = stb.WeightCache(torch.ones(I, dtype=torch.bool), H, gate.to(DEV), up.to(DEV), down.to(DEV), True)
    buf_a = torch.zeros(1, H, dtype=dtype, device=DEV)
    buf_b = torch.zeros(1, H, dtype=dtype, device=DEV)
    comb = torch.zeros(1, 2, dtype=dtype, device=DEV)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for step, r in enumerate([rows, rows, 1, rows]):
        mask = torch.rand(I, generator=g) < (0.2 + 0.1 * step)
        wc.update_active_weights(mask.to(DEV))
        x = torch.randn(r, H, generator=g).to(dtype).to(DEV)
        got = wc.sparse_forward(x, buf_a, "silu").clone()
        want = stb.sparse_mlp_forward(x, wc.get_concat_weight(), wc.get_active_down_weight(), buf_b, comb, "silu").clone()
        assert got.shape == want.shape == (r, H)
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err <= tol, (step, err)


def test_skip_mlp_fused_getters_match_reference_sequence():
    import sparse_transformers_b200 as stb

    torch.manual_seed(0)
    mlp = stb.SkipMLP(512, 1024, sparsity=0.8).to(DEV).half()
    mlp.initialize_weight_cache()
    lora = stb.FastLoRAProjection(512, 1024, 32).to(DEV).half()
    x = torch.randn(1, 512, device=DEV, dtype=torch.float16)
    stb.compute_binary_mask(x, lora, "naive", weight_cache=mlp.weight_cache)
    a = mlp(x)
    mlp.fused_getters = False
    b = mlp(x)
    assert float((a.float() - b.float()).abs().max() / b.float().abs().max()) <= 2e-2
