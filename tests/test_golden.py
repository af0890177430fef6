"""The CPU oracle against golden vectors produced by running the reference
(tests/golden/generate_golden.py)."""
import numpy as np
import pytest

from oracle import oracle as orc

SEQS = ["kat", "seq_a", "seq_b", "seq_c", "seq_nogate"]


@pytest.mark.parametrize("name", SEQS)
def test_cache_order_matches_reference_trace(golden, name):
    masks, orders, ks = golden[f"{name}_masks"], golden[f"{name}_orders"], golden[f"{name}_k"]
    I = masks.shape[1]
    c = orc.OracleCache(I)
    assert c.update(np.ones(I, bool)) == I  # the reference constructor applies an all-ones mask
    for m, o, k in zip(masks, orders, ks):
        assert c.update(m) == k
        assert c.active.tolist() == o[:k].tolist()


def test_known_answer_trace_values(golden):
    # the 12-neuron trace, spelled out
    o, k = golden["kat_orders"], golden["kat_k"]
    assert o[0][: k[0]].tolist() == [11, 1, 5, 9, 4]
    assert o[1][: k[1]].tolist() == [11, 1, 5, 7, 2]
    assert o[2][: k[2]].tolist() == [11, 1, 5, 7, 2, 0, 3]
    assert o[3][: k[3]].tolist() == [11, 3, 6]


def test_all_false_mask_raises_like_reference(golden):
    assert "No active weights" in str(golden["err_all_false"])
    c = orc.OracleCache(8)
    c.update(np.ones(8, bool))
    with pytest.raises(orc.NoActiveWeights):
        c.update(np.zeros(8, bool))


def test_mlp_against_reference_op_and_expression(golden):
    g = golden
    x, cw, dw = g["mlp_x"], g["mlp_concat"], g["mlp_down_active"]  # dw: [H,K]
    packed = np.ascontiguousarray(dw.T)
    out, comb = orc.sparse_mlp(x, cw, packed, "relu", True)
    np.testing.assert_allclose(out, g["mlp_out_op_gated"], rtol=1e-5, atol=1e-5 * np.abs(g["mlp_out_op_gated"]).max())
    np.testing.assert_allclose(comb, g["mlp_combined_op_gated"], rtol=1e-5, atol=1e-6)
    for act in ("relu", "silu", "gelu_pytorch_tanh"):
        ref = g[f"mlp_out_expr_{act}"]
        out, _ = orc.sparse_mlp(x, cw, packed, act, True)
        np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-5 * np.abs(ref).max())
    out3, _ = orc.sparse_mlp(g["mlp_x3"].reshape(-1, x.shape[1]), cw, packed, "relu", True)
    np.testing.assert_allclose(out3.reshape(g["mlp_x3"].shape), g["mlp_out3_op_gated"], rtol=1e-5, atol=1e-5)


def test_mlp_no_gate(golden):
    g = golden
    K = int(g["mlp_mask"].sum())
    c = orc.OracleCache(len(g["mlp_mask"]))
    c.update(np.ones(len(g["mlp_mask"]), bool))
    c.update(g["mlp_mask"])
    assert c.K == K
    wup = c.gather(g["mlp_up"])
    wdown = c.gather(np.ascontiguousarray(g["mlp_down"].T))
    out, comb = orc.sparse_mlp(g["mlp_x"], wup, wdown, "relu", False)
    np.testing.assert_allclose(out, g["mlp_out_op_nogate"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(comb, g["mlp_combined_op_nogate"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(out, g["mlp_out_expr_nogate_relu"], rtol=1e-5, atol=1e-5)


def test_cache_gather_reproduces_reference_tensors(golden):
    g = golden
    I = len(g["mlp_mask"])
    c = orc.OracleCache(I)
    c.update(np.ones(I, bool))
    c.update(g["mlp_mask"])
    cw = np.concatenate([c.gather(g["mlp_gate"]), c.gather(g["mlp_up"])])
    assert np.array_equal(cw, g["mlp_concat"])
    assert np.array_equal(c.gather(np.ascontiguousarray(g["mlp_down"].T)).T, g["mlp_down_active"])


@pytest.mark.parametrize("name", ["tk_a", "tk_b", "tk_c", "tk_d"])
def test_approx_topk_threshold_bit_exact(golden, name):
    thr = orc.approx_topk_threshold(golden[f"{name}_scores"], int(golden[f"{name}_k"]))
    assert np.array_equal(thr, golden[f"{name}_thr"])


def test_predictor_scores_and_rules(golden):
    g = golden
    t, s = orc.predictor(g["pred_x"], g["pred_A"], g["pred_Bm"], orc.F32)
    ref = g["pred_scores"]
    np.testing.assert_allclose(s, ref, rtol=0, atol=2e-6 * np.abs(ref).max())
    # masks agree wherever the score is not within rounding distance of the cut
    margin = 4e-6 * np.abs(ref).max()
    _, uni = orc.mask_threshold(s, orc.F32, 0.0)
    safe = (np.abs(ref) > margin).all(axis=0)
    assert np.array_equal(uni[safe], g["pred_mask_naive"][safe]) and safe.mean() > 0.99
    _, uni = orc.mask_threshold(s, orc.F32, float(g["pred_tau"]))
    safe = (np.abs(ref - g["pred_tau"]) > margin).all(axis=0)
    assert np.array_equal(uni[safe], g["pred_mask_tau"][safe]) and safe.mean() > 0.99
    # rules on the reference's own scores are exact (no ties in these fp32 rows)
    _, uni = orc.mask_topk(ref, int(g["pred_topk_k"]))
    assert np.array_equal(uni, g["pred_mask_topk"])
    _, uni, _ = orc.mask_statistical(ref, orc.F32, float(g["pred_stat_z"]))
    assert np.array_equal(uni, g["pred_mask_stat"])
