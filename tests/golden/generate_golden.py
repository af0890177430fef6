"""Generates tests/golden/reference_vectors.npz by RUNNING THE REFERENCE: its CPU operator
compiled unmodified (oracle/build_ref.py) plus torch for the Python half
(oracle/ref_python.py).  Run where the reference sources are available:

    python tests/golden/generate_golden.py

The vectors are small on purpose; they pin the oracle (tests/test_golden.py), which in turn
checks the CUDA path at sizes where running the reference is not possible.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_python as rp  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")


def tagged_weights(I, H, gen):
    gate = torch.randn(I, H, generator=gen) * 0.5
    up = torch.randn(I, H, generator=gen) * 0.5
    down = torch.randn(H, I, generator=gen) * 0.5
    up[:, 0] = torch.arange(I, dtype=torch.float32)  # tag: row n of up carries n in column 0
    return gate, up, down


def cache_trace(I, H, masks, gen, has_gate=True):
    WC, _, _ = rp.reference()
    gate, up, down = tagged_weights(I, H, gen)
    wc = WC(torch.ones(I, dtype=torch.bool), H, gate if has_gate else torch.empty(0), up, down, has_gate)
    orders, ks = [], []
    for m in masks:
        wc.update_active_weights(m)
        c = wc.get_concat_weight()
        K = c.shape[0] // 2 if has_gate else c.shape[0]
        order = c[c.shape[0] - K:, 0].round().long()
        d = wc.get_active_down_weight()
        # packed contents must be pool[order]
        assert torch.equal(c[c.shape[0] - K:], up[order]) and torch.equal(d, down[:, order])
        if has_gate:
            assert torch.equal(c[:K], gate[order])
        orders.append(np.pad(order.numpy().astype(np.int32), (0, I - K), constant_values=-1))
        ks.append(K)
    return np.stack(orders), np.array(ks, np.int32)


def random_masks(I, steps, gen, density=0.3, churn=0.15):
    m = torch.rand(I, generator=gen) < density
    out = []
    for _ in range(steps):
        flip = torch.rand(I, generator=gen) < churn
        target = torch.rand(I, generator=gen) < density
        m = torch.where(flip, target, m)
        if not m.any():
            m[int(torch.randint(0, I, (1,), generator=gen))] = True
        out.append(m.clone())
    return out


def main():
    torch.set_num_threads(1)
    gen = torch.Generator().manual_seed(1234)
    data = {}

    # 1. known-answer trace, 12 neurons
    I = 12
    masks = []
    for s in [{1, 4, 5, 9, 11}, {1, 2, 5, 7, 11}, {0, 1, 2, 3, 5, 7, 11}, {3, 6, 11}, {3, 6, 11}, {0}, set(range(12))]:
        m = torch.zeros(I, dtype=torch.bool)
        m[list(s)] = True
        masks.append(m)
    o, k = cache_trace(I, 8, masks, gen)
    data["kat_masks"] = torch.stack(masks).numpy()
    data["kat_orders"], data["kat_k"] = o, k

    # 2. random mask sequences (ragged sizes: I not a multiple of 32; removals > additions etc.)
    for name, I, steps, dens, churn in [("seq_a", 70, 40, 0.3, 0.2), ("seq_b", 257, 30, 0.6, 0.5), ("seq_c", 96, 30, 0.1, 0.05)]:
        masks = random_masks(I, steps, gen, dens, churn)
        # edge cases appended: all ones, single survivor, unchanged, additions only, removals only
        ones = torch.ones(I, dtype=torch.bool)
        single = torch.zeros(I, dtype=torch.bool); single[I // 2] = True
        grow = single.clone(); grow[: I // 3] = True
        masks += [ones, single, single.clone(), grow, single]
        o, k = cache_trace(I, 8, masks, gen)
        data[f"{name}_masks"] = torch.stack(masks).numpy()
        data[f"{name}_orders"], data[f"{name}_k"] = o, k
    # no-gate cache (OPT form)
    masks = random_masks(40, 12, gen, 0.4, 0.3)
    o, k = cache_trace(40, 8, masks, gen, has_gate=False)
    data["seq_nogate_masks"] = torch.stack(masks).numpy()
    data["seq_nogate_orders"], data["seq_nogate_k"] = o, k

    # 3. MLP forward: compiled op (always ReLU) and the expression the models run
    WC, fwd, topk = rp.reference()
    I, H, B = 48, 32, 3
    gate, up, down = (torch.randn(I, H, generator=gen) * 0.3, torch.randn(I, H, generator=gen) * 0.3,
                      torch.randn(H, I, generator=gen) * 0.3)
    m = torch.rand(I, generator=gen) < 0.5
    x = torch.randn(B, H, generator=gen)
    wc = WC(torch.ones(I, dtype=torch.bool), H, gate, up, down, True)
    wc.update_active_weights(m)
    cw, dw = wc.get_concat_weight().clone(), wc.get_active_down_weight().clone()
    db, cb = torch.zeros(1, H), torch.zeros(1, 2)
    out = fwd(x, cw, dw, db, cb, "silu", True)  # ReLU regardless of the name (sparse_mlp_op.cpp:157)
    data.update(mlp_x=x.numpy(), mlp_gate=gate.numpy(), mlp_up=up.numpy(), mlp_down=down.numpy(), mlp_mask=m.numpy(),
                mlp_concat=cw.numpy(), mlp_down_active=dw.contiguous().numpy(),
                mlp_out_op_gated=out.clone().numpy(), mlp_combined_op_gated=cb.clone().numpy())
    for act in ("relu", "silu", "gelu_pytorch_tanh"):
        data[f"mlp_out_expr_{act}"] = rp.skip_mlp_sparse(x, cw, dw, act, True).numpy()
    # 3-D input is flattened and the output viewed back (sparse_mlp_op.cpp:88-102,191)
    x3 = torch.randn(2, 3, H, generator=gen)
    data["mlp_x3"] = x3.numpy()
    data["mlp_out3_op_gated"] = fwd(x3, cw, dw, db, cb, "relu", True).clone().numpy()
    # no gate
    wc2 = WC(torch.ones(I, dtype=torch.bool), H, torch.empty(0), up, down, False)
    wc2.update_active_weights(m)
    cw2, dw2 = wc2.get_concat_weight().clone(), wc2.get_active_down_weight().clone()
    db2, cb2 = torch.zeros(1, H), torch.zeros(1, 2)
    data["mlp_out_op_nogate"] = fwd(x, cw2, dw2, db2, cb2, "relu", False).clone().numpy()
    data["mlp_combined_op_nogate"] = cb2.clone().numpy()
    data["mlp_out_expr_nogate_relu"] = rp.skip_mlp_sparse(x, cw2, dw2, "relu", False).numpy()

    # 4. approx_topk_threshold (fp32 only in the reference)
    for name, B_, I_, k_ in [("tk_a", 3, 64, 8), ("tk_b", 2, 1000, 100), ("tk_c", 1, 8192, 1638), ("tk_d", 2, 37, 37)]:
        s = torch.randn(B_, I_, generator=gen)
        data[f"{name}_scores"] = s.numpy()
        data[f"{name}_k"] = np.int32(k_)
        data[f"{name}_thr"] = topk(s, k_).numpy().reshape(-1)

    # 5. predictor + rules in torch (the Python half), fp32
    H, r, I, B = 64, 16, 200, 4
    A = torch.randn(r, H, generator=gen) * 0.1
    Bm = torch.randn(I, r, generator=gen) * 0.1
    x = torch.randn(B, H, generator=gen)
    s = rp.lora_scores(x, A, Bm)
    data.update(pred_x=x.numpy(), pred_A=A.numpy(), pred_Bm=Bm.numpy(), pred_scores=s.numpy())
    data["pred_mask_naive"] = rp.compute_binary_mask(s, "naive").numpy()
    data["pred_mask_tau"] = rp.compute_binary_mask(s, "threshold", tau=0.05).numpy()
    data["pred_tau"] = np.float32(0.05)
    data["pred_mask_topk"] = rp.compute_binary_mask(s, "topk", k=20).numpy()
    data["pred_topk_k"] = np.int32(20)
    data["pred_mask_stat"] = rp.compute_binary_mask(s, "statistical_topk", sparsity=0.8).numpy()
    data["pred_stat_sparsity"] = np.float32(0.8)
    data["pred_stat_z"] = np.float32(torch.distributions.normal.Normal(0, 1).icdf(torch.tensor(0.8)).item())

    # 6. "No active weights": an all-false mask throws (weight_cache.h:117-118)
    wc3 = WC(torch.ones(8, dtype=torch.bool), 8, torch.randn(8, 8), torch.randn(8, 8), torch.randn(8, 8), True)
    try:
        wc3.update_active_weights(torch.zeros(8, dtype=torch.bool))
        raised = ""
    except RuntimeError as e:
        raised = str(e).splitlines()[0]
    data["err_all_false"] = np.array(raised)

    np.savez_compressed(OUT, **data)
    print("wrote", OUT, os.path.getsize(OUT), "bytes;", len(data), "arrays")


if __name__ == "__main__":
    main()
