"""LlamaSkip host (dense prefill, sparse decode) on the GPU: every decode-time MLP call is
checked against the oracle on the very inputs the model fed it (mask bit-exact, output within
2e-2 as max|a-b|/max|b|), and the graph-replayed decode equals the eager one token for token."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    from sparse_transformers_b200.llama_skip import LlamaSkipConfig

    base = dict(vocab=1000, hidden=512, intermediate=2048, layers=3, heads=4, kv_heads=2, head_dim=64,
                predictor_rank=32, density=0.25, max_len=96, dtype=torch.float16)
    base.update(kw)
    return LlamaSkipConfig(**base)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_mlp_calls_match_oracle(dtype):
    from sparse_transformers_b200.llama_skip import LlamaSkipModel
    from stxgpu import ODT, rel_err

    cfg = _cfg(dtype=dtype)
    m = LlamaSkipModel(cfg, "cuda:0", seed=3)
    assert m.layers[0]["sparse"].single_row_fused(1)
    prompt = torch.randint(0, cfg.vocab, (17,), generator=torch.Generator().manual_seed(0)).to("cuda:0")
    m.prefill(prompt)
    m.trace = []
    for _ in range(5):
        m.decode_step(use_graph=False)
    torch.cuda.synchronize()
    assert len(m.trace) == 5 * cfg.layers
    f = lambda t: t.float().cpu().numpy()
    dens = []
    for li, x_pred, x_mlp, out, mask in m.trace:
        L = m.layers[li]
        _, s = orc.predictor(f(x_pred), f(L["A"]), f(L["Bm"]), ODT[dtype])
        _, ref_mask = orc.mask_threshold(s, ODT[dtype], cfg.tau)
        assert np.array_equal(mask.cpu().numpy(), ref_mask)
        idx = np.nonzero(ref_mask)[0]
        dens.append(len(idx) / cfg.intermediate)
        wcat = np.concatenate([f(L["gate"])[idx], f(L["up"])[idx]])
        ref, _ = orc.sparse_mlp(f(x_mlp), wcat, np.ascontiguousarray(f(L["down"]).T[idx]), cfg.act, True)
        assert rel_err(f(out), ref) <= 2e-2
    assert 0.1 < np.mean(dens) < 0.45
    m.close()


def test_graph_decode_equals_eager_decode():
    from sparse_transformers_b200.llama_skip import LlamaSkipModel

    cfg = _cfg()
    prompt = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(1)).to("cuda:0")
    a = LlamaSkipModel(cfg, "cuda:0", seed=5)
    ra = a.generate(prompt, 12, use_graph=False)
    b = LlamaSkipModel(cfg, "cuda:0", seed=5)
    rb = b.generate(prompt, 12, use_graph=True)
    assert torch.equal(ra["tokens"], rb["tokens"])
    assert rb["ttft_s"] > 0 and rb["output_tokens_per_s"] > 0
    # a second generation on the same model (graph reuse, other prompt length)
    prompt2 = torch.randint(0, cfg.vocab, (9,), generator=torch.Generator().manual_seed(2)).to("cuda:0")
    rb2 = b.generate(prompt2, 6, use_graph=True)
    ra2 = a.generate(prompt2, 6, use_graph=False)
    assert torch.equal(ra2["tokens"], rb2["tokens"])
    a.close()
    b.close()


def test_decode_continues_prefill():
    """Decoding token T from the cache equals prefilling T+1 tokens when the MLP is dense in both:
    with a threshold far below every score all neurons are active, so the sparse step is the
    dense MLP and the two paths must agree within half-precision tolerance."""
    from sparse_transformers_b200.llama_skip import LlamaSkipModel

    cfg = _cfg(density=0.999999)
    m = LlamaSkipModel(cfg, "cuda:0", seed=7)
    ids = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(4)).to("cuda:0")
    m.prefill(ids)
    full = m.logits.clone()
    m.prefill(ids[:-1])
    m.token.copy_(ids[-1:])
    m.decode_step(use_graph=False)
    step = m.logits.clone()
    err = (full - step).abs().max() / full.abs().max()
    assert err < 3e-2, float(err)
    m.close()
