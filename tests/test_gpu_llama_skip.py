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


@pytest.mark.parametrize("dtype,hd,heads,kv,pos", [(torch.float16, 128, 6, 2, 300), (torch.bfloat16, 64, 4, 4, 0),
                                                   (torch.float32, 64, 8, 2, 77), (torch.float16, 256, 2, 1, 513),
                                                   (torch.float16, 128, 24, 8, 3), (torch.bfloat16, 128, 24, 8, 639)])
def test_attn_decode_matches_torch(dtype, hd, heads, kv, pos):
    """RoPE + cache append + one-query attention in one kernel against the torch ops it replaces
    (rotate-half RoPE in fp32, scaled_dot_product_attention in fp32 on the rounded operands)."""
    from sparse_transformers_b200.llama_skip import LlamaSkipConfig, apply_rope, attn_decode, attn_workspace, rope_tables
    from stxgpu import rel_err

    dev, max_len = "cuda:0", 640
    cfg = LlamaSkipConfig(heads=heads, kv_heads=kv, head_dim=hd, max_len=max_len)
    cos, sin = rope_tables(cfg, dev)
    g = torch.Generator(device=dev).manual_seed(pos + hd)
    qkv = torch.randn(1, (heads + 2 * kv) * hd, generator=g, device=dev).to(dtype)
    kc = torch.randn(kv, max_len, hd, generator=g, device=dev).to(dtype)
    vc = torch.randn(kv, max_len, hd, generator=g, device=dev).to(dtype)
    kc0, vc0 = kc.clone(), vc.clone()
    p = torch.tensor([pos], dtype=torch.long, device=dev)
    ws = attn_workspace(heads, hd, dev)
    for _ in range(2):   # the second call finds the workspace as the first left it
        kc.copy_(kc0)
        vc.copy_(vc0)
        out = attn_decode(qkv, cos, sin, p, kc, vc, torch.zeros(1, heads * hd, dtype=dtype, device=dev), heads, kv, hd, ws)
    torch.cuda.synchronize()

    q, k, v = qkv.view(-1).split([heads * hd, kv * hd, kv * hd])
    q = apply_rope(q.view(heads, 1, hd), cos[pos:pos + 1], sin[pos:pos + 1])
    k = apply_rope(k.view(kv, 1, hd), cos[pos:pos + 1], sin[pos:pos + 1])
    # the cache: position pos holds the rotated key and the value, everything else is untouched
    assert torch.equal(kc[:, pos], k[:, 0]) and torch.equal(vc[:, pos], v.view(kv, hd))
    keep = torch.ones(max_len, dtype=torch.bool, device=dev)
    keep[pos] = False
    assert torch.equal(kc[:, keep], kc0[:, keep]) and torch.equal(vc[:, keep], vc0[:, keep])
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.float().unsqueeze(0), kc[:, :pos + 1].float().unsqueeze(0), vc[:, :pos + 1].float().unsqueeze(0), enable_gqa=True)
    ref = ref.squeeze(0).transpose(0, 1).reshape(1, heads * hd)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert rel_err(out.float().cpu().numpy(), ref.cpu().numpy()) <= tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("with_add", [True, False])
def test_add_rmsnorm_follows_the_reference_order(dtype, with_add):
    from sparse_transformers_b200.llama_skip import add_rmsnorm

    dev, H, eps = "cuda:0", 3072, 1e-5
    g = torch.Generator(device=dev).manual_seed(4)
    h = torch.randn(1, H, generator=g, device=dev).to(dtype)
    a = torch.randn(1, H, generator=g, device=dev).to(dtype) if with_add else None
    w = (1 + 0.1 * torch.randn(H, generator=g, device=dev)).to(dtype)
    hs = h + a if with_add else h.clone()
    x = hs.float()
    ref = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)).to(dtype) * w   # LlamaSkipRMSNorm
    hh = h.clone()
    out = add_rmsnorm(hh, a, w, eps, torch.empty_like(h))
    torch.cuda.synchronize()
    assert torch.equal(hh, hs)
    ulp = {torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7, torch.float32: 1e-6}[dtype]
    assert ((out.float() - ref.float()).abs() <= 2 * ulp * ref.float().abs() + 1e-7).all()


@pytest.mark.parametrize("qkv_proj,own_wo", [("torch", True), ("fused", True), ("gemv", False), ("torch", False)])
def test_native_glue_matches_torch_glue(qkv_proj, own_wo):
    """The same model decoded with the library's glue kernels and with torch ops: logits agree
    within the half-precision tolerance step after step (same prompt, eager steps)."""
    from sparse_transformers_b200.llama_skip import LlamaSkipModel
    from stxgpu import rel_err

    prompt = torch.randint(0, 1000, (20,), generator=torch.Generator().manual_seed(2)).to("cuda:0")
    a = LlamaSkipModel(_cfg(native_glue=True, qkv_proj=qkv_proj, own_wo=own_wo), "cuda:0", seed=7)
    b = LlamaSkipModel(_cfg(native_glue=False), "cuda:0", seed=7)
    a.prefill(prompt)
    b.prefill(prompt)
    for step in range(6):
        b.token.copy_(a.token)   # keep both on the same token even if an argmax tie breaks differently
        a.decode_step(use_graph=False)
        b.decode_step(use_graph=False)
        torch.cuda.synchronize()
        assert rel_err(a.logits.cpu().numpy(), b.logits.cpu().numpy()) <= 2e-2, step
    a.close()
    b.close()


@pytest.mark.parametrize("dtype,H,N,mode", [(torch.float16, 3072, 5120, "norm+add"), (torch.bfloat16, 512, 200, "norm"),
                                            (torch.float32, 1024, 333, "norm+add"), (torch.float16, 3072, 3072, "plain"),
                                            (torch.bfloat16, 8192, 64, "norm+add"),
                                            # a share of W larger than shared memory: the register-pipelined kernel
                                            (torch.float16, 3072, 6000, "norm+add"), (torch.float32, 2048, 4500, "plain")])
def test_norm_gemv_matches_add_rmsnorm_then_matmul(dtype, H, N, mode):
    from sparse_transformers_b200.llama_skip import add_rmsnorm, norm_gemv
    from stxgpu import rel_err

    dev, eps = "cuda:0", 1e-5
    g = torch.Generator(device=dev).manual_seed(H + N)
    h = torch.randn(1, H, generator=g, device=dev).to(dtype)
    a = torch.randn(1, H, generator=g, device=dev).to(dtype) if mode == "norm+add" else None
    w = (1 + 0.1 * torch.randn(H, generator=g, device=dev)).to(dtype) if mode != "plain" else None
    W = (torch.randn(N, H, generator=g, device=dev) * 0.02).to(dtype)
    if mode == "plain":
        y = norm_gemv(h, None, None, 0.0, W)
        ref = h.float() @ W.float().t()
    else:
        h_out, x_out = torch.empty_like(h), torch.empty_like(h)
        y = norm_gemv(h, a, w, eps, W, h_out=h_out, x_out=x_out)
        h2 = h.clone()
        x_ref = add_rmsnorm(h2, a, w, eps, torch.empty_like(h))
        torch.cuda.synchronize()
        assert torch.equal(h_out, h2)
        ulp = {torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7, torch.float32: 1e-6}[dtype]
        # same arithmetic as the stand-alone kernel up to the order of the sum of squares
        assert ((x_out.float() - x_ref.float()).abs() <= 2 * ulp * x_ref.float().abs() + 1e-7).all()
        ref = x_ref.float() @ W.float().t()
    torch.cuda.synchronize()
    assert rel_err(y.float().cpu().numpy(), ref.cpu().numpy()) <= (1e-5 if dtype == torch.float32 else 4e-3)
