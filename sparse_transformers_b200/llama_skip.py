"""Minimal LlamaSkip host: a Llama-architecture decoder whose MLP runs dense in prefill and
through the sparse layer step (predictor -> mask -> weight cache -> sparse MLP) in decode.

Mirrors the reference's inference model for this path (src/modeling_skip.py:131-266: decoder
layer with the mask computed from the input-layernorm output and the sparse MLP applied to the
post-attention-layernorm output, dense for sequences longer than one token;
src/models/llama/modelling_llama_skip.py:30-66: RMSNorm and layer wiring).  Prefill, the
projections, embedding and lm_head are ordinary torch ops: they are the host around the path.
At decode time the glue between them is the library's own (``native_glue``): residual add +
RMSNorm as one kernel, RoPE + KV-cache append + one-query attention as one kernel and the
output projection as a bulk-copy GEMV, which takes a decoder layer from about two dozen launches
to nine.
Weights are random (N(0, 0.02), seeded): checkpoints are not available offline.

The decode step (all layers, lm_head, greedy argmax, KV-cache append, position advance) is
captured once into a CUDA graph and replayed per token with no host synchronisation; each
layer's cache maintenance runs on a side stream inside the same graph.
"""
from __future__ import annotations

import ctypes
import math
import time
from dataclasses import dataclass
from statistics import NormalDist

import torch
import torch.nn.functional as F

from . import _capi as C
from .layer import SparseLayer


@dataclass
class LlamaSkipConfig:
    vocab: int = 128256
    hidden: int = 3072
    intermediate: int = 8192
    layers: int = 28
    heads: int = 24
    kv_heads: int = 8
    head_dim: int = 128
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    predictor_rank: int = 64
    density: float = 0.20          # active fraction per token the threshold aims at
    act: str = "silu"
    max_len: int = 1024
    dtype: torch.dtype = torch.float16
    wstd: float = 0.02             # initializer_range
    lazy_cache: bool = False
    native_glue: bool = True       # decode: stx_norm_gemv / stx_attn_decode / stx_add_rmsnorm instead of torch ops
    # decode projections: the output projection runs through stx_norm_gemv (measured 6 % more tokens/s than the
    # torch matmul at the 3B shape); add + RMSNorm + q/k/v projection as ONE stx_norm_gemv is available but
    # measured 7 % slower there than stx_add_rmsnorm followed by the torch matmul, so it is off by default
    qkv_proj: str = "torch"        # "torch" | "gemv" (stx_add_rmsnorm, then stx_norm_gemv without norm) | "fused"
    own_wo: bool = True

    @property
    def tau(self) -> float:
        # scores of a unit-RMS input are ~N(0, wstd^4 H r)
        return self.wstd ** 2 * math.sqrt(self.hidden * self.predictor_rank) * NormalDist().inv_cdf(1.0 - self.density)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm of modelling_llama_skip.py:41-47 (normalise in fp32, scale by the weight) as one fused op."""
    return F.rms_norm(x, (x.shape[-1],), w, eps)


_DT = {torch.float32: C.F32, torch.float16: C.F16, torch.bfloat16: C.BF16}


def add_rmsnorm(h: torch.Tensor, a: torch.Tensor | None, w: torch.Tensor, eps: float, x_out: torch.Tensor) -> torch.Tensor:
    """h <- h + a in place (a may be None), x_out <- RMSNorm(h) * w; all [1,H] contiguous on the device."""
    C.check(C.lib.stx_add_rmsnorm(h.data_ptr(), a.data_ptr() if a is not None else None, w.data_ptr(), float(eps),
                                  h.data_ptr(), x_out.data_ptr(), h.numel(), _DT[h.dtype],
                                  torch.cuda.current_stream().cuda_stream))
    return x_out


def norm_gemv(h: torch.Tensor, a: torch.Tensor | None, w_norm: torch.Tensor | None, eps: float, W: torch.Tensor,
              h_out: torch.Tensor | None = None, x_out: torch.Tensor | None = None) -> torch.Tensor:
    """y [1,N] = RMSNorm(h + a) * w_norm times W^T in one kernel (w_norm None: y = h W^T); optionally
    leaves h + a in h_out (not h itself) and the normalised vector in x_out."""
    y = torch.empty(1, W.shape[0], dtype=h.dtype, device=h.device)
    p = lambda t: t.data_ptr() if t is not None else None
    C.check(C.lib.stx_norm_gemv(h.data_ptr(), p(a), p(w_norm), float(eps), W.data_ptr(), y.data_ptr(), p(h_out), p(x_out),
                                h.numel(), W.shape[0], _DT[h.dtype], torch.cuda.current_stream().cuda_stream))
    return y


def attn_workspace(heads: int, head_dim: int, device) -> torch.Tensor:
    """Zeroed scratch of stx_attn_decode for one stream of calls."""
    n = ctypes.c_int64()
    C.check(C.lib.stx_attn_decode_workspace_bytes(heads, head_dim, ctypes.byref(n)))
    return torch.zeros(n.value, dtype=torch.uint8, device=device)


def attn_decode(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor,
                v_cache: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                workspace: torch.Tensor) -> torch.Tensor:
    """RoPE at position pos[0] (device int64), append k/v to the caches [kv_heads, max_len, head_dim] of one layer,
    attend over positions 0..pos; qkv [(heads + 2 kv_heads) * head_dim] -> out [heads * head_dim]."""
    C.check(C.lib.stx_attn_decode(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(), k_cache.data_ptr(),
                                  v_cache.data_ptr(), out.data_ptr(), heads, kv_heads, head_dim, k_cache.shape[1],
                                  _DT[qkv.dtype], workspace.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return out


def rope_tables(cfg: LlamaSkipConfig, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=device, dtype=torch.float32) / cfg.head_dim))
    ang = torch.arange(cfg.max_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos(), emb.sin()  # [max_len, head_dim] fp32


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [heads, T, hd]; cos/sin [T, hd] (rotate-half convention)."""
    h = x.shape[-1] // 2
    rot = torch.cat([-x[..., h:], x[..., :h]], dim=-1)
    return (x.float() * cos + rot.float() * sin).to(x.dtype)


class LlamaSkipModel:
    def __init__(self, cfg: LlamaSkipConfig, device: torch.device | str = "cuda", seed: int = 0):
        self.cfg, self.device = cfg, torch.device(device)
        g = torch.Generator(device=self.device).manual_seed(seed)
        dt = cfg.dtype

        def rn(*shape):
            return (torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * cfg.wstd).to(dt)

        H, I, hd = cfg.hidden, cfg.intermediate, cfg.head_dim
        self.embed = rn(cfg.vocab, H)          # tied with lm_head, as Llama-3.2 does
        self.final_norm = torch.ones(H, dtype=dt, device=self.device)
        self.layers = []
        for _ in range(cfg.layers):
            L = dict(
                wqkv=rn((cfg.heads + 2 * cfg.kv_heads) * hd, H), wo=rn(H, cfg.heads * hd),
                ln1=torch.ones(H, dtype=dt, device=self.device), ln2=torch.ones(H, dtype=dt, device=self.device),
                gate=rn(I, H), up=rn(I, H), down=rn(H, I), A=rn(cfg.predictor_rank, H), Bm=rn(I, cfg.predictor_rank))
            L["sparse"] = SparseLayer(L["gate"], L["up"], L["down"], L["A"], L["Bm"], act=cfg.act, method="threshold",
                                      param=cfg.tau, max_batch=1, alias_gate_up=True, init_all_active=True,
                                      lazy_cache=cfg.lazy_cache)
            self.layers.append(L)
        self.cos, self.sin = rope_tables(cfg, self.device)
        self.k_cache = torch.zeros(cfg.layers, cfg.kv_heads, cfg.max_len, hd, dtype=dt, device=self.device)
        self.v_cache = torch.zeros_like(self.k_cache)
        # decode state, all on the device so that the captured step needs no host input
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)
        self.gen_base = torch.zeros(1, dtype=torch.long, device=self.device)  # prompt length of the current generation
        self.token = torch.zeros(1, dtype=torch.long, device=self.device)
        self.generated = torch.zeros(cfg.max_len, dtype=torch.long, device=self.device)
        self.logits = torch.zeros(cfg.vocab, dtype=torch.float32, device=self.device)
        self._arange = torch.arange(cfg.max_len, device=self.device)
        self._side = torch.cuda.Stream(device=self.device)    # cache index plans
        self._side2 = torch.cuda.Stream(device=self.device)   # cache row copies
        self._attn_ws = attn_workspace(cfg.heads, cfg.head_dim, self.device)
        self._graph = None
        self.trace = None  # when a list: per decode step and layer (x_pred, x_mlp, mlp_out, mask) copies, eager mode only

    # ------------------------------------------------------------------ pieces
    def _attention(self, li: int, x: torch.Tensor, pos0, T: int, decode: bool) -> torch.Tensor:
        cfg, L = self.cfg, self.layers[li]
        hd, nh, nkv = cfg.head_dim, cfg.heads, cfg.kv_heads
        qkv = x @ L["wqkv"].t()                                                  # [T, (nh+2nkv)*hd]
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
        q = q.view(T, nh, hd).transpose(0, 1)
        k = k.view(T, nkv, hd).transpose(0, 1)
        v = v.view(T, nkv, hd).transpose(0, 1)
        if decode:
            idx = self.pos                                                       # device scalar [1]
            cos, sin, mask = self._step_rope                                     # made once per token in _decode_body
            qk = apply_rope(torch.cat([q, k], dim=0), cos, sin)                   # one pass over the q and k heads
            q, k = qk[:nh], qk[nh:]
            self.k_cache[li].index_copy_(1, idx, k)
            self.v_cache[li].index_copy_(1, idx, v)
            o = F.scaled_dot_product_attention(q.unsqueeze(0), self.k_cache[li].unsqueeze(0), self.v_cache[li].unsqueeze(0),
                                               attn_mask=mask, enable_gqa=True)
        else:
            cos, sin = self.cos[pos0:pos0 + T], self.sin[pos0:pos0 + T]
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            self.k_cache[li, :, pos0:pos0 + T] = k
            self.v_cache[li, :, pos0:pos0 + T] = v
            o = F.scaled_dot_product_attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), is_causal=True, enable_gqa=True)
        o = o.squeeze(0).transpose(0, 1).reshape(T, nh * hd)
        return o @ L["wo"].t()

    def _dense_mlp(self, li: int, x: torch.Tensor) -> torch.Tensor:
        L = self.layers[li]
        act = {"silu": F.silu, "relu": F.relu, "gelu_pytorch_tanh": lambda t: F.gelu(t, approximate="tanh")}[self.cfg.act]
        return (act(x @ L["gate"].t()) * (x @ L["up"].t())) @ L["down"].t()

    # ------------------------------------------------------------------ prefill (dense MLP)
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [T] on the device.  Fills the KV cache, returns the greedy next token [1] and leaves
        the decode state (position, token) ready."""
        cfg, T = self.cfg, int(ids.numel())
        h = self.embed.index_select(0, ids)
        for li, L in enumerate(self.layers):
            a = self._attention(li, rms_norm(h, L["ln1"], cfg.rms_eps), 0, T, decode=False)
            h = h + a
            h = h + self._dense_mlp(li, rms_norm(h, L["ln2"], cfg.rms_eps))
        last = rms_norm(h[-1:], self.final_norm, cfg.rms_eps)
        self.logits.copy_((last @ self.embed.t()).float().view(-1))
        nxt = self.logits.argmax().view(1)
        self.token.copy_(nxt)
        self.pos.fill_(T)
        self.generated.zero_()
        self.generated[0:1] = nxt
        self.gen_base.fill_(T)
        return nxt

    # ------------------------------------------------------------------ one decode token
    def _mlp_decode(self, li: int, x_pred: torch.Tensor, x_mlp: torch.Tensor) -> torch.Tensor:
        """Sparse MLP of layer li on the current stream, its cache upkeep on the side streams."""
        main = torch.cuda.current_stream()
        sp: SparseLayer = self.layers[li]["sparse"]
        out = torch.empty_like(x_mlp)
        sp.step_stages(C.STAGE_PREDICT | C.STAGE_MLP, x_pred, x_mlp, out, batch=1)
        self._side.wait_stream(main)                                             # cache upkeep off the critical path
        with torch.cuda.stream(self._side):
            sp.step_stages(C.STAGE_PLAN, batch=1)
        self._side2.wait_stream(self._side)
        with torch.cuda.stream(self._side2):
            sp.step_stages(C.STAGE_COPY, batch=1)
        if self.trace is not None:
            self.trace.append((li, x_pred.clone(), x_mlp.clone(), out.clone(), sp.mask().clone()))
        return out

    def _finish_token(self, last: torch.Tensor) -> None:
        self.logits.copy_((last @ self.embed.t()).float().view(-1))
        nxt = self.logits.argmax().view(1)
        self.pos.add_(1)
        self.token.copy_(nxt)
        self.generated.index_copy_(0, self.pos - self.gen_base, nxt)

    def _decode_body_native(self) -> None:
        cfg = self.cfg
        main = torch.cuda.current_stream()
        h = self.embed.index_select(0, self.token)                              # [1,H]
        h_next = torch.empty_like(h)                                            # the residual stream alternates between the two
        pending = None                                                          # MLP output not yet added to h
        for li, L in enumerate(self.layers):
            # residual add + input RMSNorm + q/k/v projection in one kernel; x_pred is the predictor's input
            x_pred = torch.empty_like(h)
            if cfg.qkv_proj == "fused":
                qkv = norm_gemv(h, pending, L["ln1"], cfg.rms_eps, L["wqkv"], h_out=h_next, x_out=x_pred)
                h, h_next = h_next, h
            elif cfg.qkv_proj == "gemv":
                qkv = norm_gemv(add_rmsnorm(h, pending, L["ln1"], cfg.rms_eps, x_pred), None, None, 0.0, L["wqkv"])
            else:
                qkv = add_rmsnorm(h, pending, L["ln1"], cfg.rms_eps, x_pred) @ L["wqkv"].t()
            o = attn_decode(qkv, self.cos, self.sin, self.pos, self.k_cache[li], self.v_cache[li],
                            torch.empty(1, cfg.heads * cfg.head_dim, dtype=h.dtype, device=h.device),
                            cfg.heads, cfg.kv_heads, cfg.head_dim, self._attn_ws)
            a = norm_gemv(o, None, None, 0.0, L["wo"]) if cfg.own_wo else o @ L["wo"].t()
            x_mlp = add_rmsnorm(h, a, L["ln2"], cfg.rms_eps, torch.empty_like(h))
            pending = self._mlp_decode(li, x_pred, x_mlp)
        main.wait_stream(self._side)
        main.wait_stream(self._side2)
        self._finish_token(add_rmsnorm(h, pending, self.final_norm, cfg.rms_eps, torch.empty_like(h)))

    def _decode_body(self) -> None:
        cfg = self.cfg
        if cfg.native_glue and cfg.head_dim in (64, 128, 256) and cfg.max_len <= 8192:
            return self._decode_body_native()
        main = torch.cuda.current_stream()
        h = self.embed.index_select(0, self.token)                              # [1,H]
        self._step_rope = (self.cos.index_select(0, self.pos), self.sin.index_select(0, self.pos),
                           (self._arange <= self.pos).view(1, 1, 1, cfg.max_len))  # keys 0..pos
        for li, L in enumerate(self.layers):
            x_pred = rms_norm(h, L["ln1"], cfg.rms_eps)                          # the predictor's input
            h = h + self._attention(li, x_pred, None, 1, decode=True)
            x_mlp = rms_norm(h, L["ln2"], cfg.rms_eps).contiguous()
            h = h + self._mlp_decode(li, x_pred.contiguous(), x_mlp)
        main.wait_stream(self._side)
        main.wait_stream(self._side2)
        self._finish_token(rms_norm(h, self.final_norm, cfg.rms_eps))

    @torch.no_grad()
    def decode_step(self, use_graph: bool = True) -> None:
        """Consumes the current token, appends the greedy next one to `generated`."""
        if not use_graph:
            self._decode_body()
            return
        if self._graph is None:
            # warm up eagerly on a side stream (allocator, function attributes), restore the state, capture
            state = (self.pos.clone(), self.token.clone(), self.generated.clone())
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_body()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            self._restore(state)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._decode_body()
            self._graph = g
            self._restore(state)
            # the two passes above advanced every layer's weight cache with this token's mask: replaying
            # the same token reproduces the same mask, which the cache treats as "no change"
        self._graph.replay()

    def _restore(self, state) -> None:
        self.pos.copy_(state[0])
        self.token.copy_(state[1])
        self.generated.copy_(state[2])

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, n_new: int, use_graph: bool = True) -> dict:
        """Greedy decoding; returns tokens and the reference's two timings (benchmark.py:255-260):
        ttft = start -> first token available; output tokens/s = (n_new - 1) / (total - ttft)."""
        assert prompt_ids.numel() + n_new <= self.cfg.max_len
        if use_graph and self._graph is None:
            # build the decode graph outside the timed region, on a throw-away state
            self.prefill(prompt_ids[: min(8, prompt_ids.numel())])
            self.decode_step(True)
            torch.cuda.synchronize()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        self.prefill(prompt_ids)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(n_new - 1):
            self.decode_step(use_graph)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        return {"tokens": self.generated[:n_new].clone(), "ttft_s": t1 - t0, "decode_s": t2 - t1,
                "output_tokens_per_s": (n_new - 1) / (t2 - t1), "total_tokens_per_s": n_new / (t2 - t0)}

    def close(self) -> None:
        self._graph = None
        for L in self.layers:
            L["sparse"].close()
