"""Fused decode step of a sparse layer and a CUDA-graph stack of layers (host side).

Thin Python owners of the C-ABI objects ``stx_cache_t`` / ``stx_layer_t`` / ``stx_stack_t``
(include/stx.h).  torch is used only for device memory and the current stream.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from . import _capi as C

_DT = {torch.float32: C.F32, torch.float16: C.F16, torch.bfloat16: C.BF16}
_ACT = {"relu": C.ACT_RELU, "silu": C.ACT_SILU, "gelu_pytorch_tanh": C.ACT_GELU_TANH, "sigmoid": C.ACT_SIGMOID, "gelu": C.ACT_GELU}
_METHOD = {"naive": C.MASK_THRESHOLD, "threshold": C.MASK_THRESHOLD, "topk": C.MASK_TOPK, "statistical_topk": C.MASK_STATISTICAL}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("sparse_transformers_b200 runs on CUDA only (got a CPU tensor)")


class SparseLayer:
    """Predictor -> mask -> differential weight cache -> sparse MLP for one layer.

    gate/up: [I,H]; down: [H,I]; lora_down (A): [r,H]; lora_up (Bm): [I,r]
    (src/modeling_skip.py:39-40,58-60).  ``method``/``param`` follow compute_binary_mask.
    """

    def __init__(self, gate, up, down, lora_down, lora_up, *, act="silu", method="threshold", param=0.0,
                 max_batch=1, has_gate=True, alias_gate_up=False, init_all_active=True, lazy_cache=False):
        _need_cuda(up, down, lora_down, lora_up)
        self.dtype = up.dtype
        self.device = up.device
        self.I, self.H = up.shape
        self.r = lora_down.shape[0]
        self.max_batch = int(max_batch)
        self.has_gate = bool(has_gate)
        self._keep = [t.contiguous() for t in ((gate, up) if has_gate else (up,))] + [lora_down.contiguous(), lora_up.contiguous()]
        up_c = self._keep[1] if has_gate else self._keep[0]
        gate_c = self._keep[0] if has_gate else None
        self.A, self.Bm = self._keep[-2], self._keep[-1]
        down_c = down.contiguous()
        init = torch.ones(self.I, dtype=torch.bool, device=self.device) if init_all_active else None
        h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            C.check(C.lib.stx_cache_create(ctypes.byref(h), self.I, self.H, _DT[self.dtype], int(has_gate),
                                           gate_c.data_ptr() if has_gate else None, up_c.data_ptr(), down_c.data_ptr(),
                                           init.data_ptr() if init is not None else None,
                                           C.CACHE_ALIAS_GATE_UP if alias_gate_up else 0, _stream()))
            torch.cuda.current_stream().synchronize()
            self._cache = h
            l = ctypes.c_void_p()
            C.check(C.lib.stx_layer_create(ctypes.byref(l), self._cache, self.A.data_ptr(), self.r, self.Bm.data_ptr(),
                                           _METHOD[method], float(param), _ACT[act], self.max_batch))
            self._layer = l
            if lazy_cache:
                C.check(C.lib.stx_layer_set_lazy_cache(self._layer, 1))
        if not alias_gate_up:
            self._keep = [self.A, self.Bm]

    def close(self) -> None:
        if getattr(self, "_layer", None):
            C.lib.stx_layer_destroy(self._layer)
            self._layer = None
        if getattr(self, "_cache", None):
            C.lib.stx_cache_destroy(self._cache)
            self._cache = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_lazy_cache(self, lazy: bool) -> None:
        """Defer (True) or perform every step (False, default) the packed-row copies of the cache;
        takes effect for steps enqueued, and stacks captured, afterwards."""
        C.check(C.lib.stx_layer_set_lazy_cache(self._layer, int(bool(lazy))))

    def set_peer(self, peer) -> None:
        """peer: sharded.PeerExchange (or None).  A step then ends with the sum of the shards'
        outputs over peer memory; every rank must step its shard in the same order."""
        self._peer = peer  # keep it alive as long as the layer points at it
        C.check(C.lib.stx_layer_set_peer(self._layer, peer.handle if peer is not None else None))

    def step(self, x_pred: torch.Tensor, x_mlp: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        x_mlp = x_pred if x_mlp is None else x_mlp
        _need_cuda(x_pred, x_mlp)
        xp = x_pred.reshape(-1, self.H).contiguous()
        xm = x_mlp.reshape(-1, self.H).contiguous()
        B = xp.shape[0]
        if out is None:
            out = torch.empty_like(xm)
        C.check(C.lib.stx_layer_step(self._layer, xp.data_ptr(), xm.data_ptr(), B, out.data_ptr(), _stream()))
        return out

    def step_stages(self, stages: int, x_pred: torch.Tensor | None = None, x_mlp: torch.Tensor | None = None,
                    out: torch.Tensor | None = None, batch: int | None = None) -> None:
        """Run only the given STAGE_* bits of a step on the current stream (tensors must already be
        contiguous [B,H]); used to put the cache maintenance on a side stream."""
        B = batch if batch is not None else (x_pred if x_pred is not None else x_mlp).reshape(-1, self.H).shape[0]
        C.check(C.lib.stx_layer_step_stages(self._layer, x_pred.data_ptr() if x_pred is not None else None,
                                            x_mlp.data_ptr() if x_mlp is not None else None, B,
                                            out.data_ptr() if out is not None else None, _stream(), stages))

    def step_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        """x_host/out_host: CPU tensors [B,H] (pinned for speed); blocks until the result is back."""
        B = x_host.reshape(-1, self.H).shape[0]
        C.check(C.lib.stx_layer_step_host(self._layer, x_host.data_ptr(), B, out_host.data_ptr(), _stream()))
        return out_host

    def single_row_fused(self, batch: int = 1) -> bool:
        """True when a step of `batch` rows runs the predictor's back half, the gather and the MLP as
        one kernel (k_mlp_b1) followed by the sum of its partial outputs (k_partial_reduce)."""
        f = ctypes.c_int()
        C.check(C.lib.stx_layer_single_row_fused(self._layer, batch, ctypes.byref(f)))
        return bool(f.value)

    # ---- introspection (each call synchronises)
    def num_active(self) -> int:
        k = ctypes.c_int64()
        C.check(C.lib.stx_cache_num_active(self._cache, ctypes.byref(k), _stream()))
        return k.value

    def active_indices(self) -> torch.Tensor:
        buf = torch.empty(self.I, dtype=torch.int32)
        k = ctypes.c_int64()
        C.check(C.lib.stx_cache_active_indices(self._cache, buf.data_ptr(), self.I, ctypes.byref(k), _stream()))
        return buf[: k.value].clone()

    def mask(self) -> torch.Tensor:
        p = ctypes.c_void_p()
        C.check(C.lib.stx_layer_mask_bits(self._layer, ctypes.byref(p)))
        out = torch.empty(self.I, dtype=torch.bool, device=self.device)
        C.check(C.lib.stx_mask_bits_to_bytes(p, self.I, out.data_ptr(), _stream()))
        return out

    def _dev_view(self, ptr: int, rows: int) -> torch.Tensor:
        es = torch.empty(0, dtype=self.dtype).element_size()
        n = rows * self.H * es

        class _Bytes:
            __cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (ptr, False), "version": 2}

        if n == 0:
            return torch.empty(0, self.H, dtype=self.dtype, device=self.device)
        return torch.as_tensor(_Bytes(), device=self.device).view(self.dtype).view(rows, self.H)

    def concat_weight(self) -> torch.Tensor:
        """WeightCache.get_concat_weight() of this layer's cache: [2K,H] (a view of cache memory)."""
        p, rows = ctypes.c_void_p(), ctypes.c_int64()
        C.check(C.lib.stx_cache_concat_weight(self._cache, ctypes.byref(p), ctypes.byref(rows), _stream()))
        return self._dev_view(p.value, rows.value)

    def active_down_weight(self) -> torch.Tensor:
        """WeightCache.get_active_down_weight(): [H,K] with strides (1,H) (a view of cache memory)."""
        p, k = ctypes.c_void_p(), ctypes.c_int64()
        C.check(C.lib.stx_cache_active_down(self._cache, ctypes.byref(p), ctypes.byref(k), _stream()))
        return self._dev_view(p.value, k.value).t()

    def update_stats(self) -> tuple[int, int, int]:
        a, r, c = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        C.check(C.lib.stx_cache_last_update_stats(self._cache, ctypes.byref(a), ctypes.byref(r), ctypes.byref(c), _stream()))
        return a.value, r.value, c.value


class SparseStack:
    """L layers fed the same x [B,H], replayed as one CUDA graph; out is [L,B,H]."""

    def __init__(self, layers: Sequence[SparseLayer], batch: int, stages: int = C.STAGE_ALL):
        self.layers = list(layers)
        self.B = int(batch)
        self.L = len(self.layers)
        self.H = self.layers[0].H
        self.dtype = self.layers[0].dtype
        self.device = self.layers[0].device
        arr = (ctypes.c_void_p * self.L)(*[l._layer for l in self.layers])
        h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            C.check(C.lib.stx_stack_create_stages(ctypes.byref(h), arr, self.L, self.B, stages))
        self._stack = h
        n = ctypes.c_int64()
        C.check(C.lib.stx_stack_launches_per_step(self._stack, ctypes.byref(n)))
        self.launches_per_step = n.value

    def close(self) -> None:
        if getattr(self, "_stack", None):
            C.lib.stx_stack_destroy(self._stack)
            self._stack = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def step(self, x: torch.Tensor | None = None, out: torch.Tensor | None = None) -> None:
        """x: device [B,H] or None (reuse the stack's input buffer); out: device [L,B,H] or None."""
        C.check(C.lib.stx_stack_step(self._stack, x.data_ptr() if x is not None else None,
                                     out.data_ptr() if out is not None else None, _stream()))

    def buffers(self) -> tuple[int, int]:
        """Device addresses of the stack's own input [B,H] and output [L,B,H] buffers."""
        a, b = ctypes.c_void_p(), ctypes.c_void_p()
        C.check(C.lib.stx_stack_buffers(self._stack, ctypes.byref(a), ctypes.byref(b)))
        return a.value, b.value

    def step_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        C.check(C.lib.stx_stack_step_host(self._stack, x_host.data_ptr(), out_host.data_ptr(), _stream()))
