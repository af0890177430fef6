"""Test-side helpers that drive the C ABI (include/stx.h) with torch-owned device memory."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from sparse_transformers_b200 import _capi as C

DT = {torch.float32: C.F32, torch.float16: C.F16, torch.bfloat16: C.BF16}
ODT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}  # oracle dtype ids
ACT = {"relu": C.ACT_RELU, "silu": C.ACT_SILU, "gelu_pytorch_tanh": C.ACT_GELU_TANH, "sigmoid": C.ACT_SIGMOID, "gelu": C.ACT_GELU}
DEV = "cuda:0"


def stream():
    return torch.cuda.current_stream().cuda_stream


class _DevBytes:
    """Library-owned device memory exposed through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class Cache:
    """stx_cache_t owner."""

    def __init__(self, gate, up, down, has_gate=True, init_mask="ones", flags=0):
        self.I, self.H = up.shape
        self.dtype = up.dtype
        self.has_gate = has_gate
        self._w = (gate, up, down)
        h = ctypes.c_void_p()
        if isinstance(init_mask, str):
            init = torch.ones(self.I, dtype=torch.bool, device=DEV)
        else:
            init = init_mask
        self._init = init
        C.check(C.lib.stx_cache_create(ctypes.byref(h), self.I, self.H, DT[self.dtype], int(has_gate),
                                       gate.data_ptr() if has_gate else None, up.data_ptr(), down.data_ptr(),
                                       init.data_ptr() if init is not None else None, flags, stream()))
        torch.cuda.synchronize()
        self.h = h

    def close(self):
        if self.h:
            C.lib.stx_cache_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def update(self, mask: torch.Tensor):
        m = mask.to(DEV, torch.bool).contiguous()
        C.check(C.lib.stx_cache_update(self.h, m.data_ptr(), stream()))
        torch.cuda.synchronize()

    def update_bits(self, bits: torch.Tensor):
        C.check(C.lib.stx_cache_update_bits(self.h, bits.data_ptr(), stream()))
        torch.cuda.synchronize()

    def num_active_status(self):
        k = ctypes.c_int64()
        rc = C.lib.stx_cache_num_active(self.h, ctypes.byref(k), stream())
        return rc, k.value

    def active(self) -> np.ndarray:
        buf = np.empty(self.I, np.int32)
        k = ctypes.c_int64()
        C.check(C.lib.stx_cache_active_indices(self.h, buf.ctypes.data_as(ctypes.c_void_p), self.I, ctypes.byref(k), stream()))
        return buf[: k.value].copy()

    def _view(self, ptr, rows):
        n = rows * self.H
        es = torch.empty(0, dtype=self.dtype).element_size()
        if n == 0:
            return torch.empty(0, self.H, dtype=self.dtype, device=DEV)
        raw = torch.as_tensor(_DevBytes(ptr, n * es), device=DEV).clone()
        return raw.view(self.dtype).view(rows, self.H)

    def concat(self) -> torch.Tensor:
        p, rows = ctypes.c_void_p(), ctypes.c_int64()
        C.check(C.lib.stx_cache_concat_weight(self.h, ctypes.byref(p), ctypes.byref(rows), stream()))
        torch.cuda.synchronize()
        return self._view(p.value, rows.value)

    def down_packed(self) -> torch.Tensor:
        p, k = ctypes.c_void_p(), ctypes.c_int64()
        C.check(C.lib.stx_cache_active_down(self.h, ctypes.byref(p), ctypes.byref(k), stream()))
        return self._view(p.value, k.value)

    def stats(self):
        a, r, c = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        C.check(C.lib.stx_cache_last_update_stats(self.h, ctypes.byref(a), ctypes.byref(r), ctypes.byref(c), stream()))
        return a.value, r.value, c.value


def mlp_forward(x, concat, down_packed, act, has_gate=True):
    """-> (out [B,H], combined [B,2K|K]) through stx_sparse_mlp_forward."""
    B, H = x.shape
    K = down_packed.shape[0]
    out = torch.full((B, H), float("nan"), dtype=x.dtype, device=DEV)
    comb = torch.full((B, concat.shape[0]), float("nan"), dtype=x.dtype, device=DEV)
    n = ctypes.c_size_t()
    C.check(C.lib.stx_mlp_scratch_bytes(B, H, K, ctypes.byref(n)))
    scratch = torch.zeros(n.value, dtype=torch.uint8, device=DEV)
    C.check(C.lib.stx_sparse_mlp_forward(x.data_ptr(), B, H, concat.data_ptr(), down_packed.data_ptr(), K, out.data_ptr(),
                                         comb.data_ptr(), ACT[act], int(has_gate), DT[x.dtype], scratch.data_ptr(), stream()))
    torch.cuda.synchronize()
    lead = 256 + (B * H * 4 + 255) // 256 * 256
    assert int(scratch[:lead].view(torch.int32).abs().sum()) == 0, "counter and accumulator must be left zeroed"
    return out, comb


def predict_mask(x, A, Bm, method=C.MASK_THRESHOLD, param=0.0, want_scores=True):
    """-> (mask bool [I] on device, scores [B,I] or None) through stx_predict_mask."""
    B, H = x.shape
    r, I = A.shape[0], Bm.shape[0]
    n = ctypes.c_size_t()
    C.check(C.lib.stx_predict_scratch_bytes(B, I, r, ctypes.byref(n)))
    scratch = torch.zeros(n.value, dtype=torch.uint8, device=DEV)
    bits = torch.zeros((I + 31) // 32, dtype=torch.int32, device=DEV)
    scores = torch.zeros(B, I, dtype=x.dtype, device=DEV) if want_scores else None
    C.check(C.lib.stx_predict_mask(x.data_ptr(), B, H, A.data_ptr(), r, Bm.data_ptr(), I, DT[x.dtype], method, float(param),
                                   bits.data_ptr(), scores.data_ptr() if want_scores else None, scratch.data_ptr(), stream()))
    mask = torch.zeros(I, dtype=torch.bool, device=DEV)
    C.check(C.lib.stx_mask_bits_to_bytes(bits.data_ptr(), I, mask.data_ptr(), stream()))
    torch.cuda.synchronize()
    return mask, scores, bits


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """max |a-b| / max |b| — the 'relative' error the tolerances refer to."""
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(np.abs(b).max(), 1e-30))
