"""ctypes front-end of the C oracle (oracle/stx_oracle.c) plus a torch restatement of the
Python half of the reference path.  TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Parity status: PINNED.  tests/test_oracle_vs_reference.py checks every function here against
the reference's own CPU operator compiled unmodified (oracle/_ref, see oracle/build_ref.py)
and tests/test_golden.py against vectors that operator generated (tests/golden/).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(HERE, "libstx_oracle.so")
_SRC = os.path.join(HERE, "stx_oracle.c")

F32, F16, BF16 = 0, 1, 2
ACT = {"relu": 0, "silu": 1, "gelu_pytorch_tanh": 2, "sigmoid": 3, "gelu": 4}

_lib = None


def build(force: bool = False) -> str:
    if force or not os.path.isfile(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off",
                               _SRC, "-o", _SO, "-lm"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.orc_cache_new.restype = vp
        L.orc_cache_new.argtypes = [i32]
        L.orc_cache_free.argtypes = [vp]
        L.orc_cache_update.restype = i32
        L.orc_cache_update.argtypes = [vp, vp, vp, vp]
        L.orc_cache_k.restype = i32
        L.orc_cache_k.argtypes = [vp]
        L.orc_cache_valid.restype = i32
        L.orc_cache_valid.argtypes = [vp]
        L.orc_cache_active.restype = ctypes.POINTER(ctypes.c_int32)
        L.orc_cache_active.argtypes = [vp]
        L.orc_gather_rows.argtypes = [vp, vp, i32, ctypes.c_size_t, vp]
        L.orc_predictor.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]
        L.orc_mask_threshold.argtypes = [vp, i32, i32, i32, f32, vp, vp]
        L.orc_mask_statistical.argtypes = [vp, i32, i32, i32, f32, vp, vp, vp]
        L.orc_mask_topk.argtypes = [vp, i32, i32, i32, vp, vp]
        L.orc_sparse_mlp.argtypes = [vp, i32, i32, vp, vp, i32, i32, i32, vp, vp]
        L.orc_approx_topk_threshold.argtypes = [vp, i32, i32, i32, vp]
        L.orc_round.restype = f32
        L.orc_round.argtypes = [f32, i32]
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


class NoActiveWeights(RuntimeError):
    """The reference throws std::runtime_error("No active weights") (weight_cache.h:117-118)."""


class OracleCache:
    """Index bookkeeping of WeightCache (weight_cache.h:229-359); see orc_cache_update."""

    def __init__(self, I: int):
        self.I = int(I)
        self._h = lib().orc_cache_new(self.I)
        self.last_added = 0
        self.last_removed = 0

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_cache_free(self._h)
            self._h = None

    def update(self, mask) -> int:
        m = np.ascontiguousarray(np.asarray(mask).astype(np.uint8))
        assert m.shape == (self.I,)
        na, nr = ctypes.c_int32(0), ctypes.c_int32(0)
        k = lib().orc_cache_update(self._h, _p(m), ctypes.byref(na), ctypes.byref(nr))
        self.last_added, self.last_removed = na.value, nr.value
        if k < 0:
            raise NoActiveWeights("No active weights")
        return k

    @property
    def K(self) -> int:
        return lib().orc_cache_k(self._h)

    @property
    def valid(self) -> bool:
        return bool(lib().orc_cache_valid(self._h))

    @property
    def active(self) -> np.ndarray:
        k = self.K
        return np.ctypeslib.as_array(lib().orc_cache_active(self._h), shape=(max(k, 1),))[:k].copy()

    def gather(self, pool: np.ndarray) -> np.ndarray:
        """Packed rows pool[active] (pool: [I, H] of any dtype)."""
        pool = np.ascontiguousarray(pool)
        act = np.ascontiguousarray(self.active.astype(np.int32))
        out = np.empty((len(act),) + pool.shape[1:], dtype=pool.dtype)
        lib().orc_gather_rows(_p(pool), _p(act), len(act), pool.strides[0], _p(out))
        return out


def predictor(x, A, Bm, dtype: int):
    """(t [B,r], scores [B,I]) as fp32 arrays holding dtype-rounded values; see orc_predictor."""
    x, A, Bm = _f32(x), _f32(A), _f32(Bm)
    B, H = x.shape
    r, I = A.shape[0], Bm.shape[0]
    assert A.shape == (r, H) and Bm.shape == (I, r)
    t = np.empty((B, r), np.float32)
    s = np.empty((B, I), np.float32)
    lib().orc_predictor(_p(x), _p(A), _p(Bm), B, H, r, I, dtype, _p(t), _p(s))
    return t, s


def mask_threshold(scores, dtype: int, tau: float):
    s = _f32(scores)
    B, I = s.shape
    rows = np.empty((B, I), np.uint8)
    uni = np.empty((I,), np.uint8)
    lib().orc_mask_threshold(_p(s), B, I, dtype, float(tau), _p(rows), _p(uni))
    return rows.astype(bool), uni.astype(bool)


def mask_statistical(scores, dtype: int, z: float):
    s = _f32(scores)
    B, I = s.shape
    rows = np.empty((B, I), np.uint8)
    uni = np.empty((I,), np.uint8)
    cut = np.empty((B,), np.float32)
    lib().orc_mask_statistical(_p(s), B, I, dtype, float(z), _p(rows), _p(uni), _p(cut))
    return rows.astype(bool), uni.astype(bool), cut


def mask_topk(scores, k: int):
    s = _f32(scores)
    B, I = s.shape
    rows = np.empty((B, I), np.uint8)
    uni = np.empty((I,), np.uint8)
    lib().orc_mask_topk(_p(s), B, I, int(k), _p(rows), _p(uni))
    return rows.astype(bool), uni.astype(bool)


def sparse_mlp(x, wcat, wdown_packed, act: str, has_gate: bool = True):
    """(out [B,H], combined [B,2K|K]); wdown_packed is [K,H] (row j = column j of [H,K])."""
    x, wcat, wd = _f32(x), _f32(wcat), _f32(wdown_packed)
    B, H = x.shape
    K = wd.shape[0]
    assert wcat.shape == ((2 * K if has_gate else K), H), (wcat.shape, K, H)
    out = np.empty((B, H), np.float32)
    comb = np.empty((B, 2 * K if has_gate else K), np.float32)
    lib().orc_sparse_mlp(_p(x), B, H, _p(wcat), _p(wd), K, ACT[act], int(has_gate), _p(out), _p(comb))
    return out, comb


def approx_topk_threshold(scores, k: int):
    s = _f32(scores)
    B, I = s.shape
    thr = np.empty((B,), np.float32)
    lib().orc_approx_topk_threshold(_p(s), B, I, int(k), _p(thr))
    return thr


def round_to(a, dtype: int) -> np.ndarray:
    a = _f32(a)
    if dtype == F32:
        return a
    L = lib()
    flat = a.ravel()
    return np.array([L.orc_round(float(v), dtype) for v in flat], np.float32).reshape(a.shape)
