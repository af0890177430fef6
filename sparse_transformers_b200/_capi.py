"""ctypes binding of libstx.so (the C ABI declared in include/stx.h).

The library is the product: if it is missing or fails to load, importing this module raises
— there is no CPU or PyTorch fallback for any entry point.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libstx.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_NO_ACTIVE, ERR_CACHE_INVALID, ERR_ALLOC, ERR_TIMEOUT, ERR_TOO_LARGE = range(9)
F32, F16, BF16 = 0, 1, 2
ACT_RELU, ACT_SILU, ACT_GELU_TANH, ACT_SIGMOID, ACT_GELU = range(5)
MASK_THRESHOLD, MASK_TOPK, MASK_STATISTICAL = range(3)
CACHE_ALIAS_GATE_UP = 1
PEER_HANDLE_BYTES = 64
STAGE_PREDICT, STAGE_PLAN, STAGE_COPY, STAGE_MLP_GATEUP, STAGE_MLP_DOWN, STAGE_MLP, STAGE_ALL = 33, 2, 4, 8, 16, 24, 63
STAGE_PREDICT_T, STAGE_PREDICT_MASK = 1, 32

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int
_u32 = ctypes.c_uint
_f32 = ctypes.c_float
_pp = ctypes.POINTER(ctypes.c_void_p)
_pi64 = ctypes.POINTER(ctypes.c_int64)
_psz = ctypes.POINTER(ctypes.c_size_t)

# name -> (restype, argtypes); mirrors include/stx.h one to one
SIGNATURES = {
    "stx_last_error": (ctypes.c_char_p, []),
    "stx_version": (_i32, []),
    "stx_status_string": (ctypes.c_char_p, [_i32]),
    "stx_act_from_name": (_i32, [ctypes.c_char_p]),
    "stx_cache_bytes": (_i32, [_i64, _i64, _i32, _i32, _u32, _psz]),
    "stx_cache_create": (_i32, [_pp, _i64, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _u32, _vp]),
    "stx_cache_destroy": (_i32, [_vp]),
    "stx_cache_update": (_i32, [_vp, _vp, _vp]),
    "stx_cache_update_bits": (_i32, [_vp, _vp, _vp]),
    "stx_cache_num_active": (_i32, [_vp, _pi64, _vp]),
    "stx_cache_concat_weight": (_i32, [_vp, _pp, _pi64, _vp]),
    "stx_cache_active_down": (_i32, [_vp, _pp, _pi64, _vp]),
    "stx_cache_flush": (_i32, [_vp, _vp]),
    "stx_cache_packed_ptrs": (_i32, [_vp, _pp, _pp, _pp, _pp]),
    "stx_cache_active_indices": (_i32, [_vp, _vp, _i64, _pi64, _vp]),
    "stx_cache_last_update_stats": (_i32, [_vp, _pi64, _pi64, _pi64, _vp]),
    "stx_predict_scratch_bytes": (_i32, [_i64, _i64, _i64, _psz]),
    "stx_predict_mask": (_i32, [_vp, _i64, _i64, _vp, _i64, _vp, _i64, _i32, _i32, _f32, _vp, _vp, _vp, _vp]),
    "stx_mask_bits_to_bytes": (_i32, [_vp, _i64, _vp, _vp]),
    "stx_mask_bytes_to_bits": (_i32, [_vp, _i64, _vp, _vp]),
    "stx_approx_topk_scratch_bytes": (_i32, [_i64, _i64, _psz]),
    "stx_approx_topk_threshold": (_i32, [_vp, _i64, _i64, _i64, _i32, _vp, _vp, _vp]),
    "stx_mlp_scratch_bytes": (_i32, [_i64, _i64, _i64, _psz]),
    "stx_sparse_mlp_forward": (_i32, [_vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "stx_sparse_mlp_forward_noalloc": (_i32, [_vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _i32, _i32, _i32, _vp]),
    "stx_cache_mlp_forward": (_i32, [_vp, _vp, _i64, _vp, _i32, _vp, _vp]),
    "stx_layer_create": (_i32, [_pp, _vp, _vp, _i64, _vp, _i32, _f32, _i32, _i64]),
    "stx_layer_destroy": (_i32, [_vp]),
    "stx_layer_step": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp]),
    "stx_layer_step_stages": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _u32]),
    "stx_layer_set_lazy_cache": (_i32, [_vp, _i32]),
    "stx_layer_mask_bits": (_i32, [_vp, _pp]),
    "stx_layer_single_row_fused": (_i32, [_vp, _i64, ctypes.POINTER(ctypes.c_int)]),
    "stx_layer_step_host": (_i32, [_vp, _vp, _i64, _vp, _vp]),
    "stx_stack_create": (_i32, [_pp, _pp, _i64, _i64]),
    "stx_stack_create_stages": (_i32, [_pp, _pp, _i64, _i64, _u32]),
    "stx_stack_destroy": (_i32, [_vp]),
    "stx_stack_buffers": (_i32, [_vp, _pp, _pp]),
    "stx_stack_step": (_i32, [_vp, _vp, _vp, _vp]),
    "stx_stack_step_host": (_i32, [_vp, _vp, _vp, _vp]),
    "stx_stack_launches_per_step": (_i32, [_vp, _pi64]),
    "stx_peer_create": (_i32, [_pp, _i32, _i32, _i64]),
    "stx_peer_destroy": (_i32, [_vp]),
    "stx_peer_ipc_handle": (_i32, [_vp, _vp]),
    "stx_peer_connect_ipc": (_i32, [_vp, _vp]),
    "stx_peer_connect_ptrs": (_i32, [_vp, _pp]),
    "stx_peer_local_buffer": (_i32, [_vp, _pp]),
    "stx_peer_allreduce": (_i32, [_vp, _vp, _i64, _i32, _vp]),
    "stx_peer_status": (_i32, [_vp, ctypes.POINTER(ctypes.c_int), _vp]),
    "stx_layer_set_peer": (_i32, [_vp, _vp]),
    "stx_attn_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i64, _i32, _vp, _vp]),
    "stx_attn_decode_workspace_bytes": (_i32, [_i32, _i32, ctypes.POINTER(_i64)]),
    "stx_add_rmsnorm": (_i32, [_vp, _vp, _vp, ctypes.c_float, _vp, _vp, _i64, _i32, _vp]),
    "stx_norm_gemv": (_i32, [_vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _vp]),
}


class StxError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def _load() -> ctypes.CDLL:
    if not os.path.isfile(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m sparse_transformers_b200.build` "
            "(needs nvcc with sm_100a support). There is no fallback path.")
    L = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError here means the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    return L


lib = _load()


def check(status: int) -> None:
    if status != OK:
        msg = lib.stx_last_error().decode(errors="replace") or lib.stx_status_string(status).decode()
        raise StxError(status, msg)


def last_error() -> str:
    return lib.stx_last_error().decode(errors="replace")
