"""The C-ABI library loads without a GPU and exports every symbol include/stx.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "stx.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(stx_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("stx_cache_create", "stx_cache_update", "stx_cache_concat_weight", "stx_cache_active_down",
                 "stx_predict_mask", "stx_sparse_mlp_forward", "stx_layer_step", "stx_stack_step"):
        assert must in syms


def test_library_exports_all_declared_symbols():
    lib = ctypes.CDLL(os.path.join(ROOT, "sparse_transformers_b200", "libstx.so"))
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in stx.h but not exported: {missing}"


def test_binding_table_matches_header():
    from sparse_transformers_b200 import _capi

    assert sorted(_capi.SIGNATURES) == declared_symbols()
    assert _capi.lib.stx_version() == 100
    assert _capi.lib.stx_act_from_name(b"silu") == _capi.ACT_SILU
    assert _capi.lib.stx_act_from_name(b"nope") == -1
    assert _capi.lib.stx_status_string(4) == b"No active weights"


def test_argument_checks_need_no_gpu():
    from sparse_transformers_b200 import _capi as C

    n = ctypes.c_size_t()
    assert C.lib.stx_cache_bytes(8192, 3072, C.F16, 1, 0, ctypes.byref(n)) == C.OK
    assert n.value >= 6 * 8192 * 3072 * 2
    assert C.lib.stx_mlp_scratch_bytes(1, 3072, 8192, ctypes.byref(n)) == C.OK and n.value >= 3072 * 4
    assert C.lib.stx_cache_update(None, None, None) == C.ERR_INVALID_ARG
    assert b"null" in C.lib.stx_last_error()
    h = ctypes.c_void_p()
    assert C.lib.stx_cache_create(ctypes.byref(h), 0, 8, C.F32, 1, None, None, None, None, 0, None) == C.ERR_INVALID_ARG


def test_torch_shim_registers_reference_names():
    import torch

    import sparse_transformers_b200 as stb

    assert "sparse_mlp.WeightCache" in str(torch.classes.sparse_mlp.WeightCache.__doc__ or "") or stb.WeightCache is not None
    assert hasattr(torch.classes.sparse_mlp, "WeightCache")
    schema = str(torch.ops.sparse_mlp.forward.default._schema)
    assert schema.startswith("sparse_mlp::forward(Tensor _0, Tensor _1, Tensor _2, Tensor _3, Tensor _4, str _5, bool _6) -> Tensor")
    # no CPU fallback: a CPU call must fail loudly
    import pytest

    with pytest.raises(RuntimeError, match="CUDA only"):
        stb.sparse_mlp_forward(torch.zeros(1, 8), torch.zeros(4, 8), torch.zeros(8, 2), torch.zeros(1, 8), torch.zeros(1, 4), "silu")
    with pytest.raises(RuntimeError, match="CUDA"):
        stb.WeightCache(torch.ones(4, dtype=torch.bool), 8, torch.zeros(4, 8), torch.zeros(4, 8), torch.zeros(8, 4), True)
