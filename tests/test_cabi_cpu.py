"""CPU tier: the C-ABI library builds, loads, exports every symbol the header declares, and
rejects bad arguments with an error code before touching a device."""
import ctypes
import pathlib
import re

import pytest

from pyhip_b200 import _lib

HEADER = pathlib.Path(__file__).resolve().parents[1] / "include" / "b200moe.h"


@pytest.fixture(scope="module")
def L():
    _lib.build()
    return _lib.lib()


def test_every_declared_symbol_is_exported(L):
    text = HEADER.read_text()
    declared = set(re.findall(r"\b(b200moe_[a-z_0-9]+)\s*\(", text))
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(L, name), name
    assert L.b200moe_version() == 3


def test_struct_sizes_match_header():
    assert ctypes.sizeof(_lib.Shape) == 60
    assert ctypes.sizeof(_lib.Io) == 12 * 8
    assert ctypes.sizeof(_lib.Workspace) == 14 * 8


def test_workspace_layout_arithmetic(L):
    s = _lib.Shape(T=64, K=4, E=128, E_route=128, H=2880, I=2880, B=32, weight_format=0, activation=0,
                   swiglu_limit=7.0, act_terms=0)
    ws = _lib.workspace_layout(s)
    assert ws.max_rows == (64 * 4 + 128 * 31 + 31) // 32 * 32
    offs = [getattr(ws, n) for n in _lib._WS_FIELDS if n.startswith("off_")]
    assert offs == sorted(offs) and all(o % 1024 == 0 for o in offs)
    assert ws.total_bytes > offs[-1]
    assert ws.off_xsf - ws.off_xq >= 3 * ws.max_rows * 3072 // 2


def test_workspace_layout_for_bf16_weights(L):
    """Unquantised weights: the row regions hold bf16 rows in sorted order (2 bytes per element), no scale regions."""
    s = _lib.Shape(T=64, K=4, E=128, E_route=128, H=2880, I=2880, B=32, weight_format=_lib.W_BF16, activation=0,
                   swiglu_limit=7.0, act_terms=0)
    ws = _lib.workspace_layout(s)
    assert ws.off_xsf - ws.off_xq >= ws.max_rows * 2880 * 2
    assert ws.off_hsf - ws.off_hq >= ws.max_rows * 2880 * 2
    assert ws.off_hq - ws.off_xsf == 1024 and ws.off_out2 - ws.off_hsf == 1024
    s.act_quant = 1
    assert L.b200moe_workspace_layout(ctypes.byref(s), ctypes.byref(_lib.Workspace())) < 0


@pytest.mark.parametrize("field,value", [("B", 40), ("H", 100), ("I", 0), ("K", 0), ("T", 1 << 24),
                                         ("weight_format", 7), ("activation", 9), ("E_route", 4), ("act_terms", 5),
                                         ("combine_mode", 2), ("act_quant", 2), ("doweight_stage1", 2), ("cta_pairs", 3)])
def test_bad_shapes_are_rejected(L, field, value):
    s = _lib.Shape(T=8, K=2, E=8, E_route=8, H=256, I=128, B=32, weight_format=0, activation=0, swiglu_limit=7.0, act_terms=0)
    setattr(s, field, value)
    ws = _lib.Workspace()
    rc = L.b200moe_workspace_layout(ctypes.byref(s), ctypes.byref(ws))
    assert rc < 0
    assert L.b200moe_last_error()
    with pytest.raises(_lib.B200MoEError):
        _lib.workspace_layout(s)


def test_null_pointers_are_rejected_without_launch(L):
    s = _lib.Shape(T=8, K=2, E=8, E_route=8, H=256, I=128, B=32, weight_format=0, activation=0, swiglu_limit=7.0, act_terms=0)
    ws = _lib.workspace_layout(s)
    assert L.b200moe_gateup(ctypes.byref(s), ctypes.byref(ws), None, None, None, None, None, None) < 0
    assert L.b200moe_down(ctypes.byref(s), ctypes.byref(ws), None, None, None, None, None, None) < 0
    assert L.b200moe_forward_ex(ctypes.byref(s), ctypes.byref(ws), None, None, None) < 0
    assert L.b200moe_static_status(ctypes.byref(s), None, None) < 0
    assert L.b200moe_forward(ctypes.byref(s), ctypes.byref(ws), None, None, None, None, None, None, None, None,
                             None, None, None) < 0
    assert L.b200moe_sort_align(None, None, 4, 2, 8, 32, None, None, None, None, None, None, None) < 0
    assert L.b200moe_debug_probe(1, None, None, None) < 0
    sb = ctypes.c_int64()
    assert L.b200moe_prepared_scale_bytes(ctypes.byref(s), 3, ctypes.byref(sb)) < 0
    assert L.b200moe_prepared_scale_bytes(ctypes.byref(s), 1, ctypes.byref(sb)) == 0
    assert sb.value == 8 * 2 * 1 * 2 * 512


def test_workspace_too_small_for_the_token_count_is_rejected(L):
    """A workspace laid out for more tokens than a call carries is accepted; a smaller one is an
    argument error raised before anything is launched (dummy non-null pointers are never touched)."""
    small = _lib.Shape(T=8, K=2, E=8, E_route=8, H=256, I=128, B=32, weight_format=0, activation=0, swiglu_limit=7.0, act_terms=0)
    big = _lib.Shape(T=4096, K=2, E=8, E_route=8, H=256, I=128, B=32, weight_format=0, activation=0, swiglu_limit=7.0, act_terms=0)
    ws_small = _lib.workspace_layout(small)
    p = ctypes.c_void_p(4096)
    rc = L.b200moe_forward(ctypes.byref(big), ctypes.byref(ws_small), p, p, p, p, None, p, p, p, p, p, None)
    assert rc < 0 and b"workspace holds" in L.b200moe_last_error()
    # enough rows but laid out for another block size / routing space: the index and scale regions are too small
    other = _lib.Shape(T=64, K=2, E=8, E_route=8, H=256, I=128, B=128, weight_format=0, activation=0, swiglu_limit=7.0, act_terms=0)
    ws_other = _lib.workspace_layout(other)
    use = _lib.Shape(T=500, K=2, E=8, E_route=8, H=256, I=128, B=16, weight_format=0, activation=0, swiglu_limit=7.0, act_terms=0)
    assert ws_other.max_rows >= _lib.workspace_layout(use).max_rows
    rc = L.b200moe_forward(ctypes.byref(use), ctypes.byref(ws_other), p, p, p, p, None, p, p, p, p, p, None)
    assert rc < 0 and b"workspace region" in L.b200moe_last_error()
    assert L.b200moe_gather_sum(None, None, 4, 2, 64, None, None) < 0
    assert L.b200moe_gather_sum(None, None, 0, 2, 64, None, None) == 0      # empty batch: nothing to do


def test_python_surface_fails_loudly_without_cuda():
    import torch
    from pyhip_b200 import QuantType, fused_moe
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        fused_moe(x, None, None, None, None, quant_type=QuantType.per_1x32)
