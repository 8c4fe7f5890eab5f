"""GPU tier, collected last: the no-allocation whole-layer entry point.

`b200moe_forward_static` serves hosts that cannot allocate device memory at call time (all HBM
already handed to a cache pool, or no allocator reachable from the host language): its scratch is
a fixed array inside the library.  The array is shared by all calls and keeps the previous call's
contents, so the check is made on two calls in a row -- the second one, with different routing and
a different token count, must not be disturbed by what the first left behind -- each compared with
`b200moe_forward` on a caller-provided workspace.  Both paths run the same kernels, so the outputs
must agree bit for bit (well inside the tolerance the other layer tests use); the result is also held
against the CPU oracle, and the status words are read back through `b200moe_static_status`.
"""
import ctypes

import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import _lib, synth
from pyhip_b200.fused_moe import get_plan, moe_forward, pick_block, prepare_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _vp(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _static_forward(shape, x, ids, tw, pw):
    y = torch.full((x.shape[0], x.shape[1]), float("nan"), dtype=torch.bfloat16, device=DEV)
    rc = _lib.lib().b200moe_forward_static(
        ctypes.byref(shape), _vp(x), _vp(ids), _vp(tw), None, _vp(pw.w1_data), _vp(pw.w1_scale), _vp(pw.w2_data),
        _vp(pw.w2_scale), _vp(y), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc, "forward_static")
    return y


def test_static_scratch_matches_workspace_path_on_two_calls_in_a_row():
    H, I, E, K = 288, 160, 16, 4
    w_host = synth.make_weights_mxfp4(E, H, I, seed=31)
    w = tuple(t.to(DEV) for t in w_host)
    pw = prepare_weights(*w)
    for call, T in enumerate((48, 5)):                       # second call: fewer rows than the first left behind
        x_host = synth.make_hidden(T, H, seed=40 + call)
        tw_host, ids_host = synth.make_routing(T, E, K, "zipf", seed=40 + call)
        x, tw, ids = x_host.to(DEV), tw_host.to(DEV), ids_host.to(DEV)
        B = pick_block(T, K, E)
        plan = get_plan(T, K, E, E, H, I, B, 0, 7.0, torch.device(DEV))
        ref = moe_forward(plan, pw, x, tw, ids)
        got = _static_forward(plan.shape, x, ids, tw, pw)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), f"call {call}"
        want = orc.torch_moe_oracle_mxfp4(x_host, *w_host, tw_host, ids_host)
        assert orc.cosine(got.cpu(), want) >= 0.9995 and orc.max_abs(got.cpu(), want) <= 2e-2, f"call {call}"
        status = (ctypes.c_int32 * 16)()
        _lib.check(_lib.lib().b200moe_static_status(ctypes.byref(plan.shape), status,
                                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
                   "static_status")
        torch.cuda.synchronize()
        assert status[0] == 0 and status[2] == 0, list(status)


def test_shape_beyond_the_built_in_scratch_is_refused():
    shape = _lib.Shape(T=8192, K=4, E=128, E_route=128, H=2880, I=2880, B=128, weight_format=0, activation=0,
                       swiglu_limit=7.0, act_terms=0)
    dummy = torch.zeros(16, dtype=torch.uint8, device=DEV)
    rc = _lib.lib().b200moe_forward_static(ctypes.byref(shape), _vp(dummy), _vp(dummy), _vp(dummy), None, _vp(dummy),
                                           _vp(dummy), _vp(dummy), _vp(dummy), _vp(dummy), None)
    assert rc < 0
    assert b"scratch" in _lib.lib().b200moe_last_error()
