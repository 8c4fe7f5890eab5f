"""Dense block-scaled linear layers on the MoE main loop.

The reference carries separate dense kernels for the projections either side of the MoE layer
(src/contrib/gemm_a4w4.py driven by tests/contrib/gemm/test_a4w4_mxfp4.py:22-58, and the FP8
block-scale GEMM of tests/contrib/gemm/test_a8w8_f32_blockscale.py:114-191).  Here a dense
`y = x @ W^T` is the down-projection grouped GEMM run with a single expert: every row sorts to
expert 0 in token order (the sort is stable), the activation quantiser gathers nothing, and the
rows the GEMM stores in sorted order are already the result.  Same kernels, same formats, same
C ABI calls (`b200moe_sort_align`, `b200moe_quant_rows[_e4m3]`, `b200moe_down`).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .fused_moe import _capacity, _ptr, _stream, get_plan, pick_block


class PreparedLinear:
    """One weight matrix [N, K] in the form the down GEMM consumes (the weights in place; MXFP4
    scales regrouped once, FP8 block scales in place)."""

    def __init__(self, weight, weight_scale, weight_format):
        if not weight.is_cuda:
            raise ValueError("weights must be CUDA tensors")
        self.fmt = weight_format
        if weight_format == _lib.W_MXFP4:
            w = (weight.view(torch.uint8) if weight.dtype != torch.uint8 else weight).contiguous()
            s = weight_scale.view(torch.uint8) if weight_scale.dtype != torch.uint8 else weight_scale
            self.N, self.K = w.shape[0], w.shape[1] * 2
            if s.numel() != self.N * (self.K // 32):
                raise ValueError("weight_scale must hold one E8M0 byte per 32 weights")
            if int(s.max()) > 254:
                raise ValueError("E8M0 scale 0xFF (NaN) is not a valid weight scale")
            shape = _lib.Shape(T=0, K=1, E=1, E_route=1, H=self.N, I=self.K, B=32, weight_format=_lib.W_MXFP4,
                               activation=0, swiglu_limit=0.0, act_terms=0, combine_mode=0, act_quant=0, doweight_stage1=0)
            sb = ctypes.c_int64()
            L = _lib.lib()
            _lib.check(L.b200moe_prepared_scale_bytes(ctypes.byref(shape), 2, ctypes.byref(sb)), "prepared_scale_bytes")
            scale = torch.empty(sb.value, dtype=torch.uint8, device=w.device)
            _lib.check(L.b200moe_prepare_scales(ctypes.byref(shape), 2, _ptr(s.contiguous()), _ptr(scale), _stream()),
                       "prepare_scales")
            self.w2_data, self.w2_scale = w, scale
        else:
            self.N, self.K = weight.shape
            if self.N % 128 or self.K % 128:
                raise ValueError("per_128x128 weights need N and K to be multiples of 128")
            if weight_scale.numel() != (self.N // 128) * (self.K // 128):
                raise ValueError("weight_scale must hold one fp32 scale per 128x128 block")
            self.w2_data = weight.contiguous().view(torch.uint8)
            self.w2_scale = weight_scale.float().contiguous()


_prepared: dict = {}          # insertion-ordered: least recently used first
_PREPARED_ENTRIES = 16


def _prepare(weight, weight_scale, fmt) -> PreparedLinear:
    key = (weight.data_ptr(), weight_scale.data_ptr(), tuple(weight.shape), fmt, weight_scale._version)
    hit = _prepared.pop(key, None)
    if hit is None:
        while len(_prepared) >= _PREPARED_ENTRIES:
            _prepared.pop(next(iter(_prepared)))
        hit = (PreparedLinear(weight, weight_scale, fmt), (weight, weight_scale))
    _prepared[key] = hit
    return hit[0]


def _linear(x, weight, weight_scale, fmt, act_terms, block_size_M):
    if not x.is_cuda:
        raise RuntimeError("block-scaled linear runs on a CUDA device only (sm_100a); there is no CPU path")
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise TypeError("x must be a bfloat16 matrix [M, K]")
    pl = _prepare(weight, weight_scale, fmt)
    M, K = x.shape
    if K != pl.K:
        raise ValueError(f"x has {K} columns, the weight {pl.K}")
    if M == 0:
        return torch.empty(0, pl.N, dtype=torch.bfloat16, device=x.device)
    B = int(block_size_M) if block_size_M else pick_block(M, 1, 1, fmt)
    M_cap = _capacity(M)
    plan = get_plan(M_cap, 1, 1, 1, pl.N, pl.K, B, _lib.ACT_SILU, 0.0, x.device, act_terms, fmt)
    plan.set_tokens(M)
    ids = torch.zeros(M, 1, dtype=torch.int32, device=x.device)
    ones = torch.ones(M, 1, dtype=torch.float32, device=x.device)
    plan.sort(ids, ones)
    plan.quant_hidden(x.contiguous())            # rows [M, 1, K]: pair (token, 0) = row token
    plan.down(pl)
    rows = plan.region("out2", plan.ws.max_rows * pl.N * 2, torch.bfloat16).view(plan.ws.max_rows, pl.N)
    return rows[:M].clone()


def linear_mxfp4(x, weight, weight_scale, act_terms: int = 0, block_size_M=None):
    """bf16 x [M, K] times MXFP4 weight [N, K/2] (E2M1 pairs, low nibble = even element) with E8M0
    scales [N, K/32] -> bf16 [M, N].  Stands where the reference calls gemm_a4w4
    (tests/contrib/gemm/test_a4w4_mxfp4.py:22-58); activations travel as `act_terms` packed-FP4 terms
    (default 3) instead of one, so the result matches a bf16-activation product."""
    return _linear(x, weight, weight_scale, _lib.W_MXFP4, act_terms, block_size_M)


def linear_fp8_128x128(x, weight, weight_scale, block_size_M=None):
    """bf16 x [M, K] times e4m3 weight [N, K] with one fp32 scale per 128x128 block [N/128, K/128]
    -> bf16 [M, N] (the reference's block-scale FP8 GEMM, tests/contrib/gemm/test_a8w8_f32_blockscale.py:114-191)."""
    return _linear(x, weight, weight_scale, _lib.W_FP8_128, 0, block_size_M)
