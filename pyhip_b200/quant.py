"""Host-side data formats of the quantised MoE layer: MXFP4 (E2M1 codes + E8M0/32 scales),
FP8-e4m3 with 128x128 block scales, and their packers.

These play the part that ``aiter.get_torch_quant(QuantType.per_1x32)`` and
``aiter.ops.quant.pertoken_quant`` play for the reference's tests
(tests/contrib/moe/test_moe.py:155-189 and :201-260): turning float weights into the packed
tensors the operator consumes.  They are plain torch ops and run on any device.

Encodings (archive/ck_tile/ck_tile/core/numeric/pk_fp4.hpp:122-129,
e8m0.hpp:12-24):
  * E2M1 code ``s e e m`` -> {0, .5, 1, 1.5, 2, 3, 4, 6} with sign bit 3.
  * two codes per byte, LOW nibble = even element.
  * E8M0 byte b -> 2**(b-127); 0xFF is NaN and is never produced here.
"""
from __future__ import annotations

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
MX_BLOCK = 32
FP8_BLOCK = 128
FP8_MAX = 448.0


def e2m1_encode(v: torch.Tensor) -> torch.Tensor:
    """Round float values to E2M1 codes (uint8 in [0,15]): round-to-nearest-even on the
    code grid, saturating at +-6 (mxfp_convert.hpp:60-216 semantics)."""
    a = v.abs().float()
    # midpoints between neighbouring magnitudes; a tie goes to the even code
    code = (a > 0.25).to(torch.uint8)
    code += (a >= 0.75).to(torch.uint8)
    code += (a > 1.25).to(torch.uint8)
    code += (a >= 1.75).to(torch.uint8)
    code += (a > 2.5).to(torch.uint8)
    code += (a >= 3.5).to(torch.uint8)
    code += (a > 5.0).to(torch.uint8)
    sign = (torch.signbit(v) & (code > 0)).to(torch.uint8) << 3
    return code | sign


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUES + tuple(-x for x in E2M1_VALUES), dtype=torch.float32,
                       device=code.device)
    return lut[code.long()]


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] uint8 codes -> [..., K/2] bytes, low nibble = even element."""
    assert codes.shape[-1] % 2 == 0
    c = codes.reshape(*codes.shape[:-1], codes.shape[-1] // 2, 2)
    return (c[..., 0] | (c[..., 1] << 4)).contiguous()


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    lo = packed & 0xF
    hi = packed >> 4
    return torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def e8m0_to_float(b: torch.Tensor) -> torch.Tensor:
    """uint8 exponent byte -> float32 power of two (b=0 gives 2**-127, a subnormal)."""
    return torch.ldexp(torch.ones(b.shape, dtype=torch.float32, device=b.device), b.int() - 127)


def quantize_mxfp4(w: torch.Tensor):
    """Quantise along the last axis in blocks of 32: shared scale 2**floor(log2(absmax/6)),
    elements rounded to E2M1 with saturation (the rule the tiny benchmark configuration states: floor(log2(absmax/6))).

    Returns (packed uint8 [..., K/2], scale uint8 [..., K/32])."""
    K = w.shape[-1]
    assert K % MX_BLOCK == 0, "K must be a multiple of 32"
    blk = w.float().reshape(*w.shape[:-1], K // MX_BLOCK, MX_BLOCK)
    amax = blk.abs().amax(dim=-1)
    # floor(log2(amax/6)) computed exactly from the float exponent of amax/6
    _, ex = torch.frexp(amax / 6.0)           # amax/6 = m * 2**ex, m in [0.5,1)
    e = (ex - 1).clamp(-127, 127)
    e = torch.where(amax > 0, e, torch.zeros_like(e))   # all-zero block: scale 1.0
    scale = torch.ldexp(torch.ones_like(amax), e)
    codes = e2m1_encode(blk / scale.unsqueeze(-1)).reshape(*w.shape)
    return pack_nibbles(codes), (e + 127).to(torch.uint8)


def dequantize_mxfp4(packed: torch.Tensor, scale: torch.Tensor,
                     dtype=torch.bfloat16) -> torch.Tensor:
    """value * 2**(e-127) per 32 along K, cast to ``dtype``
    (tests/contrib/moe/test_moe.py:164-166)."""
    vals = e2m1_decode(unpack_nibbles(packed))
    K = vals.shape[-1]
    sc = e8m0_to_float(scale)
    out = vals.reshape(*vals.shape[:-1], K // MX_BLOCK, MX_BLOCK) * sc.unsqueeze(-1)
    return out.reshape(*vals.shape).to(dtype)


def quantize_fp8_128x128(w: torch.Tensor):
    """[E, N, K] float -> e4m3 weights + fp32 scale per 128x128 block, scale = amax/448
    (the shape of tests/contrib/moe/test_moe.py:202-229)."""
    E, N, K = w.shape
    assert N % FP8_BLOCK == 0 and K % FP8_BLOCK == 0
    blk = w.float().reshape(E, N // FP8_BLOCK, FP8_BLOCK, K // FP8_BLOCK, FP8_BLOCK)
    amax = blk.abs().amax(dim=(2, 4))
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (blk / scale[:, :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(E, N, K), scale


def dequantize_fp8_128x128(q: torch.Tensor, scale: torch.Tensor,
                           dtype=torch.bfloat16) -> torch.Tensor:
    """tests/contrib/moe/test_moe.py:243-245."""
    E, N, K = q.shape
    blk = q.to(dtype).reshape(E, N // FP8_BLOCK, FP8_BLOCK, K // FP8_BLOCK, FP8_BLOCK)
    out = (blk * scale.reshape(E, N // FP8_BLOCK, 1, K // FP8_BLOCK, 1)).to(dtype)
    return out.reshape(E, N, K)


def quantize_fp8_per_row(w: torch.Tensor):
    """[E, N, K] float -> e4m3 weights + one fp32 scale per output row [E, N], scale = amax_row / 448: the
    per-token-per-channel weight format (tests/contrib/moe/test_moe.py:123-128; the arithmetic of the per-tensor
    rule at :130-137 applied row by row)."""
    amax = w.float().abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (w.float() / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def quantize_fp8_per_tensor(w: torch.Tensor):
    """[E, N, K] float -> e4m3 weights + one fp32 scale per expert [E] (tests/contrib/moe/test_moe.py:130-137)."""
    scale = w.float().abs().amax(dim=(1, 2)) / FP8_MAX
    scale = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = (w.float() / scale.view(-1, 1, 1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale
