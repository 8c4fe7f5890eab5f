"""GPU tier: dense block-scaled linear layers on the MoE main loop (single-expert down GEMM), against
the dequantise-then-matmul product the reference's dense-GEMM tests compare with
(tests/contrib/gemm/test_a4w4_mxfp4.py:60-88, tests/contrib/gemm/test_a8w8_f32_blockscale.py:114-191)."""
import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import quant, synth
from pyhip_b200.linear import linear_fp8_128x128, linear_mxfp4

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _check(y, ref, what):
    cos, mx = orc.cosine(y, ref), orc.max_abs(y, ref)
    bound = 2e-2 * max(1.0, float(ref.float().abs().max()))      # one bf16 step at the output's magnitude
    assert cos >= 0.9995 and mx <= bound, f"{what}: cosine {cos:.6f} max_abs {mx:.3e} bound {bound:.3e}"


@pytest.mark.parametrize("M,N,K", [(1, 512, 512), (33, 288, 160), (300, 2880, 2880), (1000, 384, 1024)])
def test_linear_mxfp4_matches_dequantised_product(M, N, K):
    g = torch.Generator().manual_seed(M + N)
    w = torch.randn(N, K, generator=g) * 0.02
    w_q, w_s = quant.quantize_mxfp4(w)
    x = synth.make_hidden(M, K, seed=M)
    ref = (x.float() @ orc.dequant_mxfp4(w_q, w_s, torch.bfloat16).float().t()).to(torch.bfloat16)
    y = linear_mxfp4(x.to(DEV), w_q.to(DEV), w_s.to(DEV)).cpu()
    assert y.shape == (M, N)
    _check(y, ref, f"mxfp4 {M}x{N}x{K}")


@pytest.mark.parametrize("M,N,K", [(7, 256, 128), (150, 384, 512), (600, 1024, 2048)])
def test_linear_fp8_matches_dequantised_product(M, N, K):
    g = torch.Generator().manual_seed(M + K)
    w = torch.randn(1, N, K, generator=g) * 0.02
    w_q, w_s = quant.quantize_fp8_128x128(w)
    x = synth.make_hidden(M, K, seed=M)
    ref = (x.float() @ orc.dequant_fp8_128x128(w_q[0], w_s[0], torch.bfloat16).float().t()).to(torch.bfloat16)
    y = linear_fp8_128x128(x.to(DEV), w_q[0].to(DEV), w_s[0].to(DEV)).cpu()
    _check(y, ref, f"fp8 {M}x{N}x{K}")


def test_linear_rejects_cpu_tensors():
    with pytest.raises(RuntimeError):
        linear_mxfp4(torch.zeros(4, 64, dtype=torch.bfloat16), torch.zeros(8, 32, dtype=torch.uint8),
                     torch.zeros(8, 2, dtype=torch.uint8))
