"""GPU tier: unquantised bf16 expert weights (the reference wrapper's QuantType.No, src/contrib/fused_moe.py:253)
against the torch layer oracle (tests/contrib/moe/test_moe.py:86-118), which takes bf16 weights as they are.

Tolerance: cosine >= 0.9995, max-abs <= 2e-2 scaled by max(1, |ref|max).  The golden case feeds the bf16 weights the
reference's own function was run on and compares with that function's outputs."""
import pathlib

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import ActivationType, QuantType, fused_moe, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = pathlib.Path(__file__).parent / "golden"
MAX_ABS, COS = 2e-2, 0.9995


def _bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def _run(x, tw, ids, w1, w2, **kw):
    y = fused_moe(x.to(DEV), w1.to(DEV), w2.to(DEV), tw.to(DEV), ids.to(DEV), quant_type=QuantType.No, **kw)
    torch.cuda.synchronize()
    return y.cpu()


def _close(y, ref, what):
    assert torch.isfinite(y.float()).all(), what
    cos, mx = orc.cosine(y, ref), orc.max_abs(y, ref)
    bound = MAX_ABS * max(1.0, float(ref.float().abs().max()))
    assert cos >= COS and mx <= bound, f"{what}: cosine {cos:.6f} max_abs {mx:.3e} (bound {bound:.3e})"


def test_golden_vectors_of_the_reference_layer():
    g = np.load(GOLD / "layer_mxfp4_small.npz")
    x = _bf16(g["x"])
    tw, ids = torch.from_numpy(g["topk_weight"]), torch.from_numpy(g["topk_ids"])
    w1, w2 = _bf16(g["w1_deq"]), _bf16(g["w2_deq"])
    for combine in ("gather", "fused"):
        _close(_run(x, tw, ids, w1, w2, combine=combine), _bf16(g["y_silu"]), f"golden silu {combine}")
        _close(_run(x, tw, ids, w1, w2, activation=ActivationType.Swiglu, swiglu_limit=7.0, combine=combine),
               _bf16(g["y_swiglu"]), f"golden swiglu {combine}")


@pytest.mark.parametrize("T,H,I,E,K,B", [(1, 256, 128, 8, 2, None), (7, 288, 160, 16, 4, None), (64, 512, 256, 8, 2, None),
                                         (65, 96, 32, 4, 3, 16), (300, 288, 160, 16, 4, 48), (257, 1024, 384, 8, 2, 96),
                                         (400, 320, 448, 4, 2, 128), (5, 2880, 2880, 4, 2, None)])
@pytest.mark.parametrize("combine", ["gather", "fused"])
def test_layer_matches_the_oracle(T, H, I, E, K, B, combine):
    x = synth.make_hidden(T, H, seed=T)
    tw, ids = synth.make_routing(T, E, K, "softmax", seed=T)
    w1, w2 = synth.make_weights_bf16(E, H, I, seed=T)
    ref = orc.torch_moe_oracle(x, w1, w2, tw, ids)
    kw = dict(block_size_M=B) if B else {}
    _close(_run(x, tw, ids, w1, w2, combine=combine, **kw), ref, f"T={T} H={H} I={I} B={B} {combine}")


@pytest.mark.parametrize("combine", ["gather", "fused"])
def test_mask_live_count_biases_and_stage1_weights(combine):
    T, H, I, E, K = 70, 288, 160, 8, 2
    x = synth.make_hidden(T, H, seed=3)
    tw, ids = synth.make_routing(T, E, K, "zipf", seed=3)
    w1, w2 = synth.make_weights_bf16(E, H, I, seed=3)
    g = torch.Generator().manual_seed(4)
    b1 = (torch.randn(E, 2 * I, generator=g) * 0.1).to(torch.bfloat16)
    b2 = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16)
    # per-expert biases, clamped SwiGLU
    ref = orc.torch_moe_oracle(x, w1, w2, tw, ids, activation="swiglu", swiglu_limit=7.0, bias1=b1, bias2=b2)
    y = _run(x, tw, ids, w1, w2, activation=ActivationType.Swiglu, combine=combine, bias1=b1.to(DEV), bias2=b2.to(DEV))
    _close(y, ref, "biases")
    # routing weights applied to h
    ref = orc.torch_moe_oracle(x, w1, w2, tw, ids, doweight_stage1=True)
    _close(_run(x, tw, ids, w1, w2, combine=combine, doweight_stage1=True), ref, "stage-1 weights")
    # expert mask: only the unmasked experts' weights are present
    keep = torch.tensor([1, 0, 1, 1, 0, 0, 1, 1], dtype=torch.bool)
    ref = orc.torch_moe_oracle(x, w1, w2, tw * keep[ids.long()].float(), ids)
    y = _run(x, tw, ids, w1[keep], w2[keep], combine=combine, expert_mask=keep.to(torch.int32).to(DEV))
    _close(y, ref, "mask")
    # live-token count below T: the rest of the batch is padding
    n = 41
    y = _run(x, tw, ids, w1, w2, combine=combine, num_local_tokens=n)
    assert float(y[n:].float().abs().max()) == 0.0
    _close(y[:n], orc.torch_moe_oracle(x[:n], w1, w2, tw[:n], ids[:n]), "live count")


def test_bitwise_reproducible_in_the_gather_form_and_argument_errors():
    T, H, I, E, K = 96, 256, 128, 8, 2
    x = synth.make_hidden(T, H, seed=5)
    tw, ids = synth.make_routing(T, E, K, seed=5)
    w1, w2 = synth.make_weights_bf16(E, H, I, seed=5)
    a, b = _run(x, tw, ids, w1, w2), _run(x, tw, ids, w1, w2)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    with pytest.raises((ValueError, TypeError)):
        _run(x, tw, ids, w1.float(), w2.float())
    with pytest.raises(ValueError):
        _run(x, tw, ids, w1, w2, act_terms=1)
