"""GPU tier: the router launch (logits -> top-k ids and weights) against the torch recipe the
configurations prescribe (softmax or sigmoid scores, top-k, renormalise) -- the step the reference
leaves to torch.topk / aiter's fused_topk (tests/contrib/moe/test_moe_sorting.py:81-84,
tests/contrib/moe/test_fused_moe.py:38,87).  Ids must match exactly, weights to float rounding."""
import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import QuantType, fused_moe, fused_topk, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _torch_route(logits, K, scoring, renorm):
    scores = torch.sigmoid(logits) if scoring == "sigmoid" else torch.softmax(logits, dim=-1)
    w, ids = torch.topk(scores, K, dim=-1)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32)


@pytest.mark.parametrize("T,E,K,scoring,renorm", [(64, 128, 4, "softmax", True), (1000, 256, 8, "sigmoid", True),
                                                  (8192, 128, 4, "softmax", True), (5, 8, 2, "softmax", False),
                                                  (33, 100, 6, "sigmoid", False), (7, 8, 8, "softmax", True),
                                                  (1, 1024, 40, "softmax", True)])
def test_router_matches_torch_topk(T, E, K, scoring, renorm):
    g = torch.Generator().manual_seed(T * 7 + E)
    logits = torch.randn(T, E, generator=g, dtype=torch.float32)
    w_ref, ids_ref = _torch_route(logits, K, scoring, renorm)
    w, ids = fused_topk(None, logits.to(DEV), K, renormalize=renorm, scoring=scoring)
    torch.cuda.synchronize()
    assert torch.equal(ids.cpu(), ids_ref)
    assert torch.allclose(w.cpu(), w_ref, rtol=1e-5, atol=1e-7)


def test_router_feeds_the_layer():
    """logits -> router -> fused MoE on the device equals the oracle fed with the torch routing."""
    c = synth.CONFIGS["tiny"]
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(c.T, c.E, generator=g, dtype=torch.float32)
    x = synth.make_hidden(c.T, c.H, 3)
    w = synth.make_weights_mxfp4(c.E, c.H, c.I, seed=3)
    tw_ref, ids_ref = _torch_route(logits, c.K, "softmax", True)
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw_ref, ids_ref)
    tw, ids = fused_topk(x.to(DEV), logits.to(DEV), c.K)
    wd = tuple(t.to(DEV) for t in w)
    y = fused_moe(x.to(DEV), wd[0], wd[2], tw, ids, quant_type=QuantType.per_1x32, w1_scale=wd[1], w2_scale=wd[3]).cpu()
    assert orc.cosine(y, ref) >= 0.9995 and orc.max_abs(y, ref) <= 2e-2
