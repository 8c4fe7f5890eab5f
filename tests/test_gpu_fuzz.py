"""GPU tier: seeded random layer configurations against the CPU oracle.

Each case draws a shape (ragged token counts, hidden sizes that are not multiples of the k-tile, expert counts from 2
to 64, top-k up to 8), a routing law, a sort block, a weight format (MXFP4, FP8 128x128, bf16), an activation format, the combine form, the CTA-pair switch and the
optional arguments (expert mask, a live-token count below T, biases, stage-1 weights) from one seed, runs the layer
through the public call and compares with the oracle called with the same options.  The fixed cases of the other
files pin single features; these cover their combinations.

Tolerance: cosine >= 0.9995 and max-abs <= 2e-2 * max(1, |ref|max) against the oracle of the same activation format
(bf16 activations for the default formats, the quantise-dequantise oracle for 1x128 FP8 activations); plain MXFP4
activations (act_terms = 1) take the reference's own a4w4 threshold, calc_diff <= 0.01 against the oracle that
dequantises the same quantised activations (tests/contrib/moe/test_mxfp4.py:286-299).
"""
import random

import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import ActivationType, QuantType, fused_moe, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_ABS, COS = 2e-2, 0.9995


def _close(y, ref, what, a4w4=False):
    assert torch.isfinite(y.float()).all(), what
    if a4w4:
        d = orc.calc_diff(y, ref)
        assert d <= 0.01 and orc.cosine(y, ref) >= 0.995, f"{what}: calc_diff {d:.4f} cosine {orc.cosine(y, ref):.5f}"
        return
    cos, mx = orc.cosine(y, ref), orc.max_abs(y, ref)
    bound = MAX_ABS * max(1.0, float(ref.float().abs().max()))
    assert cos >= COS and mx <= bound, f"{what}: cosine {cos:.6f} max_abs {mx:.3e} bound {bound:.3e}"


def _draw(seed, fp8, bf16=False):
    r = random.Random(seed * 7919 + (1 if fp8 else 0) + (2 if bf16 else 0))
    step = 128 if fp8 else 32
    c = dict(
        T=r.choice([1, 2, 3, 5, 8, 17, 31, 64, 65, 100, 129, 255, 300, 513]),
        H=step * r.randint(1, 1024 // step), I=step * r.randint(1, 768 // step),
        E=r.choice([2, 4, 8, 16, 32, 64]), routing=r.choice(["softmax", "sigmoid", "zipf"]),
        B=r.choice([None, None, 16, 32, 48, 64, 80, 96] + ([] if fp8 else [112, 128])),
        combine=r.choice(["gather", "fused"]), activation=r.choice(["silu", "swiglu"]),
        mask=r.random() < 0.3, live=r.random() < 0.3, bias=r.random() < 0.3, stage1=r.random() < 0.2,
        pairs=r.choice(["auto", "on", "off"]))
    c["K"] = r.randint(1, min(c["E"], 8))
    if fp8:
        c["act"] = r.choice(["terms", "terms", "1x128"])
    elif not bf16:
        c["terms"] = r.choice([0, 0, 3, 4, 1])
    return c


def _run_case(seed, fp8, bf16=False, force_T1=False):
    c = _draw(seed, fp8, bf16)
    if force_T1:
        c["T"], c["terms"], c["live"] = 1, 0, False
    T, H, I, E, K = c["T"], c["H"], c["I"], c["E"], c["K"]
    what = f"seed {seed} {c}"
    x = synth.make_hidden(T, H, seed)
    tw, ids = synth.make_routing(T, E, K, c["routing"], seed)
    if bf16:
        w1, w2 = synth.make_weights_bf16(E, H, I, seed=seed)
        w = (w1, None, w2, None)
    else:
        w = (synth.make_weights_fp8 if fp8 else synth.make_weights_mxfp4)(E, H, I, seed=seed)
    g = torch.Generator().manual_seed(seed)
    kw, okw = {}, {}
    if c["bias"]:
        b1 = (torch.randn(E, 2 * I, generator=g) * 0.1).to(torch.bfloat16)
        b2 = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16)
        kw.update(bias1=b1, bias2=b2)
        okw.update(bias1=b1, bias2=b2)
    if c["stage1"]:
        kw["doweight_stage1"] = okw["doweight_stage1"] = True
        if c["bias"] and c["mask"]:      # a zero routing weight no longer silences a dropped expert's bias2: no mask
            c["mask"] = False
    n = T
    if c["live"] and T > 1:
        n = random.Random(seed).randint(0, T - 1)
        kw["num_local_tokens"] = n
    keep = torch.ones(E, dtype=torch.bool)
    if c["mask"]:
        keep = torch.rand(E, generator=g) < 0.6
        keep[int(ids[0, 0])] = True                       # at least one expert stays
        kw["expert_mask"] = keep.to(torch.int32).to(DEV)
    w_local = tuple(None if t is None else t[keep].to(DEV) for t in w)
    if "bias1" in kw:
        kw["bias1"], kw["bias2"] = kw["bias1"][keep].to(DEV), kw["bias2"][keep].to(DEV)
    if fp8:
        kw["act_quant"] = c["act"]
        if c["act"] == "1x128":
            okw["act_quant"] = "fp8_1x128"
    elif not bf16:
        kw["act_terms"] = c["terms"]
        if c["terms"] == 1:
            okw["act_quant"] = "mxfp4"
    if c["B"]:
        kw["block_size_M"] = c["B"]
    act = ActivationType.Silu if c["activation"] == "silu" else ActivationType.Swiglu
    qt = QuantType.No if bf16 else QuantType.per_128x128 if fp8 else QuantType.per_1x32
    y = fused_moe(x.to(DEV), w_local[0], w_local[2], tw.to(DEV), ids.to(DEV), quant_type=qt,
                  w1_scale=w_local[1], w2_scale=w_local[3], activation=act, combine=c["combine"],
                  cta_pairs=c["pairs"], **kw)
    torch.cuda.synchronize()
    y = y.cpu()
    assert y.shape == (T, H), what
    if n < T:
        assert float(y[n:].float().abs().max()) == 0.0, what + " (rows beyond the live count)"
    if n == 0:
        return
    # the masked layer is the full one with the dropped experts' routing weights set to zero
    tw_m = tw * keep[ids.long()].float()
    if bf16:
        ref = orc.torch_moe_oracle(x[:n], w[0], w[2], tw_m[:n], ids[:n], activation=c["activation"], swiglu_limit=7.0, **okw)
    else:
        oracle = orc.torch_moe_oracle_fp8 if fp8 else orc.torch_moe_oracle_mxfp4
        ref = oracle(x[:n], *w, tw_m[:n], ids[:n], activation=c["activation"], swiglu_limit=7.0, **okw)
    _close(y[:n], ref, what, a4w4=c.get("terms") == 1)
    if T == 1 and not fp8 and not bf16 and c.get("terms") == 0 and K <= 8:
        # the same call down the batch-1 path (no sort, no activation quantiser)
        y1 = fused_moe(x.to(DEV), w_local[0], w_local[2], tw.to(DEV), ids.to(DEV), quant_type=qt, w1_scale=w_local[1],
                       w2_scale=w_local[3], activation=act, combine=c["combine"], method="batch1",
                       **{k: v for k, v in kw.items() if k != "block_size_M"})
        torch.cuda.synchronize()
        _close(y1.cpu()[:n], ref, what + " (batch-1 path)")


@pytest.mark.parametrize("seed", range(28))
def test_random_mxfp4_layers(seed):
    _run_case(seed, fp8=False)


@pytest.mark.parametrize("seed", range(100, 112))
def test_random_single_token_layers_on_both_paths(seed):
    _run_case(seed, fp8=False, force_T1=True)


@pytest.mark.parametrize("seed", range(16))
def test_random_fp8_layers(seed):
    _run_case(seed, fp8=True)


@pytest.mark.parametrize("seed", range(16))
def test_random_bf16_weight_layers(seed):
    _run_case(seed, fp8=False, bf16=True)
