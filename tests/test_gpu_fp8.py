"""GPU tier: FP8 (e4m3) weights with fp32 scales per 128x128 block -- parity of the CUDA path with
the torch dequantise-then-matmul oracle (bf16 activations), tolerance max-abs <= 2e-2 and
cosine >= 0.9995 as for the MXFP4 path."""
import pathlib

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import QuantType, _lib, fused_moe, synth
from pyhip_b200.fused_moe import get_plan, prepare_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = pathlib.Path(__file__).parent / "golden"
MAX_ABS, COS = 2e-2, 0.9995


def _bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def _run(x, tw, ids, w, **kw):
    w1_q, w1_s, w2_q, w2_s = (t.to(DEV) for t in w)
    y = fused_moe(x.to(DEV), w1_q, w2_q, tw.to(DEV), ids.to(DEV), quant_type=QuantType.per_128x128,
                  w1_scale=w1_s, w2_scale=w2_s, **kw)
    torch.cuda.synchronize()
    return y.cpu()


def _close(y, ref, what):
    assert torch.isfinite(y.float()).all(), what
    cos, mx = orc.cosine(y, ref), orc.max_abs(y, ref)
    # bf16 spacing exceeds 2e-2 above magnitude 4: the absolute bound scales with the output range there
    bound = MAX_ABS * max(1.0, float(ref.float().abs().max()))
    assert cos >= COS and mx <= bound, f"{what}: cosine {cos:.6f} max_abs {mx:.3e} (bound {bound:.3e})"


def test_e4m3_rows_match_oracle_bit_for_bit():
    T, H, I, E, K, B = 40, 256, 128, 8, 2, 32
    x = synth.make_hidden(T, H, 4)
    tw, ids = synth.make_routing(T, E, K, seed=4)
    plan = get_plan(T, K, E, E, H, I, B, 0, 7.0, torch.device(DEV), weight_format=_lib.W_FP8_128)
    s_ids, _, _, nv, _ = plan.sort(ids.to(DEV), tw.to(DEV))
    plan.quant_input(x.to(DEV))
    torch.cuda.synchronize()
    n, L = int(nv[0]), plan.ws.max_rows
    q = plan.region("xq", 2 * L * H).cpu().numpy().reshape(2, L, H)[:, :n]
    sf = plan.region("xsf", L // B * (H // 128) * 2 * 512).cpu().numpy().reshape(-1, H // 128, 2, 32, 4, 4)
    sf = sf.transpose(0, 2, 4, 3, 1, 5).reshape(sf.shape[0], 2, 128, H // 32)[:, :, :B]    # [blk, term, r, kb*4+j]
    sf = sf.transpose(1, 0, 2, 3).reshape(2, -1, H // 32)[:, :n]
    sid = s_ids.cpu().numpy().view(np.uint32)[:n]
    tok, kk = sid & 0xFFFFFF, sid >> 24
    eq, ee = orc.e4m3_terms_quant(x, 2)
    eq = eq.float().numpy()
    got = torch.from_numpy(q.copy()).view(torch.float8_e4m3fn).float().numpy()
    for r in range(n):
        if kk[r] < K:
            assert np.array_equal(got[:, r], eq[:, tok[r]]), r
            assert np.array_equal(sf[:, r], ee[:, tok[r]]), r


@pytest.mark.parametrize("T,H,I,E,K,B", [(32, 256, 128, 4, 2, 32), (150, 256, 384, 4, 2, 64), (300, 384, 128, 4, 2, 96), (260, 256, 256, 4, 2, 80),
                                         (7, 512, 256, 8, 2, 16)])
def test_stage_chain_matches_layer_oracle(T, H, I, E, K, B):
    x = synth.make_hidden(T, H, T)
    tw, ids = synth.make_routing(T, E, K, seed=T)
    w = synth.make_weights_fp8(E, H, I, seed=T)
    pw = prepare_weights(*(t.to(DEV) for t in w), weight_format=_lib.W_FP8_128)
    plan = get_plan(T, K, E, E, H, I, B, 0, 7.0, torch.device(DEV), weight_format=_lib.W_FP8_128)
    plan.sort(ids.to(DEV), tw.to(DEV))
    plan.quant_input(x.to(DEV))
    h = torch.zeros(T, K, I, dtype=torch.bfloat16, device=DEV)
    plan.gateup(pw, h)
    torch.cuda.synchronize()
    plan.check_status()
    srt = orc.moe_sorting_oracle(ids, tw, E, B)
    w1 = orc.dequant_fp8_128x128(w[0], w[1])
    ref_h = orc.moe_gemm_oracle(K, B, srt[0], srt[2], srt[1], srt[3], x, w1, True)
    _close(h.cpu(), ref_h, "fp8 gate-up")
    plan.quant_hidden(h)
    plan.down(pw)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    plan.combine(tw.to(DEV), y)
    torch.cuda.synchronize()
    plan.check_status()
    _close(y.cpu(), orc.torch_moe_oracle_fp8(x, *w, tw, ids), "fp8 stage chain")


def test_layer_matches_reference_golden_vectors():
    g = np.load(GOLD / "layer_fp8_small.npz")
    x = _bf16(g["x"])
    tw, ids = torch.from_numpy(g["topk_weight"]), torch.from_numpy(g["topk_ids"])
    w = (torch.from_numpy(g["w1_q"]).view(torch.float8_e4m3fn), torch.from_numpy(g["w1_s"]),
         torch.from_numpy(g["w2_q"]).view(torch.float8_e4m3fn), torch.from_numpy(g["w2_s"]))
    _close(_run(x, tw, ids, w), _bf16(g["y"]), "fp8 golden")


@pytest.mark.parametrize("T", [1, 33, 257])
def test_fused_layer_ragged_and_skewed(T):
    H, I, E, K = 384, 256, 16, 4
    x = synth.make_hidden(T, H, T)
    tw, ids = synth.make_routing(T, E, K, "zipf", seed=T)
    w = synth.make_weights_fp8(E, H, I, seed=3)
    _close(_run(x, tw, ids, w), orc.torch_moe_oracle_fp8(x, *w, tw, ids), f"fp8 T={T}")


def test_deepseek_shaped_slice():
    """H=7168, I=2048 (the config-3 shape) with a handful of experts: sigmoid routing, top-8."""
    T, H, I, E, K = 16, 7168, 2048, 8, 8
    x = synth.make_hidden(T, H, 1)
    tw, ids = synth.make_routing(T, E, K, "sigmoid", seed=1)
    w = synth.make_weights_fp8(E, H, I, seed=1)
    _close(_run(x, tw, ids, w), orc.torch_moe_oracle_fp8(x, *w, tw, ids), "dsv3 slice")


# --------------------------------------------------------------------------------------------
# per-token 1x128 activations (the reference's own FP8 activation format), fused combine
# --------------------------------------------------------------------------------------------
def test_1x128_rows_match_oracle_bit_for_bit():
    T, H, I, E, K, B = 40, 384, 256, 8, 2, 32
    x = synth.make_hidden(T, H, 4)
    x[3, 128:256] = 0                                    # an all-zero block takes scale 1.0
    tw, ids = synth.make_routing(T, E, K, seed=4)
    plan = get_plan(T, K, E, E, H, I, B, 0, 7.0, torch.device(DEV), weight_format=_lib.W_FP8_128, act_quant=_lib.ACTQ_1X128)
    s_ids, _, _, nv, _ = plan.sort(ids.to(DEV), tw.to(DEV))
    plan.quant_input(x.to(DEV))
    torch.cuda.synchronize()
    n, L = int(nv[0]), plan.ws.max_rows
    q = plan.region("xq", L * H).cpu().view(torch.float8_e4m3fn).float().numpy().reshape(L, H)[:n]
    sc = plan.region("xsf", L // B * (H // 128) * B * 4, torch.float32).cpu().numpy().reshape(L // B, H // 128, B)
    sid = s_ids.cpu().numpy().view(np.uint32)[:n]
    tok, kk = sid & 0xFFFFFF, sid >> 24
    eq, es = orc.act_quant_fp8_1x128(x)
    eq, es = eq.float().numpy(), es.numpy()
    for r in range(n):
        if kk[r] < K:
            assert np.array_equal(q[r], eq[tok[r]]), r
            assert np.array_equal(sc[r // B, :, r % B], es[tok[r]]), r


def _close_q(y, ref_q, ref, what):
    """Against the oracle that dequantises the same 1x128-quantised activations; the distance to the
    bf16-activation oracle is reported."""
    assert torch.isfinite(y.float()).all(), what
    cos, mx = orc.cosine(y, ref_q), orc.max_abs(y, ref_q)
    bound = MAX_ABS * max(1.0, float(ref_q.float().abs().max()))
    print(f"{what}: vs 1x128 oracle cosine {cos:.6f} max_abs {mx:.3e}; vs bf16-activation oracle cosine {orc.cosine(y, ref):.6f}")
    assert cos >= COS and mx <= bound, f"{what}: cosine {cos:.6f} max_abs {mx:.3e} (bound {bound:.3e})"


@pytest.mark.parametrize("T,H,I,E,K,B", [(32, 256, 128, 4, 2, 32), (150, 256, 384, 4, 2, 64), (300, 384, 128, 4, 2, 96),
                                         (7, 512, 256, 8, 2, 16)])
def test_1x128_stage_chain_matches_its_oracle(T, H, I, E, K, B):
    x = synth.make_hidden(T, H, T)
    tw, ids = synth.make_routing(T, E, K, seed=T)
    w = synth.make_weights_fp8(E, H, I, seed=T)
    pw = prepare_weights(*(t.to(DEV) for t in w), weight_format=_lib.W_FP8_128)
    plan = get_plan(T, K, E, E, H, I, B, 0, 7.0, torch.device(DEV), weight_format=_lib.W_FP8_128, act_quant=_lib.ACTQ_1X128)
    plan.sort(ids.to(DEV), tw.to(DEV))
    plan.quant_input(x.to(DEV))
    h = torch.zeros(T, K, I, dtype=torch.bfloat16, device=DEV)
    plan.gateup(pw, h)
    plan.quant_hidden(h)
    plan.down(pw)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    plan.combine(tw.to(DEV), y)
    torch.cuda.synchronize()
    plan.check_status()
    _close_q(y.cpu(), orc.torch_moe_oracle_fp8(x, *w, tw, ids, act_quant="fp8_1x128"),
             orc.torch_moe_oracle_fp8(x, *w, tw, ids), "1x128 stage chain")


@pytest.mark.parametrize("T", [1, 8, 33, 257])
@pytest.mark.parametrize("combine", ["gather", "fused"])
def test_1x128_fused_layer(T, combine):
    H, I, E, K = 384, 256, 16, 4
    x = synth.make_hidden(T, H, T)
    tw, ids = synth.make_routing(T, E, K, "zipf", seed=T)
    w = synth.make_weights_fp8(E, H, I, seed=3)
    _close_q(_run(x, tw, ids, w, act_quant="1x128", combine=combine),
             orc.torch_moe_oracle_fp8(x, *w, tw, ids, act_quant="fp8_1x128"), orc.torch_moe_oracle_fp8(x, *w, tw, ids),
             f"1x128 layer T={T} {combine}")


@pytest.mark.parametrize("act_quant", ["terms", "1x128"])
def test_fp8_fused_combine_biases_and_stage1_weights(act_quant):
    T, H, I, E, K = 70, 256, 128, 8, 2
    x = synth.make_hidden(T, H, 5)
    tw, ids = synth.make_routing(T, E, K, seed=5)
    w = synth.make_weights_fp8(E, H, I, seed=5)
    g = torch.Generator().manual_seed(9)
    b1 = (torch.randn(E, 2 * I, generator=g) * 0.1).to(torch.bfloat16)
    b2 = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16)
    okw = {} if act_quant == "terms" else {"act_quant": "fp8_1x128"}
    for combine in ("gather", "fused"):
        for kw, ok in ((dict(), dict()), (dict(bias1=b1.to(DEV), bias2=b2.to(DEV)), dict(bias1=b1, bias2=b2)),
                       (dict(doweight_stage1=True), dict(doweight_stage1=True))):
            ref = orc.torch_moe_oracle_fp8(x, *w, tw, ids, **ok, **okw)
            _close(_run(x, tw, ids, w, combine=combine, act_quant=act_quant, **kw), ref, f"fp8 {act_quant} {combine} {sorted(kw)}")


def test_deepseek_shaped_slice_1x128():
    T, H, I, E, K = 100, 7168, 2048, 8, 8
    x = synth.make_hidden(T, H, 1)
    tw, ids = synth.make_routing(T, E, K, "sigmoid", seed=1)
    w = synth.make_weights_fp8(E, H, I, seed=1)
    _close_q(_run(x, tw, ids, w, act_quant="1x128", combine="fused"),
             orc.torch_moe_oracle_fp8(x, *w, tw, ids, act_quant="fp8_1x128"), orc.torch_moe_oracle_fp8(x, *w, tw, ids),
             "dsv3 slice 1x128")


# --------------------------------------------------------------------------------------------
# row-scaled FP8 weights: per-token-per-channel and per-tensor (tests/contrib/moe/test_moe.py:123-138,190-200)
# --------------------------------------------------------------------------------------------
def _rows_case(T, H, I, E, K, seed, per_tensor):
    from pyhip_b200 import quant
    g = torch.Generator().manual_seed(seed)
    w1f = torch.randn(E, 2 * I, H, generator=g) * 0.02
    w2f = torch.randn(E, H, I, generator=g) * 0.02
    # uneven row magnitudes, so that a wrong row <-> scale pairing cannot pass
    w1f *= torch.linspace(0.5, 2.0, 2 * I)[None, :, None]
    w2f *= torch.linspace(2.0, 0.5, H)[None, :, None]
    q = quant.quantize_fp8_per_tensor if per_tensor else quant.quantize_fp8_per_row
    (w1_q, w1_s), (w2_q, w2_s) = q(w1f), q(w2f)
    x = synth.make_hidden(T, H, seed)
    tw, ids = synth.make_routing(T, E, K, seed=seed)
    return x, tw, ids, (w1_q, w1_s, w2_q, w2_s)


@pytest.mark.parametrize("per_tensor", [False, True])
@pytest.mark.parametrize("T,H,I,E,K", [(1, 256, 128, 4, 2), (70, 384, 256, 8, 2), (300, 256, 384, 4, 2), (40, 2048, 512, 8, 4)])
def test_row_scaled_fp8_weights_match_the_layer_oracle(per_tensor, T, H, I, E, K):
    x, tw, ids, w = _rows_case(T, H, I, E, K, 60 + T, per_tensor)
    ref = orc.torch_moe_oracle_fp8(x, *w, tw, ids, row_scaled=True)
    qt = QuantType.per_Tensor if per_tensor else QuantType.per_Token
    for combine in ("gather", "fused"):
        w1_q, w1_s, w2_q, w2_s = (t.to(DEV) for t in w)
        y = fused_moe(x.to(DEV), w1_q, w2_q, tw.to(DEV), ids.to(DEV), quant_type=qt, w1_scale=w1_s, w2_scale=w2_s,
                      combine=combine)
        torch.cuda.synchronize()
        _close(y.cpu(), ref, f"row-scaled fp8 per_tensor={per_tensor} T={T} {combine}")
