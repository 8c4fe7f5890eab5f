"""CPU tier: the oracle against the golden vectors produced by the reference's own functions,
known-answer tests of the encodings, and the sorting contract."""
import pathlib

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import quant, synth

GOLD = pathlib.Path(__file__).parent / "golden"


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


# ------------------------------------------------------------------ encodings
def test_e2m1_table_and_nibble_order():
    # pk_fp4.hpp:128-129 value table; low nibble = even element (pk_fp4.hpp:122-125)
    codes = torch.arange(16, dtype=torch.uint8)
    vals = quant.e2m1_decode(codes)
    assert vals.tolist() == [0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]
    packed = quant.pack_nibbles(torch.tensor([[1, 2, 3, 4]], dtype=torch.uint8))
    assert packed.tolist() == [[0x21, 0x43]]
    assert quant.unpack_nibbles(packed).tolist() == [[1, 2, 3, 4]]
    # the oracle's independent decoder agrees on all 16 codes
    allc = quant.pack_nibbles(torch.arange(32, dtype=torch.uint8).reshape(1, 32) % 16)
    one = torch.full((1, 1), 127, dtype=torch.uint8)
    assert torch.equal(orc.dequant_mxfp4(allc, one, torch.float32),
                       quant.dequantize_mxfp4(allc, one, torch.float32))


def test_e2m1_round_to_nearest_even_and_saturation():
    v = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, 100.0, -0.25, -0.76, 0.2, 0.26])
    got = quant.e2m1_decode(quant.e2m1_encode(v)).tolist()
    assert got == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, 6.0, 0.0, -1.0, 0.0, 0.5]


def test_e8m0_known_answers():
    b = torch.tensor([127, 128, 126, 0, 254], dtype=torch.uint8)
    f = quant.e8m0_to_float(b)
    assert f[0] == 1.0 and f[1] == 2.0 and f[2] == 0.5
    assert f[4] == 2.0 ** 127 and f[3] == 2.0 ** -127


def test_mxfp4_scale_rule_and_roundtrip():
    torch.manual_seed(0)
    w = torch.randn(8, 96) * 0.02
    q, s = quant.quantize_mxfp4(w)
    assert q.shape == (8, 48) and s.shape == (8, 3)
    amax = w.reshape(8, 3, 32).abs().amax(-1)
    expect = torch.floor(torch.log2(amax.double() / 6.0)).int() + 127
    assert torch.equal(s.int(), expect.int())
    deq = quant.dequantize_mxfp4(q, s, torch.float32)
    # quantising an already-representable tensor is the identity
    q2, s2 = quant.quantize_mxfp4(deq)
    deq2 = quant.dequantize_mxfp4(q2, s2, torch.float32)
    assert torch.equal(deq, deq2)
    # oracle's decoder == package's decoder
    assert torch.equal(orc.dequant_mxfp4(q, s, torch.float32), deq)
    # zero block: scale byte 127, zero codes
    qz, sz = quant.quantize_mxfp4(torch.zeros(1, 32))
    assert sz.tolist() == [[127]] and int(qz.sum()) == 0


def test_fp8_block_roundtrip():
    torch.manual_seed(1)
    w = torch.randn(2, 256, 128) * 0.02
    q, s = quant.quantize_fp8_128x128(w)
    assert s.shape == (2, 2, 1)
    assert torch.equal(orc.dequant_fp8_128x128(q, s), quant.dequantize_fp8_128x128(q, s))
    err = (quant.dequantize_fp8_128x128(q, s, torch.float32) - w).abs().max()
    assert err < 0.02 * 4 * 2 ** -3


# ------------------------------------------------------------------ golden: layer
def test_layer_oracle_matches_reference_golden_mxfp4():
    g = np.load(GOLD / "layer_mxfp4_small.npz")
    x = _bf16(g["x"])
    tw, ids = torch.from_numpy(g["topk_weight"]), torch.from_numpy(g["topk_ids"])
    w1_q, w1_s = torch.from_numpy(g["w1_q"]), torch.from_numpy(g["w1_s"])
    w2_q, w2_s = torch.from_numpy(g["w2_q"]), torch.from_numpy(g["w2_s"])
    # dequantised weights the reference consumed == oracle's dequantiser output
    assert torch.equal(orc.dequant_mxfp4(w1_q, w1_s).view(torch.int16), _bf16(g["w1_deq"]).view(torch.int16))
    assert torch.equal(orc.dequant_mxfp4(w2_q, w2_s).view(torch.int16), _bf16(g["w2_deq"]).view(torch.int16))
    y = orc.torch_moe_oracle_mxfp4(x, w1_q, w1_s, w2_q, w2_s, tw, ids)
    assert torch.equal(y.view(torch.int16), _bf16(g["y_silu"]).view(torch.int16))
    y2 = orc.torch_moe_oracle_mxfp4(x, w1_q, w1_s, w2_q, w2_s, tw, ids, activation="swiglu",
                                    swiglu_limit=7.0)
    assert torch.equal(y2.view(torch.int16), _bf16(g["y_swiglu"]).view(torch.int16))


def test_layer_oracle_matches_reference_golden_fp8():
    g = np.load(GOLD / "layer_fp8_small.npz")
    x = _bf16(g["x"])
    tw, ids = torch.from_numpy(g["topk_weight"]), torch.from_numpy(g["topk_ids"])
    w1_q = torch.from_numpy(g["w1_q"]).view(torch.float8_e4m3fn)
    w2_q = torch.from_numpy(g["w2_q"]).view(torch.float8_e4m3fn)
    y = orc.torch_moe_oracle_fp8(x, w1_q, torch.from_numpy(g["w1_s"]), w2_q,
                                 torch.from_numpy(g["w2_s"]), tw, ids)
    assert torch.equal(y.view(torch.int16), _bf16(g["y"]).view(torch.int16))


def test_inputs_regenerate_from_seed():
    """The synthetic generators reproduce the tensors stored in the fixture."""
    g = np.load(GOLD / "layer_mxfp4_small.npz")
    x = synth.make_hidden(16, 256, seed=3)
    tw, ids = synth.make_routing(16, 4, 2, "softmax", seed=3)
    w1_q, w1_s, _, _ = synth.make_weights_mxfp4(4, 256, 128, seed=3)
    assert torch.equal(x.view(torch.int16), _bf16(g["x"]).view(torch.int16))
    assert np.array_equal(ids.numpy(), g["topk_ids"]) and np.array_equal(tw.numpy(), g["topk_weight"])
    assert np.array_equal(w1_q.numpy(), g["w1_q"]) and np.array_equal(w1_s.numpy(), g["w1_s"])


# ------------------------------------------------------------------ sorting
def test_sorting_matches_reference_golden_b256():
    g = np.load(GOLD / "sorting_b256.npz")
    s_ids, s_w, s_e, nv = orc.moe_sorting_oracle(g["topk_ids"], g["topk_weight"], int(g["E"]), int(g["B"]))
    n = int(g["num_valid"])
    assert nv[0] == n and nv[1] == g["topk_ids"].shape[0]
    assert np.array_equal(s_ids[:n], g["sorted_ids"])
    assert np.array_equal(s_w[:n].view(np.uint32), g["sorted_weights"].view(np.uint32))
    assert np.array_equal(s_e[: n // int(g["B"])], g["sorted_expert_ids"])


CK_IDS = [[0, 3, 5], [2, 3, 5], [1, 3, 5], [1, 2, 3], [1, 3, 5]]


def test_sorting_ck_tile_worked_example():
    """archive/ck_tile/.../moe_sorting_kernel.hpp:35-82 (E=6, K=3, B=4, T=5, skip empty)."""
    ids = np.array(CK_IDS, dtype=np.int32)
    w = np.arange(15, dtype=np.float32).reshape(5, 3) + 1
    s_ids, s_w, s_e, nv = orc.moe_sorting_oracle(ids, w, 6, 4)
    assert nv[0] == 24
    assert (s_ids[:24] & 0xFFFFFF).tolist() == [0, 5, 5, 5, 2, 3, 4, 5, 1, 3, 5, 5, 0, 1, 2, 3,
                                                4, 5, 5, 5, 0, 1, 2, 4]
    assert s_e[:6].tolist() == [0, 1, 2, 3, 3, 5]
    # k is carried in the high byte; padding carries k = topk
    assert (s_ids[:4] >> 24).tolist() == [0, 3, 3, 3]
    assert s_w[:8].tolist() == [1.0, 0, 0, 0, 7.0, 10.0, 13.0, 0]


def test_sorting_ck_tile_masked_example():
    """moe_sorting_kernel.hpp:84-97: mask out experts 1 and 4 -> local ids [0,1,2,2,3]."""
    ids = np.array(CK_IDS, dtype=np.int32)
    w = np.ones((5, 3), dtype=np.float32)
    _, _, s_e, nv = orc.moe_sorting_oracle(ids, w, 6, 4, expert_mask=[1, 0, 1, 1, 0, 1])
    assert nv[0] == 20 and s_e[:5].tolist() == [0, 1, 2, 2, 3]


@pytest.mark.parametrize("T,E,K,B", [(1, 8, 2, 16), (3, 128, 4, 32), (77, 8, 2, 32), (500, 32, 8, 64)])
def test_sorting_against_brute_force(T, E, K, B):
    tw, ids = synth.make_routing(T, E, K, "zipf", seed=T)
    s_ids, s_w, s_e, nv = orc.moe_sorting_oracle(ids, tw, E, B)
    exp_ids, exp_w, exp_e = [], [], []
    for e in range(E):
        n0 = len(exp_ids)
        for t in range(T):
            for k in range(K):
                if int(ids[t, k]) == e:
                    exp_ids.append((k << 24) | t)
                    exp_w.append(float(tw[t, k]))
        if len(exp_ids) > n0:
            while len(exp_ids) % B:
                exp_ids.append((K << 24) | T)
                exp_w.append(0.0)
            exp_e += [e] * ((len(exp_ids) - n0) // B)
    assert nv[0] == len(exp_ids)
    assert s_ids[:nv[0]].tolist() == exp_ids
    assert s_w[:nv[0]].tolist() == exp_w
    assert s_e[:nv[0] // B].tolist() == exp_e


# ------------------------------------------------------------------ per-stage form and hilo8
def test_block_form_agrees_with_layer_form():
    T, H, I, E, K, B = 24, 128, 64, 4, 2, 16
    x = synth.make_hidden(T, H, seed=11)
    tw, ids = synth.make_routing(T, E, K, seed=11)
    w1_q, w1_s, w2_q, w2_s = synth.make_weights_mxfp4(E, H, I, seed=11)
    w1, w2 = orc.dequant_mxfp4(w1_q, w1_s), orc.dequant_mxfp4(w2_q, w2_s)
    srt = orc.moe_sorting_oracle(ids, tw, E, B)
    h = orc.moe_gemm_oracle(K, B, srt[0], srt[2], srt[1], srt[3], x, w1, True)
    y = orc.moe_gemm_oracle(K, B, srt[0], srt[2], srt[1], srt[3], h, w2, False)
    ref = orc.torch_moe_oracle(x, w1, w2, tw, ids)
    assert orc.cosine(y, ref) > 0.9999 and orc.max_abs(y, ref) < 2e-3


def test_fp4_term_expansion_converges():
    """The packed-FP4 term expansion of the device quantiser: error relative to the block maximum
    shrinks ~6x per term; four terms are exact for most bf16 inputs."""
    x = synth.make_hidden(64, 256, seed=2)
    xf = x.float()
    errs = []
    for nt in (1, 2, 3, 4):
        c, e = orc.fp4_terms_quant(x, nt)
        assert c.shape == (nt, 64, 256) and e.shape == (nt, 64, 8) and int(e.max()) < 255
        back = orc.fp4_terms_dequant(c, e)
        errs.append(float((back - xf).norm() / xf.norm()))
    assert errs[0] < 0.2 and errs[1] < 0.03 and errs[2] < 4e-3 and errs[3] < 3e-4
    c, e = orc.fp4_terms_quant(x, 4)
    assert float((orc.fp4_terms_dequant(c, e) == xf).float().mean()) > 0.9
    # zero rows stay zero with the smallest scale
    c0, e0 = orc.fp4_terms_quant(torch.zeros(1, 32, dtype=torch.bfloat16), 3)
    assert not (c0 & 7).any() and not e0.any()


def test_tiny_config_parity_bar_is_meaningful():
    """Config 0 end to end on the CPU: three FP4 terms per activation row stay well inside the
    north-star tolerance against the bf16-activation oracle; one term (plain MXFP4 activations)
    does not reach the cosine bar -- the reason the kernels carry several terms."""
    c = synth.CONFIGS["tiny"]
    x = synth.make_hidden(c.T, c.H)
    tw, ids = synth.make_routing(c.T, c.E, c.K)
    w1_q, w1_s, w2_q, w2_s = synth.make_weights_mxfp4(c.E, c.H, c.I)
    ref = orc.torch_moe_oracle_mxfp4(x, w1_q, w1_s, w2_q, w2_s, tw, ids)
    x3 = orc.fp4_terms_dequant(*orc.fp4_terms_quant(x, 3)).to(torch.bfloat16)
    got = orc.torch_moe_oracle_mxfp4(x3, w1_q, w1_s, w2_q, w2_s, tw, ids)
    assert orc.cosine(got, ref) >= 0.9999 and orc.max_abs(got, ref) <= 2e-2
    x1 = orc.fp4_terms_dequant(*orc.fp4_terms_quant(x, 1)).to(torch.bfloat16)
    got1 = orc.torch_moe_oracle_mxfp4(x1, w1_q, w1_s, w2_q, w2_s, tw, ids)
    assert orc.cosine(got1, ref) < 0.9995


# ------------------------------------------------------------------ synthetic routing
def test_zipf_routing_follows_the_stated_load_law():
    """The skewed-routing configuration asks for Zipf(s = 1.2) expert load.  `make_routing(..., "zipf")` adds
    b_e = -c ln(rank_e) to N(0,1) logits before softmax / top-2, with c calibrated on the measured load: the
    share of (token, expert) pairs per expert, ordered by popularity rank, must fall like rank^-1.2 (log-log
    slope within 0.15 of -1.2), stay within 0.08 of the Zipf(1.2) shares (top-k without replacement caps the
    head at 1/K), and leave no expert empty."""
    from pyhip_b200 import synth
    T, E, K = 16384, 8, 2
    _, ids = synth.make_routing(T, E, K, "zipf", seed=0, skew_seed=0)
    share = np.bincount(ids.flatten().numpy(), minlength=E) / (T * K)
    gp = torch.Generator().manual_seed(0 * 1000003 + 41)
    rank = torch.randperm(E, generator=gp).numpy() + 1           # rank_e used by make_routing
    by_rank = share[np.argsort(rank)]
    assert np.all(np.diff(by_rank) < 0), by_rank                  # strictly falling with the popularity rank
    assert by_rank[0] <= 1.0 / K + 1e-9 and by_rank[-1] > 0.0
    slope = np.polyfit(np.log(np.arange(1, E + 1)), np.log(by_rank), 1)[0]
    assert abs(slope + 1.2) < 0.15, (slope, by_rank)
    zipf = 1.0 / np.arange(1, E + 1) ** 1.2
    zipf /= zipf.sum()
    assert np.abs(by_rank - zipf).max() < 0.08, (by_rank, zipf)
    print("measured share by rank", np.round(by_rank, 4).tolist(), "Zipf(1.2)", np.round(zipf, 4).tolist(), "slope", slope)


def test_calc_diff_matches_its_definition_and_thresholds():
    """calc_diff (src/misc.py:131-141) is 0 for identical tensors, 1 for orthogonal ones, and grows with noise:
    the reference's thresholds (0.02 layer, 0.01 a4w4 gate-up, 1e-3 bf16 path) are ordered accordingly."""
    g = torch.Generator().manual_seed(0)
    a = torch.randn(64, 128, generator=g)
    assert orc.calc_diff(a, a) == 0.0
    b = torch.zeros_like(a)
    b[0, 0], a2 = 1.0, torch.zeros_like(a)
    a2[0, 1] = 1.0
    assert abs(orc.calc_diff(a2, b) - 1.0) < 1e-12
    noisy = a + 0.05 * torch.randn(64, 128, generator=g)
    d = orc.calc_diff(a, noisy)
    assert 1e-3 < d < 0.01
    assert abs(d - (1 - orc.cosine(a, noisy))) < 2e-3           # for nearly equal norms the two agree


def test_activation_quantiser_modes_of_the_oracle():
    """act_quant = mxfp4 / fp8_1x128 quantise x and h before the products; the known distances to the
    bf16-activation layer (cosine ~0.98 and ~0.999) show why those modes are judged against their own oracle."""
    from pyhip_b200 import synth
    c = synth.CONFIGS["tiny"]
    x = synth.make_hidden(c.T, c.H)
    tw, ids = synth.make_routing(c.T, c.E, c.K)
    w = synth.make_weights_mxfp4(c.E, c.H, c.I)
    r0 = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    r1 = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids, act_quant="mxfp4")
    assert 0.95 < orc.cosine(r0, r1) < 0.9995
    wf = synth.make_weights_fp8(c.E, c.H, c.I)
    q0 = orc.torch_moe_oracle_fp8(x, *wf, tw, ids)
    q1 = orc.torch_moe_oracle_fp8(x, *wf, tw, ids, act_quant="fp8_1x128")
    assert 0.998 < orc.cosine(q0, q1) < 0.99999
    # the 1x128 quantiser: scale = amax/448, values round-trip within one e4m3 step of the block maximum
    q, s = orc.act_quant_fp8_1x128(x)
    assert s.shape == (c.T, c.H // 128) and q.dtype == torch.float8_e4m3fn
    back = orc.act_dequant_fp8_1x128(q, s)
    amax = x.float().reshape(c.T, -1, 128).abs().amax(-1, keepdim=True)
    assert float(((back - x.float()).reshape(c.T, -1, 128).abs() / amax).max()) <= 2 ** -4 + 1e-6
    assert torch.equal(q.float().reshape(c.T, -1, 128).abs().amax(-1), torch.full((c.T, c.H // 128), 448.0))
