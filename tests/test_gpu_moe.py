"""GPU tier: parity of the CUDA path (through the C ABI) with the CPU oracle.

Tolerances are the north-star's: routing / sort indices bit-exact, bf16 outputs max-abs <= 2e-2
and cosine >= 0.9995 against the torch dequantise-then-matmul oracle with bf16 activations.
"""
import pathlib

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from pyhip_b200 import ActivationType, QuantType, fused_moe, synth
from pyhip_b200.fused_moe import get_plan, pick_block, prepare_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = pathlib.Path(__file__).parent / "golden"
MAX_ABS, COS = 2e-2, 0.9995


def _bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def _case(T, H, I, E, K, routing="softmax", seed=0):
    x = synth.make_hidden(T, H, seed)
    tw, ids = synth.make_routing(T, E, K, routing, seed)
    w = synth.make_weights_mxfp4(E, H, I, seed)
    return x, tw, ids, w


def _run_layer(x, tw, ids, w, **kw):
    w1_q, w1_s, w2_q, w2_s = (t.to(DEV) for t in w)
    y = fused_moe(x.to(DEV), w1_q, w2_q, tw.to(DEV), ids.to(DEV), quant_type=QuantType.per_1x32,
                  w1_scale=w1_s, w2_scale=w2_s, **kw)
    torch.cuda.synchronize()
    return y.cpu()


def _assert_close(y, ref, what=""):
    assert torch.isfinite(y.float()).all(), what
    cos, mx = orc.cosine(y, ref), orc.max_abs(y, ref)
    assert cos >= COS and mx <= MAX_ABS, f"{what}: cosine {cos:.6f} max_abs {mx:.3e}"


def _sf_rows(sf: np.ndarray, rows: int, KB: int, B: int, NT: int, TS: int) -> np.ndarray:
    """Scale chunks [blocks, KB, chunks, 512] -> [NT, rows, KB*4].  Term t, block-local row r sit at
    virtual row v = t*TS + r: chunk v/128, byte (v%32)*16 + ((v%128)/32)*4 + j."""
    chunks = (NT * TS + 127) // 128
    c = sf.reshape(-1, KB, chunks, 32, 4, 4)                      # [blk, kb, chunk, v%32, (v%128)/32, j]
    v = c.transpose(0, 2, 4, 3, 1, 5).reshape(c.shape[0], chunks * 128, KB * 4)   # [blk, v, kb*4+j]
    return np.stack([v[:, t * TS:t * TS + B].reshape(-1, KB * 4)[:rows] for t in range(NT)])


_E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


@pytest.mark.parametrize("NT", [3, 4, 2, 1])
def test_quantised_rows_match_oracle_bit_for_bit(NT):
    T, H, I, E, K, B = 40, 288, 160, 8, 2, 32      # H, I multiples of 32 but not of 128
    x, tw, ids, w = _case(T, H, I, E, K, seed=4)
    plan = get_plan(T, K, E, E, H, I, B, 0, 7.0, torch.device(DEV), act_terms=NT)
    s_ids, _, _, nv, _ = plan.sort(ids.to(DEV), tw.to(DEV))
    plan.quant_input(x.to(DEV))
    torch.cuda.synchronize()
    n = int(nv[0])
    L = plan.ws.max_rows
    HP = (H + 255) // 256 * 256
    packed = plan.region("xq", NT * L * HP // 2).cpu().numpy().reshape(NT, L, HP // 2)[:, :n]
    codes = np.empty((NT, n, HP), dtype=np.uint8)
    codes[..., 0::2], codes[..., 1::2] = packed & 0xF, packed >> 4
    # the gate-up GEMM stacks the terms along N when that fits tensor memory twice over
    TS = B if (NT * B <= 256 and 2 * 2 * NT * B <= 448) else 128
    nch = L // B * (HP // 128) * ((NT * TS + 127) // 128) * 512
    sf = _sf_rows(plan.region("xsf", nch).cpu().numpy(), n, HP // 128, B, NT, TS)
    sid = s_ids.cpu().numpy().view(np.uint32)[:n]
    tok, kk = sid & 0xFFFFFF, sid >> 24
    ecodes, eexps = orc.fp4_terms_quant(x, NT)
    for r in range(n):
        if kk[r] < K:           # padding rows of a block are left unwritten by design
            assert np.array_equal(_E2M1[codes[:, r, :H]], _E2M1[ecodes[:, tok[r]]]), r
            assert np.array_equal(sf[:, r, :H // 32], eexps[:, tok[r]]), r
            assert not (codes[:, r, H:] & 7).any()


@pytest.mark.parametrize("T,H,I,E,K,B", [(32, 512, 256, 8, 2, 32), (40, 288, 160, 8, 2, 32), (40, 288, 160, 8, 2, 16),
                                         (150, 256, 384, 4, 2, 64), (300, 384, 128, 4, 2, 128)])
def test_gateup_stage_matches_block_oracle(T, H, I, E, K, B):
    x, tw, ids, w = _case(T, H, I, E, K, seed=T)
    pw = prepare_weights(*(t.to(DEV) for t in w))
    plan = get_plan(T, K, E, E, H, I, B, 0, 7.0, torch.device(DEV))
    plan.sort(ids.to(DEV), tw.to(DEV))
    plan.quant_input(x.to(DEV))
    h = torch.zeros(T, K, I, dtype=torch.bfloat16, device=DEV)
    plan.gateup(pw, h)
    torch.cuda.synchronize()
    plan.check_status()
    srt = orc.moe_sorting_oracle(ids, tw, E, B)
    w1 = orc.dequant_mxfp4(w[0], w[1])
    ref = orc.moe_gemm_oracle(K, B, srt[0], srt[2], srt[1], srt[3], x, w1, True)
    _assert_close(h.cpu(), ref, "gate-up")


@pytest.mark.parametrize("T,H,I,E,K,B", [(32, 512, 256, 8, 2, 32), (40, 288, 160, 8, 2, 32), (40, 288, 160, 8, 2, 16),
                                         (150, 256, 384, 4, 2, 64), (300, 384, 128, 4, 2, 128)])
def test_unfused_stage_chain_matches_layer_oracle(T, H, I, E, K, B):
    x, tw, ids, w = _case(T, H, I, E, K, seed=T + 1)
    pw = prepare_weights(*(t.to(DEV) for t in w))
    plan = get_plan(T, K, E, E, H, I, B, 0, 7.0, torch.device(DEV))
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
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    _assert_close(y.cpu(), ref, "stage chain")


@pytest.mark.parametrize("terms", [0, 2, 4])
def test_tiny_config_layer(terms):
    c = synth.CONFIGS["tiny"]
    x, tw, ids, w = _case(c.T, c.H, c.I, c.E, c.K)
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    y = _run_layer(x, tw, ids, w, act_terms=terms)
    _assert_close(y, ref, f"tiny terms={terms}")
    if terms != 2:
        assert orc.cosine(y, ref) > 0.9999


def test_layer_matches_reference_golden_vectors():
    g = np.load(GOLD / "layer_mxfp4_small.npz")
    x = _bf16(g["x"])
    tw, ids = torch.from_numpy(g["topk_weight"]), torch.from_numpy(g["topk_ids"])
    w = tuple(torch.from_numpy(g[k]) for k in ("w1_q", "w1_s", "w2_q", "w2_s"))
    _assert_close(_run_layer(x, tw, ids, w), _bf16(g["y_silu"]), "golden silu")
    _assert_close(_run_layer(x, tw, ids, w, activation=ActivationType.Swiglu, swiglu_limit=7.0),
                  _bf16(g["y_swiglu"]), "golden swiglu")


@pytest.mark.parametrize("T", [1, 2, 7, 33, 64, 257])
def test_ragged_token_counts(T):
    H, I, E, K = 288, 160, 16, 4
    x, tw, ids, w = _case(T, H, I, E, K, seed=T)
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    _assert_close(_run_layer(x, tw, ids, w), ref, f"T={T}")


@pytest.mark.parametrize("B", [16, 32, 48, 64, 80, 96, 112, 128])
def test_block_sizes_and_skew(B):
    T, H, I, E, K = 400, 256, 256, 8, 2
    x, tw, ids, w = _case(T, H, I, E, K, routing="zipf", seed=9)
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    _assert_close(_run_layer(x, tw, ids, w, block_size_M=B), ref, f"B={B}")


def test_expert_mask_drops_masked_experts():
    """Expert-parallel convention (tests/contrib/moe/test_fused_moe.py:35-44,70-81): only the
    unmasked experts' weights are present and their contributions are summed."""
    T, H, I, E, K = 64, 256, 128, 8, 2
    x, tw, ids, w = _case(T, H, I, E, K, seed=21)
    mask = torch.tensor([1, 1, 0, 0, 1, 0, 1, 0], dtype=torch.int32)
    keep = mask.bool()
    w_local = tuple(t[keep] for t in w)
    y = _run_layer(x, tw, ids, w_local, expert_mask=mask.to(DEV))
    tw_masked = tw * keep[ids.long()].float()
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw_masked, ids)
    _assert_close(y, ref, "masked")


@pytest.mark.parametrize("combine", ["gather", "fused"])
def test_single_local_expert(combine):
    """One expert of eight lives here (expert parallelism with one expert per GPU): every sorted block carries local
    id 0 and most (token, expert) pairs are dropped by the mask."""
    T, H, I, E, K = 200, 256, 128, 8, 2
    x, tw, ids, w = _case(T, H, I, E, K, routing="zipf", seed=33)
    for e in (0, 5):
        keep = torch.zeros(E, dtype=torch.bool)
        keep[e] = True
        y = _run_layer(x, tw, ids, tuple(t[keep] for t in w), expert_mask=keep.to(torch.int32).to(DEV), combine=combine)
        ref = orc.torch_moe_oracle_mxfp4(x, *w, tw * keep[ids.long()].float(), ids)
        _assert_close(y, ref, f"only expert {e} local, {combine}")


def test_deterministic_bitwise():
    T, H, I, E, K = 96, 256, 128, 8, 2
    x, tw, ids, w = _case(T, H, I, E, K, seed=5)
    a = _run_layer(x, tw, ids, w)
    b = _run_layer(x, tw, ids, w)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_empty_batch_and_argument_errors():
    H, I, E, K = 256, 128, 4, 2
    _, _, _, w = _case(4, H, I, E, K)
    w1_q, w1_s, w2_q, w2_s = (t.to(DEV) for t in w)
    y = fused_moe(torch.empty(0, H, dtype=torch.bfloat16, device=DEV), w1_q, w2_q,
                  torch.empty(0, K, device=DEV), torch.empty(0, K, dtype=torch.int32, device=DEV),
                  quant_type=QuantType.per_1x32, w1_scale=w1_s, w2_scale=w2_s)
    assert y.shape == (0, H)
    with pytest.raises(NotImplementedError):
        fused_moe(torch.zeros(1, H, dtype=torch.bfloat16, device=DEV), w1_q, w2_q, torch.ones(1, K, device=DEV),
                  torch.zeros(1, K, dtype=torch.int32, device=DEV), quant_type=QuantType.per_1x128, w1_scale=w1_s,
                  w2_scale=w2_s)
    with pytest.raises(ValueError):          # QuantType.No means bf16 weights: packed bytes are refused
        fused_moe(torch.zeros(1, H, dtype=torch.bfloat16, device=DEV), w1_q, w2_q, torch.ones(1, K, device=DEV),
                  torch.zeros(1, K, dtype=torch.int32, device=DEV), quant_type=QuantType.No)
    with pytest.raises(RuntimeError):
        fused_moe(torch.zeros(1, H, dtype=torch.bfloat16), w1_q, w2_q, torch.ones(1, K), torch.zeros(1, K),
                  quant_type=QuantType.per_1x32, w1_scale=w1_s, w2_scale=w2_s)


def test_gptoss_shape_decode_round_trip_properties():
    """Full-size shape (H = I = 2880, E = 128, top-4): the oracle is run on the experts that
    were hit only; linearity in the routing weights is checked at full size."""
    c = synth.CONFIGS["gptoss_decode"]
    T = 8
    x = synth.make_hidden(T, c.H, 1)
    tw, ids = synth.make_routing(T, c.E, c.K, seed=1)
    hit = sorted(set(ids.flatten().tolist()))
    w = synth.make_weights_mxfp4(c.E, c.H, c.I, seed=1, experts=hit)
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    y = _run_layer(x, tw, ids, w)
    _assert_close(y, ref, "gpt-oss T=8")
    y2 = _run_layer(x, tw * 0.5, ids, w)
    assert orc.cosine(y2.float() * 2, y.float()) > 0.99999


def test_gptoss_prefill_slice_scaled_bound():
    """Compute-bound regime (token tile 96, per-term MMAs) on an 8-expert slice of the gpt-oss shape.
    Outputs reach magnitude 2, where one bf16 step is 1.56e-2: the absolute bound is scaled by
    max(1, |ref|max) there (two roundings of the oracle's own chain already differ by a step)."""
    T, H, I, E, K = 1024, 2880, 2880, 8, 4
    x = synth.make_hidden(T, H, 2)
    tw, ids = synth.make_routing(T, E, K, seed=2)
    w = synth.make_weights_mxfp4(E, H, I, seed=2)
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    y = _run_layer(x, tw, ids, w)
    cos, mx = orc.cosine(y, ref), orc.max_abs(y, ref)
    bound = MAX_ABS * max(1.0, float(ref.float().abs().max()))
    assert cos >= 0.9999 and mx <= bound, f"cosine {cos:.6f} max_abs {mx:.3e} bound {bound:.3e}"


def test_gather_sum_kernel_matches_fp32_sum():
    """Expert-parallel combine kernel: fp32 accumulation in slot order, one rounding."""
    from pyhip_b200 import ep
    T, S, H, n = 300, 8, 2880, 1200
    g = torch.Generator().manual_seed(5)
    rows = torch.randn(n, H, generator=g).to(torch.bfloat16)
    pos = torch.randint(-1, n, (T, S), generator=g, dtype=torch.int32)
    pos[7] = -1                                    # a token nobody answered stays zero
    want = ep.gather_sum(rows, pos)                # CPU arithmetic
    got = ep.gather_sum(rows.to(DEV), pos.to(DEV)).cpu()
    assert torch.equal(got, want)
    assert float(got[7].float().abs().max()) == 0.0


def test_varying_token_counts_share_one_workspace():
    """Beyond 512 tokens the wrapper lays the workspace out for the count rounded up to 512, so calls whose
    batch varies (expert-parallel dispatch) reuse one allocation; results must not depend on the capacity."""
    import importlib
    fm = importlib.import_module("pyhip_b200.fused_moe")
    H, I, E, K = 512, 256, 8, 2
    w = synth.make_weights_mxfp4(E, H, I, seed=6)
    fm._workspace_cache.clear()
    for T in (600, 1000, 1024, 513):
        x = synth.make_hidden(T, H, T)
        tw, ids = synth.make_routing(T, E, K, seed=T)
        ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
        _assert_close(_run_layer(x, tw, ids, w, block_size_M=64), ref, f"T={T}")
    assert len(fm._workspace_cache) == 1


def test_num_local_tokens_padded_batch_and_graph_replay():
    """A batch padded to a fixed T with the live count on the device (the reference's num_local_tokens,
    src/contrib/fused_moe.py:48-49): live rows equal the unpadded call bit for bit, padding rows are zero,
    and one captured graph serves every count."""
    import importlib
    fm = importlib.import_module("pyhip_b200.fused_moe")
    T, H, I, E, K, B = 64, 512, 256, 8, 2, 16
    x = synth.make_hidden(T, H, 11)
    tw, ids = synth.make_routing(T, E, K, seed=11)
    w = tuple(t.to(DEV) for t in synth.make_weights_mxfp4(E, H, I, seed=11))
    xd, twd, idsd = x.to(DEV), tw.to(DEV), ids.to(DEV)
    kw = dict(quant_type=QuantType.per_1x32, w1_scale=w[1], w2_scale=w[3], block_size_M=B)
    n_dev = torch.zeros(1, dtype=torch.int32, device=DEV)
    pw = fm.prepare_weights(*w)
    plan = fm.get_plan(T, K, E, E, H, I, B, 0, 7.0, torch.device(DEV))
    y = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    graph, _ = fm.capture_forward(plan, pw, xd, twd, idsd, None, y, num_local_tokens=n_dev)
    for n in (40, 1, 64, 0, 17):
        n_dev.fill_(n)
        graph.replay()
        torch.cuda.synchronize()
        got = y.cpu()
        assert float(got[n:].float().abs().max()) == 0.0 if n < T else True
        if n:
            want = fused_moe(xd[:n], w[0], w[2], twd[:n], idsd[:n], **kw).cpu()
            assert torch.equal(got[:n], want), n
        # the public call with a host integer takes the same route
        assert torch.equal(fused_moe(xd, w[0], w[2], twd, idsd, num_local_tokens=n, **kw).cpu(), got)
    plan.check_status()


# --------------------------------------------------------------------------------------------
# fused combine, decode-sized (three-launch) path, plain MXFP4 activations, biases, stage-1 weights
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T", [1, 2, 7, 8, 33, 64, 65, 300])
def test_fused_combine_matches_oracle_and_the_gather_form(T):
    """The down epilogue that multiplies by the routing weight and adds into the output (the reference kernels'
    own epilogue, src/contrib/moe.py:703-787) against the layer oracle; the gather form is the anchor: the two
    differ only in the order of a token's K bf16 additions."""
    H, I, E, K = 288, 160, 16, 4
    x, tw, ids, w = _case(T, H, I, E, K, seed=100 + T)
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    y_f = _run_layer(x, tw, ids, w, combine="fused")
    y_g = _run_layer(x, tw, ids, w, combine="gather")
    _assert_close(y_f, ref, f"fused T={T}")
    _assert_close(y_g, ref, f"gather T={T}")
    assert orc.max_abs(y_f, y_g) <= 2 ** -7 * max(1.0, float(ref.float().abs().max()))   # a bf16 step or two


@pytest.mark.parametrize("T,E,K,mask", [(1, 128, 4, False), (2, 16, 4, False), (7, 16, 4, True), (8, 128, 4, False),
                                        (64, 128, 4, False), (32, 256, 8, False), (64, 16, 4, True)])
def test_small_batch_path_sorts_bit_exactly(T, E, K, mask):
    """Up to 256 (token, expert) pairs the sort runs inside the quantiser launch (every CTA repeats it): the
    sort arrays it leaves in the workspace must equal the oracle's over the defined prefix."""
    H, I = 256, 128
    x = synth.make_hidden(T, H, T)
    tw, ids = synth.make_routing(T, E, K, seed=T + E)
    m = None
    if mask:
        m = torch.tensor([1, 0] * (E // 2), dtype=torch.int32)
    E_local = E if m is None else int(m.sum())
    w = synth.make_weights_mxfp4(E_local, H, I, seed=3)
    pw = prepare_weights(*(t.to(DEV) for t in w))
    B = 16
    plan = get_plan(T, K, E_local, E, H, I, B, 0, 7.0, torch.device(DEV), combine_mode=1)
    from pyhip_b200.fused_moe import moe_forward
    y = moe_forward(plan, pw, x.to(DEV), tw.to(DEV), ids.to(DEV), None if m is None else m.to(DEV))
    torch.cuda.synchronize()
    plan.check_status()
    s_ids, s_w, s_e, nv, loc = (t.cpu().numpy() for t in plan.sort_outputs())
    exp = orc.moe_sorting_oracle(ids, tw, E, B, expert_mask=None if m is None else m.tolist())
    n = int(exp[3][0])
    assert nv.tolist() == exp[3].tolist()
    assert np.array_equal(s_ids.view(np.uint32)[:n], exp[0][:n])
    assert np.array_equal(s_w[:n].view(np.uint32), exp[1][:n].view(np.uint32))
    assert np.array_equal(s_e[:n // B], exp[2][:n // B])
    # loc is the inverse map: pair (t, k) -> sorted position, -1 when its expert is masked out
    live = (exp[0][:n] >> 24) < K
    pos = np.nonzero(live)[0]
    pair = (exp[0][:n][live] & 0xFFFFFF) * K + (exp[0][:n][live] >> 24)
    want = np.full(T * K, -1, dtype=np.int32)
    want[pair] = pos
    assert np.array_equal(loc[:T * K], want)
    tw_m = tw if m is None else tw * m.bool()[ids.long()].float()
    keep = None if m is None else m.bool()
    w_full = w if m is None else tuple(_expand(t, keep) for t in w)
    _assert_close(y.cpu(), orc.torch_moe_oracle_mxfp4(x, *w_full, tw_m, ids), "small path layer")


@pytest.mark.parametrize("H,I,E,K", [(256, 128, 8, 2), (288, 160, 16, 4), (2880, 2880, 8, 4), (1024, 96, 4, 1), (96, 4096, 16, 8)])
def test_batch1_path_matches_the_oracle(H, I, E, K):
    """method="batch1": one token in two launches, no sort and no activation quantiser (the reference's
    moe_gemm_batch1, src/contrib/moe.py:41-188).  Against the layer oracle with bf16 activations; bitwise
    reproducible; the default (sorted tensor-core) path on the same input agrees to a bf16 step."""
    from pyhip_b200.fused_moe import batch1_eligible
    from pyhip_b200 import _lib
    assert batch1_eligible(1, K, H, I, _lib.W_MXFP4, 0) and not batch1_eligible(2, K, H, I, _lib.W_MXFP4, 0)
    assert not batch1_eligible(1, K, H, I, _lib.W_MXFP4, 1) and not batch1_eligible(1, K, H, I, _lib.W_FP8_128, 0)
    x, tw, ids, w = _case(1, H, I, E, K, seed=H + K)
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    y = _run_layer(x, tw, ids, w, method="batch1")
    _assert_close(y, ref, "batch-1")
    assert torch.equal(y.view(torch.int16), _run_layer(x, tw, ids, w, method="batch1").view(torch.int16))
    y_s = _run_layer(x, tw, ids, w)
    _assert_close(y_s, ref, "sorted path, one token")
    with pytest.raises(ValueError):
        _run_layer(torch.cat([x, x]), torch.cat([tw, tw]), torch.cat([ids, ids]), w, method="batch1")
    assert orc.max_abs(y, y_s) <= 2 ** -6 * max(1.0, float(ref.float().abs().max()))


@pytest.mark.parametrize("activation", ["silu", "swiglu"])
def test_batch1_mask_biases_stage1_weights_and_padding(activation):
    H, I, E, K = 288, 160, 8, 3
    x, tw, ids, w = _case(1, H, I, E, K, seed=77)
    g = torch.Generator().manual_seed(5)
    b1 = (torch.randn(E, 2 * I, generator=g) * 0.1).to(torch.bfloat16)
    b2 = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16)
    act = ActivationType.Silu if activation == "silu" else ActivationType.Swiglu
    okw = dict(activation=activation, swiglu_limit=7.0)
    y = _run_layer(x, tw, ids, w, activation=act, bias1=b1.to(DEV), bias2=b2.to(DEV), method="batch1")
    _assert_close(y, orc.torch_moe_oracle_mxfp4(x, *w, tw, ids, bias1=b1, bias2=b2, **okw), "biases")
    y = _run_layer(x, tw, ids, w, activation=act, doweight_stage1=True, method="batch1")
    _assert_close(y, orc.torch_moe_oracle_mxfp4(x, *w, tw, ids, doweight_stage1=True, **okw), "stage-1 weights")
    keep = torch.ones(E, dtype=torch.bool)
    keep[int(ids[0, 0])] = False                       # the token's first expert lives on another rank
    keep[(int(ids[0, 1]) + 1) % E] = keep[(int(ids[0, 1]) + 1) % E] and True
    y = _run_layer(x, tw, ids, tuple(t[keep] for t in w), activation=act, expert_mask=keep.to(torch.int32).to(DEV),
                   method="batch1")
    _assert_close(y, orc.torch_moe_oracle_mxfp4(x, *w, tw * keep[ids.long()].float(), ids, **okw), "mask")
    y = _run_layer(x, tw, ids, w, activation=act, num_local_tokens=0, method="batch1")
    assert float(y.float().abs().max()) == 0.0


def _expand(t, keep):
    """local expert tensors -> full-size tensor with the masked experts left at zero."""
    full = torch.zeros((keep.numel(),) + tuple(t.shape[1:]), dtype=t.dtype)
    full[keep] = t
    return full


@pytest.mark.parametrize("T,H,I,E,K", [(32, 512, 256, 8, 2), (300, 288, 160, 16, 4), (5, 2880, 2880, 4, 2)])
def test_plain_mxfp4_activations_match_the_a4w4_oracle(T, H, I, E, K):
    """act_terms = 1 is the reference's a4w4 arithmetic (per-1x32 MXFP4 activations): parity is against the
    oracle that dequantises the same quantised activations, with the reference's own threshold
    (calc_diff <= 0.01, tests/contrib/moe/test_mxfp4.py:286-299); the distance to the bf16-activation oracle is
    reported, not asserted."""
    x, tw, ids, w = _case(T, H, I, E, K, seed=T + 7)
    ref_q = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids, act_quant="mxfp4")
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
    for combine in ("gather", "fused"):
        y = _run_layer(x, tw, ids, w, act_terms=1, combine=combine)
        d = orc.calc_diff(y, ref_q)
        assert d <= 0.01 and orc.cosine(y, ref_q) >= 0.995, f"{combine}: calc_diff {d:.4f} cosine {orc.cosine(y, ref_q):.5f}"
        print(f"a4w4 T={T} {combine}: calc_diff vs a4w4 oracle {d:.2e}, cosine vs bf16-activation oracle "
              f"{orc.cosine(y, ref):.5f}")


@pytest.mark.parametrize("combine", ["gather", "fused"])
@pytest.mark.parametrize("activation", ["silu", "swiglu"])
def test_biases_and_stage1_weights(combine, activation):
    T, H, I, E, K = 70, 288, 160, 8, 2
    x, tw, ids, w = _case(T, H, I, E, K, seed=51)
    g = torch.Generator().manual_seed(9)
    b1 = (torch.randn(E, 2 * I, generator=g) * 0.1).to(torch.bfloat16)
    b2 = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16)
    act = ActivationType.Silu if activation == "silu" else ActivationType.Swiglu
    for kw, okw in ((dict(bias1=b1.to(DEV), bias2=b2.to(DEV)), dict(bias1=b1, bias2=b2)),
                    (dict(doweight_stage1=True), dict(doweight_stage1=True)),
                    (dict(bias1=b1.to(DEV), doweight_stage1=True), dict(bias1=b1, doweight_stage1=True))):
        ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids, activation=activation, swiglu_limit=7.0, **okw)
        y = _run_layer(x, tw, ids, w, activation=act, combine=combine, **kw)
        _assert_close(y, ref, f"{sorted(kw)} {combine} {activation}")


def test_prepared_scale_image_known_answer():
    """b200moe_prepare_scales against the byte formula of the scale chunks: chunk (e, m-tile, k-block, part),
    byte (r % 32) * 16 + (r / 32) * 4 + j holds the scale of weight row r of the tile and 32-block 4*kb + j;
    rows and k-blocks that do not exist read 127."""
    E, H, I = 3, 288, 160            # neither a multiple of 128
    g = torch.Generator().manual_seed(2)
    s1 = torch.randint(100, 140, (E, 2 * I, H // 32), dtype=torch.uint8, generator=g)
    s2 = torch.randint(100, 140, (E, H, I // 32), dtype=torch.uint8, generator=g)
    w1 = torch.zeros(E, 2 * I, H // 2, dtype=torch.uint8)
    w2 = torch.zeros(E, H, I // 2, dtype=torch.uint8)
    pw = prepare_weights(w1.to(DEV), s1.to(DEV), w2.to(DEV), s2.to(DEV))
    torch.cuda.synchronize()
    for which, src, rows, Kd, got in ((1, s1.numpy(), I, H, pw.w1_scale.cpu().numpy()),
                                      (2, s2.numpy(), H, I, pw.w2_scale.cpu().numpy())):
        KB = (Kd + 255) // 256 * 2
        MT = (rows + 127) // 128 if which == 1 else (rows + 255) // 256
        img = got.reshape(E, MT, KB, 2, 512)
        want = np.full_like(img, 127)
        for e in range(E):
            for mt in range(MT):
                for part in range(2):
                    for r in range(128):
                        row_in = mt * 128 + r if which == 1 else (2 * mt + part) * 128 + r
                        if row_in >= rows:
                            continue
                        row = part * rows + row_in if which == 1 else row_in
                        for kb in range(KB):
                            for j in range(4):
                                if kb * 4 + j < Kd // 32:
                                    want[e, mt, kb, part, (r % 32) * 16 + (r // 32) * 4 + j] = src[e, row, kb * 4 + j]
        assert np.array_equal(img, want), which


# --------------------------------------------------------------------------------------------
# CTA pairs (tcgen05.mma.cta_group::2): the same layer, bit for bit
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,H,I,E,K,B,terms", [(300, 384, 128, 4, 2, 96, 0), (150, 256, 384, 4, 2, 64, 4), (400, 512, 256, 8, 2, 80, 3),
                                               (260, 288, 160, 4, 2, 96, 1), (1, 256, 128, 4, 2, 96, 0), (700, 2880, 384, 4, 2, 96, 0)])
def test_cta_pairs_match_the_single_cta_kernels_bit_for_bit(T, H, I, E, K, B, terms):
    """Two CTAs of a cluster share one token tile (each fetches half of it, the even CTA issues M = 256 MMAs for both):
    products and accumulation order per output element are those of the single-CTA kernels, so the deterministic
    (GATHER) layer output must be identical bit for bit -- and within the tolerance of the oracle like any other."""
    x, tw, ids, w = _case(T, H, I, E, K, seed=300 + T)
    kw = dict(block_size_M=B, act_terms=terms, combine="gather")
    y_off = _run_layer(x, tw, ids, w, cta_pairs="off", **kw)
    y_on = _run_layer(x, tw, ids, w, cta_pairs="on", **kw)
    assert torch.equal(y_on.view(torch.int16), y_off.view(torch.int16))
    ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids, **({"act_quant": "mxfp4"} if terms == 1 else {}))
    if terms == 1:
        assert orc.calc_diff(y_on, ref) <= 0.01
    else:
        cos, mx = orc.cosine(y_on, ref), orc.max_abs(y_on, ref)
        assert cos >= COS and mx <= MAX_ABS * max(1.0, float(ref.float().abs().max())), (cos, mx)
    y_f = _run_layer(x, tw, ids, w, cta_pairs="on", block_size_M=B, act_terms=terms, combine="fused")
    assert orc.max_abs(y_f, y_on) <= 2 ** -6 * max(1.0, float(ref.float().abs().max()))
