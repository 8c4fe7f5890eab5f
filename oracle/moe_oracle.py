"""CPU oracle for the quantised fused-MoE path.  TEST INFRASTRUCTURE ONLY.

This file restates, for the CPU, the algorithms the reference (tingqli/pyhip) uses to judge
its own MoE kernels.  Nothing in the shipped package imports it: only tests, the smoke check
and the benchmark's CPU-baseline leg do.  Each function names the reference lines it follows.

Pinning: `torch_moe_oracle` and `moe_sorting_oracle` are checked bit-for-bit against outputs of
the reference's own functions (extracted from its test files and executed on CPU) stored under
tests/golden/, and the sorter additionally against the worked example in the reference's
sorting-kernel documentation.  The MXFP4 / FP8 weight quantisers of the reference live in an
un-vendored third-party module (aiter, no pinned version); for them the parity is unpinned and
the encodings follow ck_tile's numeric headers instead (pk_fp4.hpp, e8m0.hpp).
"""
from __future__ import annotations

import numpy as np
import torch

_E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                  -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


# --------------------------------------------------------------------------------------
# metrics
# --------------------------------------------------------------------------------------
def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x,y>/(|x|^2+|y|^2) in float64 (src/misc.py:131-141)."""
    x, y = x.double(), y.double()
    den = (x * x + y * y).sum()
    if den == 0:
        return 0.0
    return float(1 - 2 * (x * y).sum() / den)


def cosine(x: torch.Tensor, y: torch.Tensor) -> float:
    x, y = x.double().flatten(), y.double().flatten()
    den = x.norm() * y.norm()
    if den == 0:
        return 1.0 if x.norm() == y.norm() else 0.0
    return float((x @ y) / den)


def max_abs(x: torch.Tensor, y: torch.Tensor) -> float:
    return float((x.double() - y.double()).abs().max()) if x.numel() else 0.0


# --------------------------------------------------------------------------------------
# weight formats
# --------------------------------------------------------------------------------------
_E2M1_PAIRS = torch.from_numpy(np.stack([_E2M1[np.arange(256) & 0xF], _E2M1[np.arange(256) >> 4]], axis=1))


def dequant_mxfp4(packed: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """Packed E2M1 (low nibble = even element) times 2**(e-127) per 32 along K, then cast
    (tests/contrib/moe/test_moe.py:164-166; pk_fp4.hpp:122-129; e8m0.hpp:12-24).  A 256-entry table maps a
    byte to its two values, so the work is one gather and one multiply (threaded by torch)."""
    packed = packed.cpu()
    vals = _E2M1_PAIRS[packed.long()].reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    K = vals.shape[-1]
    sc = torch.ldexp(torch.ones(scale.shape, dtype=torch.float32), scale.cpu().int() - 127)
    out = vals.reshape(*vals.shape[:-1], K // 32, 32) * sc.unsqueeze(-1)
    return out.reshape(vals.shape).to(dtype)


def dequant_fp8_128x128(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """e4m3 value cast to bf16, times the fp32 scale of its 128x128 block, cast to bf16
    (tests/contrib/moe/test_moe.py:243-245)."""
    *lead, N, K = q.shape
    blk = q.to(dtype).reshape(*lead, N // 128, 128, K // 128, 128)
    out = (blk * scale.reshape(*lead, N // 128, 1, K // 128, 1)).to(dtype)
    return out.reshape(*lead, N, K)


def dequant_fp8_rows(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """e4m3 value cast to bf16 times the fp32 scale of its output row (or of its expert), cast to bf16
    (tests/contrib/moe/test_moe.py:127,136).  q [..., N, K]; scale [..., N] or [...] (per tensor)."""
    sc = scale.float()
    sc = sc.reshape(*sc.shape, 1, 1) if sc.dim() == q.dim() - 2 else sc.unsqueeze(-1)
    return (q.to(dtype) * sc).to(dtype)


# --------------------------------------------------------------------------------------
# token -> expert sort / align
# --------------------------------------------------------------------------------------
def moe_sorting_oracle(topk_ids, topk_weights, num_experts: int, block_size: int,
                       expert_mask=None):
    """Group (token, k) pairs by expert, stable in token-major order, pad every non-empty
    expert to a multiple of ``block_size`` with the sentinel (topk<<24)|num_tokens and weight
    0, one expert id per block.

    Follows src/contrib/fused_moe.py:56-100 (with the pad length being ``block_size`` rather
    than that function's literal 256) and ck_tile's reference_moe_sorting with
    skip_experts_with_zero_token=true and the (k<<24)|token packing
    (archive/ck_tile/ck_tile/host/reference/reference_moe_sorting.hpp:14-117): a masked-out
    expert emits nothing and does not advance the emitted (local) expert id; an empty
    unmasked expert emits nothing but does advance it.

    Returns numpy arrays (sorted_ids u32, sorted_weights f32, sorted_expert_ids i32,
    num_valid_ids i32[2]); the arrays are sized to the worst case and only the prefix
    [0, num_valid_ids[0]) is defined (the tail is filled with sentinel / 0 / -1 here)."""
    ids = np.asarray(topk_ids.cpu() if torch.is_tensor(topk_ids) else topk_ids).astype(np.int64)
    w = np.asarray(topk_weights.cpu() if torch.is_tensor(topk_weights) else topk_weights,
                   dtype=np.float32)
    T, K = ids.shape
    B = block_size
    nblk_max = (T * K + num_experts * (B - 1) + B - 1) // B
    sentinel = np.uint32((K << 24) | T)
    sorted_ids = np.full(nblk_max * B, sentinel, dtype=np.uint32)
    sorted_w = np.zeros(nblk_max * B, dtype=np.float32)
    sorted_e = np.full(nblk_max, -1, dtype=np.int32)

    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")           # token-major, then k, inside an expert
    counts = np.bincount(flat, minlength=num_experts)[:num_experts]
    tok = (order // K).astype(np.uint32)
    kk = (order % K).astype(np.uint32)
    packed = (kk << np.uint32(24)) | tok
    starts = np.concatenate([[0], np.cumsum(counts)])

    pos = 0
    local_id = 0
    for e in range(num_experts):
        if expert_mask is not None and int(expert_mask[e]) == 0:
            continue
        n = int(counts[e])
        if n == 0:
            local_id += 1
            continue
        sl = slice(starts[e], starts[e] + n)
        sorted_ids[pos:pos + n] = packed[sl]
        sorted_w[pos:pos + n] = w.reshape(-1)[order[sl]]
        nb = (n + B - 1) // B
        sorted_e[pos // B: pos // B + nb] = local_id
        pos += nb * B
        local_id += 1
    num_valid = np.array([pos, T], dtype=np.int32)
    return sorted_ids, sorted_w, sorted_e, num_valid


# --------------------------------------------------------------------------------------
# end-to-end layer
# --------------------------------------------------------------------------------------
def _gateup_activation(gate, up, activation="silu", swiglu_limit=None):
    """tests/contrib/moe/test_moe.py:73-83."""
    if activation == "silu":
        return torch.nn.functional.silu(gate) * up
    if activation == "swiglu":
        lim = float(swiglu_limit) if swiglu_limit else 7.0
        dt = gate.dtype
        g = gate.float().clamp(max=lim)
        u = up.float().clamp(min=-lim, max=lim)
        return (g * torch.sigmoid(1.702 * g) * (u + 1.0)).to(dt)
    raise ValueError(activation)


def act_quant_mxfp4(x: torch.Tensor) -> torch.Tensor:
    """Per-1x32 MXFP4 activation quantiser followed by its dequantisation: E8M0 scale
    2**(floor(log2 amax) - 2) per 32 along K (the OCP MX rule), E2M1 codes rounded to nearest even with
    saturation.  This is the a4w4 activation format of the reference (aiter's per_1x32 quantiser,
    tests/contrib/moe/test_moe.py:665-679; dequantised for the check exactly as
    tests/contrib/moe/test_mxfp4.py:102-236 and src/contrib/moe_gemm_ref.py:82-89,114-123 do).  aiter itself is
    not vendored, so its rounding of ties / the scale is unpinned; encodings follow pk_fp4.hpp / e8m0.hpp."""
    codes, exps = fp4_terms_quant(x, 1)
    return fp4_terms_dequant(codes, exps).to(x.dtype)


def act_quant_fp8_1x128(x: torch.Tensor):
    """Per-token, per-128-channel e4m3 quantiser with an fp32 scale = amax / 448 (1.0 for an all-zero block):
    the reference's per_1x128 activation format (src/contrib/fused_moe.py:276-281,375-381; the only in-repo
    statement of the rule is the per-tensor one, tests/contrib/moe/test_moe.py:130-137).
    Returns (q float8_e4m3fn [..., K], scale float32 [..., K/128])."""
    xf = x.float()
    K = xf.shape[-1]
    blk = xf.reshape(*xf.shape[:-1], K // 128, 128)
    amax = blk.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (blk / scale.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.reshape(xf.shape), scale


def act_dequant_fp8_1x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 values of a 1x128-quantised tensor (src/contrib/moe_gemm_ref.py:72-80)."""
    K = q.shape[-1]
    return (q.float().reshape(*q.shape[:-1], K // 128, 128) * scale.unsqueeze(-1)).reshape(q.shape)


def torch_moe_oracle(hidden, w1, w2, topk_weight, topk_ids, activation="silu",
                     swiglu_limit=None, expert_weights=None, act_quant="none", bias1=None, bias2=None,
                     doweight_stage1=False):
    """The reference's dequantise-then-matmul layer (tests/contrib/moe/test_moe.py:86-118):
    expert by expert, bf16 matmuls, silu(gate)*up, times the routing weight, cast to the
    activation dtype and accumulated into the output with index_add_ in expert order.

    ``w1`` [E,2I,H] / ``w2`` [E,H,I] are dequantised weights in the activation dtype, or
    ``expert_weights(e) -> (w1_e, w2_e)`` produces them one expert at a time (bounds host
    memory for the large configurations).

    ``act_quant``: "none" (bf16 activations, the layer oracle as written), "mxfp4" (x and h pass through
    the per-1x32 MXFP4 quantiser first: the a4w4 check of tests/contrib/moe/test_mxfp4.py) or "fp8_1x128"
    (x and h pass through the per-token 1x128 e4m3 quantiser and the products are formed in fp32, as
    src/contrib/moe_gemm_ref.py:72-80,126 does).
    ``bias1`` [E, 2I] / ``bias2`` [E, H]: per-expert biases added to the (bf16) projection outputs -- the
    reference asserts them absent (src/contrib/fused_moe.py:262-263), the semantics are the gpt-oss layer's.
    ``doweight_stage1``: the routing weight multiplies h instead of the down output
    (tests/contrib/moe/test_fused_moe.py:280,311)."""
    T, H = hidden.shape
    ids = topk_ids.long()
    out = torch.zeros((T, H), dtype=hidden.dtype)
    E = w1.shape[0] if expert_weights is None else None
    e_list = range(E) if expert_weights is None else sorted(e for e in set(ids.flatten().tolist()) if e >= 0)
    ids_kt = ids.t().contiguous()                     # [K, T]: where() walks k-major like the
    if act_quant == "mxfp4":
        hidden_q = act_quant_mxfp4(hidden)
    elif act_quant == "fp8_1x128":
        hidden_q = act_dequant_fp8_1x128(*act_quant_fp8_1x128(hidden))       # fp32
    elif act_quant == "none":
        hidden_q = hidden
    else:
        raise ValueError(act_quant)

    def mm(a, w):
        if act_quant == "fp8_1x128":
            return (a.float() @ w.float().t()).to(hidden.dtype)
        return a @ w.t()

    for e in e_list:                                  # reference's permuted one-hot mask
        k_idx, t_idx = torch.where(ids_kt == e)
        if t_idx.numel() == 0:
            continue
        w1_e, w2_e = (w1[e], w2[e]) if expert_weights is None else expert_weights(e)
        inter = w1_e.shape[0] // 2
        cur = hidden_q[t_idx]
        gate, up = mm(cur, w1_e[:inter]), mm(cur, w1_e[inter:])
        if bias1 is not None:
            gate = gate + bias1[e, :inter].to(gate.dtype)
            up = up + bias1[e, inter:].to(up.dtype)
        act = _gateup_activation(gate, up, activation, swiglu_limit)
        wts = topk_weight[t_idx, k_idx, None]
        if doweight_stage1:
            act = (act * wts).to(hidden.dtype)
        if act_quant == "mxfp4":
            act = act_quant_mxfp4(act)
        elif act_quant == "fp8_1x128":
            act = act_dequant_fp8_1x128(*act_quant_fp8_1x128(act))
        y = mm(act, w2_e)
        if bias2 is not None:
            y = y + bias2[e].to(y.dtype)
        if not doweight_stage1:
            y = y * wts
        out.index_add_(0, t_idx, y.to(hidden.dtype))
    return out


def torch_moe_oracle_mxfp4(hidden, w1_q, w1_s, w2_q, w2_s, topk_weight, topk_ids, **kw):
    """Same layer from packed MXFP4 tensors; dequantises one expert at a time."""
    def ew(e):
        return dequant_mxfp4(w1_q[e], w1_s[e], hidden.dtype), dequant_mxfp4(w2_q[e], w2_s[e], hidden.dtype)
    return torch_moe_oracle(hidden, None, None, topk_weight, topk_ids, expert_weights=ew, **kw)


def torch_moe_oracle_fp8(hidden, w1_q, w1_s, w2_q, w2_s, topk_weight, topk_ids, row_scaled=False, **kw):
    def ew(e):
        if row_scaled:
            return dequant_fp8_rows(w1_q[e], w1_s[e], hidden.dtype), dequant_fp8_rows(w2_q[e], w2_s[e], hidden.dtype)
        return (dequant_fp8_128x128(w1_q[e], w1_s[e], hidden.dtype),
                dequant_fp8_128x128(w2_q[e], w2_s[e], hidden.dtype))
    return torch_moe_oracle(hidden, None, None, topk_weight, topk_ids, expert_weights=ew, **kw)


# --------------------------------------------------------------------------------------
# per-stage (sorted-block) form, as the reference's block reference does it
# --------------------------------------------------------------------------------------
def moe_gemm_oracle(topk: int, block_m: int, sorted_ids, sorted_expert_ids, sorted_weights,
                    num_valid_ids, inp, weight, is_gateup: bool, out_dtype=torch.bfloat16):
    """One grouped GEMM driven by the sort arrays, fp32 matmul per live block
    (src/contrib/moe_gemm_ref.py:93-141).  ``weight`` is dequantised [E, OC, IC].
    gate-up: inp [T,H] -> out [T,topk,OC/2] (silu(g)*u);  down: inp [T,topk,IC] -> out [T,OC]
    accumulated with the routing weights in block order."""
    sorted_ids = torch.as_tensor(np.asarray(sorted_ids).astype(np.int64))
    sorted_expert_ids = np.asarray(sorted_expert_ids)
    sorted_weights = torch.as_tensor(np.asarray(sorted_weights))
    T = inp.shape[0]
    OC = weight.shape[1]
    out = torch.zeros((T, topk, OC // 2) if is_gateup else (T, OC), dtype=out_dtype)
    for b in range(len(sorted_expert_ids)):
        if b * block_m >= int(num_valid_ids[0]):
            break
        ids = sorted_ids[b * block_m:(b + 1) * block_m]
        tok, kk = ids & 0xFFFFFF, ids >> 24
        valid = kk < topk
        w_e = weight[int(sorted_expert_ids[b])].float()
        src = inp[tok[valid]] if is_gateup else inp[tok[valid], kk[valid]]
        act = src.float() @ w_e.t()
        if is_gateup:
            act = torch.nn.functional.silu(act[:, :OC // 2]) * act[:, OC // 2:]
            out[tok[valid], kk[valid]] = act.to(out_dtype)
        else:
            tw = sorted_weights[b * block_m:(b + 1) * block_m][valid]
            out[tok[valid]] += act.to(out_dtype) * tw[:, None]
    return out


# --------------------------------------------------------------------------------------
# activation quantiser used by the sm_100a kernels (sum of packed-FP4 terms, E8M0 scale per 32)
# --------------------------------------------------------------------------------------
def _biased_exponent(a: np.ndarray) -> np.ndarray:
    """Biased exponent field of float32 ``a`` (= floor(log2 a)+127 for normal a)."""
    return ((a.astype(np.float32).view(np.uint32) >> 23) & 0xFF).astype(np.int32)


def _e2m1_rne(v: np.ndarray) -> np.ndarray:
    """float32 -> E2M1 code (round to nearest, ties to the even code, saturating at 6; the sign
    bit is kept even when the magnitude rounds to zero)."""
    a = np.abs(v)
    code = ((a > 0.25).astype(np.uint8) + (a >= 0.75) + (a > 1.25) + (a >= 1.75) + (a > 2.5)
            + (a >= 3.5) + (a > 5.0)).astype(np.uint8)
    return code | (np.signbit(v).astype(np.uint8) << 3)


def fp4_terms_quant(x: torch.Tensor, terms: int = 3):
    """Restatement of the device activation quantiser.  Per 32 along K and per term t:
    e = max(biased_exponent(amax(r)) - 2, 0), code = e2m1_rne(r * 2**(127-e)),
    r <- r - value(code) * 2**(e-127), starting from r = x.
    Returns (codes uint8 [terms, ..., K], exps uint8 [terms, ..., K/32])."""
    xf = x.float().numpy()
    K = xf.shape[-1]
    r = xf.reshape(xf.shape[:-1] + (K // 32, 32)).copy()
    codes, exps = [], []
    for _ in range(terms):
        amax = np.abs(r).max(axis=-1)
        e = np.maximum(_biased_exponent(amax) - 2, 0)
        inv = np.ldexp(np.float32(1.0), 127 - e).astype(np.float32)
        c = _e2m1_rne(r * inv[..., None])
        r = r - _E2M1[c] * np.ldexp(np.float32(1.0), e - 127).astype(np.float32)[..., None]
        codes.append(c.reshape(xf.shape))
        exps.append(e.astype(np.uint8))
    return np.stack(codes), np.stack(exps)


def fp4_terms_dequant(codes: np.ndarray, exps: np.ndarray) -> torch.Tensor:
    K = codes.shape[-1]
    v = _E2M1[codes].reshape(codes.shape[:-1] + (K // 32, 32))
    v = v * np.ldexp(np.float32(1.0), exps.astype(np.int32) - 127).astype(np.float32)[..., None]
    return torch.from_numpy(v.reshape(codes.shape).sum(axis=0))


def e4m3_terms_quant(x: torch.Tensor, terms: int = 2):
    """Activation operand of the FP8 GEMMs: per 32 along K and per term,
    e = max(biased_exponent(amax(r)) - 7, 0), q = e4m3_rne(r * 2**(127-e)), r <- r - q * 2**(e-127).
    Returns (q float8_e4m3fn [terms, ..., K], exps uint8 [terms, ..., K/32])."""
    xf = x.float().numpy()
    K = xf.shape[-1]
    r = xf.reshape(xf.shape[:-1] + (K // 32, 32)).copy()
    qs, exps = [], []
    for _ in range(terms):
        amax = np.abs(r).max(axis=-1)
        e = np.maximum(_biased_exponent(amax) - 7, 0)
        inv = np.ldexp(np.float32(1.0), 127 - e).astype(np.float32)
        q = torch.from_numpy(np.ascontiguousarray(r * inv[..., None], dtype=np.float32)).clamp(-448.0, 448.0) \
            .to(torch.float8_e4m3fn)
        r = r - q.float().numpy() * np.ldexp(np.float32(1.0), e - 127).astype(np.float32)[..., None]
        qs.append(q.reshape(xf.shape))
        exps.append(e.astype(np.uint8))
    return torch.stack(qs), np.stack(exps)
