"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (the reference measures on no public dataset; its tests draw random tensors,
tests/contrib/moe/test_moe.py:140-270).

Weights are drawn per expert from generator seed (seed, e) so that large configurations never
materialise a full fp32 tensor; routing follows each configuration's stated recipe.
"""
from __future__ import annotations

import dataclasses
import math

import torch

from . import quant


@dataclasses.dataclass(frozen=True)
class MoEShape:
    name: str
    H: int
    I: int
    E: int
    K: int
    T: int
    wq: str = "mxfp4"           # "mxfp4" | "fp8_128"
    routing: str = "softmax"    # "softmax" | "sigmoid" | "zipf"


CONFIGS = {
    "tiny": MoEShape("tiny", 512, 256, 8, 2, 32),
    "gptoss_decode": MoEShape("gptoss_decode", 2880, 2880, 128, 4, 64),
    "gptoss_prefill": MoEShape("gptoss_prefill", 2880, 2880, 128, 4, 8192),
    "dsv3_ep": MoEShape("dsv3_ep", 7168, 2048, 256, 8, 4096, wq="fp8_128", routing="sigmoid"),
    "mixtral_skew": MoEShape("mixtral_skew", 4096, 14336, 8, 2, 16384, routing="zipf"),
}


ZIPF_BIAS = 1.0


def make_routing(T: int, E: int, K: int, routing: str = "softmax", seed: int = 0, skew_seed=None):
    """fp32 N(0,1) logits -> (topk_weight f32 [T,K], topk_ids i32 [T,K]).

    softmax: softmax -> top-k -> renormalise.  sigmoid: sigmoid -> top-k -> renormalise.
    zipf: logits + b_e with b_e = -ZIPF_BIAS*ln(rank_e) under a seeded rank permutation, then the softmax
    recipe.  The coefficient is calibrated on the measured load, not taken from the target law: with N(0,1)
    logit noise and top-k selection without replacement a coefficient of 1.2 gives a load that falls like
    rank^-1.48; 1.0 gives rank^-1.23, the closest to the Zipf(s = 1.2) load the configuration names
    (measured shares at T=16384, E=8, top-2: 0.361 0.221 0.139 0.096 0.066 0.050 0.037 0.030 against
    Zipf(1.2) 0.429 0.187 0.115 0.081 0.062 0.050 0.042 0.035; the head is capped at 1/K by top-k).
    ``skew_seed``: draw that permutation from its own generator, so that ranks with different ``seed``
    share one expert popularity order."""
    g = torch.Generator().manual_seed(seed * 1000003 + 17)
    logits = torch.randn(T, E, generator=g, dtype=torch.float32)
    if routing == "zipf":
        gp = g if skew_seed is None else torch.Generator().manual_seed(skew_seed * 1000003 + 41)
        rank = torch.randperm(E, generator=gp).float() + 1.0
        logits = logits + (-ZIPF_BIAS * torch.log(rank))[None, :]
    scores = torch.sigmoid(logits) if routing == "sigmoid" else torch.softmax(logits, dim=-1)
    w, ids = torch.topk(scores, K, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return w.contiguous(), ids.to(torch.int32).contiguous()


def make_hidden(T: int, H: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed * 1000003 + 29)
    return torch.randn(T, H, generator=g, dtype=torch.float32).to(torch.bfloat16)


def _expert_weight(e: int, rows: int, cols: int, seed: int, which: int) -> torch.Tensor:
    g = torch.Generator().manual_seed((seed * 1000003 + 31 + which) * 65537 + e)
    return torch.randn(rows, cols, generator=g, dtype=torch.float32) * 0.02


def make_weights_mxfp4(E: int, H: int, I: int, seed: int = 0, experts=None):
    """w1 [E,2I,H] (gate rows then up rows) and w2 [E,H,I], N(0,0.02), MXFP4-quantised.
    Returns (w1_q u8 [E,2I,H/2], w1_s u8 [E,2I,H/32], w2_q u8 [E,H,I/2], w2_s u8 [E,H,I/32]).
    ``experts``: optional iterable of expert ids to actually draw (others stay zero)."""
    w1_q = torch.zeros(E, 2 * I, H // 2, dtype=torch.uint8)
    w1_s = torch.full((E, 2 * I, H // 32), 127, dtype=torch.uint8)
    w2_q = torch.zeros(E, H, I // 2, dtype=torch.uint8)
    w2_s = torch.full((E, H, I // 32), 127, dtype=torch.uint8)
    for e in (range(E) if experts is None else experts):
        w1_q[e], w1_s[e] = quant.quantize_mxfp4(_expert_weight(e, 2 * I, H, seed, 0))
        w2_q[e], w2_s[e] = quant.quantize_mxfp4(_expert_weight(e, H, I, seed, 1))
    return w1_q, w1_s, w2_q, w2_s


def make_weights_bf16(E: int, H: int, I: int, seed: int = 0):
    """Unquantised weights of the same draw: w1 bf16 [E,2I,H] (gate rows then up rows), w2 bf16 [E,H,I]."""
    w1 = torch.stack([_expert_weight(e, 2 * I, H, seed, 0) for e in range(E)]).to(torch.bfloat16)
    w2 = torch.stack([_expert_weight(e, H, I, seed, 1) for e in range(E)]).to(torch.bfloat16)
    return w1, w2


def make_weights_mxfp4_fast(E: int, H: int, I: int, seed: int = 0, device="cpu", distinct: int = 8):
    """Benchmark-sized MXFP4 weights: ``distinct`` experts are drawn and quantised exactly as
    in make_weights_mxfp4, the rest repeat them cyclically with their bytes rolled by the
    expert index (same distribution, every expert's bytes distinct); cheap enough to build a
    128-expert layer in seconds."""
    base = make_weights_mxfp4(distinct, H, I, seed)
    outs = []
    for t in base:
        t = t.to(device)
        reps = [torch.roll(t[e % distinct], shifts=e // distinct, dims=0) for e in range(E)]
        outs.append(torch.stack(reps))
    return tuple(outs)


def make_weights_fp8(E: int, H: int, I: int, seed: int = 0, experts=None):
    w1_q = torch.zeros(E, 2 * I, H, dtype=torch.float8_e4m3fn)
    w1_s = torch.ones(E, 2 * I // 128, H // 128, dtype=torch.float32)
    w2_q = torch.zeros(E, H, I, dtype=torch.float8_e4m3fn)
    w2_s = torch.ones(E, H // 128, I // 128, dtype=torch.float32)
    for e in (range(E) if experts is None else experts):
        q, s = quant.quantize_fp8_128x128(_expert_weight(e, 2 * I, H, seed, 0)[None])
        w1_q[e], w1_s[e] = q[0], s[0]
        q, s = quant.quantize_fp8_128x128(_expert_weight(e, H, I, seed, 1)[None])
        w2_q[e], w2_s[e] = q[0], s[0]
    return w1_q, w1_s, w2_q, w2_s


def make_weights_fp8_fast(E: int, H: int, I: int, seed: int = 0, device="cpu", distinct: int = 4):
    """Benchmark-sized FP8 weights: ``distinct`` experts drawn and quantised as in make_weights_fp8,
    the others repeat them with rows rolled by the expert index."""
    base = make_weights_fp8(distinct, H, I, seed)
    outs = []
    for t in base:
        t = t.to(device)
        if t.dtype == torch.float8_e4m3fn:      # roll whole 128-row blocks so data and scales stay aligned
            reps = [torch.roll(t[e % distinct].view(torch.uint8), shifts=128 * (e // distinct), dims=0) for e in range(E)]
            outs.append(torch.stack(reps).view(torch.float8_e4m3fn))
        else:
            reps = [torch.roll(t[e % distinct], shifts=e // distinct, dims=0) for e in range(E)]
            outs.append(torch.stack(reps))
    return tuple(outs)


class FastWeights:
    """Benchmark-sized expert weights that never exist in full on the host: ``distinct`` experts are drawn
    and quantised exactly as make_weights_mxfp4 / make_weights_fp8 do; expert e is base expert e % distinct with
    its rows rolled by e // distinct (whole 128-row blocks for FP8 data, so data and block scales stay aligned).
    `device_tensors` stacks all E experts on a device; `expert(e)` rebuilds one expert on the host for the CPU
    oracle.  make_weights_*_fast return the same tensors as `device_tensors`."""

    def __init__(self, E: int, H: int, I: int, seed: int = 0, wq: str = "mxfp4", distinct: int = 8):
        self.E, self.wq, self.distinct = E, wq, min(distinct, E)
        self.base = (make_weights_fp8 if wq == "fp8_128" else make_weights_mxfp4)(self.distinct, H, I, seed)

    def _one(self, t, e):
        b, shift = t[e % self.distinct], e // self.distinct
        if t.dtype == torch.float8_e4m3fn:
            return torch.roll(b.view(torch.uint8), shifts=128 * shift, dims=0).view(torch.float8_e4m3fn)
        return torch.roll(b, shifts=shift, dims=0)

    def expert(self, e: int):
        """(w1_q, w1_s, w2_q, w2_s) of expert e, on the host."""
        return tuple(self._one(t, e) for t in self.base)

    def device_tensors(self, device):
        outs = []
        for t in self.base:
            td = t.to(device)
            if td.dtype == torch.float8_e4m3fn:
                reps = [torch.roll(td[e % self.distinct].view(torch.uint8), shifts=128 * (e // self.distinct), dims=0)
                        for e in range(self.E)]
                outs.append(torch.stack(reps).view(torch.float8_e4m3fn))
            else:
                outs.append(torch.stack([torch.roll(td[e % self.distinct], shifts=e // self.distinct, dims=0)
                                         for e in range(self.E)]))
        return tuple(outs)


def algorithmic_flops(T: int, K: int, H: int, I: int) -> float:
    """6*H*I*T*K (tests/contrib/moe/test_moe.py:274)."""
    return 6.0 * H * I * T * K


def algorithmic_bytes(T: int, H: int, I: int, experts_hit: int, wq: str = "mxfp4") -> float:
    """Distinct experts' weight+scale bytes plus bf16 input and output."""
    per = 3.0 * H * I * ((0.5 + 1.0 / 32) if wq == "mxfp4" else 2.0 if wq == "bf16" else (1.0 + 4.0 / 16384))
    return experts_hit * per + 2.0 * T * H * 2


def expected_experts_hit(T: int, E: int, K: int) -> float:
    return E * (1.0 - math.pow(1.0 - K / E, T))
