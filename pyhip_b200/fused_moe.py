"""`fused_moe` -- the reference's operator surface (src/contrib/fused_moe.py:128-155 of
tingqli/pyhip) in front of the sm_100a kernels.

Same positional / keyword names and argument meaning as the reference; the aiter enums it takes
(`ActivationType`, `QuantType`) are re-declared here because aiter is not a dependency.  The
reference wrapper accepts QuantType.No (bf16 weights, no scales) and per_128x128 and reaches MXFP4
only through its raw kernels (tests/contrib/moe/test_moe.py:347-374, 638-771); this wrapper takes
both and adds per_1x32 to the same signature: ``w1``/``w2`` are packed E2M1 (uint8 or float4_e2m1fn_x2, low nibble = even element)
and ``w1_scale``/``w2_scale`` are E8M0 bytes ``[E*N, Kd/32]`` (or ``[E, N, Kd/32]``).

Work is enqueued on ``torch.cuda.current_stream()`` and never synchronises.
"""
from __future__ import annotations

import ctypes
import math
import enum

import torch

from . import _lib


class ActivationType(enum.IntEnum):
    No = -1
    Silu = 0
    Gelu = 1
    Swiglu = 2


class QuantType(enum.IntEnum):
    No = 0
    per_Tensor = 1
    per_Token = 2
    per_1x32 = 3
    per_1x128 = 4
    per_128x128 = 5


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def pick_block(T: int, K: int, E: int, weight_format: int = _lib.W_MXFP4) -> int:
    """Rows per sorted block (= token tile of the GEMMs).  Small when few tokens reach each
    expert so the weight-streaming regime wastes no tensor work on padding; the reference makes
    the same decode/prefill split on T*K/E (src/contrib/fused_moe.py:285-300,358-362).

    In the compute-bound regime the tile is chosen by a cost model: an expert that receives n
    rows costs ceil(n/B) MMA column tiles, each reading a 128-row weight tile plus B token rows
    from shared memory, so cost(B) = E[ceil(n/B)] * (128 + B) with n ~ Normal(mu, mu(1-1/E)) under
    uniform routing.  96 is the largest tile whose two accumulator buffers fit tensor memory.
    Measured on the gpt-oss shape: T=4096 0.94 ms at 80 vs 1.06 ms at 96, T=8192 1.60 ms at 96 vs 1.70 ms
    at 80, as the model predicts.  The FP8 kernels pay a fixed promotion cost per tile and k-block on top (modelled as
    64 more rows), so fewer tiles win more often there: 96 unless a smaller tile covers the experts' rows with the same
    number of tiles (about 128 rows per expert: two tiles of 80 instead of two of 96)."""
    per_expert = (T * K) / max(E, 1)
    if per_expert <= 4:
        return 16
    if per_expert <= 20:
        return 32
    if per_expert <= 48:
        return 64
    fp8 = weight_format in (_lib.W_FP8_128, _lib.W_FP8_ROW)
    sigma = math.sqrt(max(per_expert * (1.0 - 1.0 / max(E, 1)), 1e-6))
    lo, hi = max(1, int(per_expert - 4 * sigma)), int(per_expert + 4 * sigma) + 1
    best, best_cost = 96, None
    for B in ((96, 80, 64) if fp8 else (96, 80, 64, 48)):
        wsum = cost = 0.0
        for n in range(lo, hi + 1):
            wgt = math.exp(-0.5 * ((n - per_expert) / sigma) ** 2)
            wsum += wgt
            cost += wgt * (-(-n // B)) * (128 + B + (64 if fp8 else 0))
        cost /= wsum
        if best_cost is None or cost < best_cost * 0.98:      # prefer the larger tile on a near tie
            best, best_cost = B, cost
    return best


class PreparedWeights:
    """One layer's MXFP4 expert weights as the kernels consume them: the packed E2M1 tensors in
    place (canonical layout, no copy) plus a regrouped image of their E8M0 scales, built once
    (the counterpart of the reference's scale pre-shuffle, tests/contrib/moe/test_moe.py:167)."""

    def __init__(self, w1, w1_scale, w2, w2_scale):
        if not w1.is_cuda:
            raise ValueError("weights must be CUDA tensors")
        w1 = (w1.view(torch.uint8) if w1.dtype != torch.uint8 else w1).contiguous()
        w2 = (w2.view(torch.uint8) if w2.dtype != torch.uint8 else w2).contiguous()
        s1 = w1_scale.view(torch.uint8) if w1_scale.dtype != torch.uint8 else w1_scale
        s2 = w2_scale.view(torch.uint8) if w2_scale.dtype != torch.uint8 else w2_scale
        E, N1, Kh = w1.shape
        self.E, self.I, self.H = E, N1 // 2, Kh * 2
        if tuple(w2.shape) != (E, self.H, self.I // 2):
            raise ValueError(f"w2 shape {tuple(w2.shape)} does not match w1 {tuple(w1.shape)}")
        if s1.numel() != E * N1 * (self.H // 32) or s2.numel() != E * self.H * (self.I // 32):
            raise ValueError("scale tensors must hold one E8M0 byte per 32 weights")
        if int(s1.max()) > 254 or int(s2.max()) > 254:
            raise ValueError("E8M0 scale 0xFF (NaN) is not a valid weight scale")
        L = _lib.lib()
        shape = _lib.Shape(T=0, K=1, E=E, E_route=E, H=self.H, I=self.I, B=32, weight_format=_lib.W_MXFP4,
                           activation=0, swiglu_limit=0.0, act_terms=0, combine_mode=0, act_quant=0, doweight_stage1=0)
        out = []
        for which, ws in ((1, s1), (2, s2)):
            sb = ctypes.c_int64()
            _lib.check(L.b200moe_prepared_scale_bytes(ctypes.byref(shape), which, ctypes.byref(sb)),
                       "prepared_scale_bytes")
            scale = torch.empty(sb.value, dtype=torch.uint8, device=w1.device)
            _lib.check(L.b200moe_prepare_scales(ctypes.byref(shape), which, _ptr(ws.contiguous()), _ptr(scale),
                                                _stream()), "prepare_scales")
            out.append(scale)
        self.w1_data, self.w2_data = w1, w2            # consumed in place
        self.w1_scale, self.w2_scale = out
        self.w1_scale_raw, self.w2_scale_raw = s1.contiguous(), s2.contiguous()   # canonical layout: the batch-1 path reads it
        self.device = w1.device


class PreparedWeightsFP8:
    """FP8 (e4m3) expert weights, consumed entirely in place, with either one fp32 scale per 128x128 block
    (tests/contrib/moe/test_moe.py:201-260) or one per output row -- the reference's per-token-per-channel format,
    scales [E, N] or [E, N, 1]; its per-tensor format, scales [E], is expanded to one value per row here
    (tests/contrib/moe/test_moe.py:123-138)."""

    def __init__(self, w1, w1_scale, w2, w2_scale, row_scaled=False):
        if not w1.is_cuda:
            raise ValueError("weights must be CUDA tensors")
        E, N1, H = w1.shape
        self.E, self.I, self.H = E, N1 // 2, H
        if tuple(w2.shape) != (E, H, self.I):
            raise ValueError(f"w2 shape {tuple(w2.shape)} does not match w1 {tuple(w1.shape)}")
        if H % 128 or self.I % 128:
            raise ValueError("FP8 weights need H and I to be multiples of 128")
        if row_scaled:
            def rows(sc, n):
                sc = sc.float().to(w1.device)
                if sc.numel() == E:                           # per-tensor: one scale per expert
                    sc = sc.reshape(E, 1).expand(E, n)
                elif sc.numel() != E * n:
                    raise ValueError("scale tensors must hold one fp32 scale per expert or per output row")
                return sc.reshape(E, n).contiguous()
            self.w1_scale, self.w2_scale = rows(w1_scale, N1), rows(w2_scale, H)
        else:
            if w1_scale.numel() != E * (N1 // 128) * (H // 128) or w2_scale.numel() != E * (H // 128) * (self.I // 128):
                raise ValueError("scale tensors must hold one fp32 scale per 128x128 block")
            self.w1_scale, self.w2_scale = w1_scale.float().contiguous(), w2_scale.float().contiguous()
        self.w1_data, self.w2_data = w1.contiguous().view(torch.uint8), w2.contiguous().view(torch.uint8)
        self.device = w1.device


class PreparedWeightsBF16:
    """Unquantised bf16 expert weights (the reference wrapper's QuantType.No, src/contrib/fused_moe.py:253):
    w1 [E, 2I, H], w2 [E, H, I], consumed in place; there are no scales."""

    def __init__(self, w1, w2):
        if not w1.is_cuda:
            raise ValueError("weights must be CUDA tensors")
        if w1.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16:
            raise TypeError("QuantType.No takes bfloat16 weights")
        E, N1, H = w1.shape
        self.E, self.I, self.H = E, N1 // 2, H
        if tuple(w2.shape) != (E, H, self.I):
            raise ValueError(f"w2 shape {tuple(w2.shape)} does not match w1 {tuple(w1.shape)}")
        if H % 32 or self.I % 32:
            raise ValueError("H and I must be multiples of 32")
        self.w1_data, self.w2_data = w1.contiguous(), w2.contiguous()
        self.w1_scale = self.w2_scale = None
        self.device = w1.device


_prepared_cache: dict = {}          # insertion-ordered: least recently used first
_workspace_cache: dict = {}
_PREPARED_CACHE_ENTRIES = 8


def prepare_weights(w1, w1_scale, w2, w2_scale, weight_format=_lib.W_MXFP4):
    """Prepared form of one layer's weights, cached by the identity of the four tensors and the in-place
    version counters of the scale tensors (scales updated in place are prepared again).  The cache keeps the
    `_PREPARED_CACHE_ENTRIES` most recently used layers alive -- an entry references the caller's weight tensors
    -- and `release_prepared()` drops them all."""
    if weight_format == _lib.W_BF16:
        key = (w1.data_ptr(), 0, w2.data_ptr(), 0, tuple(w1.shape), weight_format, 0, 0)
    else:
        key = (w1.data_ptr(), w1_scale.data_ptr(), w2.data_ptr(), w2_scale.data_ptr(), tuple(w1.shape), weight_format,
               w1_scale._version, w2_scale._version)
    hit = _prepared_cache.pop(key, None)
    if hit is None:
        while len(_prepared_cache) >= _PREPARED_CACHE_ENTRIES:
            _prepared_cache.pop(next(iter(_prepared_cache)))
        if weight_format == _lib.W_MXFP4:
            pw = PreparedWeights(w1, w1_scale, w2, w2_scale)
        elif weight_format == _lib.W_BF16:
            pw = PreparedWeightsBF16(w1, w2)
        else:
            pw = PreparedWeightsFP8(w1, w1_scale, w2, w2_scale, row_scaled=weight_format == _lib.W_FP8_ROW)
        hit = (pw, (w1, w1_scale, w2, w2_scale))      # the sources stay alive, so their addresses identify them
    _prepared_cache[key] = hit
    return hit[0]


def release_prepared():
    """Forget every cached prepared weight set and workspace (frees the HBM they pin)."""
    _prepared_cache.clear()
    _workspace_cache.clear()


class MoEPlan:
    """Shape, workspace layout and workspace tensor of one (T, K, E, H, I, B) problem."""

    def __init__(self, T, K, E, E_route, H, I, B, activation, swiglu_limit, device, act_terms=0,
                 weight_format=_lib.W_MXFP4, combine_mode=_lib.COMBINE_GATHER, act_quant=_lib.ACTQ_TERMS,
                 doweight_stage1=False, cta_pairs=0):
        self.shape = _lib.Shape(T=T, K=K, E=E, E_route=E_route, H=H, I=I, B=B, weight_format=weight_format,
                                activation=activation, swiglu_limit=float(swiglu_limit), act_terms=act_terms,
                                combine_mode=combine_mode, act_quant=act_quant,
                                doweight_stage1=1 if doweight_stage1 else 0, cta_pairs=cta_pairs)
        self.capacity = T
        self.terms = act_terms or 3
        self.fp8 = weight_format in (_lib.W_FP8_128, _lib.W_FP8_ROW)
        self.bf16 = weight_format == _lib.W_BF16
        self.aq = act_quant
        self.ws = _lib.workspace_layout(self.shape)
        self.buf = torch.empty(self.ws.total_bytes + 1024, dtype=torch.uint8, device=device)
        off = (-self.buf.data_ptr()) % 1024
        self.base = self.buf.data_ptr() + off
        self._view = self.buf[off:off + self.ws.total_bytes]
        sb = ctypes.c_int64()
        _lib.check(_lib.lib().b200moe_sort_scratch_bytes(E_route, ctypes.byref(sb)), "sort_scratch_bytes")
        self.sort_scratch_bytes = sb.value if T * K >= 8192 else 0     # the layout reserves it from that size up
        self.status().zero_()

    def set_tokens(self, T: int):
        """Run the next calls with T tokens (T <= the token count the workspace was laid out for)."""
        if T > self.capacity:
            raise ValueError(f"plan holds {self.capacity} tokens, {T} requested")
        self.shape.T = T

    def region(self, name: str, nbytes: int, dtype=torch.uint8):
        off = getattr(self.ws, "off_" + name)
        return self._view[off:off + nbytes].view(dtype)

    def status(self):
        return self.region("status", 64, torch.int32)

    def sort_outputs(self):
        L, B = self.ws.max_rows, self.shape.B
        return (self.region("sorted_ids", L * 4, torch.int32), self.region("sorted_w", L * 4, torch.float32),
                self.region("sorted_e", L // B * 4, torch.int32), self.region("num_valid", 8, torch.int32),
                self.region("loc", max(self.capacity * self.shape.K, 1) * 4, torch.int32))

    # ---- stage-by-stage entry points (the raw-kernel surface the reference's tests drive,
    # tests/contrib/moe/test_moe.py:638-771) -------------------------------------------------
    def _args(self):
        return ctypes.byref(self.shape), ctypes.byref(self.ws), ctypes.c_void_p(self.base)

    def sort(self, topk_ids, topk_weight, expert_mask=None):
        s = self.shape
        ids_o, w_o, e_o, nv_o, loc_o = self.sort_outputs()
        _lib.check(_lib.lib().b200moe_sort_align_ws(
            _ptr(topk_ids), _ptr(topk_weight), s.T, s.K, s.E_route, s.B, _ptr(expert_mask), None, _ptr(ids_o),
            _ptr(w_o), _ptr(e_o), _ptr(nv_o), _ptr(loc_o), ctypes.c_void_p(self.base + self.ws.off_sort_scratch),
            self.sort_scratch_bytes, _stream()), "sort_align")
        return ids_o, w_o, e_o, nv_o, loc_o

    def quant_input(self, x):
        s, ws = self.shape, self.ws
        ids_o, _, _, nv_o, _ = self.sort_outputs()
        base = self.base
        if self.bf16:
            raise NotImplementedError("bf16 weights: the stage-by-stage surface starts at the whole-layer call")
        if self.fp8:
            fn = _lib.lib().b200moe_quant_rows_fp8_1x128 if self.aq else _lib.lib().b200moe_quant_rows_e4m3
            _lib.check(fn(_ptr(x), 0, _ptr(ids_o), _ptr(nv_o), s.T, s.K, s.H, s.B, ws.max_rows,
                          ctypes.c_void_p(base + ws.off_xq), ctypes.c_void_p(base + ws.off_xsf), _stream()), "quant_rows (fp8)")
            return
        _lib.check(_lib.lib().b200moe_quant_rows(
            _ptr(x), 0, _ptr(ids_o), _ptr(nv_o), s.T, s.K, s.H, s.B, self.terms, ws.max_rows,
            ctypes.c_void_p(base + ws.off_xq), ctypes.c_void_p(base + ws.off_xsf), _stream()),
            "quant_rows")

    def quant_hidden(self, h):
        """h: bf16 [T, K, I] -> operand rows of the down GEMM."""
        s, ws = self.shape, self.ws
        ids_o, _, _, nv_o, _ = self.sort_outputs()
        base = self.base
        if self.fp8:
            fn = _lib.lib().b200moe_quant_rows_fp8_1x128 if self.aq else _lib.lib().b200moe_quant_rows_e4m3
            _lib.check(fn(_ptr(h), 1, _ptr(ids_o), _ptr(nv_o), s.T, s.K, s.I, s.B, ws.max_rows,
                          ctypes.c_void_p(base + ws.off_hq), ctypes.c_void_p(base + ws.off_hsf), _stream()), "quant_rows (fp8)")
            return
        _lib.check(_lib.lib().b200moe_quant_rows(
            _ptr(h), 1, _ptr(ids_o), _ptr(nv_o), s.T, s.K, s.I, s.B, self.terms, ws.max_rows,
            ctypes.c_void_p(base + ws.off_hq), ctypes.c_void_p(base + ws.off_hsf), _stream()),
            "quant_rows")

    def gateup(self, pw, h_out=None, bias1=None):
        _lib.check(_lib.lib().b200moe_gateup(*self._args(), _ptr(pw.w1_data), _ptr(pw.w1_scale), _ptr(bias1),
                                             _ptr(h_out), _stream()), "gateup")

    def down(self, pw, bias2=None, y=None):
        """``y`` (zeroed bf16 [T, H]) is the target of the fused combine when the plan was built with
        combine_mode FUSED; otherwise the rows land in the workspace for `combine`."""
        _lib.check(_lib.lib().b200moe_down(*self._args(), _ptr(pw.w2_data), _ptr(pw.w2_scale), _ptr(bias2), _ptr(y),
                                           _stream()), "down")

    def combine(self, topk_weight, y):
        _lib.check(_lib.lib().b200moe_combine(*self._args(), _ptr(topk_weight), _ptr(y), _stream()), "combine")

    def check_status(self):
        """Host read of the device-side error words (synchronises; for tests and debugging)."""
        st = self.status().cpu().tolist()
        if st[0] != 0 or st[2] != 0:
            raise _lib.B200MoEError(f"device status: wait gave up at 0x{st[0]:x} in CTA {st[1]}, "
                                    f"bad expert id flag {st[2]}")


_WORKSPACE_CACHE_ENTRIES = 16


def _capacity(T: int) -> int:
    """Token capacity a cached workspace is laid out for: the next power of two up to 512, multiples of 512
    beyond, so that a decode loop whose batch size wanders reuses a handful of allocations."""
    if T <= 512:
        return 1 << max(0, (T - 1).bit_length())
    return -(-T // 512) * 512


def get_plan(T, K, E, E_route, H, I, B, activation, swiglu_limit, device, act_terms=0,
             weight_format=_lib.W_MXFP4, combine_mode=_lib.COMBINE_GATHER, act_quant=_lib.ACTQ_TERMS,
             doweight_stage1=False, cta_pairs=0) -> MoEPlan:
    """Cached plan (shape + workspace).  One workspace per (shape, CUDA stream): calls enqueued on different
    streams never share scratch memory.  The least recently used entry is dropped when the cache is full."""
    stream_id = torch.cuda.current_stream(device).cuda_stream if torch.cuda.is_available() else 0
    key = (T, K, E, E_route, H, I, B, activation, float(swiglu_limit), str(device), act_terms, weight_format,
           combine_mode, act_quant, bool(doweight_stage1), cta_pairs, stream_id)
    plan = _workspace_cache.pop(key, None)
    if plan is None:
        while len(_workspace_cache) >= _WORKSPACE_CACHE_ENTRIES:
            _workspace_cache.pop(next(iter(_workspace_cache)))
        plan = MoEPlan(T, K, E, E_route, H, I, B, activation, swiglu_limit, device, act_terms, weight_format,
                       combine_mode, act_quant, doweight_stage1, cta_pairs)
    _workspace_cache[key] = plan          # (re)insert at the recent end
    return plan


BATCH1_MAX_TOPK, BATCH1_MAX_DIM = 8, 8192


def batch1_eligible(T: int, K: int, H: int, I: int, weight_format: int, act_terms: int) -> bool:
    """Whether a call can take the two-launch batch-1 path (one token, MXFP4 weights, default activation format; no
    sort, no quantiser: matrix-vector products from the bf16 input itself), the counterpart of the reference's
    moe_gemm_batch1 (src/contrib/moe.py:41-188).  It is selected with ``method="batch1"`` only: on this GPU the
    sorted tensor-core path is the faster one even for a single token (gpt-oss shape: 31.5 us against 38.6 us)."""
    return (T == 1 and weight_format == _lib.W_MXFP4 and act_terms == 0 and K <= BATCH1_MAX_TOPK and
            H <= BATCH1_MAX_DIM and I <= BATCH1_MAX_DIM)


def moe_forward(plan: MoEPlan, pw: PreparedWeights, hidden_states, topk_weight, topk_ids, expert_mask=None,
                out=None, num_local_tokens=None, bias1=None, bias2=None, batch1=None):
    """One layer call through the C ABI (sort -> quantise -> gate-up -> down [-> combine]; decode-sized batches
    fold the first two into one launch; ``batch1=True`` sends a single token down the batch-1 path instead).
    ``num_local_tokens``: optional int32 device tensor; tokens at and beyond its value are padding (their output
    rows are zero)."""
    T, H = hidden_states.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.bfloat16, device=hidden_states.device)
    if T == 0:
        return out
    s = plan.shape
    if batch1:
        if not batch1_eligible(T, s.K, s.H, s.I, s.weight_format, s.act_terms):
            raise ValueError("the batch-1 path takes one token, MXFP4 weights, default act_terms and top-k <= 8")
        need = ctypes.c_int64()
        _lib.check(_lib.lib().b200moe_batch1_scratch_bytes(ctypes.byref(s), ctypes.byref(need)), "batch1_scratch_bytes")
        if plan.ws.off_hsf - plan.ws.off_hq < need.value:
            raise ValueError("workspace too small for the batch-1 scratch")
        _lib.check(_lib.lib().b200moe_forward_batch1(
            ctypes.byref(s), _ptr(hidden_states), _ptr(topk_ids), _ptr(topk_weight), _ptr(expert_mask),
            _ptr(num_local_tokens), _ptr(pw.w1_data), _ptr(pw.w1_scale_raw), _ptr(pw.w2_data), _ptr(pw.w2_scale_raw),
            _ptr(bias1), _ptr(bias2), ctypes.c_void_p(plan.base + plan.ws.off_hq), _ptr(out), _stream()), "forward_batch1")
        return out
    io = _lib.Io(x_bf16=hidden_states.data_ptr(), topk_ids=topk_ids.data_ptr(), topk_weight=topk_weight.data_ptr(),
                 expert_mask=None if expert_mask is None else expert_mask.data_ptr(),
                 num_local_tokens=None if num_local_tokens is None else num_local_tokens.data_ptr(),
                 w1_q=pw.w1_data.data_ptr(), w1_scale_prepared=None if pw.w1_scale is None else pw.w1_scale.data_ptr(),
                 w2_q=pw.w2_data.data_ptr(), w2_scale_prepared=None if pw.w2_scale is None else pw.w2_scale.data_ptr(),
                 bias1=None if bias1 is None else bias1.data_ptr(),
                 bias2=None if bias2 is None else bias2.data_ptr(), y_bf16=out.data_ptr())
    _lib.check(_lib.lib().b200moe_forward_ex(ctypes.byref(plan.shape), ctypes.byref(plan.ws),
                                             ctypes.c_void_p(plan.base), ctypes.byref(io), _stream()), "forward")
    return out


def launches_per_call(T: int, K: int, E_route: int, combine_mode: int, batch1: bool = False) -> int:
    """Kernel launches of one whole-layer call: sort + quantise (one launch up to 256 (token, expert) pairs, two
    below 8192 pairs, four from there on: the sort is then count / scan / scatter), gate-up, down, and the
    gather-sum unless the combine is fused into the down epilogue.  The batch-1 path is two launches."""
    if batch1:
        return 2
    pairs = T * K
    front = 1 if (pairs <= 256 and E_route <= 1024) else (4 if pairs >= 8192 else 2)
    return front + 2 + (0 if combine_mode == _lib.COMBINE_FUSED else 1)


def capture_forward(plan: MoEPlan, pw, hidden_states, topk_weight, topk_ids, expert_mask=None, out=None,
                    num_local_tokens=None):
    """Capture one layer call (three to five kernel launches, no host synchronisation inside) into a CUDA
    graph.  Returns (graph, out): ``graph.replay()`` re-runs the layer on the same tensors -- the
    caller refreshes their contents in place between replays, including the int32 device tensor
    ``num_local_tokens`` when the batch is padded to a fixed T (the reference's use of that argument,
    src/contrib/fused_moe.py:48-49)."""
    T, H = hidden_states.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.bfloat16, device=hidden_states.device)
    moe_forward(plan, pw, hidden_states, topk_weight, topk_ids, expert_mask, out, num_local_tokens)   # first-use set-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        moe_forward(plan, pw, hidden_states, topk_weight, topk_ids, expert_mask, out, num_local_tokens)
    return graph, out


def fused_moe(hidden_states, w1, w2, topk_weight, topk_ids, expert_mask=None,
              activation=ActivationType.Silu, quant_type=QuantType.No, doweight_stage1=False,
              w1_scale=None, w2_scale=None, a1_scale=None, a2_scale=None, block_size_M=None,
              num_local_tokens=None, moe_sorting_dispatch_policy=0, dtype=None, hidden_pad=0,
              intermediate_pad=0, bias1=None, bias2=None, splitk=0, method="auto",
              swiglu_limit=7.0, act_terms=0, combine="auto", act_quant="terms", cta_pairs="auto"):
    """bf16 hidden states [T,H], router top-k ids [T,K] int32 and weights [T,K] fp32, packed
    expert weights with their scales -> bf16 [T,H].  Unsupported combinations raise, as the
    reference asserts (src/contrib/fused_moe.py:252-266).

    Arguments beyond the reference's signature:
      ``act_terms`` (MXFP4; 0 = default 3): packed-FP4 terms that carry one activation row inside the GEMMs.
        1 = plain per-1x32 MXFP4 activations, the arithmetic of the reference's a4w4 kernels
        (tests/contrib/moe/test_moe.py:665-679); 3 keeps the layer within the bf16-activation tolerance.
      ``combine``: "gather" (deterministic: sorted rows + a gather-sum launch in expert order), "fused" (the down
        epilogue multiplies by the routing weight and adds into the output with packed-bf16 reductions, the
        reference kernels' own epilogue, src/contrib/moe.py:703-787) or "auto" (= "gather", the reproducible one).
      ``act_quant`` (FP8 weights): "terms" (default: two e4m3 terms with E8M0 scales per 32, exact for bf16 inputs
        to ~2^-9 of the block maximum) or "1x128" (the reference's own per-token, per-128-channel e4m3 format with
        fp32 scales, src/contrib/fused_moe.py:375-381: half the operand bytes and MMA work, judged against the
        oracle that dequantises the same quantised activations).
      ``bias1`` [E, 2I] / ``bias2`` [E, H]: per-expert biases of the two projections (gpt-oss style).
      ``method``: "batch1" takes the two-launch batch-1 path (one token, MXFP4 weights: no sort, no activation
        quantiser, bitwise reproducible; slower than the default on this GPU); any other value, the reference's
        "auto" / "jit" / "gluon" among them, takes the sorted grouped GEMMs.
      ``cta_pairs`` (MXFP4): "auto" runs the GEMMs on CTA pairs (tcgen05.mma.cta_group::2) in the compute-bound regime,
        "off" never, "on" wherever the tile allows it.
    """
    if not hidden_states.is_cuda:
        raise RuntimeError("fused_moe runs on a CUDA device only (sm_100a); there is no CPU path")
    if hidden_states.dtype != torch.bfloat16:
        raise TypeError("hidden_states must be bfloat16")
    fmt = {int(QuantType.No): _lib.W_BF16, int(QuantType.per_1x32): _lib.W_MXFP4,
           int(QuantType.per_128x128): _lib.W_FP8_128, int(QuantType.per_Token): _lib.W_FP8_ROW,
           int(QuantType.per_Tensor): _lib.W_FP8_ROW}.get(int(quant_type))
    if fmt is None:
        raise NotImplementedError(f"quant_type={quant_type!r}: No (bf16 weights), per_1x32 (MXFP4), per_128x128, per_Token "
                                  "and per_Tensor (FP8) are implemented")
    if int(activation) not in (ActivationType.Silu, ActivationType.Swiglu):
        raise NotImplementedError(f"activation={activation!r}: Silu and Swiglu are implemented")
    if a1_scale is not None or a2_scale is not None:
        raise NotImplementedError("pre-quantised activations (a1_scale / a2_scale) are not implemented: pass bf16")
    if hidden_pad or intermediate_pad:
        raise NotImplementedError("padding arguments are not implemented")
    if fmt != _lib.W_BF16 and (w1_scale is None or w2_scale is None):
        raise ValueError("quantised weights need w1_scale and w2_scale")
    if fmt == _lib.W_BF16 and (act_terms or w1.dtype != torch.bfloat16):
        raise ValueError("quant_type=No takes bfloat16 weights and no act_terms (activations stay bf16)")
    if dtype not in (None, torch.bfloat16):
        raise NotImplementedError("output dtype must be bfloat16")
    if combine not in ("auto", "gather", "fused"):
        raise ValueError(f"combine={combine!r}: 'auto', 'gather' or 'fused'")
    if act_quant not in ("terms", "1x128"):
        raise ValueError(f"act_quant={act_quant!r}: 'terms' or '1x128'")
    if cta_pairs not in ("auto", "off", "on"):
        raise ValueError(f"cta_pairs={cta_pairs!r}: 'auto', 'off' or 'on'")
    if act_quant == "1x128" and fmt != _lib.W_FP8_128:
        raise ValueError("act_quant='1x128' belongs to per_128x128 (FP8) weights; MXFP4 weights take act_terms")
    T, H = hidden_states.shape
    K = topk_ids.shape[1]
    pw = prepare_weights(w1, w1_scale, w2, w2_scale, fmt)
    if pw.H != H:
        raise ValueError(f"hidden size {H} does not match weights ({pw.H})")
    E_route = pw.E if expert_mask is None else int(expert_mask.numel())
    B = int(block_size_M) if block_size_M else pick_block(T, K, pw.E, fmt)
    act = _lib.ACT_SILU if int(activation) == ActivationType.Silu else _lib.ACT_SWIGLU
    cm = _lib.COMBINE_FUSED if combine == "fused" else _lib.COMBINE_GATHER
    aq = _lib.ACTQ_1X128 if act_quant == "1x128" else _lib.ACTQ_TERMS
    b1 = b2 = None
    if bias1 is not None:
        if tuple(bias1.shape) != (pw.E, 2 * pw.I):
            raise ValueError(f"bias1 must be [E, 2I] = [{pw.E}, {2 * pw.I}]")
        b1 = bias1.float().contiguous()
    if bias2 is not None:
        if tuple(bias2.shape) != (pw.E, H):
            raise ValueError(f"bias2 must be [E, H] = [{pw.E}, {H}]")
        b2 = bias2.float().contiguous()
    plan = get_plan(_capacity(T), K, pw.E, E_route, H, pw.I, B, act, swiglu_limit, hidden_states.device, act_terms, fmt,
                    cm, aq, bool(doweight_stage1), {"auto": 0, "off": 1, "on": 2}[cta_pairs])
    plan.set_tokens(T)
    ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
    tw = topk_weight if topk_weight.dtype == torch.float32 else topk_weight.float()
    mask = None if expert_mask is None else expert_mask.to(torch.int32).contiguous()
    return moe_forward(plan, pw, hidden_states.contiguous(), tw.contiguous(), ids.contiguous(), mask,
                       num_local_tokens=_num_local(num_local_tokens, hidden_states.device), bias1=b1, bias2=b2,
                       batch1=method == "batch1")


def fused_topk(hidden_states, gating_output, topk: int, renormalize: bool = True, scoring: str = "softmax"):
    """Router step with the call shape of aiter's fused_topk as the reference uses it
    (tests/contrib/moe/test_fused_moe.py:38,87): fp32 logits [T, E] -> (topk_weights f32 [T, topk],
    topk_ids i32 [T, topk]), ids in descending score order.  `hidden_states` is only consulted for the
    token count, as in the reference."""
    if not gating_output.is_cuda:
        raise RuntimeError("fused_topk runs on a CUDA device only (sm_100a); there is no CPU path")
    T, E = gating_output.shape
    if hidden_states is not None and hidden_states.shape[0] != T:
        raise ValueError("hidden_states and gating_output disagree on the token count")
    logits = gating_output.float().contiguous()
    ids = torch.empty(T, topk, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, topk, dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().b200moe_route_topk(_ptr(logits), T, E, topk, {"softmax": 0, "sigmoid": 1}[scoring],
                                             1 if renormalize else 0, _ptr(ids), _ptr(w), _stream()), "route_topk")
    return w, ids


def _num_local(num_local_tokens, device):
    """The reference's num_local_tokens argument (src/contrib/fused_moe.py:48-49): a device tensor holding the
    number of leading tokens that are real; the rest of the batch is padding."""
    if num_local_tokens is None:
        return None
    if not torch.is_tensor(num_local_tokens):
        return torch.tensor([int(num_local_tokens)], dtype=torch.int32, device=device)
    return num_local_tokens.to(device=device, dtype=torch.int32).reshape(-1)[:1].contiguous()


def moe_sorting(topk_ids, topk_weights, num_experts, model_dim, moebuf_dtype, block_size=32, expert_mask=None,
                num_local_tokens=None, dispatch_policy=0):
    """Same outputs as the reference's sorter (src/contrib/fused_moe.py:56-100):
    (sorted_ids, sorted_weights, sorted_expert_ids, num_valid_ids, moe_out)."""
    T, K = topk_ids.shape
    dev = topk_ids.device
    nlt = _num_local(num_local_tokens, dev)
    nblk = (T * K + num_experts * (block_size - 1) + block_size - 1) // block_size
    sorted_ids = torch.empty(nblk * block_size, dtype=torch.int32, device=dev)
    sorted_w = torch.empty(nblk * block_size, dtype=torch.float32, device=dev)
    sorted_e = torch.empty(nblk, dtype=torch.int32, device=dev)
    num_valid = torch.empty(2, dtype=torch.int32, device=dev)
    moe_out = torch.zeros((T, model_dim), dtype=moebuf_dtype, device=dev)
    mask = None if expert_mask is None else expert_mask.to(torch.int32).contiguous()
    sb = ctypes.c_int64()
    _lib.check(_lib.lib().b200moe_sort_scratch_bytes(num_experts, ctypes.byref(sb)), "sort_scratch_bytes")
    scratch = torch.empty(sb.value, dtype=torch.uint8, device=dev) if T * K >= 8192 else None   # several CTAs from there
    _lib.check(_lib.lib().b200moe_sort_align_ws(
        _ptr(topk_ids.to(torch.int32).contiguous()), _ptr(topk_weights.float().contiguous()), T, K, num_experts,
        block_size, _ptr(mask), _ptr(nlt), _ptr(sorted_ids), _ptr(sorted_w), _ptr(sorted_e), _ptr(num_valid), None,
        _ptr(scratch), sb.value if scratch is not None else 0, _stream()), "sort_align")
    return sorted_ids, sorted_w, sorted_e, num_valid, moe_out
