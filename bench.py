"""Benchmark of the fused-MoE hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload W] [--tokens T] [--no-extras]
                    [--weights bf16] [--method batch1]

One "step" is one MoE layer call on one batch of synthetic tokens.  At N=1 the default workload is
the gpt-oss-120b-shaped MXFP4 layer (H=I=2880, E=128, top-4) at T=64 decode tokens -- the
weight-streaming regime the headline metric is quoted on.  `--workload` selects the other
configurations: gptoss_prefill (T=8192), dsv3_ep (DeepSeek-V3-shaped FP8 128x128, T=4096 per GPU),
mixtral_skew (E=8, Zipf load, T=16384 in total).  At N>1 the layer runs expert-parallel, one process
per GPU (torchrun), with the exchange over NCCL inside the timed region: all-gather + reduce-scatter
at decode sizes, all-to-all-v dispatch/combine above 512 tokens per GPU; before anything is timed a
small expert-parallel layer is checked against the CPU oracle on every rank (`parity`, non-zero exit
on a miss).

Prints ONE JSON line (rank 0).  The timed region of exactly K steps (CUDA events, barrier and
synchronise on both sides, max over ranks) is repeated until about a second of GPU time has been
spent; `ms_per_step` / `value` are the median region, the spread is in `ms_per_step_min/max`.
`value` = tokens/s with inputs resident in HBM (a CUDA-graph replay of the call's launches at N=1);
`e2e` = the same through the public `fused_moe` call with pinned host buffers copied in and the
result copied out every step; `roofline` = the gate-up grouped GEMM (the dominant kernel) timed
alone against the measured HBM copy rate; `cpu_baseline` = the CPU oracle timed on a bounded sample
of the same workload.  `--impl reference` times only that CPU path (every expert the batch hits,
once per step).

Unless `--no-extras` is given the default run also measures, each with its own clock record:
`sweep` (decode T in {1, 8, 32, 256}; batches whose expert set fits L2 rotate over several routing
sets so that weights are streamed from HBM every step), `batch1_T1` (one token down the sort-free
matrix-vector path, `--method batch1`, beside the sweep's T=1 entry), `prefill` (gpt-oss shape, T=8192: the default
three-term activation format and the plain MXFP4 a4w4 format, scored against the dense FP4 rate --
nominal 9 PFLOP/s and the rate the library's MMA probe measures in the same run), `config3`
(DeepSeek-V3-shaped FP8 layer, T=4096 per GPU, expert-parallel at N>1) and `config4` (Mixtral-shaped
layer under Zipf load).
"""
import argparse
import dataclasses
import json
import math
import os
import pathlib
import re
import statistics
import subprocess
import sys
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
L2_BYTES = 126e6
PAIRS = {"auto": 0, "off": 1, "on": 2}
FP4_NOMINAL_TFLOPS = 9000.0
FP8_NOMINAL_TFLOPS = 4500.0
BF16_NOMINAL_TFLOPS = 2250.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="tokens per GPU per step (0 = the workload's own)")
    ap.add_argument("--workload", default="gptoss_decode", choices=["gptoss_decode", "gptoss_prefill", "dsv3_ep", "mixtral_skew"],
                    help="gptoss_*: MXFP4 weights (decode / prefill); dsv3_ep: FP8 128x128 weights; mixtral_skew: MXFP4, Zipf load")
    ap.add_argument("--experts", type=int, default=0,
                    help="override the number of experts (0 = the workload's own); for small profiling captures")
    ap.add_argument("--ep-chunks", type=int, default=0,
                    help="N>1: slices of the pipelined dispatch/combine exchange (0 = chosen from the shape)")
    ap.add_argument("--combine", default="fused", choices=["fused", "gather"],
                    help="fused: weighted scatter-add in the down epilogue; gather: sorted rows + deterministic gather-sum")
    ap.add_argument("--act-terms", type=int, default=0, help="MXFP4 activation terms (0 = default 3; 1 = plain a4w4)")
    ap.add_argument("--act-quant", default="terms", choices=["terms", "1x128"],
                    help="FP8 weights: two e4m3 terms with E8M0 scales (default) or the per-token 1x128 fp32-scale format")
    ap.add_argument("--weights", default="native", choices=["native", "bf16"],
                    help="bf16: the same shape with unquantised bf16 weights (QuantType.No; one GPU, implies --no-extras)")
    ap.add_argument("--method", default="auto", choices=["auto", "batch1"],
                    help="batch1: the sort-free one-token path (needs --tokens 1 and MXFP4 weights)")
    ap.add_argument("--cta-pairs", default="auto", choices=["auto", "off", "on"],
                    help="MXFP4 GEMMs on CTA pairs (tcgen05.mma.cta_group::2): auto = in the compute-bound regime")
    ap.add_argument("--no-extras", action="store_true", help="only the headline workload (no sweep / prefill / config3 / config4)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time direct launches instead of CUDA-graph replays")
    ap.add_argument("--repeat-ms", type=float, default=1000.0, help="GPU time to spend repeating the K-step region")
    return ap.parse_args()


def profiled_traffic(shape, T):
    """DRAM bytes per gate-up launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture) from the
    committed summary of this shape and token count, else None."""
    name = {(2880, 2880, 128, 64, "mxfp4"): "gemm_mxf4_gptoss_decode_T64.md",
            (2880, 2880, 128, 8192, "mxfp4"): "gemm_mxf4_gptoss_prefill_T8192.md",
            (7168, 2048, 32, 4096, "fp8_128"): "gemm_fp8_dsv3_E32_T4096.md"}.get((shape.H, shape.I, shape.E, T, shape.wq))
    f = ROOT / "profiles" / name if name else None
    if f is not None and f.exists():
        m = re.search(r"roofline\.traffic[^\n]*gate-up (\d+) bytes", f.read_text())
        if m:
            return float(m.group(1))
    return None


def measured_peaks(key="hbm_gbs"):
    """(peak, "measured"|"fallback") from the driver-written peaks file; `key` is hbm_gbs,
    bf16_tflops (burst) or bf16_tflops_sustained."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        if key in d:
            return float(d[key]), "measured " + key
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}[key], "fallback " + key


_dense_rate_cache = {}


def dense_mma_rate(dev, kind=0, n=256, count=40000):
    """Dense tensor rate of the whole chip in TFLOP/s for kind 0 (block-scaled FP4, kind::mxf4) or 1 (e4m3,
    kind::mxf8f6f4): every SM issues `count` MMAs of 128 x n x (64 | 32) from resident shared-memory tiles
    (the library's rate probe), timed with stream events after one warm-up launch."""
    import ctypes
    import torch
    from pyhip_b200 import _lib
    if kind in _dense_rate_cache:
        return _dense_rate_cache[kind]
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    cfg = torch.tensor([kind, n, count, 0, 0, 0, 0, 0], dtype=torch.int32, device=dev)
    out = torch.zeros(sms * 3, dtype=torch.int32, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run():
        _lib.check(_lib.lib().b200moe_debug_probe(4, ctypes.c_void_p(cfg.data_ptr()), ctypes.c_void_p(out.data_ptr()), st),
                   "debug_probe")
    run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        run()
    e1.record()
    torch.cuda.synchronize()
    rate = None
    if int(out.view(-1, 3)[:, 2].abs().max()) == 0:
        k = 64 if kind == 0 else 32
        rate = 3.0 * sms * count * 2.0 * 128 * n * k / (e0.elapsed_time(e1) * 1e-3) / 1e12
    _dense_rate_cache[kind] = rate
    return rate


class ClockSampler:
    """nvidia-smi clock/throttle sampling during the timed region (read-only query)."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------
# CPU oracle timing (the reference arm and the cpu_baseline leg)
# ---------------------------------------------------------------------------------------------------
def cpu_oracle_pass(T, shape, seed=0, max_experts=None, budget_s=None):
    """One pass of the CPU oracle (torch dequantise-then-matmul, weights dequantised inside the expert loop as
    the baseline definition says) over the experts the batch hits -- all of them, or the first `max_experts`,
    or as many as fit `budget_s` seconds.  Returns (seconds, experts done, experts hit, pairs done, pairs)."""
    import torch
    from oracle import moe_oracle as orc
    from pyhip_b200 import synth
    torch.set_num_threads(os.cpu_count() or 1)
    x = synth.make_hidden(T, shape.H, seed)
    tw, ids = synth.make_routing(T, shape.E, shape.K, shape.routing, seed, skew_seed=0)
    hit = sorted(set(ids.flatten().tolist()))
    fp8 = shape.wq == "fp8_128"
    fw = synth.FastWeights(shape.E, shape.H, shape.I, seed, shape.wq, distinct=2 if 3.0 * shape.H * shape.I > 1e8 else 4)
    deq = orc.dequant_fp8_128x128 if fp8 else orc.dequant_mxfp4
    todo = hit if max_experts is None else hit[:max_experts]
    done, pairs_done, spent = 0, 0, 0.0
    for e in todo:
        keep = ids == e
        ids_e = torch.where(keep, ids, torch.full_like(ids, -1))
        wq = fw.expert(e)
        t0 = time.perf_counter()

        def ew(_e, wq=wq):
            return deq(wq[0], wq[1], x.dtype), deq(wq[2], wq[3], x.dtype)
        orc.torch_moe_oracle(x, None, None, tw, ids_e, expert_weights=ew)
        spent += time.perf_counter() - t0
        done += 1
        pairs_done += int(keep.sum())
        if budget_s is not None and spent > budget_s:
            break
    return spent, done, len(hit), pairs_done, ids.numel()


def cpu_rate(T, shape, budget_s):
    """tokens/s of the CPU oracle from a bounded pass, scaled to the whole batch by experts where dequantising an
    expert dominates (fewer than 64 rows per expert) and by pairs where the matmuls do."""
    spent, done, hit, pairs_done, pairs = cpu_oracle_pass(T, shape, budget_s=budget_s)
    by_pairs = pairs / shape.E >= 64
    full = spent * ((pairs / max(pairs_done, 1)) if by_pairs else (hit / max(done, 1)))
    text = (f"torch dequantise-then-matmul oracle on {done} of {hit} hit experts ({spent:.2f} s)" +
            ("" if done == hit else f", scaled to the whole batch by {'pairs' if by_pairs else 'experts'}"))
    return T / full, text


def run_reference(args):
    from pyhip_b200 import synth
    shape = synth.CONFIGS[args.workload]
    if args.experts:
        shape = dataclasses.replace(shape, E=args.experts)
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.tokens or shape.T
    # one step = the oracle over EVERY expert the batch hits (no extrapolation) where that takes seconds;
    # the large configurations (minutes per pass on a host CPU) use a bounded pass and say so
    big = 6.0 * shape.H * shape.I * T * shape.K > 2e11
    budget = 20.0 if big else None
    t_start = time.perf_counter()
    cpu_oracle_pass(T, shape, max_experts=2)                       # warm-up (thread pools, allocator)
    times, text = [], ""
    for _ in range(max(1, args.steps)):
        if budget is None:
            spent, done, hit, _, _ = cpu_oracle_pass(T, shape)
            times.append(spent)
            text = f"torch dequantise-then-matmul oracle over all {hit} hit experts, every step"
        else:
            r, text = cpu_rate(T, shape, budget)
            times.append(T / r)
        if time.perf_counter() - t_start > 240:
            break
    sec = statistics.median(times)
    v = T / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times),
        "warmup": 1, "ms_per_step": 1e3 * sec, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload} H{shape.H} I{shape.I} E{shape.E} top{shape.K} T{T} {shape.wq}",
                   "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": text},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# timing
# ---------------------------------------------------------------------------------------------------
def time_steps(fn, steps, warmup, dist=None):
    """Milliseconds of exactly `steps` calls (CUDA events on the current stream, barrier + synchronise on both
    sides, max over ranks)."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def time_repeated(fn, steps, warmup, dist=None, total_ms=1000.0, min_rep=5, max_rep=200):
    """The K-step region repeated until about `total_ms` of GPU time: returns per-step milliseconds
    {"ms", "min", "max", "repeats"} with ms = the median region."""
    first = time_steps(fn, steps, warmup, dist)
    reps = int(min(max_rep, max(min_rep, math.ceil(total_ms / max(first, 1e-3)))))
    regions = [first] + [time_steps(fn, steps, 0, dist) for _ in range(reps - 1)]
    per = sorted(r / steps for r in regions)
    return {"ms": statistics.median(per), "min": per[0], "max": per[-1], "repeats": len(per)}


# ---------------------------------------------------------------------------------------------------
# one GPU
# ---------------------------------------------------------------------------------------------------
def dtype_text(fp8, act_terms, bf16=False):
    if bf16:
        return "bf16 weights x bf16 activations (kind::f16), f32 accumulate"
    if fp8:
        return "fp8-e4m3 128x128-block weights x 2-term e4m3 activations (kind::mxf8f6f4), f32 accumulate"
    nt = act_terms or 3
    return (f"mxfp4 weights x {nt}-term fp4 activations (kind::mxf4), f32 accumulate" if nt > 1 else
            "mxfp4 weights x mxfp4 activations (a4w4, kind::mxf4), f32 accumulate")


class Case:
    """Weights, prepared weights and helpers of one workload on one device."""

    def __init__(self, workload, dev, experts=0, weights="native"):
        import torch
        from pyhip_b200 import QuantType, _lib, synth
        from pyhip_b200.fused_moe import prepare_weights
        shape = synth.CONFIGS[workload]
        if experts:
            shape = dataclasses.replace(shape, E=experts)
        self.bf16 = weights == "bf16"
        if self.bf16:
            # the same shape with unquantised weights, drawn on the device (N(0, 0.02), as the quantised sets are)
            shape = dataclasses.replace(shape, wq="bf16")
            self.workload, self.shape, self.dev = workload, shape, dev
            self.fp8, self.fmt, self.qt, self.wbytes = False, _lib.W_BF16, QuantType.No, 2.0
            g = torch.Generator(device=dev).manual_seed(0)
            w1 = (torch.randn(shape.E, 2 * shape.I, shape.H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            w2 = (torch.randn(shape.E, shape.H, shape.I, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            self.w = (w1, None, w2, None)
            self.pw = prepare_weights(w1, None, w2, None, weight_format=self.fmt)
            torch.cuda.synchronize()
            return
        self.workload, self.shape, self.dev = workload, shape, dev
        self.fp8 = shape.wq == "fp8_128"
        self.fmt = 1 if self.fp8 else 0
        self.qt = QuantType.per_128x128 if self.fp8 else QuantType.per_1x32
        self.wbytes = (1.0 + 4.0 / 16384) if self.fp8 else (0.5 + 1.0 / 32)
        distinct = 2 if 3.0 * shape.H * shape.I > 1e8 else (4 if self.fp8 else 8)
        make_w = synth.make_weights_fp8_fast if self.fp8 else synth.make_weights_mxfp4_fast
        self.w = make_w(shape.E, shape.H, shape.I, seed=0, device=dev, distinct=min(distinct, shape.E))
        self.pw = prepare_weights(*self.w, weight_format=self.fmt)
        torch.cuda.synchronize()

    def dtype_text(self, act_terms):
        return dtype_text(self.fp8, act_terms, self.bf16)

    def inputs(self, T, seed=0):
        from pyhip_b200 import synth
        s = self.shape
        x = synth.make_hidden(T, s.H, seed)
        tw, ids = synth.make_routing(T, s.E, s.K, s.routing, seed, skew_seed=0)
        return x, tw, ids


def measure_layer(case, T, args, steps, warmup, combine, act_terms=0, local=0, total_ms=None, act_quant=0, batch1=False):
    """Whole-layer timing at T tokens: graph replay of the call's launches; batches whose expert set fits L2
    rotate over enough different routing sets that every step streams its weights from HBM."""
    import torch
    from pyhip_b200 import _lib, synth
    from pyhip_b200.fused_moe import capture_forward, get_plan, launches_per_call, moe_forward, pick_block
    s, dev = case.shape, case.dev
    x0, tw0, ids0 = case.inputs(T, 0)
    hit0 = len(set(ids0.flatten().tolist()))
    step_bytes = hit0 * 3.0 * s.H * s.I * case.wbytes
    n_sets = 1 if step_bytes > 4 * L2_BYTES else int(min(64, math.ceil(6 * L2_BYTES / max(step_bytes, 1.0))))
    sets = [tuple(t.to(dev) for t in case.inputs(T, i)) for i in range(n_sets)]
    hits = [len(set(st[2].flatten().tolist())) for st in sets]
    B = pick_block(T, s.K, s.E, case.fmt)
    cm = _lib.COMBINE_FUSED if combine == "fused" else _lib.COMBINE_GATHER
    plan = get_plan(T, s.K, s.E, s.E, s.H, s.I, B, 0, 7.0, dev, act_terms=act_terms, weight_format=case.fmt, combine_mode=cm,
                    act_quant=act_quant, cta_pairs=PAIRS[args.cta_pairs])
    y = torch.empty(T, s.H, dtype=torch.bfloat16, device=dev)

    def one_round():
        for xs, tws, idss in sets:
            moe_forward(plan, case.pw, xs, tws, idss, None, y, batch1=batch1)

    launch_mode = "direct launches"
    fn = one_round
    if not args.no_graph:
        try:
            one_round()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                one_round()
            fn = graph.replay
            launch_mode = "cuda graph replay"
        except Exception as exc:  # noqa: BLE001 - capture is an optimisation, direct launches still measure the path
            launch_mode = f"direct launches (graph capture failed: {type(exc).__name__})"
    rounds = max(1, steps // n_sets)
    sampler = ClockSampler(local)
    r = time_repeated(fn, rounds, max(1, warmup // n_sets), total_ms=args.repeat_ms if total_ms is None else total_ms)
    clocks = sampler.stop()
    plan.check_status()
    ms = r["ms"] / n_sets
    hit = statistics.mean(hits)
    peak, _ = measured_peaks()
    layer_bytes = synth.algorithmic_bytes(T, s.H, s.I, hit, s.wq)
    return {"T": T, "ms_per_step": ms, "ms_per_step_min": r["min"] / n_sets, "ms_per_step_max": r["max"] / n_sets,
            "repeats": r["repeats"], "steps_per_region": rounds * n_sets, "tokens_per_s": T / (ms * 1e-3),
            "experts_hit": hit, "block": B, "combine": combine,
            "act_terms": 0 if case.bf16 else (1 if act_quant else 2) if case.fp8 else (act_terms or 3),
            "launch": launch_mode, "launches_per_step": launches_per_call(T, s.K, s.E, cm, batch1),
            "path": "batch-1 (no sort, CUDA cores)" if batch1 else "sorted grouped GEMMs (tensor cores)",
            "routing_sets_rotated": n_sets,
            "layer_gbs": layer_bytes / (ms * 1e-3) / 1e9,
            "frac_of_hbm_measured": layer_bytes / (ms * 1e-3) / 1e9 / peak,
            "frac_of_hbm_nominal_8tbs": layer_bytes / (ms * 1e-3) / 1e9 / 8000.0,
            "layer_tflops": synth.algorithmic_flops(T, s.K, s.H, s.I) / (ms * 1e-3) / 1e12,
            "clocks": clocks}


def measure_gemms(case, T, args, steps, warmup, act_terms=0, act_quant=0):
    """The two grouped GEMMs timed alone on the layer's own sorted / quantised inputs: returns the roofline record
    of the gate-up launch (the dominant kernel)."""
    import torch
    from pyhip_b200.fused_moe import get_plan, pick_block
    s, dev = case.shape, case.dev
    x, tw, ids = (t.to(dev) for t in case.inputs(T, 0))
    hit = len(set(ids.flatten().tolist()))
    B = pick_block(T, s.K, s.E, case.fmt)
    plan = get_plan(T, s.K, s.E, s.E, s.H, s.I, B, 0, 7.0, dev, act_terms=act_terms, weight_format=case.fmt, act_quant=act_quant,
                    cta_pairs=PAIRS[args.cta_pairs])
    if case.bf16:
        # no stage-by-stage front end for unquantised weights: one whole call leaves the sort arrays and the bf16
        # rows of both stages in the workspace, and the two GEMMs are then timed on them
        from pyhip_b200.fused_moe import moe_forward
        moe_forward(plan, case.pw, x, tw, ids, None, torch.empty(T, s.H, dtype=torch.bfloat16, device=dev))
    else:
        plan.sort(ids, tw)
        plan.quant_input(x)
    k = max(3, min(steps, 200 if T <= 512 else 20))
    gu = time_repeated(lambda: plan.gateup(case.pw, None), k, 3, total_ms=300.0)
    dn = time_repeated(lambda: plan.down(case.pw), k, 3, total_ms=300.0)
    plan.check_status()
    per_launch_s = gu["ms"] * 1e-3
    gu_bytes = hit * 2.0 * s.H * s.I * case.wbytes + T * s.H * 2.0
    gu_flops = 4.0 * T * s.K * s.H * s.I
    peak, peak_kind = measured_peaks()
    hbm_time = gu_bytes / (peak * 1e9)
    nominal = BF16_NOMINAL_TFLOPS if case.bf16 else FP8_NOMINAL_TFLOPS if case.fp8 else FP4_NOMINAL_TFLOPS
    common = {"kernel": ("moe_grouped_gemm_bf16_kernel<gate-up>" if case.bf16 else
                         "moe_grouped_gemm_fp8_kernel<gate-up>" if case.fp8 else "moe_grouped_gemm_kernel<gate-up>"),
              "us_per_launch": per_launch_s * 1e6, "us_per_launch_min": gu["min"] * 1e3,
              "down_us_per_launch": dn["ms"] * 1e3, "traffic": profiled_traffic(s, T) if not (act_terms == 1 or act_quant) else None,
              "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture summarised under profiles/ "
                                "(same kernel and shape; not measured in this run)"}
    # weight-streaming regime (few rows per expert): HBM roofline; from 64 rows per expert on the launch is scored
    # against the dense tensor rate of its format, as the configurations state (the gpt-oss prefill shape sits at
    # the ridge: at the nominal rates its tensor time is 0.7 of its HBM time)
    if T * s.K / s.E >= 64 or gu_flops / (nominal * 1e12) > hbm_time:
        ach = gu_flops / per_launch_s / 1e12
        bf16, bf16_kind = measured_peaks("bf16_tflops_sustained" if gu["ms"] > 0.5 else "bf16_tflops")
        if case.bf16:       # scored against the measured cuBLAS bf16 rate, with the nominal dense figure beside it
            return {"bound": "tensor", "achieved": ach, "peak": bf16, "unit": "TFLOP/s", "frac": ach / bf16,
                    "peak_kind": bf16_kind, "frac_of_nominal_bf16_2250": ach / nominal, "algorithmic_flops": gu_flops,
                    "mma_work_over_algorithmic": 1.0, **common}
        probe = dense_mma_rate(dev, 1 if case.fp8 else 0)
        return {"bound": "tensor", "achieved": ach, "peak": nominal, "unit": "TFLOP/s", "frac": ach / nominal,
                "peak_kind": ("nominal dense FP8 (4.5 PFLOP/s)" if case.fp8 else "nominal dense FP4 (9 PFLOP/s)"),
                "peak_probe_tflops": probe, "frac_of_probe": ach / probe if probe else None,
                "peak_probe_kind": "block-scaled MMAs from resident tiles on every SM, this run (the library's rate probe)",
                "frac_of_bf16_" + bf16_kind.replace(" ", "_"): ach / bf16, "algorithmic_flops": gu_flops,
                "mma_work_over_algorithmic": ((1.0 if act_quant else 2.0) if case.fp8 else float(act_terms or 3)), **common}
    achieved = gu_bytes / per_launch_s / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_kind": peak_kind, "algorithmic_bytes": gu_bytes, **common}


def measure_e2e(case, T, args, steps, warmup, combine, act_terms=0, act_quant='terms'):
    import torch
    from pyhip_b200 import fused_moe
    s, dev = case.shape, case.dev
    x, tw, ids = case.inputs(T, 0)
    xh, twh, idsh = x.pin_memory(), tw.pin_memory(), ids.pin_memory()
    yh = torch.empty(T, s.H, dtype=torch.bfloat16).pin_memory()
    w = case.w

    def step_e2e():
        xg = xh.to(dev, non_blocking=True)
        tg = twh.to(dev, non_blocking=True)
        ig = idsh.to(dev, non_blocking=True)
        out = fused_moe(xg, w[0], w[2], tg, ig, quant_type=case.qt, w1_scale=w[1], w2_scale=w[3], combine=combine,
                        act_terms=act_terms, act_quant=act_quant if case.fp8 else "terms", cta_pairs=args.cta_pairs,
                        method=args.method)
        yh.copy_(out, non_blocking=True)

    r = time_repeated(step_e2e, steps, warmup, total_ms=min(args.repeat_ms, 500.0))
    return {"value": T / (r["ms"] * 1e-3), "unit": UNIT, "ms_per_step": r["ms"], "repeats": r["repeats"],
            "h2d_bytes_per_step": x.numel() * 2 + tw.numel() * 4 + ids.numel() * 4, "d2h_bytes_per_step": T * s.H * 2}


def run_single(args, dev, local):
    import torch
    from pyhip_b200 import release_prepared, synth
    case = Case(args.workload, dev, args.experts, args.weights)
    is_bf16 = case.bf16
    if is_bf16:
        args.no_extras, args.no_cpu_baseline, args.act_terms = True, True, 0
    s = case.shape
    T = args.tokens or s.T
    aq = 1 if (args.act_quant == '1x128' and case.fp8) else 0
    b1 = args.method == "batch1"
    head = measure_layer(case, T, args, args.steps, args.warmup, args.combine, args.act_terms, local, act_quant=aq, batch1=b1)
    other = "gather" if args.combine == "fused" else "fused"
    alt = measure_layer(case, T, args, args.steps, args.warmup, other, args.act_terms, local, total_ms=300.0, act_quant=aq,
                        batch1=b1)
    e2e = measure_e2e(case, T, args, args.steps, args.warmup, args.combine, args.act_terms, args.act_quant)
    if b1:       # two matrix-vector launches: the whole call against the HBM rate
        peak, peak_kind = measured_peaks()
        roofline = {"bound": "hbm", "achieved": head["layer_gbs"], "peak": peak, "unit": "GB/s",
                    "frac": head["layer_gbs"] / peak, "peak_kind": peak_kind, "traffic": None,
                    "kernel": "batch1_gateup_kernel + batch1_down_kernel (whole call)",
                    "us_per_launch": head["ms_per_step"] * 1e3 / 2}
    else:
        roofline = measure_gemms(case, T, args, args.steps, args.warmup, args.act_terms, act_quant=aq)
    extras = {}
    default_run = not args.no_extras and args.workload == "gptoss_decode" and not args.tokens and not args.experts
    if default_run:
        st = max(20, min(args.steps, 200))
        extras["sweep"] = [measure_layer(case, Ts, args, st, 3, args.combine, args.act_terms, local, total_ms=300.0)
                           for Ts in (1, 8, 32, 256)]
        # the reference-style sort-free path for one token beside the sweep's T = 1 entry
        extras["batch1_T1"] = measure_layer(case, 1, args, st, 3, args.combine, 0, local, total_ms=200.0, batch1=True)
        Tp = synth.CONFIGS["gptoss_prefill"].T
        pre = {}
        for nt, name in ((0, "three_term"), (1, "a4w4")):
            m = measure_layer(case, Tp, args, 20, 3, args.combine, nt, local, total_ms=300.0)
            m["roofline"] = measure_gemms(case, Tp, args, 20, 3, nt)
            m["dtype"] = case.dtype_text(nt)
            m["parity_oracle"] = ("bf16-activation oracle (cosine >= 0.9995)" if nt == 0 else
                                  "a4w4 oracle that dequantises the same MXFP4 activations (calc_diff <= 0.01)")
            pre[name] = m
        extras["prefill"] = pre
    cpu = None
    if not args.no_cpu_baseline:
        r, text = cpu_rate(T, s, 12.0)
        cpu = {"value": r, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": text}
    if default_run:
        del case
        release_prepared()
        torch.cuda.empty_cache()
        for key, wl in (("config3", "dsv3_ep"), ("config4", "mixtral_skew")):
            c2 = Case(wl, dev)
            m = measure_layer(c2, c2.shape.T, args, 10, 3, args.combine, 0, local, total_ms=300.0)
            m["roofline"] = measure_gemms(c2, c2.shape.T, args, 10, 3, 0)
            m["dtype"] = c2.dtype_text(0)
            m["workload"] = f"{wl} H{c2.shape.H} I{c2.shape.I} E{c2.shape.E} top{c2.shape.K} T{c2.shape.T} {c2.shape.wq}"
            if c2.fp8:
                # the reference's own activation format beside the default: per-token 1x128 e4m3 with fp32 scales
                m2 = measure_layer(c2, c2.shape.T, args, 10, 3, args.combine, 0, local, total_ms=300.0, act_quant=1)
                m2["roofline"] = measure_gemms(c2, c2.shape.T, args, 10, 3, 0, act_quant=1)
                m2["dtype"] = "fp8-e4m3 128x128-block weights x e4m3 activations with fp32 scales per 1x128, f32 accumulate"
                m2["parity_oracle"] = "oracle that dequantises the same 1x128-quantised activations (cosine >= 0.9995)"
                m["act_1x128"] = m2
            extras[key] = m
            del c2
            release_prepared()
            torch.cuda.empty_cache()
    hit = head["experts_hit"]
    line = {"metric": METRIC, "value": head["tokens_per_s"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "ms_per_step_min": head["ms_per_step_min"],
            "ms_per_step_max": head["ms_per_step_max"], "repeats": head["repeats"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": dtype_text(s.wq == "fp8_128", args.act_terms, is_bf16), "data": "synthetic",
            "config": {"workload": f"{args.workload} H{s.H} I{s.I} E{s.E} top{s.K} T{T} {s.wq}", "block": head["block"],
                       "combine": args.combine, "launch": head["launch"],
                       "l2": ("inputs larger than L2: %.2f GB of expert weights streamed per step" %
                              (hit * 3.0 * s.H * s.I * (2.0 if is_bf16 else (1.0 + 4.0 / 16384) if s.wq == "fp8_128" else (0.5 + 1.0 / 32)) / 1e9)
                              + (f"; {head['routing_sets_rotated']} routing sets rotated" if head["routing_sets_rotated"] > 1 else ""))},
            "clocks": head["clocks"], "e2e": e2e, "gpu_launches": head["launches_per_step"] * head["steps_per_region"],
            "roofline": roofline, "cpu_baseline": cpu,
            "layer": {k: head[k] for k in ("layer_gbs", "frac_of_hbm_measured", "frac_of_hbm_nominal_8tbs", "layer_tflops",
                                           "experts_hit", "launches_per_step")},
            "other_combine": {k: alt[k] for k in ("combine", "ms_per_step", "tokens_per_s", "launches_per_step")}}
    line.update(extras)
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# expert parallel, N > 1
# ---------------------------------------------------------------------------------------------------
def ep_parity(rank, world, dev, dist):
    """A small expert-parallel layer through both exchange forms on the GPUs, every rank's output against the CPU
    oracle of the unsharded layer on its own tokens (the reference's expert-parallel check,
    tests/contrib/moe/test_fused_moe.py:35-44,70-81).  Returns the worst figures over all ranks."""
    import torch
    from oracle import moe_oracle as orc
    from pyhip_b200 import ep, synth
    H, I, K = 512, 256, 4
    E = 16 * world
    El = E // world
    w = synth.make_weights_mxfp4(E, H, I, seed=3)
    w_loc = tuple(t[rank * El:(rank + 1) * El].to(dev) for t in w)
    out = {}
    for name, T, kw in (("dispatch", 96, dict(exchange="dispatch")), ("gathered", 32, dict(tokens_per_rank=32)),
                        ("dispatch_fused_combine", 70 + rank, dict(exchange="dispatch", combine="fused"))):
        layer = ep.ExpertParallelMoE(*w_loc, E, rank, world, **kw)
        x = synth.make_hidden(T, H, seed=20 + rank)
        tw, ids = synth.make_routing(T, E, K, "zipf", seed=20 + rank, skew_seed=1)
        y = layer.forward(x.to(dev), tw.to(dev), ids.to(dev))
        torch.cuda.synchronize()
        ref = orc.torch_moe_oracle_mxfp4(x, *w, tw, ids)
        t = torch.tensor([1.0 - orc.cosine(y.cpu(), ref), orc.max_abs(y.cpu(), ref)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = {"worst_cosine": 1.0 - float(t[0]), "worst_max_abs": float(t[1])}
    ok = all(v["worst_cosine"] >= 0.9995 and v["worst_max_abs"] <= 2e-2 for v in out.values())
    return {"ok": ok, "oracle": "CPU torch dequantise-then-matmul layer, unsharded, bf16 activations",
            "tolerance": "cosine >= 0.9995, max-abs <= 2e-2", **out}


def measure_ep(workload, args, rank, world, local, dev, dist, steps, warmup, total_ms):
    import torch
    from pyhip_b200 import QuantType, ep, synth
    from pyhip_b200.fused_moe import get_plan, pick_block, prepare_weights
    shape = synth.CONFIGS[workload]
    if args.experts and workload == args.workload:
        shape = dataclasses.replace(shape, E=args.experts)
    H, I, E, K = shape.H, shape.I, shape.E, shape.K
    T = (args.tokens if (args.tokens and workload == args.workload) else shape.T)
    strong = workload == "mixtral_skew"        # this configuration states a global token count
    if strong:
        T //= world
    fp8 = shape.wq == "fp8_128"
    qt = QuantType.per_128x128 if fp8 else QuantType.per_1x32
    fmt = 1 if fp8 else 0
    wbytes = (1.0 + 4.0 / 16384) if fp8 else (0.5 + 1.0 / 32)
    distinct = 2 if 3.0 * H * I > 1e8 else (4 if fp8 else 8)
    make_w = synth.make_weights_fp8_fast if fp8 else synth.make_weights_mxfp4_fast
    E_local = E // world
    w_full = make_w(E_local, H, I, seed=rank, device=dev, distinct=min(distinct, E_local))
    layer = ep.ExpertParallelMoE(w_full[0], w_full[1], w_full[2], w_full[3], E, rank, world, quant_type=qt,
                                 dispatch_chunks=args.ep_chunks or None, tokens_per_rank=T, combine=args.combine,
                                 **({'act_quant': args.act_quant} if fp8 else {'cta_pairs': args.cta_pairs}))
    x = synth.make_hidden(T, H, rank)
    tw, ids = synth.make_routing(T, E, K, shape.routing, rank, skew_seed=0)
    xd, twd, idsd = x.to(dev), tw.to(dev), ids.to(dev)

    def step():
        layer.forward(xd, twd, idsd)

    sampler = ClockSampler(local)
    r = time_repeated(step, steps, warmup, dist, total_ms=total_ms)
    clocks = sampler.stop()
    xh, twh, idsh = x.pin_memory(), tw.pin_memory(), ids.pin_memory()
    yh = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        out = layer.forward(xh.to(dev, non_blocking=True), twh.to(dev, non_blocking=True),
                            idsh.to(dev, non_blocking=True))
        yh.copy_(out, non_blocking=True)

    ms_e2e = time_steps(step_e2e, steps, min(warmup, 3), dist) / steps

    # ---- per-rank time inside the local experts (load balance), three extra steps
    layer.busy_events = []
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    busy = statistics.median(a.elapsed_time(b) for a, b in layer.busy_events) if layer.busy_events else 0.0
    layer.busy_events = None
    # ---- where one step's time goes on rank 0 (marks inside the dispatch/combine call), one extra step
    phases = None
    if layer.exchange == "dispatch":
        layer.trace = []
        step()
        torch.cuda.synchronize()
        tr, layer.trace = layer.trace, None
        phases = [(tr[i + 1][0], round(tr[i][1].elapsed_time(tr[i + 1][1]), 3)) for i in range(len(tr) - 1)]
    busy_t = torch.tensor([busy], device=dev)
    busy_all = [torch.zeros_like(busy_t) for _ in range(world)]
    dist.all_gather(busy_all, busy_t)

    # ---- dominant kernel on this rank's rows (gate-up grouped GEMM), timed alone on rank 0
    roofline = None
    if rank == 0 and layer.last_local is not None:
        xr, twr, idr = layer.last_local
        n = xr.shape[0]
        pw = prepare_weights(*w_full, weight_format=fmt)
        plan = get_plan(n, K, E_local, E_local, H, I, pick_block(n, K, E, fmt), 0, 7.0, dev, weight_format=fmt)
        plan.sort(idr.contiguous(), twr.contiguous())
        plan.quant_input(xr)
        k_steps = max(3, min(steps, 50))
        ms_gu = time_steps(lambda: plan.gateup(pw, None), k_steps, 3)
        plan.check_status()
        idc = idr.flatten()
        hit_l = int(torch.unique(idc[(idc >= 0) & (idc < E_local)]).numel())
        pairs_l = int(((idc >= 0) & (idc < E_local)).sum())
        per = ms_gu * 1e-3 / k_steps
        peak, peak_kind = measured_peaks()
        gu_bytes = hit_l * 2.0 * H * I * wbytes + n * H * 2.0
        roofline = {"bound": "hbm", "achieved": gu_bytes / per / 1e9, "peak": peak, "unit": "GB/s",
                    "frac": gu_bytes / per / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                    "kernel": "gate-up grouped GEMM on rank 0's received rows", "us_per_launch": per * 1e6,
                    "algorithmic_bytes": gu_bytes, "tflops": 4.0 * pairs_l * H * I / per / 1e12,
                    "frac_of_tensor_nominal": 4.0 * pairs_l * H * I / per / 1e12 / (FP8_NOMINAL_TFLOPS if fp8 else FP4_NOMINAL_TFLOPS),
                    "rows": n, "pairs": pairs_l, "experts_hit": hit_l, "block": plan.shape.B}
    dist.barrier()
    from pyhip_b200 import release_prepared
    ms = r["ms"]
    rec = {"workload": f"{workload} H{H} I{I} E{E} top{K} T{T}/gpu {shape.wq} expert-parallel",
           "tokens_per_gpu": T, "scaling": "strong" if strong else "weak",
           "ms_per_step": ms, "ms_per_step_min": r["min"], "ms_per_step_max": r["max"], "repeats": r["repeats"],
           "tokens_per_s": T * world / (ms * 1e-3), "e2e_tokens_per_s": T * world / (ms_e2e * 1e-3),
           "exchange": "all-gather + reduce-scatter" if layer.exchange == "gathered" else "all-to-all-v dispatch and combine",
           "clocks": clocks, "roofline": roofline,
           "local_expert_ms_per_rank": [round(float(b.item()), 4) for b in busy_all], "rank0_phase_ms": phases,
           "h2d_bytes_per_step": x.numel() * 2 + tw.numel() * 4 + ids.numel() * 4, "d2h_bytes_per_step": T * H * 2,
           "launches_per_step": None}
    del layer, w_full
    release_prepared()
    torch.cuda.empty_cache()
    return rec, shape, fp8


def run_ep(args, rank, world, local, dev, dist):
    parity = ep_parity(rank, world, dev, dist)
    if not parity["ok"]:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "error": "expert-parallel parity check failed", "parity": parity}), flush=True)
        dist.destroy_process_group()
        sys.exit(3)
    head, shape, fp8 = measure_ep(args.workload, args, rank, world, local, dev, dist, args.steps, args.warmup, args.repeat_ms)
    extras = {}
    if not args.no_extras and args.workload == "gptoss_decode" and not args.tokens and not args.experts:
        for key, wl in (("config3", "dsv3_ep"), ("config4", "mixtral_skew")):
            extras[key], _, _ = measure_ep(wl, args, rank, world, local, dev, dist, 10, 3, 300.0)
    if rank == 0:
        gathered = head["exchange"].startswith("all-gather")
        T = head["tokens_per_gpu"]
        small = T * world * shape.K <= 256
        per_step = (3 if small else 4) + (0 if args.combine == "fused" else 1) + (0 if gathered else 2)
        line = {"metric": METRIC, "value": head["tokens_per_s"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "ms_per_step_min": head["ms_per_step_min"],
                "ms_per_step_max": head["ms_per_step_max"], "repeats": head["repeats"], "higher_is_better": True,
                "scaling": head["scaling"], "vs_baseline": None,
                "dtype": dtype_text(fp8, args.act_terms), "data": "synthetic",
                "config": {"workload": head["workload"], "parallelism": f"ep{world}", "combine": args.combine,
                           "l2": "inputs larger than L2 (expert weights streamed)", "exchange": head["exchange"]},
                "clocks": head["clocks"],
                "e2e": {"value": head["e2e_tokens_per_s"], "unit": UNIT, "h2d_bytes_per_step": head["h2d_bytes_per_step"],
                        "d2h_bytes_per_step": head["d2h_bytes_per_step"]},
                # this library's kernels per step on every rank (NCCL's kernels are not counted): the layer's own
                # launches plus, in the dispatch form, the plan and the gather-sum
                "gpu_launches": per_step * args.steps,
                "roofline": head["roofline"], "cpu_baseline": None, "parity": parity,
                "local_expert_ms_per_rank": head["local_expert_ms_per_rank"], "rank0_phase_ms": head["rank0_phase_ms"]}
        line.update(extras)
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def run_b200(args):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        run_ep(args, rank, world, local, dev, dist)
    else:
        run_single(args, dev, local)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_b200(a)
