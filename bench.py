"""Benchmark of the fused-MoE hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload W] [--tokens T] [--sweep]

One "step" is one MoE layer call on one batch of synthetic tokens.  At N=1 the default workload is
the gpt-oss-120b-shaped MXFP4 layer (H=I=2880, E=128, top-4) at T=64 decode tokens -- the
weight-streaming regime the headline metric is quoted on.  `--workload` selects the other
configurations: gptoss_prefill (T=8192), dsv3_ep (DeepSeek-V3-shaped FP8 128x128, T=4096 per GPU),
mixtral_skew (E=8, Zipf load, T=16384 in total).  At N>1 the layer runs expert-parallel, one process
per GPU (torchrun), with the exchange over NCCL inside the timed region: all-gather + reduce-scatter
at decode sizes, all-to-all-v dispatch/combine above 512 tokens per GPU.

Prints ONE JSON line (rank 0).  `value` = tokens/s with inputs resident in HBM, timed with CUDA
events over exactly K steps (a CUDA-graph replay of the call's five launches at N=1); `e2e` = the
same through the public `fused_moe` call with pinned host buffers copied in and the result copied
out every step; `roofline` = the gate-up grouped GEMM (the dominant kernel) timed alone: against the
measured HBM copy rate where the launch is bandwidth-bound, against the measured dense bf16 rate --
with the dense FP4 MMA rate measured in the same run beside it -- where it is compute-bound;
`cpu_baseline` = the CPU oracle timed on a bounded sample of the same workload.  `--impl reference`
times only that CPU path.  Extra keys: `layer` (whole-call GB/s and TFLOP/s), `sweep`, and at N>1
`local_expert_ms_per_rank` (load balance) and `rank0_phase_ms` (where a step's time goes).
"""
import argparse
import dataclasses
import json
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


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="tokens per GPU per step (0 = the workload's own)")
    ap.add_argument("--workload", default="gptoss_decode", choices=["gptoss_decode", "gptoss_prefill", "dsv3_ep", "mixtral_skew"],
                    help="gptoss_*: MXFP4 weights (BASELINE configs 1, 2); dsv3_ep: FP8 128x128 weights (config 3)")
    ap.add_argument("--experts", type=int, default=0,
                    help="override the number of experts (0 = the workload's own); for small profiling captures")
    ap.add_argument("--ep-chunks", type=int, default=0,
                    help="N>1: slices of the pipelined dispatch/combine exchange (0 = chosen from the shape)")
    ap.add_argument("--sweep", action="store_true", help="also time T in {1,8,32,64,256,8192} (extra keys)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time direct launches instead of CUDA-graph replays")
    return ap.parse_args()


def profiled_traffic(workload, T, E):
    """DRAM bytes per gate-up launch from the committed ncu summary of this workload, else None."""
    name = {("gptoss_decode", 64, 128): "gemm_mxf4_gptoss_decode_T64.md",
            ("gptoss_prefill", 8192, 128): "gemm_mxf4_gptoss_prefill_T8192.md",
            ("dsv3_ep", 4096, 32): "gemm_fp8_dsv3_E32_T4096.md"}.get((workload, T, E))
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


def fp4_dense_rate(dev, n=256, count=40000):
    """Dense FP4 tensor rate of the whole chip in TFLOP/s: every SM issues `count` block-scaled
    kind::mxf4 MMAs of 128 x n x 64 from resident shared-memory tiles (the library's rate probe),
    timed with stream events after one warm-up launch."""
    import ctypes
    import torch
    from pyhip_b200 import _lib
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    cfg = torch.tensor([0, n, count, 1, 0, 0, 0, 0], dtype=torch.int32, device=dev)
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
    if int(out.view(-1, 3)[:, 2].abs().max()) != 0:
        return None
    return 3.0 * sms * count * 2.0 * 128 * n * 64 / (e0.elapsed_time(e1) * 1e-3) / 1e12


class ClockSampler:
    """nvidia-smi clock/throttle sampling during the timed region."""
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
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
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


def cpu_oracle_rate(T, shape, sample_experts, seed=0, target_seconds=10.0):
    """tokens/s of the CPU oracle, measured on the first experts that the batch hits (weights
    dequantised inside the expert loop, as the baseline definition says) and scaled to the whole
    batch: by experts hit where dequantising an expert dominates (fewer than 64 rows per expert),
    by (token, expert) pairs where the matmuls do.  A first pass over `sample_experts` experts
    sizes a second pass of about `target_seconds` of CPU work."""
    import torch
    from oracle import moe_oracle as orc
    from pyhip_b200 import synth
    torch.set_num_threads(os.cpu_count() or 1)
    x = synth.make_hidden(T, shape.H, seed)
    tw, ids = synth.make_routing(T, shape.E, shape.K, shape.routing, seed, skew_seed=0)
    hit = sorted(set(ids.flatten().tolist()))
    fp8 = shape.wq == "fp8_128"
    make = synth.make_weights_fp8 if fp8 else synth.make_weights_mxfp4
    run = orc.torch_moe_oracle_fp8 if fp8 else orc.torch_moe_oracle_mxfp4

    def one(n):
        sample = hit[:n]
        w = make(max(sample) + 1, shape.H, shape.I, seed, experts=sample)
        keep = torch.zeros(shape.E, dtype=torch.bool)
        keep[sample] = True
        ids_s = torch.where(keep[ids.long()], ids, torch.full_like(ids, -1))
        t0 = time.perf_counter()
        run(x, *w, tw, ids_s)
        return time.perf_counter() - t0, len(sample), int(keep[ids.long()].sum())

    dt, n, pairs_s = one(min(sample_experts, len(hit)))
    more = min(len(hit), 32, int(n * target_seconds / max(dt, 1e-3)))
    if more > n:
        dt, n, pairs_s = one(more)
    pairs = ids.numel()
    by_pairs = pairs / shape.E >= 64
    full = dt * (pairs / pairs_s if by_pairs else len(hit) / n)
    return T / full, {"experts_hit": len(hit), "experts_sampled": n, "sample_seconds": round(dt, 3),
                      "scaled_by": "pairs" if by_pairs else "experts"}


def cpu_sample_text(info):
    return (f"torch dequantise-then-matmul oracle on {info['experts_sampled']} of {info['experts_hit']} hit experts "
            f"({info['sample_seconds']} s), scaled to the whole batch by {info['scaled_by']}")


def run_reference(args):
    from pyhip_b200 import synth
    shape = synth.CONFIGS[args.workload]
    if args.experts:
        shape = dataclasses.replace(shape, E=args.experts)
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.tokens or shape.T
    n_sample = 4 if T * shape.K / shape.E < 64 else 1
    rates, info = [], None
    t_start = time.perf_counter()
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_oracle_rate(T, shape, n_sample, target_seconds=0.0)
    for _ in range(max(1, args.steps)):
        r, info = cpu_oracle_rate(T, shape, n_sample)
        rates.append(r)
        if time.perf_counter() - t_start > 120:
            break
    v = statistics.median(rates)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": len(rates),
        "warmup": args.warmup, "ms_per_step": 1e3 * T / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload} H{shape.H} I{shape.I} E{shape.E} top{shape.K} T{T} {shape.wq}",
                   "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                         "sample": cpu_sample_text(info)},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def time_steps(fn, steps, warmup, dist=None):
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


def run_b200(args):
    import torch
    from pyhip_b200 import QuantType, fused_moe, synth
    from pyhip_b200.fused_moe import get_plan, moe_forward, pick_block, prepare_weights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=dev)
        dist = dist_mod

    shape = synth.CONFIGS[args.workload]
    if args.experts:
        shape = dataclasses.replace(shape, E=args.experts)
    T, H, I, E, K = (args.tokens or shape.T), shape.H, shape.I, shape.E, shape.K
    strong = args.workload == "mixtral_skew"        # this configuration states a global token count
    if strong and world > 1:
        T //= world
    launches_per_step = 5
    fp8 = shape.wq == "fp8_128"
    qt = QuantType.per_128x128 if fp8 else QuantType.per_1x32
    fmt = 1 if fp8 else 0
    distinct = 2 if 3.0 * H * I > 1e8 else (4 if fp8 else 8)   # experts drawn on the host (the rest repeat them)
    make_w = synth.make_weights_fp8_fast if fp8 else synth.make_weights_mxfp4_fast
    wbytes = (1.0 + 4.0 / 16384) if fp8 else (0.5 + 1.0 / 32)
    dtype_s = ("fp8-e4m3 128x128-block weights x 2-term e4m3 activations (kind::mxf8f6f4), f32 accumulate" if fp8 else
               "mxfp4 weights x 3-term fp4 activations (kind::mxf4), f32 accumulate")

    if world == 1:
        w = make_w(E, H, I, seed=0, device=dev, distinct=min(distinct, E))
        pw = prepare_weights(*w, weight_format=fmt)
        x = synth.make_hidden(T, H, 0)
        tw, ids = synth.make_routing(T, E, K, shape.routing, 0, skew_seed=0)
        hit = len(set(ids.flatten().tolist()))
        xd, twd, idsd = x.to(dev), tw.to(dev), ids.to(dev)
        B = pick_block(T, K, E, fmt)
        plan = get_plan(T, K, E, E, H, I, B, 0, 7.0, dev, weight_format=fmt)
        y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

        def step():
            moe_forward(plan, pw, xd, twd, idsd, None, y)

        launch_mode = "direct launches"
        if not args.no_graph:
            try:
                from pyhip_b200.fused_moe import capture_forward
                graph, _ = capture_forward(plan, pw, xd, twd, idsd, None, y)
                step = graph.replay
                launch_mode = "cuda graph replay of the five launches"
            except Exception as exc:  # noqa: BLE001 - capture is an optimisation, direct launches still measure the path
                launch_mode = f"direct launches (graph capture failed: {type(exc).__name__})"

        sampler = ClockSampler(local)
        ms = time_steps(step, args.steps, args.warmup)
        clocks = sampler.stop()
        plan.check_status()
        value = T * args.steps / (ms * 1e-3)

        # ---- end to end through the public call, host buffers in and out
        xh, twh, idsh = x.pin_memory(), tw.pin_memory(), ids.pin_memory()
        yh = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()

        def step_e2e():
            xg = xh.to(dev, non_blocking=True)
            tg = twh.to(dev, non_blocking=True)
            ig = idsh.to(dev, non_blocking=True)
            out = fused_moe(xg, w[0], w[2], tg, ig, quant_type=qt, w1_scale=w[1], w2_scale=w[3])
            yh.copy_(out, non_blocking=True)

        ms_e2e = time_steps(step_e2e, args.steps, args.warmup)
        e2e = {"value": T * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": x.numel() * 2 + tw.numel() * 4 + ids.numel() * 4,
               "d2h_bytes_per_step": T * H * 2}

        # ---- dominant kernel (gate-up grouped GEMM) timed alone, same inputs
        plan.sort(idsd, twd)
        plan.quant_input(xd)
        ms_gu = time_steps(lambda: plan.gateup(pw, None), args.steps, args.warmup)
        ms_dn = time_steps(lambda: plan.down(pw), args.steps, args.warmup)
        per_launch_s = ms_gu * 1e-3 / args.steps
        gu_bytes = hit * 2.0 * H * I * wbytes + T * H * 2.0
        gu_flops = 4.0 * T * K * H * I
        peak, peak_kind = measured_peaks()
        achieved = gu_bytes / per_launch_s / 1e9
        hbm_time = gu_bytes / (peak * 1e9)
        tpeak, tpeak_kind = measured_peaks("bf16_tflops_sustained" if ms_gu > 500 else "bf16_tflops")
        if gu_flops / (tpeak * 1e12) > hbm_time:
            # compute-bound launch: report against the measured dense bf16 rate (the only tensor peak the
            # peaks file carries) and, beside it, the dense FP4 MMA rate measured here on every SM at once
            fp4 = fp4_dense_rate(dev)
            ach = gu_flops / per_launch_s / 1e12
            roofline = {"bound": "tensor", "achieved": ach, "peak": tpeak, "unit": "TFLOP/s", "frac": ach / tpeak,
                        "traffic": profiled_traffic(args.workload, T, E), "kernel": "moe_grouped_gemm_kernel<gate-up>",
                        "peak_kind": tpeak_kind + " (dense bf16 GEMM)", "us_per_launch": per_launch_s * 1e6,
                        "down_us_per_launch": ms_dn * 1e3 / args.steps, "algorithmic_flops": gu_flops,
                        "fp4_dense_measured_tflops": fp4}
            if fp8:
                roofline.update({"frac_of_fp8_nominal_4p5pf": ach / 4500.0,
                                 "frac_of_half_fp4_measured": 2 * ach / fp4 if fp4 else None,
                                 "note": "two e4m3 activation terms per product: the MMA work is 2x the algorithmic "
                                         "flops; the FP8 tensor rate is half the FP4 rate measured here"})
            else:
                roofline.update({"frac_of_fp4_measured": ach / fp4 if fp4 else None,
                                 "frac_of_fp4_nominal_9pf": ach / 9000.0,
                                 "note": "three packed-FP4 activation terms per product: the MMA work is 3x the "
                                         "algorithmic flops"})
        else:
            roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "traffic": profiled_traffic(args.workload, T, E), "kernel": "moe_grouped_gemm_kernel<gate-up>",
                        "peak_kind": peak_kind, "us_per_launch": per_launch_s * 1e6,
                        "down_us_per_launch": ms_dn * 1e3 / args.steps, "algorithmic_bytes": gu_bytes}
        layer_bytes = synth.algorithmic_bytes(T, H, I, hit, shape.wq)
        extra = {"layer_gbs": layer_bytes / (ms * 1e-3 / args.steps) / 1e9,
                 "layer_frac_of_hbm_peak": layer_bytes / (ms * 1e-3 / args.steps) / 1e9 / peak,
                 "layer_tflops": synth.algorithmic_flops(T, K, H, I) / (ms * 1e-3 / args.steps) / 1e12,
                 "experts_hit": hit}
        sweep = None
        if args.sweep and args.workload.startswith("gptoss"):
            sweep = []
            for Ts in (1, 8, 32, 64, 256, 8192):
                xs = synth.make_hidden(Ts, H, 0).to(dev)
                tws, idss = (t.to(dev) for t in synth.make_routing(Ts, E, K, shape.routing, 0))
                pl = get_plan(Ts, K, E, E, H, I, pick_block(Ts, K, E), 0, 7.0, dev)
                ys = torch.empty(Ts, H, dtype=torch.bfloat16, device=dev)
                st = 10 if Ts > 1000 else args.steps
                fn = lambda: moe_forward(pl, pw, xs, tws, idss, None, ys)   # noqa: E731
                if not args.no_graph:
                    try:
                        fn = capture_forward(pl, pw, xs, tws, idss, None, ys)[0].replay
                    except Exception:  # noqa: BLE001
                        pass
                m = time_steps(fn, st, 3)
                u = len(set(idss.flatten().tolist()))
                us = m * 1e3 / st
                sweep.append({"T": Ts, "us": us, "tokens_per_s": Ts / (us * 1e-6), "experts_hit": u,
                              "gbs": synth.algorithmic_bytes(Ts, H, I, u) / (us * 1e-6) / 1e9,
                              "tflops": synth.algorithmic_flops(Ts, K, H, I) / (us * 1e-6) / 1e12})
        cpu = None
        if not args.no_cpu_baseline:
            r, info = cpu_oracle_rate(T, shape, 4 if T * K / E < 64 else 1)
            cpu = {"value": r, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": cpu_sample_text(info)}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": dtype_s,
                "data": "synthetic",
                "config": {"workload": f"{args.workload} H{H} I{I} E{E} top{K} T{T} {shape.wq}", "block": B,
                           "launch": launch_mode,
                           "l2": "inputs larger than L2: %.2f GB of expert weights streamed per step" %
                                 (hit * 3.0 * H * I * wbytes / 1e9)},
                "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
                "roofline": roofline, "cpu_baseline": cpu, "layer": extra}
        if sweep:
            line["sweep"] = sweep
        print(json.dumps(line), flush=True)
        return

    # ------------------------------------------------------------------ expert parallel, N > 1
    from pyhip_b200 import ep
    E_local = E // world
    w_full = make_w(E_local, H, I, seed=rank, device=dev, distinct=min(distinct, E_local))
    layer = ep.ExpertParallelMoE(w_full[0], w_full[1], w_full[2], w_full[3], E, rank, world, quant_type=qt,
                                 dispatch_chunks=args.ep_chunks or None)
    x = synth.make_hidden(T, H, rank)
    tw, ids = synth.make_routing(T, E, K, shape.routing, rank, skew_seed=0)
    xd, twd, idsd = x.to(dev), tw.to(dev), ids.to(dev)

    def step():
        layer.forward(xd, twd, idsd)

    sampler = ClockSampler(local)
    ms = time_steps(step, args.steps, args.warmup, dist)
    clocks = sampler.stop()
    value = T * world * args.steps / (ms * 1e-3)
    xh, twh, idsh = x.pin_memory(), tw.pin_memory(), ids.pin_memory()
    yh = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        out = layer.forward(xh.to(dev, non_blocking=True), twh.to(dev, non_blocking=True),
                            idsh.to(dev, non_blocking=True))
        yh.copy_(out, non_blocking=True)

    ms_e2e = time_steps(step_e2e, args.steps, args.warmup, dist)

    # ---- per-rank time inside the local experts (load balance), three extra steps
    layer.busy_events = []
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    busy = statistics.median(a.elapsed_time(b) for a, b in layer.busy_events) if layer.busy_events else 0.0
    layer.busy_events = None
    # ---- where one step's time goes on rank 0 (marks inside the dispatch/combine call), one extra step
    phases = None
    if T > layer.small_batch:
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
        plan = get_plan(n, K, E_local, E_local, H, I, pick_block(n, K, E_local, fmt), 0, 7.0, dev, weight_format=fmt)
        plan.sort(idr.contiguous(), twr.contiguous())
        plan.quant_input(xr)
        k_steps = max(3, min(args.steps, 50))
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
                    "kernel": "moe_grouped_gemm_kernel<gate-up> on rank 0's received rows", "us_per_launch": per * 1e6,
                    "algorithmic_bytes": gu_bytes, "tflops": 4.0 * pairs_l * H * I / per / 1e12,
                    "rows": n, "pairs": pairs_l, "experts_hit": hit_l}
    dist.barrier()
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "strong" if strong else "weak",
                "vs_baseline": None, "dtype": dtype_s,
                "data": "synthetic",
                "config": {"workload": f"{args.workload} H{H} I{I} E{E} top{K} T{T}/gpu {shape.wq} expert-parallel",
                           "parallelism": f"ep{world}", "l2": "inputs larger than L2 (expert weights streamed)",
                           "exchange": "all-gather + reduce-scatter" if T <= layer.small_batch else
                                       "all-to-all-v dispatch and combine"},
                "clocks": clocks,
                "e2e": {"value": T * world * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": x.numel() * 2 + tw.numel() * 4 + ids.numel() * 4,
                        "d2h_bytes_per_step": T * H * 2},
                # this library's kernels per step on every rank: the five of the layer, plus the gather-sum
                # combine in the dispatch form of the exchange (NCCL's kernels are not counted)
                "gpu_launches": (launches_per_step + (1 if T > layer.small_batch else 0)) * args.steps,
                "roofline": roofline, "cpu_baseline": None,
                "local_expert_ms_per_rank": [round(float(b.item()), 4) for b in busy_all],
                "rank0_phase_ms": phases}
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_b200(a)
