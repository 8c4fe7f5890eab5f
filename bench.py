"""Benchmark of the fused-MoE hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--tokens T]

One "step" is one MoE layer call on one batch of synthetic tokens.  At N=1 the workload is the
gpt-oss-120b-shaped MXFP4 layer (H=I=2880, E=128, top-4) at T=64 decode tokens -- the
weight-streaming regime the headline metric is quoted on.  At N>1 the same layer runs
expert-parallel, one process per GPU (torchrun), T tokens per GPU, with the dispatch/combine
all-to-all over NCCL inside the timed region.

Prints ONE JSON line (rank 0).  `value` = tokens/s with inputs resident in HBM, timed with CUDA
events over exactly K steps; `e2e` = the same through the public `fused_moe` call with pinned
host buffers copied in and the result copied out every step; `roofline` = the gate-up grouped
GEMM (the dominant kernel) against the measured HBM copy rate; `cpu_baseline` = the CPU oracle
timed on a bounded sample of the same workload.  `--impl reference` times only that CPU path.
"""
import argparse
import json
import os
import pathlib
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
    ap.add_argument("--workload", default="gptoss_decode", choices=["gptoss_decode", "gptoss_prefill", "dsv3_ep"],
                    help="gptoss_*: MXFP4 weights (BASELINE configs 1, 2); dsv3_ep: FP8 128x128 weights (config 3)")
    ap.add_argument("--sweep", action="store_true", help="also time T in {1,8,32,64,256,8192} (extra keys)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time direct launches instead of CUDA-graph replays")
    return ap.parse_args()


def profiled_traffic(workload, T):
    """DRAM bytes per gate-up launch from the committed ncu capture of this workload, else None."""
    f = ROOT / "profiles" / "gemm_mxf4_gptoss_decode_T64_traffic.json"
    if workload == "gptoss_decode" and T == 64 and f.exists():
        return json.loads(f.read_text()).get("gateup_dram_bytes")
    return None


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


def cpu_oracle_rate(T, shape, sample_experts, seed=0, repeats=1):
    """tokens/s of the CPU oracle, measured on the first `sample_experts` experts that the batch
    hits (weights dequantised inside the expert loop, as the baseline definition says) and scaled
    by (experts hit / experts sampled)."""
    import torch
    from oracle import moe_oracle as orc
    from pyhip_b200 import synth
    torch.set_num_threads(os.cpu_count() or 1)
    x = synth.make_hidden(T, shape.H, seed)
    tw, ids = synth.make_routing(T, shape.E, shape.K, shape.routing, seed)
    hit = sorted(set(ids.flatten().tolist()))
    sample = hit[:sample_experts]
    w = synth.make_weights_mxfp4(max(sample) + 1, shape.H, shape.I, seed, experts=sample)
    keep = torch.zeros(shape.E, dtype=torch.bool)
    keep[sample] = True
    ids_s = torch.where(keep[ids.long()], ids, torch.full_like(ids, -1))
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.torch_moe_oracle_mxfp4(x, *w, tw, ids_s)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    full = best * len(hit) / len(sample)
    return T / full, {"experts_hit": len(hit), "experts_sampled": len(sample), "sample_seconds": round(best, 3)}


def run_reference(args):
    from pyhip_b200 import synth
    shape = synth.CONFIGS["gptoss_decode"]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.tokens or shape.T
    rates, info = [], None
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_oracle_rate(T, shape, 2)
    t_start = time.perf_counter()
    for _ in range(max(1, args.steps)):
        r, info = cpu_oracle_rate(T, shape, 4)
        rates.append(r)
        if time.perf_counter() - t_start > 150:
            break
    v = statistics.median(rates)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": len(rates),
        "warmup": args.warmup, "ms_per_step": 1e3 * T / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"gptoss_decode H2880 I2880 E128 top4 T{T} mxfp4", "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                         "sample": f"torch dequantise-then-matmul oracle on {info['experts_sampled']} of "
                                   f"{info['experts_hit']} hit experts per step, scaled to all hit experts"},
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
    T, H, I, E, K = (args.tokens or shape.T), shape.H, shape.I, shape.E, shape.K
    launches_per_step = 5
    fp8 = shape.wq == "fp8_128"
    qt = QuantType.per_128x128 if fp8 else QuantType.per_1x32
    fmt = 1 if fp8 else 0
    make_w = synth.make_weights_fp8_fast if fp8 else synth.make_weights_mxfp4_fast
    wbytes = (1.0 + 4.0 / 16384) if fp8 else (0.5 + 1.0 / 32)
    dtype_s = ("fp8-e4m3 128x128-block weights x 2-term e4m3 activations (kind::mxf8f6f4), f32 accumulate" if fp8 else
               "mxfp4 weights x 3-term fp4 activations (kind::mxf4), f32 accumulate")

    if world == 1:
        w = make_w(E, H, I, seed=0, device=dev)
        pw = prepare_weights(*w, weight_format=fmt)
        x = synth.make_hidden(T, H, 0)
        tw, ids = synth.make_routing(T, E, K, shape.routing, 0)
        hit = len(set(ids.flatten().tolist()))
        xd, twd, idsd = x.to(dev), tw.to(dev), ids.to(dev)
        B = pick_block(T, K, E)
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
        peak, peak_kind = measured_peaks()
        achieved = gu_bytes / per_launch_s / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": profiled_traffic(args.workload, T), "kernel": "moe_grouped_gemm_kernel<gate-up>", "peak_kind": peak_kind,
                    "us_per_launch": per_launch_s * 1e6, "down_us_per_launch": ms_dn * 1e3 / args.steps,
                    "algorithmic_bytes": gu_bytes}
        layer_bytes = synth.algorithmic_bytes(T, H, I, hit, shape.wq)
        extra = {"layer_gbs": layer_bytes / (ms * 1e-3 / args.steps) / 1e9,
                 "layer_frac_of_hbm_peak": layer_bytes / (ms * 1e-3 / args.steps) / 1e9 / peak,
                 "layer_tflops": synth.algorithmic_flops(T, K, H, I) / (ms * 1e-3 / args.steps) / 1e12,
                 "experts_hit": hit}
        sweep = None
        if args.sweep and not fp8:
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
        if not args.no_cpu_baseline and not fp8:
            r, info = cpu_oracle_rate(T, shape, 4)
            cpu = {"value": r, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                   "sample": f"torch dequantise-then-matmul oracle on {info['experts_sampled']} of "
                             f"{info['experts_hit']} hit experts ({info['sample_seconds']} s), scaled to all hit experts"}
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
    experts = list(range(rank * E_local, (rank + 1) * E_local))
    w_full = make_w(E_local, H, I, seed=rank, device=dev)
    layer = ep.ExpertParallelMoE(w_full[0], w_full[1], w_full[2], w_full[3], E, rank, world, quant_type=qt)
    x = synth.make_hidden(T, H, rank)
    tw, ids = synth.make_routing(T, E, K, shape.routing, rank)
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
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": dtype_s,
                "data": "synthetic",
                "config": {"workload": f"{args.workload} H{H} I{I} E{E} top{K} T{T}/gpu {shape.wq} expert-parallel",
                           "parallelism": f"ep{world}", "l2": "inputs larger than L2 (expert weights streamed)"},
                "clocks": clocks,
                "e2e": {"value": T * world * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": x.numel() * 2 + tw.numel() * 4 + ids.numel() * 4,
                        "d2h_bytes_per_step": T * H * 2},
                "gpu_launches": launches_per_step * args.steps}
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_b200(a)
