#!/usr/bin/env python
"""Benchmark of the MoE expert bank on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline workload `olmoe_q4k_decode`: the OLMoE-shaped layer in decode form (hidden 2048, 64 experts,
top-8 without renormalisation, intermediate 1024, GGUF Q4_K experts quantised from seeded
N(0, 0.02) weights, f16 N(0, 1) activations) at T=64 tokens.  One step = one pass of T tokens
through 16 distinct layers' banks (3.6 GB of Q4_K in rotation, so weights come from HBM, not L2).
metric = MoE-layer tokens/s = T * layers / step time.  On N > 1 GPUs the experts are sharded
(expert parallelism over peer memory) and every GPU brings its own T tokens.

The same JSON line carries the other targets as sub-records: `sweep` (T = 1 .. 64), `prefill`
(T = 4096, bf16, Zipf-skewed routing, tensor-core grouped GEMMs), `olmoe_decode` (the whole
OLMoE-1B-7B-shaped model, greedy decode at batch 1 and 32) and, at every N, `ep_qwen3` (the
Qwen3-30B-A3B-shaped expert-parallel stack, T = 16384 per step over all GPUs: strong scaling).
`--workload` runs one of them alone as the headline.  Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

os.environ["NCCL_DEBUG"] = os.environ.get("MUMMU_NCCL_DEBUG", "WARN")   # stdout carries one JSON line only

H, I, E, K = 2048, 1024, 64, 8
EXPERT_BYTES_Q4K = 3 * H * I * 144 // 256          # 3,538,944 B: gate + up + down of one expert
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the gate/up kernel, from ncu captures
# (summaries under profiles/), keyed by (tokens, experts hit); other shapes report null
GATE_UP_TRAFFIC = {(64, 64): 156.35e6}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all",
                    choices=["all", "olmoe_q4k_decode", "olmoe_bf16_prefill", "olmoe_decode", "ep_qwen3", "ep_skew"])
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--ep-layers", type=int, default=48, help="layers of the Qwen3-shaped expert-parallel stack")
    ap.add_argument("--new-tokens", type=int, default=128, help="decode steps of the olmoe_decode workload")
    ap.add_argument("--batches", default="1,32", help="batch sizes of the olmoe_decode workload")
    ap.add_argument("--ep-form", default="auto", choices=["auto", "gathered", "hops"],
                    help="decode-sized expert-parallel steps: tokens to every GPU (gathered) or the three-hop exchange")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub", action="store_true", help="headline only (profiling runs)")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 9:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(float(s[1]) for s in self.samples)
        reasons = set()
        for s in self.samples:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(self.samples[0][2]),
                "reasons": sorted(reasons), "samples": len(self.samples),
                "power_w_max": max(float(s[3]) for s in self.samples)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return {"hbm": float(d["hbm_gbs"]), "tc": float(d["bf16_tflops"]),
                    "tc_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "kind": "measured"}
        except Exception:
            pass
    return {"hbm": 6650.0, "tc": 1590.0, "tc_sustained": 1400.0, "kind": "fallback"}


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle (a port of the reference's algorithm; the reference itself is Rust and cannot
# be built on this image) timed on the host cores, on a bounded sample of the same workload
# ----------------------------------------------------------------------------------------------
def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_sample(tokens: int, sample_layers: int, seed: int = 0):
    from oracle import oracle as O
    from mummu_b200 import q4k, synth
    O.set_num_threads(host_cores())          # a launcher may have exported OMP_NUM_THREADS=1
    layers = []
    for l in range(sample_layers):
        router, gate, up, down, x = synth.moe_layer(H, I, E, tokens, cfg_seed=seed, layer=l)
        layers.append((router, q4k.quantize(gate), q4k.quantize(up), q4k.quantize(down),
                       x.astype(np.float16).astype(np.float32)))

    def run():
        for router, gq, uq, dq, x in layers:
            O.moe_forward(x, router, gq, uq, dq, K, False, q4k=True)
    return run, O.num_threads()


def decode_config(tokens: int, layers: int, world: int) -> dict:
    name = f"olmoe_q4k_decode_T{tokens}" + ("_per_gpu" if world > 1 else "")
    return {"workload": name, "hidden": H, "intermediate": I, "experts": E, "top_k": K, "norm_topk_prob": False,
            "tokens": tokens * world, "layers_per_step": layers}


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return 0
    sample_layers = 1
    run, cores = cpu_sample(args.tokens, sample_layers)
    warm = min(args.warmup, 1)
    for _ in range(warm):
        run()
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    value = args.tokens * sample_layers / dt
    sample = (f"{sample_layers} layer of the workload per step (T={args.tokens}, all 64 experts' Q4_K banks, "
              f"quantised from SplitMix64 N(0,0.02) weights), {steps} timed steps on {cores} host threads")
    cfg = decode_config(args.tokens, sample_layers, world)
    cfg["note"] = ("CPU restatement of the reference's routed Q4_K expert bank (dequantise rows, f32 dots), one "
                   "process on the host cores; the reference is Rust and cannot be built on this image; the "
                   "metric is per layer-token, so a one-layer sample compares with the 16-layer GPU step")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------------------------
# timing helpers
# ----------------------------------------------------------------------------------------------
class Ctx:
    def __init__(self, args, rank, world, local_rank):
        import torch
        self.torch, self.args, self.rank, self.world, self.local_rank = torch, args, rank, world, local_rank
        self.device = torch.device("cuda", local_rank)
        torch.cuda.set_device(self.device)
        self.dist = None
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.device)
            self.dist = dist
        self.stream = torch.cuda.Stream(self.device)
        torch.cuda.set_stream(self.stream)      # every launch and every event below is on this stream
        self.peaks = measured_peaks()

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def max_over_ranks(self, v: float) -> float:
        if self.dist is None:
            return v
        t = self.torch.tensor([v], device=self.device, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def windows(self, run, steps: int, warmup: int, min_total_ms: float = 600.0, max_windows: int = 40,
                sync_ranks: bool = True):
        """ms per step of windows of EXACTLY `steps` steps each, timed with CUDA events on the launching
        stream between a barrier + synchronize on both sides, maximum over ranks per window; after
        `warmup` untimed steps.  Windows repeat until about `min_total_ms` of device time is covered
        (a 20-step window of a 1.5 ms step alone would be 30 ms)."""
        torch = self.torch
        for _ in range(warmup):
            run()
        out, total = [], 0.0
        while len(out) < 3 or (total < min_total_ms and len(out) < max_windows):
            torch.cuda.synchronize()
            if sync_ranks:
                self.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for _ in range(steps):
                run()
            b.record()
            torch.cuda.synchronize()
            if sync_ranks:
                self.barrier()
            ms = a.elapsed_time(b)
            if sync_ranks:
                ms = self.max_over_ranks(ms)
            out.append(ms / steps)
            total += ms
        return out


def graphed(torch, step):
    """`step` captured once in a CUDA graph on the current stream (the CPU's launch cost leaves the
    device's critical path); returns the replay callable."""
    step()
    torch.cuda.current_stream().synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=torch.cuda.current_stream()):
        step()
    return g.replay


def kernel_profile(torch, handles, step, reps: int, spin_cycles: int = 200_000_000):
    """Average launch duration per internal kernel (CUDA event pairs on the launching stream), taken
    behind a device-side spin so that no launch waits for the CPU."""
    for h in handles:
        h.set_profiling(True)
    step()                                  # creates the event pool outside the measured pass
    torch.cuda.synchronize()
    for h in handles:
        h.take_profile()
    torch.cuda._sleep(spin_cycles)
    for _ in range(reps):
        step()
    torch.cuda.synchronize()
    prof = {}
    for h in handles:
        for name, (n, avg_ms) in h.take_profile().items():
            cur = prof.setdefault(name, [0, 0.0])
            cur[0] += n
            cur[1] += avg_ms * n
        h.set_profiling(False)
    return {name: {"launches": n, "avg_us": 1e3 * tot / n} for name, (n, tot) in prof.items() if n}


# ----------------------------------------------------------------------------------------------
# headline at N = 1: Q4_K decode, T tokens through NL layers
# ----------------------------------------------------------------------------------------------
def build_decode_layers(ctx, layers: int, tokens: int, seed: int):
    torch = ctx.torch
    from mummu_b200 import _lib as L, moe
    gen = torch.Generator(device=ctx.device)
    gen.manual_seed(seed)
    out = []
    for l in range(layers):
        m = moe.SparseMoeConfig(H, I, E, K).init(device=ctx.device.index, act_dtype=L.F16,
                                                 weight_dtype=L.Q4_K, max_tokens=max(tokens, 64))
        m.set_router((torch.randn(H, E, generator=gen, device=ctx.device) * 0.02).cpu().numpy())
        for which, shape in ((L.BANK_GATE, (E, I, H)), (L.BANK_UP, (E, I, H)), (L.BANK_DOWN, (E, H, I))):
            w = torch.randn(shape, generator=gen, device=ctx.device) * 0.02
            m.set_bank(which, moe.q4k_quantize_device(w))
            del w
        out.append(m)
    torch.cuda.synchronize(ctx.device)
    return out, gen


def experts_hit(torch, layers, xs):
    hit = []
    for m, x in zip(layers, xs):
        ids, _ = m.route_flat(x, K, False)
        hit.append(int(torch.unique(ids).numel()))
    torch.cuda.synchronize()
    return float(np.mean(hit))


def measure_decode(ctx, line: dict):
    torch, args = ctx.torch, ctx.args
    T, NL = args.tokens, args.layers or 16
    layers, gen = build_decode_layers(ctx, NL, T, seed=1234 + ctx.rank)
    xs = [torch.randn(T, H, generator=gen, device=ctx.device).to(torch.float16) for _ in range(NL)]
    u_mean = experts_hit(torch, layers, xs)

    def step():
        for m, x in zip(layers, xs):
            m.forward(x, K, False)

    launches0 = sum(m.launch_count() for m in layers)
    step()
    launches_per_step = sum(m.launch_count() for m in layers) - launches0
    replay = graphed(torch, step)
    with ClockSampler(ctx.local_rank) as clocks:
        win = ctx.windows(replay, args.steps, args.warmup, min_total_ms=800.0)
    ms = statistics.median(win)
    eager = statistics.median(ctx.windows(step, args.steps, 2, min_total_ms=100.0, max_windows=3, sync_ranks=False))
    value = T * NL / (ms * 1e-3)

    kern = kernel_profile(torch, layers, step, max(3, min(args.steps, 10)))
    peaks = ctx.peaks
    gu_bytes = u_mean * 2 * H * I * 144 / 256 + T * H * 2 + T * K * I * 2     # weights + x read + hact write
    roof = None
    if "q4k_gate_up" in kern:
        ach = gu_bytes / (kern["q4k_gate_up"]["avg_us"] * 1e-6) / 1e9
        roof = {"bound": "hbm", "kernel": "q4k_gate_up", "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": ach / peaks["hbm"], "peak_kind": peaks["kind"],
                "traffic": GATE_UP_TRAFFIC.get((T, int(round(u_mean)))),
                "algorithmic_bytes_per_launch": gu_bytes, "frac_of_nominal_8TBs": ach / 8000.0}
    layer_bytes = u_mean * EXPERT_BYTES_Q4K + H * E * 4 + 2 * T * H * 2

    # ---- end to end through the host-pointer C ABI call: pinned host buffers in and out ----
    hx = [x.cpu().pin_memory() for x in xs]
    hx_np = [h.numpy() for h in hx]
    hy_np = [torch.empty_like(h).pin_memory().numpy() for h in hx]      # results land in pinned memory too

    def e2e_step():
        for m, xn, yn in zip(layers, hx_np, hy_np):
            m.forward(xn, K, False, out=yn)     # H2D copy, layer, D2H copy, stream sync: all inside the call
    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    e2e_steps = max(3, min(args.steps, 20))
    e2e_win = []
    for _ in range(5):
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_win.append((time.perf_counter() - t0) * 1e3 / e2e_steps)
    e2e_ms = statistics.median(e2e_win)

    cpu = None
    if not args.no_cpu_baseline:
        run, cores = cpu_sample(T, 1)
        run()
        reps = 3
        t0 = time.perf_counter()
        for _ in range(reps):
            run()
        dt = (time.perf_counter() - t0) / reps
        cpu = {"value": T / dt, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"1 layer of the workload (T={T}, 64 experts Q4_K), {reps} repetitions after 1 warm-up; "
                         "CPU restatement of the reference algorithm (oracle/), OpenMP"}

    cfg = decode_config(T, NL, 1)
    cfg.update({"l2": "inputs larger than L2: %d distinct layer banks (%.2f GB Q4_K) rotate every step"
                      % (NL, NL * E * EXPERT_BYTES_Q4K / 1e9),
                "launch": "one CUDA graph per step (%d layer calls captured from the C ABI)" % NL,
                "parallelism": "single GPU", "experts_hit_mean": u_mean})
    line.update({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "ms_per_step_min": min(win), "timed_windows": len(win), "eager_ms_per_step": eager,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 activations x Q4_K weights, f32 accumulate", "data": "synthetic", "config": cfg,
        "e2e": {"value": T * NL / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": NL * T * H * 2,
                "d2h_bytes_per_step": NL * T * H * 2, "ms_per_step": e2e_ms},
        "gpu_launches": int(launches_per_step * args.steps), "gpu_launches_per_step": int(launches_per_step),
        "clocks": clocks.summary(), "roofline": roof,
        "layer": {"algorithmic_bytes": layer_bytes, "us": 1e3 * ms / NL,
                  "GBps": layer_bytes * NL / (ms * 1e-3) / 1e9,
                  "frac_of_measured_hbm": layer_bytes * NL / (ms * 1e-3) / 1e9 / peaks["hbm"],
                  "frac_of_nominal_8TBs": layer_bytes * NL / (ms * 1e-3) / 1e9 / 8000.0},
        "kernels": kern, "cpu_baseline": cpu,
    })

    # ---- sweep over T: the decode regime from one token up ----
    if not args.no_sub:
        sweep = {}
        for t_s in (1, 2, 4, 8, 16, 32, 64):
            xs_s = [torch.randn(t_s, H, generator=gen, device=ctx.device).to(torch.float16) for _ in range(NL)]
            u = experts_hit(torch, layers, xs_s)

            def step_s():
                for m, x in zip(layers, xs_s):
                    m.forward(x, K, False)
            ms_s = statistics.median(ctx.windows(graphed(torch, step_s), args.steps, 3, min_total_ms=150.0,
                                                 max_windows=10, sync_ranks=False))
            b = u * EXPERT_BYTES_Q4K + H * E * 4 + 2 * t_s * H * 2
            gbs = b * NL / (ms_s * 1e-3) / 1e9
            sweep[str(t_s)] = {"us_per_layer": 1e3 * ms_s / NL, "tokens_per_s": t_s * NL / (ms_s * 1e-3),
                               "experts_hit": u, "layer_bytes": b, "layer_GBps": gbs,
                               "frac_of_measured_hbm": gbs / peaks["hbm"], "frac_of_nominal_8TBs": gbs / 8000.0}
        line["sweep"] = sweep
    for m in layers:
        m.close()
    torch.cuda.empty_cache()


# ----------------------------------------------------------------------------------------------
# prefill: T=4096, bf16, Zipf-skewed routing, tensor-core grouped GEMMs
# ----------------------------------------------------------------------------------------------
def measure_prefill(ctx) -> dict:
    torch, args = ctx.torch, ctx.args
    from mummu_b200 import _lib as L, moe, synth
    T = 4096
    NL = 2
    gen = torch.Generator(device=ctx.device)
    gen.manual_seed(4321 + ctx.rank)
    layers = []
    for l in range(NL):
        m = moe.SparseMoeConfig(H, I, E, K).init(device=ctx.device.index, act_dtype=L.BF16, weight_dtype=L.BF16,
                                                 max_tokens=T)
        m._router_np = (torch.randn(H, E, generator=gen, device=ctx.device) * 0.02).cpu().numpy()
        m.set_router(m._router_np)
        for which, shape in ((L.BANK_GATE, (E, I, H)), (L.BANK_UP, (E, I, H)), (L.BANK_DOWN, (E, H, I))):
            m.set_bank(which, (torch.randn(shape, generator=gen, device=ctx.device) * 0.02).to(torch.bfloat16))
        layers.append(m)
    xs = [torch.randn(T, H, generator=gen, device=ctx.device).to(torch.bfloat16) for _ in range(NL)]
    # router-logit bias b_e = -alpha * 1.1 * ln(rank_e): alpha calibrated so hottest / mean load ~ 8
    alpha, ratio = None, None
    for cand in (0.5, 1.0, 1.5, 2.0, 2.5, 3.0, 4.0, 6.0):
        layers[0].set_router(layers[0]._router_np, bias=synth.zipf_router_bias(E, cand))
        ids, _ = layers[0].route_flat(xs[0], K, False)
        load = torch.bincount(ids.reshape(-1).long(), minlength=E).float()
        alpha, ratio = cand, float(load.max() / load.mean())
        if ratio >= 7.6:
            break
    for m in layers:
        m.set_router(m._router_np, bias=synth.zipf_router_bias(E, alpha))
    torch.cuda.synchronize()

    def step():
        for m, x in zip(layers, xs):
            m.forward(x, K, False)
    l0 = sum(m.launch_count() for m in layers)
    step()
    launches_per_step = sum(m.launch_count() for m in layers) - l0
    win = ctx.windows(step, args.steps, max(args.warmup, 3), min_total_ms=500.0, sync_ranks=False)
    ms = statistics.median(win)
    kern = kernel_profile(torch, layers, step, 5, spin_cycles=100_000_000)
    peaks = ctx.peaks
    flops_gu, flops_dn = T * K * 2 * 2 * H * I, T * K * 2 * H * I
    out = {"workload": f"olmoe_bf16_prefill_T{T}", "tokens": T, "layers_per_step": NL, "zipf_alpha": alpha,
           "hottest_over_mean_load": ratio, "dtype": "bf16 x bf16, f32 accumulate",
           "tokens_per_s": T * NL / (ms * 1e-3), "ms_per_step": ms, "us_per_layer": 1e3 * ms / NL,
           "launch": "eager", "gpu_launches_per_step": int(launches_per_step), "kernels": kern,
           "l2": "inputs larger than L2: %.2f GB of bf16 banks per layer, %d layers rotate" % (3 * E * H * I * 2 / 1e9, NL)}
    layer_tflops = (flops_gu + flops_dn) * NL / (ms * 1e-3) / 1e12
    out["whole_layer"] = {"TFLOPs": layer_tflops, "frac_of_burst_peak": layer_tflops / peaks["tc"],
                          "frac_of_sustained_peak": layer_tflops / peaks["tc_sustained"]}
    if "tc_gate_up" in kern and "tc_down" in kern:
        gu = flops_gu / (kern["tc_gate_up"]["avg_us"] * 1e-6) / 1e12
        dn = flops_dn / (kern["tc_down"]["avg_us"] * 1e-6) / 1e12
        both = (flops_gu + flops_dn) / ((kern["tc_gate_up"]["avg_us"] + kern["tc_down"]["avg_us"]) * 1e-6) / 1e12
        out["roofline"] = {"bound": "tensor", "kernel": "tc_gate_up", "achieved": gu, "peak": peaks["tc"],
                           "unit": "TFLOP/s", "frac": gu / peaks["tc"], "frac_of_sustained_peak": gu / peaks["tc_sustained"],
                           "peak_kind": peaks["kind"], "traffic": None, "flops_per_launch": flops_gu,
                           "tc_down_TFLOPs": dn, "tc_down_frac_of_burst": dn / peaks["tc"],
                           "both_gemms_TFLOPs": both, "both_gemms_frac_of_burst": both / peaks["tc"],
                           "both_gemms_frac_of_sustained": both / peaks["tc_sustained"]}
    for m in layers:
        m.close()
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------------------------
# whole-model decode: OLMoE-1B-7B-shaped, random weights, Q4_K experts, f16 trunk
# ----------------------------------------------------------------------------------------------
def measure_model(ctx) -> dict:
    torch = ctx.torch
    from mummu_b200 import _lib as L
    from mummu_b200.olmoe import OlmoeConfig, OlmoeDecoder
    cfg = OlmoeConfig()
    prompt, n_new = 512, ctx.args.new_tokens
    peaks = ctx.peaks
    results = {}
    for B in [int(b) for b in ctx.args.batches.split(",")]:
        chunk = max(1, 2048 // B)                       # prompt fed in chunks of <= 2048 tokens over the batch
        dec = OlmoeDecoder(cfg, device=ctx.local_rank, expert_dtype=L.Q4_K, max_batch=B, max_ctx=prompt + n_new,
                           max_tokens=B * chunk)
        dec.random_init(seed=11)
        gen = torch.Generator(device=ctx.device)
        gen.manual_seed(5 + B)
        ids = torch.randint(0, cfg.vocab_size, (B, prompt), generator=gen, device=ctx.device)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        toks, ms, launches = dec.greedy_generate_static(ids, n_new, chunk=chunk, timed=True)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        # bytes one decode step has to read: routed experts, attention weights, lm_head, the KV cache so far
        hit = E * (1.0 - (1.0 - K / E) ** B)
        ctx_mean = prompt + n_new / 2
        step_bytes = (cfg.num_hidden_layers * (hit * EXPERT_BYTES_Q4K + 4 * cfg.hidden_size ** 2 * 2
                                               + B * ctx_mean * 2 * cfg.hidden_size * 2)
                      + cfg.vocab_size * cfg.hidden_size * 2)
        results[f"batch_{B}"] = {"decode_tok_per_s": B * n_new / (ms * 1e-3), "ms_per_token_step": ms / n_new,
                                 "prefill_plus_decode_wall_s": wall, "step_bytes": step_bytes,
                                 "GBps": step_bytes / (ms / n_new * 1e-3) / 1e9,
                                 "frac_of_measured_hbm": step_bytes / (ms / n_new * 1e-3) / 1e9 / peaks["hbm"],
                                 "launches_per_step": launches}
        dec.close()
        del dec
        torch.cuda.empty_cache()
    return {"workload": "olmoe_1b_7b_shaped_greedy_decode", "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "experts": cfg.num_experts, "top_k": cfg.num_experts_per_tok,
            "vocab": cfg.vocab_size, "prompt": prompt, "new_tokens": n_new, "dtype": "f16 trunk, Q4_K experts",
            "launch": "one CUDA graph per decode step", **results}


# ----------------------------------------------------------------------------------------------
# expert-parallel stacks (N >= 1): the decode workload sharded (weak) and the Qwen3-shaped one (strong)
# ----------------------------------------------------------------------------------------------
def measure_ep(ctx, shape: dict) -> dict:
    torch, args, world, rank = ctx.torch, ctx.args, ctx.world, ctx.rank
    from mummu_b200 import _lib as L, moe
    from mummu_b200.ep import ExpertParallelMoe, PeerWorkspace
    h, i, e, k = shape["hidden"], shape["inter"], shape["experts"], shape["top_k"]
    T, NL, q4 = shape["tokens_per_rank"], shape["layers"], shape["q4k"]
    act, wdt = (L.F16, L.Q4_K) if q4 else (L.BF16, L.BF16)
    tdt = torch.float16 if q4 else torch.bfloat16
    el = e // world
    cfg = moe.SparseMoeConfig(h, i, e, k)
    gen = torch.Generator(device=ctx.device)
    plan = shape.get("placement")                                   # None: contiguous shards
    bias = shape.get("bias")
    slots_total = plan.virtual_experts if plan is not None else e
    mine = plan.rank_experts(rank).tolist() if plan is not None else list(range(rank * el, rank * el + el))
    # decode-sized steps take the small-batch form (every token to every rank), whose return buffer
    # is indexed by the common sorted order: as many rows as all ranks route together
    gathered = q4 and (args.ep_form == "gathered" or (args.ep_form == "auto" and world * T * k <= 1024))
    ws = (PeerWorkspace(None, ctx.local_rank, world * T * k, h, slots_total, back_rows=world * T * k if gathered else 0)
          if world > 1 else None)
    layers = []
    for l in range(NL):
        gen.manual_seed(9000 + l)                                   # router: same on every rank
        router = (torch.randn(h, e, generator=gen, device=ctx.device) * 0.02).cpu().numpy()
        if world > 1:
            m = ExpertParallelMoe(cfg, device=ctx.local_rank, act_dtype=act, weight_dtype=wdt, max_tokens=T,
                                  workspace=ws, scratch_donor=layers[0][0] if layers else None, placement=plan)
            handle = m.moe
        else:
            m = cfg.init(device=ctx.local_rank, act_dtype=act, weight_dtype=wdt, max_tokens=T if not layers else 0)
            if layers:
                m.adopt_scratch(layers[0][0])
            handle = m
        m.set_router(router, bias=bias)
        for which, shp in ((L.BANK_GATE, (i, h)), (L.BANK_UP, (i, h)), (L.BANK_DOWN, (h, i))):
            parts = []
            for ex in mine:                                         # an expert's weights follow the expert, not the rank
                gen.manual_seed(100000 + 1000 * l + 8 * ex + which)
                parts.append(torch.randn(shp, generator=gen, device=ctx.device) * 0.02)
            wt = torch.stack(parts)
            handle.set_bank(which, moe.q4k_quantize_device(wt) if q4 else wt.to(tdt))
            del wt, parts
        layers.append((m, handle))
    gen.manual_seed(777 + rank)
    xs = [torch.randn(T, h, generator=gen, device=ctx.device).to(tdt) for _ in range(min(NL, 8))]
    torch.cuda.synchronize()

    def step():
        for n, (m, _) in enumerate(layers):
            m.forward(xs[n % len(xs)], k, False)

    l0 = sum(hd.launch_count() for _, hd in layers)
    step()
    launches_per_step = sum(hd.launch_count() for _, hd in layers) - l0
    # decode-sized steps are launch-bound: replay one CUDA graph per step (the ranks signal each other
    # through peer memory, so the multi-GPU step holds no library collective and is captured too)
    run, is_graph = step, False
    if q4:
        try:
            torch.cuda.synchronize()
            ctx.barrier()
            run, is_graph = graphed(torch, step), True
            torch.cuda.synchronize()
        except Exception as exc:                                  # keep the eager step
            sys.stderr.write(f"graph capture of the expert-parallel step failed, running eagerly: {exc}\n")
            torch.cuda.synchronize()
            run = step
    steps = args.steps if q4 else max(3, min(args.steps, 5))
    with ClockSampler(ctx.local_rank) as clocks:
        win = ctx.windows(run, steps, max(args.warmup, 3) if q4 else 3, min_total_ms=600.0, max_windows=20 if q4 else 3)
    ms = statistics.median(win)

    hx = [x.cpu().pin_memory() for x in xs]

    def e2e_step():
        for n, (m, _) in enumerate(layers):
            xd = hx[n % len(hx)].to(ctx.device, non_blocking=True)
            m.forward(xd, k, False).cpu()
    e2e_ms = statistics.median(ctx.windows(e2e_step, max(2, min(steps, 5)), 1, min_total_ms=0.0, max_windows=3))
    kern = kernel_profile(torch, [hd for _, hd in layers], step, 2, spin_cycles=50_000_000)
    for _, hd in layers:
        hd.sync()                               # raises if a bounded device-side wait ran out or a row was dropped

    hits = None
    if shape.get("want_hits"):
        hits = np.zeros(e, dtype=np.uint64)
        for m, _ in layers:
            m.take_hits()                                           # drop what warm-up and timing counted
        step()
        torch.cuda.synchronize()
        for m, _ in layers:
            hits += m.take_hits()
        if world > 1:
            t_h = torch.from_numpy(hits.astype(np.int64)).to(ctx.device)
            ctx.dist.all_reduce(t_h)
            hits = t_h.cpu().numpy().astype(np.uint64)
    total_tokens = T * world
    flops = total_tokens * k * 6 * h * i * NL
    out = {"workload": shape["name"], "scaling": shape["scaling"], "hidden": h, "intermediate": i, "experts": e,
           "top_k": k, "norm_topk_prob": False, "tokens_per_gpu": T, "tokens": total_tokens, "layers_per_step": NL,
           "n_gpus": world, "steps": steps, "ms_per_step": ms, "ms_per_step_min": min(win), "timed_windows": len(win),
           "tokens_per_s": total_tokens * NL / (ms * 1e-3), "us_per_layer": 1e3 * ms / NL,
           "launch": "one CUDA graph per step" if is_graph else "eager",
           "parallelism": ((f"ep{world}: {el} experts per GPU, " +
                            ("tokens pushed to every GPU, replicated bit-reproducible routing, expert outputs pushed back"
                             if gathered and plan is None else
                             "rows pushed to the experts' GPUs, expert outputs pushed back from the down GEMM's epilogue") +
                            ": peer stores over NVLink, one-way device-side signals, no host sync, no collective")
                           if world > 1 else "single GPU"),
           "l2": "inputs larger than L2: %.2f GB of expert weights per GPU rotate every step"
                 % (NL * el * 3 * h * i * (144 / 256 if q4 else 2) / 1e9),
           "e2e": {"value": total_tokens * NL / (e2e_ms * 1e-3), "unit": UNIT,
                   "h2d_bytes_per_step": NL * T * h * 2 * world, "d2h_bytes_per_step": NL * T * h * 2 * world,
                   "ms_per_step": e2e_ms},
           "gpu_launches_per_step": int(launches_per_step), "clocks": clocks.summary(), "kernels_rank0": kern}
    if not q4:
        peaks = ctx.peaks
        tf = flops / (ms * 1e-3) / 1e12
        out["TFLOPs_all_gpus"] = tf
        out["frac_of_burst_peak_all_gpus"] = tf / (peaks["tc"] * world)
        if world > 1:
            # rows that leave the GPU: (world - 1) / world of T * k rows of hidden 16-bit values, each way
            nv = T * k * h * 2 * (world - 1) / world
            for name in ("ep_dispatch", "ep_return"):
                if name in kern:
                    out[name + "_GBps_per_gpu"] = nv / (kern[name]["avg_us"] * 1e-6) / 1e9
            out["nvlink_bytes_per_gpu_per_layer_each_way"] = nv
    if hits is not None:
        out["_hits"] = hits
    for m, _ in reversed(layers):
        m.close()
    torch.cuda.synchronize()
    if ws is not None:
        ctx.barrier()
        ws.close()
    torch.cuda.empty_cache()
    return out


def measure_ep_skew(ctx) -> dict:
    """The prefill configuration's skewed router (Zipf bias over 64 experts) sharded over the GPUs:
    once with contiguous shards, once with the placement planned from the first run's hit counters
    (experts moved between the ranks, the hottest held on several).  Same tokens, same weights per
    expert; the outputs are bit-equal (tested), the busiest rank's rows and the step time are not."""
    from mummu_b200 import placement as P, synth
    args, world = ctx.args, ctx.world
    total = 4096
    bias = synth.zipf_router_bias(E, 1.0)
    base = dict(hidden=H, inter=I, experts=E, top_k=K, tokens_per_rank=total // world, layers=min(args.ep_layers, 16),
                q4k=False, scaling="strong", bias=bias)
    plain = measure_ep(ctx, dict(base, name=f"olmoe_bf16_zipf_ep_T{total}", want_hits=True))
    hits = plain.pop("_hits")
    hot = P.smooth_hotness([], [int(v) for v in hits], 1.0)
    slots = E // world + 2
    plan = P.plan_placement(hot, E, world, slots)
    placed = measure_ep(ctx, dict(base, name=f"olmoe_bf16_zipf_ep_T{total}_placed", placement=plan))
    share = lambda p: float(p.rank_loads(hot).max() * world)
    keep = ("ms_per_step", "us_per_layer", "tokens_per_s", "gpu_launches_per_step", "kernels_rank0", "clocks")
    return {"workload": f"olmoe_bf16_zipf_ep_T{total}", "n_gpus": world, "layers_per_step": base["layers"],
            "zipf_alpha": 1.0, "slots_per_gpu": slots, "experts_per_gpu_plain": E // world,
            "copies_of_hottest": max(len(hs) for hs in plan.hosts),
            "experts_held_twice_or_more": int(sum(len(hs) > 1 for hs in plan.hosts)),
            "busiest_gpu_load_over_fair_share": {"contiguous": share(P.contiguous_placement(E, world)), "placed": share(plan)},
            "contiguous": {k2: plain[k2] for k2 in keep}, "placed": {k2: placed[k2] for k2 in keep},
            "speedup": plain["ms_per_step"] / placed["ms_per_step"]}


def qwen3_shape(args, world: int) -> dict:
    total = 16384
    return dict(name=f"qwen3_30b_a3b_shaped_ep_T{total}", hidden=2048, inter=768, experts=128, top_k=8,
                tokens_per_rank=total // world, layers=args.ep_layers, q4k=False, scaling="strong")


def main() -> int:
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    ctx = Ctx(args, rank, world, local_rank)
    line: dict = {}
    rc = 0

    def sub(name, fn):
        """A sub-record must not cost the headline its line."""
        nonlocal rc
        if args.no_sub:
            return
        try:
            line[name] = fn()
        except Exception as exc:                                   # reported, and the exit status says so
            import traceback
            traceback.print_exc()
            line[name] = {"error": f"{type(exc).__name__}: {exc}"}
            rc = 4

    if args.workload in ("all", "olmoe_q4k_decode"):
        if world == 1:
            measure_decode(ctx, line)
            if args.workload == "all":
                sub("prefill", lambda: measure_prefill(ctx))
                sub("olmoe_decode", lambda: measure_model(ctx))
        else:
            # the headline on N GPUs: same layer, experts sharded, every GPU brings its own T tokens
            r = measure_ep(ctx, dict(name=f"olmoe_q4k_decode_T{args.tokens}_per_gpu", hidden=H, inter=I, experts=E,
                                     top_k=K, tokens_per_rank=args.tokens, layers=args.layers or 16, q4k=True,
                                     scaling="weak"))
            cfg = decode_config(args.tokens, r["layers_per_step"], world)
            cfg.update({k2: r[k2] for k2 in ("tokens_per_gpu", "launch", "parallelism", "l2")})
            line.update({"metric": METRIC, "value": r["tokens_per_s"], "unit": UNIT, "n_gpus": world,
                         "steps": r["steps"], "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"],
                         "ms_per_step_min": r["ms_per_step_min"], "timed_windows": r["timed_windows"],
                         "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                         "dtype": "f16 activations x Q4_K weights, f32 accumulate", "data": "synthetic",
                         "config": cfg, "e2e": r["e2e"],
                         "gpu_launches": int(r["gpu_launches_per_step"] * r["steps"]),
                         "gpu_launches_per_step": r["gpu_launches_per_step"], "clocks": r["clocks"], "roofline": None,
                         "kernels_rank0": r["kernels_rank0"], "cpu_baseline": None})
        if args.workload == "all":
            sub("ep_qwen3", lambda: measure_ep(ctx, qwen3_shape(args, world)))
            if world > 1:
                sub("ep_skew", lambda: measure_ep_skew(ctx))
    elif args.workload == "olmoe_bf16_prefill":
        r = measure_prefill(ctx)
        line.update({"metric": METRIC, "value": r["tokens_per_s"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                     "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                     "scaling": "weak", "vs_baseline": None, "dtype": r["dtype"], "data": "synthetic",
                     "config": {"workload": r["workload"], "tokens": r["tokens"], "layers_per_step": r["layers_per_step"]},
                     "roofline": r.get("roofline"), "prefill": r})
    elif args.workload == "olmoe_decode":
        r = measure_model(ctx)
        big = r["batch_" + str(max(int(b) for b in args.batches.split(",")))]
        line.update({"metric": "olmoe_decode_tokens_per_s", "value": big["decode_tok_per_s"], "unit": UNIT,
                     "n_gpus": 1, "steps": r["new_tokens"], "warmup": 0, "ms_per_step": big["ms_per_token_step"],
                     "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": r["dtype"],
                     "data": "synthetic", "config": {"workload": r["workload"]}, "olmoe_decode": r})
    elif args.workload == "ep_qwen3":
        r = measure_ep(ctx, qwen3_shape(args, world))
        line.update({"metric": METRIC, "value": r["tokens_per_s"], "unit": UNIT, "n_gpus": world, "steps": r["steps"],
                     "warmup": 3, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                     "vs_baseline": None, "dtype": "bf16 x bf16, f32 accumulate", "data": "synthetic",
                     "config": {"workload": r["workload"], "tokens": r["tokens"], "layers_per_step": r["layers_per_step"]},
                     "e2e": r["e2e"], "ep_qwen3": r})
    elif args.workload == "ep_skew":
        if world < 2:
            raise SystemExit("the ep_skew workload shards experts over GPUs: run it with --gpus 2, 4 or 8")
        r = measure_ep_skew(ctx)
        line.update({"metric": METRIC, "value": r["placed"]["tokens_per_s"], "unit": UNIT, "n_gpus": world,
                     "steps": args.steps, "warmup": 3, "ms_per_step": r["placed"]["ms_per_step"], "higher_is_better": True,
                     "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x bf16, f32 accumulate", "data": "synthetic",
                     "config": {"workload": r["workload"], "layers_per_step": r["layers_per_step"]}, "ep_skew": r})
    if rank == 0:
        print(json.dumps(line), flush=True)
    if ctx.dist is not None:
        # the line is out; a peer that never reaches the teardown must not hold the GPUs for ever
        watchdog = threading.Timer(120.0, lambda: os._exit(3))
        watchdog.daemon = True
        watchdog.start()
        ctx.dist.barrier()
        ctx.dist.destroy_process_group()
        watchdog.cancel()
    return rc


if __name__ == "__main__":
    sys.exit(main())
