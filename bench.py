#!/usr/bin/env python
"""Benchmark of the MoE expert bank on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `olmoe_q4k_decode`: the OLMoE-shaped layer in decode form (hidden 2048, 64 experts,
top-8 without renormalisation, intermediate 1024, GGUF Q4_K experts quantised from seeded
N(0, 0.02) weights, f16 N(0, 1) activations) at T=64 tokens.  One step = one pass of T tokens
through 16 distinct layers' banks (3.6 GB of Q4_K in rotation, so weights come from HBM, not L2).
metric = MoE-layer tokens/s = T * layers / step time.  Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
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


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="olmoe_q4k_decode")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--sweep", action="store_true", help="also time T in 1,2,4,...,64 (extra key)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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


def measured_peak_hbm():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle (a port of the reference's algorithm; the reference itself is Rust and cannot
# be built on this image) timed on the host cores, on a bounded sample of the same workload
# ----------------------------------------------------------------------------------------------
def cpu_sample(tokens: int, sample_layers: int, seed: int = 0):
    from oracle import oracle as O
    from mummu_b200 import q4k, synth
    layers = []
    e_sample = E
    for l in range(sample_layers):
        router, gate, up, down, x = synth.moe_layer(H, I, e_sample, tokens, cfg_seed=seed, layer=l)
        layers.append((router, q4k.quantize(gate), q4k.quantize(up), q4k.quantize(down),
                       x.astype(np.float16).astype(np.float32)))
    def run():
        for router, gq, uq, dq, x in layers:
            O.moe_forward(x, router, gq, uq, dq, K, False, q4k=True)
    return run, O.num_threads()


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    sample_layers = 1
    run, cores = cpu_sample(args.tokens, sample_layers)
    for _ in range(min(args.warmup, 1)):
        run()
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    value = args.tokens * sample_layers / dt
    sample = (f"{sample_layers} layer(s) of the workload per step (T={args.tokens}, all 64 experts' Q4_K banks, "
              f"quantised from SplitMix64 N(0,0.02) weights), {steps} timed steps")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"olmoe_q4k_decode_T{args.tokens}", "hidden": H, "intermediate": I,
                   "experts": E, "top_k": K, "tokens": args.tokens, "layers_per_step": sample_layers,
                   "note": "CPU restatement of the reference's routed Q4_K expert bank "
                           "(dequantise rows, f32 dots); the reference is Rust and cannot be built here"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def build_layers(torch, moe, L, device, layers: int, tokens: int, seed: int):
    """`layers` distinct OLMoE-shaped Q4_K layers on the device + one f16 input batch per layer."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = []
    for l in range(layers):
        m = moe.SparseMoeConfig(H, I, E, K).init(device=device.index, act_dtype=L.F16,
                                                 weight_dtype=L.Q4_K, max_tokens=max(tokens, 64))
        router = (torch.randn(H, E, generator=gen, device=device) * 0.02).cpu().numpy()
        m.set_router(router)
        for which, shape in ((L.BANK_GATE, (E, I, H)), (L.BANK_UP, (E, I, H)), (L.BANK_DOWN, (E, H, I))):
            w = torch.randn(shape, generator=gen, device=device) * 0.02
            m.set_bank(which, moe.q4k_quantize_device(w))
            del w
        out.append(m)
    torch.cuda.synchronize(device)
    return out, gen


def time_steps(torch, layers, xs, steps: int, warmup: int, barrier, graph: bool = True):
    """ms per step on the current torch stream: CUDA events around exactly `steps` steps, after
    `warmup` untimed ones.  With graph=True one step (all layers) is captured once in a CUDA graph
    and replayed, so the CPU's launch cost is off the device's critical path."""
    def step():
        for m, x in zip(layers, xs):
            m.forward(x, K, False)
    run = step
    if graph:
        step()
        torch.cuda.current_stream().synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=torch.cuda.current_stream()):
            step()
        run = g.replay
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    barrier()
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(steps):
        run()
    b.record()
    torch.cuda.synchronize()
    barrier()
    return a.elapsed_time(b) / steps


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    from mummu_b200 import _lib as L, moe
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if dist is not None:
            dist.barrier()

    T, NL = args.tokens, args.layers
    stream = torch.cuda.Stream(device)
    torch.cuda.set_stream(stream)          # every launch and every event below is on this stream
    layers, gen = build_layers(torch, moe, L, device, NL, T, seed=1234 + rank)
    xs = [torch.randn(T, H, generator=gen, device=device).to(torch.float16) for _ in range(NL)]

    # distinct experts hit per layer (for the algorithmic byte count)
    hit = []
    for m, x in zip(layers, xs):
        ids, _ = m.route_flat(x, K, False)
        hit.append(int(torch.unique(ids).numel()))
    torch.cuda.synchronize()

    launches0 = sum(m.launch_count() for m in layers)
    for m, x in zip(layers, xs):
        m.forward(x, K, False)
    launches_per_step = sum(m.launch_count() for m in layers) - launches0
    with ClockSampler(local_rank) as clocks:
        ms = time_steps(torch, layers, xs, args.steps, args.warmup, barrier, graph=True)
        if ms * args.steps < 800:   # very short timed region: keep the same load up so that the
            # 200 ms sampler sees clocks under this kernel mix (not part of the reported time)
            time_steps(torch, layers, xs, int(800 / max(ms, 1e-3)) + 1, 0, lambda: None, graph=True)
    eager_ms = time_steps(torch, layers, xs, args.steps, args.warmup, lambda: None, graph=False)

    if dist is not None:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = world * T * NL / (ms * 1e-3)

    # ---- per-kernel launch durations (CUDA events on the launching stream), second pass ----
    for m in layers:
        m.set_profiling(True)
    for m, x in zip(layers, xs):            # creates the event pool outside the measured pass
        m.forward(x, K, False)
    torch.cuda.synchronize()
    for m in layers:
        m.take_profile()
    torch.cuda._sleep(200_000_000)          # ~0.1 s of device spin: the queue fills behind it, so no
    # kernel below waits for the CPU and its event pair times the kernel alone
    for _ in range(max(3, min(args.steps, 10))):
        for m, x in zip(layers, xs):
            m.forward(x, K, False)
    torch.cuda.synchronize()
    prof = {}
    for m in layers:
        for name, (n, avg_ms) in m.take_profile().items():
            cur = prof.setdefault(name, [0, 0.0])
            cur[0] += n
            cur[1] += avg_ms * n
        m.set_profiling(False)
    kern = {name: {"launches": n, "avg_us": 1e3 * tot / n} for name, (n, tot) in prof.items() if n}
    peak, peak_kind = measured_peak_hbm()
    u_mean = float(np.mean(hit))
    gu_bytes = u_mean * 2 * H * I * 144 / 256 + T * H * 2 + T * K * I * 2     # weights + x read + hact write
    roof = None
    if "q4k_gate_up" in kern:
        ach = gu_bytes / (kern["q4k_gate_up"]["avg_us"] * 1e-6) / 1e9
        roof = {"bound": "hbm", "kernel": "q4k_gate_up", "achieved": ach, "peak": peak, "unit": "GB/s",
                "frac": ach / peak, "peak_kind": peak_kind,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this very shape
                # (T=64, 64 experts hit), from an ncu capture of this kernel (summary under profiles/)
                "traffic": 156.7e6 if (T == 64 and u_mean == 64.0) else None,
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
    barrier()
    e2e_steps = max(3, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    if dist is not None:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * T * NL / (e2e_ms * 1e-3)

    sweep = None
    if args.sweep and rank == 0:
        sweep = {}
        for t_s in (1, 2, 4, 8, 16, 32, 64):
            xs_s = [torch.randn(t_s, H, generator=gen, device=device).to(torch.float16) for _ in range(NL)]
            u = []
            for m, x in zip(layers, xs_s):
                ids, _ = m.route_flat(x, K, False)
                u.append(int(torch.unique(ids).numel()))
            ms_s = time_steps(torch, layers, xs_s, args.steps, args.warmup, lambda: None, graph=True)
            b = float(np.mean(u)) * EXPERT_BYTES_Q4K + H * E * 4 + 2 * t_s * H * 2
            sweep[str(t_s)] = {"us_per_layer": 1e3 * ms_s / NL, "tokens_per_s": t_s * NL / (ms_s * 1e-3),
                               "experts_hit": float(np.mean(u)), "layer_GBps": b * NL / (ms_s * 1e-3) / 1e9,
                               "frac_of_measured_hbm": b * NL / (ms_s * 1e-3) / 1e9 / peak}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
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

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "eager_ms_per_step": eager_ms,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 activations x Q4_K weights, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"olmoe_q4k_decode_T{T}", "hidden": H, "intermediate": I, "experts": E,
                       "top_k": K, "norm_topk_prob": False, "tokens": T, "layers_per_step": NL,
                       "l2": "inputs larger than L2: %d distinct layer banks (%.2f GB Q4_K) rotate every step"
                             % (NL, NL * E * EXPERT_BYTES_Q4K / 1e9),
                       "launch": "one CUDA graph per step (16 layer calls captured from the C ABI)",
                       "parallelism": "single GPU" if world == 1 else f"{world} replicas, tokens per GPU fixed",
                       "experts_hit_mean": u_mean},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": NL * T * H * 2,
                    "d2h_bytes_per_step": NL * T * H * 2, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches_per_step * args.steps),
            "gpu_launches_per_step": int(launches_per_step),
            "clocks": clocks.summary(),
            "roofline": roof,
            "layer": {"algorithmic_bytes": layer_bytes, "us": 1e3 * ms / NL,
                      "GBps": layer_bytes * NL / (ms * 1e-3) / 1e9,
                      "frac_of_measured_hbm": layer_bytes * NL / (ms * 1e-3) / 1e9 / peak},
            "kernels": kern,
            "cpu_baseline": cpu,
        }
        if sweep:
            line["sweep"] = sweep
        print(json.dumps(line), flush=True)
    for m in layers:
        m.close()
    if dist is not None:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------
# prefill workload: T=4096, bf16, Zipf-skewed routing, tensor-core grouped GEMMs
# ----------------------------------------------------------------------------------------------
def measured_peak_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
        except Exception:
            pass
    return 1590.0, 1400.0, "fallback"


def run_prefill(args, rank: int, world: int, local_rank: int):
    import torch
    from mummu_b200 import _lib as L, moe, synth
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    stream = torch.cuda.Stream(device)
    torch.cuda.set_stream(stream)
    T = args.tokens if args.tokens != 64 else 4096
    NL = min(args.layers, 4)
    gen = torch.Generator(device=device)
    gen.manual_seed(4321 + rank)
    layers = []
    for l in range(NL):
        m = moe.SparseMoeConfig(H, I, E, K).init(device=device.index, act_dtype=L.BF16, weight_dtype=L.BF16,
                                                 max_tokens=T)
        m._router_np = (torch.randn(H, E, generator=gen, device=device) * 0.02).cpu().numpy()
        m.set_router(m._router_np)
        for which, shape in ((L.BANK_GATE, (E, I, H)), (L.BANK_UP, (E, I, H)), (L.BANK_DOWN, (E, H, I))):
            m.set_bank(which, (torch.randn(shape, generator=gen, device=device) * 0.02).to(torch.bfloat16))
        layers.append(m)
    xs = [torch.randn(T, H, generator=gen, device=device).to(torch.bfloat16) for _ in range(NL)]
    # router-logit bias b_e = -alpha * 1.1 * ln(rank_e): alpha calibrated so hottest / mean load ~ 8
    alpha, ratio = None, None
    for cand in (0.5, 1.0, 1.5, 2.0, 2.5, 3.0, 4.0, 6.0):
        bias = synth.zipf_router_bias(E, cand)
        layers[0].set_router(layers[0]._router_np, bias=bias)
        ids, _ = layers[0].route_flat(xs[0], K, False)
        load = torch.bincount(ids.reshape(-1).long(), minlength=E).float()
        r = float(load.max() / load.mean())
        alpha, ratio = cand, r
        if r >= 7.6:
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
    with ClockSampler(local_rank) as clocks:
        ms = time_steps(torch, layers, xs, args.steps, max(args.warmup, 3), lambda: None, graph=False)
        if ms * args.steps < 800:
            time_steps(torch, layers, xs, int(800 / max(ms, 1e-3)) + 1, 0, lambda: None, graph=False)
    for m in layers:
        m.set_profiling(True)
    step()
    torch.cuda.synchronize()
    for m in layers:
        m.take_profile()
    torch.cuda._sleep(100_000_000)
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    prof = {}
    for m in layers:
        for name, (n, avg_ms) in m.take_profile().items():
            cur = prof.setdefault(name, [0, 0.0])
            cur[0] += n
            cur[1] += avg_ms * n
    kern = {name: {"launches": n, "avg_us": 1e3 * tot / n} for name, (n, tot) in prof.items() if n}
    burst, sustained, kind = measured_peak_tflops()
    flops_gu = T * K * 2 * 2 * H * I
    flops_dn = T * K * 2 * H * I
    roof = None
    if "tc_gate_up" in kern:
        ach = flops_gu / (kern["tc_gate_up"]["avg_us"] * 1e-6) / 1e12
        roof = {"bound": "tensor", "kernel": "tc_gate_up", "achieved": ach, "peak": burst, "unit": "TFLOP/s",
                "frac": ach / burst, "frac_of_sustained_peak": ach / sustained, "peak_kind": kind, "traffic": None,
                "flops_per_launch": flops_gu}
        if "tc_down" in kern:
            roof["down_TFLOPs"] = flops_dn / (kern["tc_down"]["avg_us"] * 1e-6) / 1e12
            both = (flops_gu + flops_dn) / ((kern["tc_gate_up"]["avg_us"] + kern["tc_down"]["avg_us"]) * 1e-6) / 1e12
            roof["both_gemms_TFLOPs"] = both
    layer_tflops = (flops_gu + flops_dn) * NL / (ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": T * NL / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 x bf16, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"olmoe_bf16_prefill_T{T}", "hidden": H, "intermediate": I, "experts": E, "top_k": K,
                   "tokens": T, "layers_per_step": NL, "zipf_alpha": alpha, "hottest_over_mean_load": ratio,
                   "l2": "inputs larger than L2: %.2f GB of bf16 banks per layer" % (3 * E * H * I * 2 / 1e9)},
        "gpu_launches": int(launches_per_step * args.steps), "gpu_launches_per_step": int(launches_per_step),
        "clocks": clocks.summary(), "roofline": roof,
        "layer": {"us": 1e3 * ms / NL, "TFLOPs_whole_layer": layer_tflops, "frac_of_burst_peak": layer_tflops / burst},
        "kernels": kern,
    }
    print(json.dumps(line), flush=True)
    for m in layers:
        m.close()


# ----------------------------------------------------------------------------------------------
# expert-parallel runs (N > 1 of the default workload, and the Qwen3-30B-A3B-shaped stack at any N)
# ----------------------------------------------------------------------------------------------
def run_ep(args, rank: int, world: int, local_rank: int, shape: dict):
    import torch
    from mummu_b200 import _lib as L, moe
    from mummu_b200.ep import ExpertParallelMoe
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)
    stream = torch.cuda.Stream(device)
    torch.cuda.set_stream(stream)
    h, i, e, k = shape["hidden"], shape["inter"], shape["experts"], shape["top_k"]
    T, NL, q4 = shape["tokens_per_rank"], shape["layers"], shape["q4k"]
    act = L.F16 if q4 else L.BF16
    wdt = L.Q4_K if q4 else L.BF16
    tdt = torch.float16 if q4 else torch.bfloat16
    el = e // world
    cfg = moe.SparseMoeConfig(h, i, e, k)
    gen = torch.Generator(device=device)
    layers = []
    ws = None
    if world > 1 and not os.environ.get("MUMMU_EP_NCCL"):
        from mummu_b200.ep import PeerWorkspace
        ws = PeerWorkspace(None, local_rank, world * T * k, h, e)  # rows move by peer stores / loads
    for l in range(NL):
        gen.manual_seed(9000 + l)                                   # router: same on every rank
        router = (torch.randn(h, e, generator=gen, device=device) * 0.02).cpu().numpy()
        gen.manual_seed(100000 + 1000 * l + rank)                   # this rank's experts
        if world > 1:
            m = ExpertParallelMoe(cfg, device=local_rank, act_dtype=act, weight_dtype=wdt, max_tokens=T,
                                  workspace=ws, scratch_donor=layers[0][0] if layers else None)
            handle = m.moe
        else:
            m = cfg.init(device=local_rank, act_dtype=act, weight_dtype=wdt, max_tokens=T if not layers else 0)
            if layers:
                m.adopt_scratch(layers[0][0])
            handle = m
        m.set_router(router)
        for which, shp in ((L.BANK_GATE, (el, i, h)), (L.BANK_UP, (el, i, h)), (L.BANK_DOWN, (el, h, i))):
            wt = torch.randn(shp, generator=gen, device=device) * 0.02
            handle.set_bank(which, moe.q4k_quantize_device(wt) if q4 else wt.to(tdt))
            del wt
        layers.append((m, handle))
    gen.manual_seed(777 + rank)
    xs = [torch.randn(T, h, generator=gen, device=device).to(tdt) for _ in range(NL)]
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()

    def step():
        for (m, _), x in zip(layers, xs):
            m.forward(x, k, False)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        barrier()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        barrier()
        ms = a.elapsed_time(b) / steps
        if dist is not None:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    l0 = sum(hd.launch_count() for _, hd in layers)
    step()
    launches_per_step = sum(hd.launch_count() for _, hd in layers) - l0
    # decode-sized steps are launch-bound: replay one CUDA graph per step.  With the ranks signalling
    # each other through peer memory the multi-GPU step holds no NCCL kernel and is captured too (a
    # captured graph that held NCCL kernels kept the process group from shutting down, so the NCCL
    # exchange stays eager)
    run, graphed = step, False
    device_sync = world > 1 and ws is not None
    if q4 and (world == 1 or device_sync) and not os.environ.get("MUMMU_NO_GRAPH"):
        try:
            torch.cuda.synchronize()
            barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=torch.cuda.current_stream()):
                step()
            g.replay()
            torch.cuda.synchronize()
            run, graphed = g.replay, True
        except Exception as exc:                                  # keep the eager step
            sys.stderr.write(f"graph capture of the EP step failed, running eagerly: {exc}\n")
            torch.cuda.synchronize()
    with ClockSampler(local_rank) as clocks:
        ms = timed(run, args.steps, max(args.warmup, 3))
        if ms * args.steps < 800:
            timed(run, int(800 / max(ms, 1e-3)) + 1, 0)

    hx = [x.cpu().pin_memory() for x in xs]
    def e2e_step():
        for (m, _), hxi in zip(layers, hx):
            xd = hxi.to(device, non_blocking=True)
            m.forward(xd, k, False).cpu()
    e2e_ms = timed(e2e_step, max(3, min(args.steps, 10)), 2)

    for _, hd in layers:
        hd.set_profiling(True)
    step()
    torch.cuda.synchronize()
    for _, hd in layers:
        hd.take_profile()
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    prof = {}
    for _, hd in layers:
        for name, (n, avg_ms) in hd.take_profile().items():
            cur = prof.setdefault(name, [0, 0.0])
            cur[0] += n
            cur[1] += avg_ms * n
    kern = {name: {"launches": n, "avg_us": 1e3 * tot / n} for name, (n, tot) in prof.items() if n}

    total_tokens = T * world
    if rank == 0:
        flops = total_tokens * k * 6 * h * i * NL
        line = {
            "metric": METRIC, "value": total_tokens * NL / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": shape["scaling"], "vs_baseline": None,
            "dtype": "f16 activations x Q4_K weights, f32 accumulate" if q4 else "bf16 x bf16, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": shape["name"], "hidden": h, "intermediate": i, "experts": e, "top_k": k,
                       "norm_topk_prob": False, "tokens_per_gpu": T, "tokens": total_tokens, "layers_per_step": NL,
                       "launch": "one CUDA graph per step" if graphed else "eager",
                       "parallelism": (f"ep{world}: {el} experts per GPU, "
                                       + ("dispatch by peer stores and combine by peer loads over NVLink, no host sync"
                                          if ws is not None else "NCCL all-to-all dispatch and combine"))
                       if world > 1 else "single GPU",
                       "l2": "inputs larger than L2: %.2f GB of expert weights per GPU rotate every step"
                             % (NL * el * 3 * h * i * (144 / 256 if q4 else 2) / 1e9)},
            "e2e": {"value": total_tokens * NL / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": NL * T * h * 2 * world,
                    "d2h_bytes_per_step": NL * T * h * 2 * world, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches_per_step * args.steps), "gpu_launches_per_step": int(launches_per_step),
            "clocks": clocks.summary(),
            "roofline": None if q4 else {"bound": "tensor", "kernel": "whole step (all ranks)",
                                         "achieved": flops / (ms * 1e-3) / 1e12, "peak": measured_peak_tflops()[0] * world,
                                         "unit": "TFLOP/s", "frac": flops / (ms * 1e-3) / 1e12 / (measured_peak_tflops()[0] * world),
                                         "traffic": None, "peak_kind": measured_peak_tflops()[2]},
            "kernels_rank0": kern, "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    # the result is out: never let a stuck shutdown of peers / NCCL hold the GPUs
    threading.Timer(30.0, lambda: os._exit(0)).start()
    for m, _ in reversed(layers):
        m.close()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        if ws is not None:
            ws.close()
        dist.destroy_process_group()
    os._exit(0)


# ----------------------------------------------------------------------------------------------
# whole-model decode: OLMoE-1B-7B-shaped, random weights, Q4_K experts, f16 trunk
# ----------------------------------------------------------------------------------------------
def run_model(args, rank: int, world: int, local_rank: int):
    import torch
    from mummu_b200 import _lib as L
    from mummu_b200.olmoe import OlmoeConfig, OlmoeDecoder
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    cfg = OlmoeConfig()
    prompt, n_new = 512, 128
    results = {}
    for B in (1, 32):
        chunk = max(1, 2048 // B)                       # prompt fed in chunks of <= 2048 tokens over the batch
        dec = OlmoeDecoder(cfg, device=local_rank, expert_dtype=L.Q4_K, max_batch=B, max_ctx=prompt + n_new,
                           max_tokens=B * chunk)
        dec.random_init(seed=11)
        gen = torch.Generator(device=device)
        gen.manual_seed(5 + B)
        ids = torch.randint(0, cfg.vocab_size, (B, prompt), generator=gen, device=device)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        past, logits = 0, None
        while past < prompt:
            logits = dec.forward(ids[:, past:past + chunk], past)
            past += min(chunk, prompt - past)
        torch.cuda.synchronize()
        t_prefill = time.perf_counter() - t0
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = sum(l["mlp"].launch_count() for l in dec.layers)
        dec._decode_static(torch.zeros(B, 1, dtype=torch.int64, device=device),
                           torch.tensor([prompt + n_new - 1], device=device))     # counts one step's launches
        launches1 = sum(l["mlp"].launch_count() for l in dec.layers)
        g, ids_buf, pos_buf, logits_buf = dec.make_decode_graph(B)              # one CUDA graph per decode step
        torch.cuda.synchronize()
        a.record()
        for _ in range(n_new):
            ids_buf.copy_(logits.argmax(-1)[:, None])
            pos_buf.fill_(past)
            g.replay()
            logits = logits_buf
            past += 1
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        results[B] = dict(decode_tok_per_s=B * n_new / (ms * 1e-3), ms_per_token_step=ms / n_new,
                          prefill_s=t_prefill,
                          moe_launches_per_step=launches1 - launches0)
        dec.close()
        del dec
        torch.cuda.empty_cache()
    line = {"metric": "olmoe_decode_tokens_per_s", "value": results[32]["decode_tok_per_s"], "unit": "tokens/s",
            "n_gpus": 1, "steps": n_new, "warmup": 0, "ms_per_step": results[32]["ms_per_token_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 trunk, Q4_K experts", "data": "synthetic",
            "config": {"workload": "olmoe_1b_7b_shaped_greedy_decode", "layers": cfg.num_hidden_layers,
                       "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "experts": cfg.num_experts,
                       "top_k": cfg.num_experts_per_tok, "vocab": cfg.vocab_size, "prompt": prompt, "new_tokens": n_new,
                       "launch": "one CUDA graph per decode step (trunk in torch, MoE layers through the C ABI)"},
            "batch_1": results[1], "batch_32": results[32]}
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.layers is None:
            args.layers = 16
        run_reference(args, rank, world)
        return
    if args.workload == "olmoe_bf16_prefill":
        if args.layers is None:
            args.layers = 4
        run_prefill(args, rank, world, local_rank)
        return
    if args.workload == "olmoe_decode":
        run_model(args, rank, world, local_rank)
        return
    if args.workload == "ep_qwen3":
        total = args.tokens if args.tokens != 64 else 16384
        run_ep(args, rank, world, local_rank, dict(
            name=f"qwen3_30b_a3b_shaped_ep_T{total}", hidden=2048, inter=768, experts=128, top_k=8,
            tokens_per_rank=total // world, layers=args.layers or 48, q4k=False, scaling="strong"))
        return
    if args.layers is None:
        args.layers = 16
    if world > 1:
        # the default workload on N GPUs: same layer, experts sharded, every GPU brings its own T tokens
        run_ep(args, rank, world, local_rank, dict(
            name=f"olmoe_q4k_decode_T{args.tokens}_per_gpu", hidden=H, inter=I, experts=E, top_k=K,
            tokens_per_rank=args.tokens, layers=args.layers, q4k=True, scaling="weak"))
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
