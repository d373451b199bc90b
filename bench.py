#!/usr/bin/env python
"""Benchmark of the quantized MoE feed-forward layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens T] [--layers L]

Workload (N = 1): the decode configuration -- a Qwen3.5-35B-A3B-shaped MoE layer (H 2048, 256 experts,
top-8, expert width 512, one sigmoid-gated shared expert), gate/up in IQ3_S, down in Q4_0, activations
Q8_1, T concurrent tokens (default 8, the top of the 1/2/4/8 sweep).  One STEP is one pass of the T-token
batch through L independent layers (default 16, seeded synthetic weights ~N(0, 0.02), fresh input per
layer).  The weights of consecutive calls differ, and one cycle touches L x ~99 MB > the 126 MB L2, so the
timed calls stream their weights from HBM.  metric = tokens x layer-calls per second.

The JSON line also carries: `roofline` for the dominant kernel (gate/up GEMV), measured live with CUDA
events; `sweep` with the layer-level numbers for T = 1, 2, 4, 8; `e2e` through the host-buffer C entry
(pinned host x in, y out, per layer call); `cpu_baseline`: the CPU oracle port timed on this host.

--impl reference times the CPU port of the reference's path (the reference's own CPU code needs ik_llama's
ggml, which is neither vendored nor pinned, so it cannot be built here) with all host threads on a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "moe_layer_decode_tokens_per_s"
UNIT = "tokens*layers/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                       "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [r.strip().split(", ") for r in open(self.f.name) if r.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[5:9]):
                if v.strip().lower() == "active":
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


_CPU_LAYERS = {}


def cpu_port_tokens_per_s(cfg, T, n_layers, threads=None, min_seconds=0.0):
    """The oracle's layer forward on the host cores: tokens x layer-calls per second.  The sample is `n_layers` seeded
    layers (built once per process) walked round-robin until at least `min_seconds` have passed (at least one pass)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    from chimere_b200 import configs
    if threads:
        oracle.lib().orc_set_num_threads(threads)
    key = (cfg.name, T, n_layers)
    if key not in _CPU_LAYERS:
        _CPU_LAYERS[key] = ([configs.make_layer(cfg, device="cpu", seed=9000 + i) for i in range(n_layers)],
                            [configs.make_input(cfg, T, seed=77 + i).numpy() for i in range(n_layers)])
        oracle.moe_forward(_CPU_LAYERS[key][0][0], _CPU_LAYERS[key][1][0], taps=False)  # warm
    layers, xs = _CPU_LAYERS[key]
    calls = 0
    t0 = time.perf_counter()
    while True:
        for w, x in zip(layers, xs):
            oracle.moe_forward(w, x, taps=False)
        calls += n_layers
        dt = time.perf_counter() - t0
        if dt >= min_seconds:
            break
    return T * calls / dt, oracle.lib().orc_num_threads(), dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from chimere_b200 import configs
    cfg = configs.QWEN_IQ3S
    T = args.tokens
    sample_layers = 2
    vals = []
    # one step = a bounded sample: the layers walked for about `per_step` seconds, sized so that the whole run stays
    # within a few minutes whatever --steps says
    per_step = min(2.0, 120.0 / max(1, args.steps + args.warmup))
    for _ in range(args.warmup):
        cpu_port_tokens_per_s(cfg, T, sample_layers, min_seconds=per_step)
    t_total = 0.0
    for _ in range(args.steps):
        v, threads, dt = cpu_port_tokens_per_s(cfg, T, sample_layers, min_seconds=per_step)
        vals.append(v); t_total += dt
    v = statistics.median(vals)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * t_total / max(1, args.steps), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 block dots, f32 accumulate", "data": "synthetic",
            "config": workload_config(cfg, T, sample_layers),
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"T={T} tokens through {sample_layers} layers, repeated for {per_step:.1f} s per step (CPU restatement in oracle/, OpenMP)"},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def workload_config(cfg, T, L):
    return {"workload": f"{cfg.name}: H={cfg.H} E={cfg.E} top{cfg.top_k} F={cfg.F} shared F_s={cfg.F_s}; gate/up IQ3_S, down Q4_0, "
                        f"Q8_1 activations; T={T} tokens x {L} independent layers per step",
            "tokens": T, "layers": L,
            "l2": f"weights rotate over {L} layers; one cycle touches more than the 126 MB L2, inputs differ per layer"}


def measure_prefill(lib, dev, tokens_list):
    """Secondary measurement: the prefill configuration (all experts Q8_0, Zipf-skewed routing) on one layer, with the
    large experts on the tcgen05 grouped GEMM and, for comparison, everything on the GEMV kernels."""
    import torch
    from chimere_b200 import configs
    from chimere_b200.layer import MoeScratch, MoeWeightsPrefill, MoeWeightsTiled, forward_moe, forward_moe_prefill
    cfg = configs.QWEN_Q8_0
    raw = configs.make_layer(cfg, device=dev)
    tiled, pw = MoeWeightsTiled(raw), MoeWeightsPrefill(raw)
    del raw
    out = []
    for T in tokens_list:
        x = configs.make_input(cfg, T, device=dev)
        sc = MoeScratch(tiled, T, device=dev)
        sc.enable_prefill()
        y = torch.empty_like(x)
        res = {"T": T}
        for name, fn in (("gemm", lambda: forward_moe_prefill(tiled, pw, sc, x, y)), ("gemv", lambda: forward_moe(tiled, sc, x, y))):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 5
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            res[name] = {"us_per_layer_call": us, "tokens_per_s": T / (us * 1e-6), "int8_tops": configs.int8_ops(cfg, T) / (us * 1e-6) / 1e12}
        res["device_status"] = sc.status()
        out.append(res)
        del sc, x, y
    return {"workload": f"{cfg.name}: one layer, all experts Q8_0, Zipf(1.1) logit bias, weights 0.86 GB (> L2)", "results": out}


def run_expert_parallel(args, cfg, dev, rank, world, local, dist, hbm_peak, peak_kind):
    """N > 1: the same layer with its experts sharded over the ranks (E/N each, contiguous), router and shared
    expert replicated, T tokens per rank (weak scaling), dispatch and combine by NCCL all-to-all."""
    import torch
    from chimere_b200 import configs, formats
    from chimere_b200.ep import ExpertParallelMoE
    T, L, K, W = args.tokens, args.layers, args.steps, args.warmup
    layers = []
    for i in range(L):
        full = configs.make_layer(cfg, device=dev, seed=1000 + i)          # same weights on every rank, then sharded
        layers.append(ExpertParallelMoE(full, max_tokens=T, rank=rank, world=world, device=dev))
        del full
    xs = [configs.make_input(cfg, T, device=dev, seed=31 * (rank + 1) + i) for i in range(L)]
    ys = [torch.empty_like(x) for x in xs]

    padded = T * cfg.top_k <= 1024          # decode-size: fixed-size exchange, no host sync per layer

    def step():
        for ep, x, y in zip(layers, xs, ys):
            (ep.forward_padded if padded else ep.forward)(x, y)

    # one step = one CUDA graph when the exchange is fixed-size (NCCL all-to-alls are captured with the kernels)
    timing_note = "eager launches"
    graph = None
    if padded:
        try:
            step(); step()
            torch.cuda.synchronize(); dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            torch.cuda.synchronize()
            timing_note = "CUDA graph replay of one step (kernels and NCCL all-to-alls captured together)"
        except Exception as exc:  # keep the eager path if this torch/NCCL pair cannot capture collectives
            graph = None
            timing_note = f"eager launches (graph capture failed: {type(exc).__name__})"
            print(f"[bench] graph capture failed: {exc}", file=sys.stderr)
            torch.cuda.synchronize()
    run_step = graph.replay if graph is not None else step

    def timed(fn, k, w):
        for _ in range(w):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(k):
            fn()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local)
    secs = timed(run_step, K, W)
    clocks = sampler.stop()
    value = world * T * L * K / secs

    hx = [x.cpu().pin_memory() for x in xs]
    hy = [torch.empty(T, cfg.H).pin_memory() for _ in xs]

    def e2e_step():
        for ep, a, b, x, y in zip(layers, hx, hy, xs, ys):
            x.copy_(a, non_blocking=True)
            (ep.forward_padded if padded else ep.forward)(x, y)
            b.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    e2e_secs = timed(e2e_step, K, W)
    recv = torch.tensor([float(sum(ep.last_recv_rows for ep in layers)) / L], device=dev)
    rmax = recv.clone(); dist.all_reduce(rmax, op=dist.ReduceOp.MAX)
    rsum = recv.clone(); dist.all_reduce(rsum, op=dist.ReduceOp.SUM)
    if rank == 0:
        b_gu = cfg.F * formats.row_bytes(cfg.type_gate_up, cfg.H)
        b_dn = cfg.H * formats.row_bytes(cfg.type_down, cfg.F)
        rows_mean = float(rsum.item()) / world
        layer_us = secs / (K * L) * 1e6
        # per rank and layer call: every received pair's expert (upper bound on distinct experts: one per pair) + shared + router
        alg = min(rows_mean, cfg.E / world) * (2 * b_gu + b_dn) + (2 * b_gu + b_dn) + 4 * cfg.E * cfg.H + 8 * T * cfg.H
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": 1e3 * secs / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "int8 block dots (dp4a), f32 accumulate", "data": "synthetic",
                "config": dict(workload_config(cfg, T, L), parallelism=f"ep{world}: {cfg.E // world} experts per GPU, router + shared expert replicated, "
                               f"{T} tokens per GPU; dispatch Q8_1 planes / combine fp32 rows by NCCL all-to-all",
                               timing="CUDA events around K steps, max over ranks; " + timing_note,
                               exchange=("fixed-size (padded to T*k rows per destination), no host sync" if padded
                                         else "exact split sizes, one host sync per layer call"),
                               weight_layout="tiled"),
                "roofline": {"bound": "hbm", "kernel": "expert-parallel layer call (per rank)", "achieved": alg / (layer_us * 1e-6) / 1e9,
                             "peak": hbm_peak, "unit": "GB/s", "frac": alg / (layer_us * 1e-6) / 1e9 / hbm_peak, "peak_kind": peak_kind,
                             "traffic": None, "us_per_layer_call": layer_us,
                             "pairs_received_per_rank_mean": rows_mean, "pairs_received_per_rank_max": float(rmax.item()),
                             "nvlink_bytes_per_rank_per_call": rows_mean * (cfg.H + 4 * ((cfg.H // 32 + 3) & ~3) + 4 + 4 * cfg.H)},
                "cpu_baseline": None,
                "e2e": {"value": world * T * L * K / e2e_secs, "unit": UNIT, "h2d_bytes_per_step": L * T * cfg.H * 4,
                        "d2h_bytes_per_step": L * T * cfg.H * 4, "ms_per_step": 1e3 * e2e_secs / K},
                "gpu_launches": 7 * L * K, "clocks": clocks}
        print(json.dumps(line), flush=True)
    # leave without tearing the communicator down: with a captured graph still holding NCCL work the
    # teardown has been seen to wait for the watchdog; every rank is past its last collective here
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--prefill-tokens", default="512,2048,8192", help="comma list of T for the secondary prefill measurement ('' = skip)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="run only the secondary prefill measurement and print its JSON (used for profiling the grouped GEMM)")
    ap.add_argument("--layout", default="tiled", choices=["tiled", "ggml"],
                    help="weight layout the layer entry runs on: the library's tiled32 repack (default) or raw ggml blocks")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    from chimere_b200 import abi, configs
    from chimere_b200.layer import MoeScratch, MoeWeightsTiled

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    lib = abi.load()
    if args.prefill_only:
        print(json.dumps({"prefill": measure_prefill(lib, dev, [int(t) for t in args.prefill_tokens.split(",") if t])}))
        return 0
    cfg = configs.QWEN_IQ3S
    T, L, K, W = args.tokens, args.layers, args.steps, args.warmup
    hbm_peak, peak_kind = peaks()
    if world > 1:
        return run_expert_parallel(args, cfg, dev, rank, world, local, dist, hbm_peak, peak_kind)

    # ---- resident state: L layers of weights, one scratch per (layer), inputs, outputs ----
    # each layer: seeded ggml blocks -> one-time load-side rewrite into the library's tiled32 layout
    layers = []
    for i in range(L):
        raw = configs.make_layer(cfg, device=dev, seed=1000 * (rank + 1) + i)
        layers.append(raw if args.layout == "ggml" else MoeWeightsTiled(raw, keep_raw=False))
        del raw
    scratch = [MoeScratch(w, max(T, 8), device=dev) for w in layers]
    xs = [configs.make_input(cfg, max(T, 8), device=dev, seed=31 * (rank + 1) + i) for i in range(L)]
    ys = [torch.empty_like(x) for x in xs]
    stream = torch.cuda.Stream(device=dev)
    sptr = stream.cuda_stream

    def enqueue_layers(Tn):
        for w, sc, x, y in zip(layers, scratch, xs, ys):
            rc = lib.chimere_b200_moe_forward(C.byref(w.as_struct()), x.data_ptr(), y.data_ptr(), Tn, C.byref(sc.ws), sptr)
            if rc:
                raise RuntimeError(f"chimere_b200_moe_forward rc={rc}")

    def make_graph(Tn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            enqueue_layers(Tn)  # warm (also sets kernel attributes outside capture)
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                enqueue_layers(Tn)
        return g

    def time_steps(run, k, w):
        """k timed repetitions of run() on `stream` after w warm-ups; returns seconds (device time)."""
        with torch.cuda.stream(stream):
            for _ in range(w):
                run()
            stream.synchronize()
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(k):
                run()
            e1.record(stream)
            stream.synchronize()
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
        return e0.elapsed_time(e1) * 1e-3

    def distinct_experts(Tn):
        return [int(torch.unique(sc.topk_indices(Tn)).numel()) for sc in scratch]

    # ---- headline: graph replay of one step = L layer calls ----
    graph = make_graph(T)
    sampler = ClockSampler(local)
    secs = time_steps(graph.replay, K, W)
    clocks = sampler.stop()
    if dist is not None:
        t = torch.tensor([secs], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())
    value = world * T * L * K / secs
    U = distinct_experts(T)
    layer_bytes = sum(configs.algorithmic_bytes(cfg, T, u) for u in U) / L
    layer_us = secs / (K * L) * 1e6
    layer_gbs = layer_bytes / (layer_us * 1e-6) / 1e9

    # ---- roofline of the dominant kernel (gate/up GEMV), timed alone over the rotating layers ----
    def gate_up_all():
        for w, sc in zip(layers, scratch):
            rc = lib.chimere_b200_moe_gate_up(C.byref(w.as_struct()), T, C.byref(sc.ws), sptr)
            if rc:
                raise RuntimeError(f"gate_up rc={rc}")

    def down_all():
        for w, sc, y in zip(layers, scratch, ys):
            rc = lib.chimere_b200_moe_down_combine(C.byref(w.as_struct()), y.data_ptr(), T, C.byref(sc.ws), sptr)
            if rc:
                raise RuntimeError(f"down rc={rc}")

    from chimere_b200 import formats
    b_gu = cfg.F * formats.row_bytes(cfg.type_gate_up, cfg.H)
    b_gu_sh = cfg.F_s * formats.row_bytes(cfg.type_gate_up, cfg.H)
    b_dn = cfg.H * formats.row_bytes(cfg.type_down, cfg.F)
    b_dn_sh = cfg.H * formats.row_bytes(cfg.type_down, cfg.F_s)
    xq_row = cfg.H // 32 * 36
    iq_row = max(cfg.F, cfg.F_s) // 32 * 36
    pairs = T * cfg.top_k + T
    gu_bytes = sum(2 * (u * b_gu + b_gu_sh) + T * xq_row + pairs * (cfg.F // 32 * 36) for u in U) / L
    dn_bytes = sum(u * b_dn + b_dn_sh + pairs * iq_row + T * cfg.H * 4 for u in U) / L
    def graph_of(fn):
        """L launches as one CUDA graph, so that the device time is not hidden behind the host's launch rate."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                fn()
        return g

    def route_all():
        for w, sc, x in zip(layers, scratch, xs):
            rc = lib.chimere_b200_moe_route(C.byref(w.as_struct()), x.data_ptr(), T, C.byref(sc.ws), sptr)
            if rc:
                raise RuntimeError(f"route rc={rc}")

    gu_secs = time_steps(graph_of(gate_up_all).replay, max(5, K), 3) / (max(5, K) * L)
    dn_secs = time_steps(graph_of(down_all).replay, max(5, K), 3) / (max(5, K) * L)
    rt_secs = time_steps(graph_of(route_all).replay, max(5, K), 3) / (max(5, K) * L)
    roof = {"bound": "hbm", "kernel": ("bulk_kernel<IQ3_S, gate_up>" if args.layout == "tiled" else "gate_up_kernel<IQ3_S>"), "achieved": gu_bytes / gu_secs / 1e9, "peak": hbm_peak,
            "unit": "GB/s", "frac": gu_bytes / gu_secs / 1e9 / hbm_peak, "peak_kind": peak_kind,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at these sizes, from an ncu capture of
            # the two-layer case (one launch = one layer); IQ3_S is streamed as 4-bit codes: +22 % over the ggml bytes
            "traffic": (67008256 + 735488) if (args.layout == "tiled" and T == 8) else None,
            "us_per_launch": gu_secs * 1e6, "algorithmic_bytes_per_launch": gu_bytes,
            "down_kernel": {"achieved": dn_bytes / dn_secs / 1e9, "frac": dn_bytes / dn_secs / 1e9 / hbm_peak,
                            "us_per_launch": dn_secs * 1e6, "algorithmic_bytes_per_launch": dn_bytes},
            "route_kernel": {"us_per_launch": rt_secs * 1e6},
            "layer": {"achieved": layer_gbs, "frac": layer_gbs / hbm_peak, "us_per_layer_call": layer_us,
                      "algorithmic_bytes_per_call": layer_bytes, "distinct_experts_mean": sum(U) / L}}

    # ---- sweep over T (layer level, graph replay) ----
    sweep = []
    if not args.no_sweep and rank == 0:
        for Tn in (1, 2, 4, 8):
            g = make_graph(Tn)
            s = time_steps(g.replay, max(5, K), 3) / max(5, K)
            Un = distinct_experts(Tn)
            b = sum(configs.algorithmic_bytes(cfg, Tn, u) for u in Un) / L
            us = s / L * 1e6
            sweep.append({"T": Tn, "us_per_layer_call": us, "tokens_layers_per_s": Tn * L / s,
                          "hbm_gbs": b / (us * 1e-6) / 1e9, "hbm_frac": b / (us * 1e-6) / 1e9 / hbm_peak,
                          "distinct_experts_mean": sum(Un) / L})
    elif dist is not None:
        pass

    # ---- end to end through the host-buffer C entry: pinned x in, y out, every layer call ----
    hx = [x[:T].cpu().pin_memory() for x in xs]
    hy = [torch.empty(T, cfg.H).pin_memory() for _ in xs]

    # the argument lists are what a C caller would hold ready: only the calls themselves are timed
    host_calls = [(C.byref(w.as_struct()), a.data_ptr(), b.data_ptr(), T, sc.x_dev.data_ptr(), sc.y_dev.data_ptr(), C.byref(sc.ws), sptr)
                  for w, sc, a, b in zip(layers, scratch, hx, hy)]
    forward_host = lib.chimere_b200_moe_forward_host

    def e2e_step():
        for call in host_calls:
            rc = forward_host(*call)
            if rc:
                raise RuntimeError(f"forward_host rc={rc}")

    for _ in range(W):
        e2e_step()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(K):
        e2e_step()
    torch.cuda.synchronize()
    e2e_secs = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_secs], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_secs = float(t.item())
    e2e = {"value": world * T * L * K / e2e_secs, "unit": UNIT, "h2d_bytes_per_step": L * T * cfg.H * 4,
           "d2h_bytes_per_step": L * T * cfg.H * 4, "ms_per_step": 1e3 * e2e_secs / K}

    status = max(sc.status() for sc in scratch)
    prefill = None
    if rank == 0 and args.prefill_tokens and args.layout == "tiled":
        del graph
        layers.clear(); scratch.clear(); xs.clear(); ys.clear()
        torch.cuda.empty_cache()
        prefill = measure_prefill(lib, dev, [int(t) for t in args.prefill_tokens.split(",") if t])
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    cpu = None
    if not args.no_cpu_baseline:
        v, threads, dt = cpu_port_tokens_per_s(cfg, T, 2, min_seconds=10.0)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"T={T} tokens through 2 layers, repeated for {dt:.1f} s; CPU restatement in oracle/ with OpenMP"}

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": 1e3 * secs / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 block dots (dp4a), f32 accumulate", "data": "synthetic",
            "config": dict(workload_config(cfg, T, L), parallelism=("single GPU" if world == 1 else f"{world} independent replicas"),
                           timing="CUDA graph replay of one step, CUDA events on the launching stream",
                           weight_layout=args.layout),
            "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": 3 * L * K, "clocks": clocks,
            "sweep": sweep, "prefill": prefill, "device_status": status}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
