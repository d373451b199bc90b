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


def pct(vals):
    """median / p10 / p90 of a list of numbers."""
    v = sorted(vals)
    if not v:
        return None
    q = lambda f: v[min(len(v) - 1, max(0, int(round(f * (len(v) - 1)))))]
    return {"p50": statistics.median(v), "p10": q(0.10), "p90": q(0.90), "n": len(v)}


def captured_traffic(kernel, shape):
    """DRAM bytes per launch of `kernel` at `shape` from the committed ncu capture table (profiles/dram_traffic.json),
    or None when no capture of that kernel and shape has been recorded."""
    try:
        table = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))
    except (OSError, ValueError):
        return None, None
    ent = table.get(f"{kernel} | {shape}")
    if not ent:
        return None, None
    return int(ent["dram_bytes_read"]) + int(ent["dram_bytes_write"]), ent.get("source")


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
    conf = workload_config(cfg, T, sample_layers)
    conf["sample"] = (f"each step walks {sample_layers} seeded layers (not the GPU arm's 16) for about {per_step:.1f} s: the same T and shapes, a rate "
                      "metric; two layers' weights (0.8 GB) still exceed the host's caches")
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * t_total / max(1, args.steps), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 block dots, f32 accumulate", "data": "synthetic",
            "config": conf, "steps_stats": pct(vals),
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


def measure_int8_peak(lib, dev):
    """The int8 tensor-pipe rate of this GPU with nothing read back (tcgen05.mma kind::i8 issued back to back from
    shared-memory operands by one CTA per SM): the denominator for the compute side of the prefill roofline."""
    import torch
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    out = {}
    for n_cols in (128, 256):
        n_mma = 16384
        best = None
        for rep in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ctas = lib.chimere_b200_mma_i8_probe(n_mma, n_cols, 512 // n_cols, status.data_ptr(), st)
            e1.record()
            torch.cuda.synchronize()
            if ctas <= 0:
                return {"error": ctas}
            ms = e0.elapsed_time(e1)
            if rep > 0:
                best = ms if best is None else min(best, ms)
        ops = ctas * n_mma * 2 * 128 * n_cols * 32
        out[f"m128_n{n_cols}_k32"] = {"tops": ops / (best * 1e-3) / 1e12, "ms": best, "ctas": ctas, "mma_per_cta": n_mma}
    out["device_status"] = int(status[0].item())
    out["how"] = "one CTA per SM, tcgen05.mma kind::i8 accumulating in TMEM, no read-back; best of 3 after one warm-up"
    return out


class L2Flush:
    """Writes a buffer twice the size of the L2 between timed calls, so that a call cannot find its weights there."""

    def __init__(self, dev):
        import torch
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.fill_(1)


def timed_calls(fn, reps, flush):
    """Device time of `reps` single calls of fn(), each after an L2 flush (events on the current stream); microseconds."""
    import torch
    times = []
    for _ in range(reps):
        flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    return times


def measure_secondary(lib, dev, hbm_peak, i8_peak_tops, prefill_tokens):
    """The configurations beside the headline one, each on one seeded layer, one layer call per timed sample with the L2
    flushed before it: the prefill configuration (all experts Q8_0, Zipf-skewed routing) at the given batch sizes on the
    tensor-core path (and, for comparison, everything on the GEMV kernels), the Nemotron-H-style layer at T = 1 and 256,
    the CPU-runnable Q4_0 layer at T = 16, and the production mix (IQ3_S / Q4_0 routed experts, Q5_K shared expert) at
    T = 1 and 8.  Every entry carries its algorithmic bytes (with the measured number of
    distinct experts), its int8 operations and frac = max(bytes / HBM peak, ops / int8 peak) / time."""
    import torch
    from chimere_b200 import configs
    from chimere_b200.layer import MoeScratch, MoeWeightsPrefill, MoeWeightsTiled, forward_moe, forward_moe_prefill
    flush = L2Flush(dev)
    plan = []
    if prefill_tokens:
        plan.append((configs.QWEN_Q8_0, [(T, ("gemm", "gemv")) for T in prefill_tokens]))
    plan.append((configs.NEMOTRON_Q4_0, [(1, ("gemv",)), (256, ("gemm", "gemv"))]))
    plan.append((configs.QWEN_Q4_0, [(16, ("gemv", "gemm"))]))
    plan.append((configs.QWEN_IQ3S_Q5K, [(1, ("gemv",)), (8, ("gemv",))]))   # the production mix: shared expert in Q5_K super-blocks
    out = []
    for cfg, cases in plan:
        raw = configs.make_layer(cfg, device=dev)
        tiled, pw = MoeWeightsTiled(raw), MoeWeightsPrefill(raw)
        del raw
        for T, paths in cases:
            x = configs.make_input(cfg, T, device=dev)
            sc = MoeScratch(tiled, T, device=dev)
            sc.enable_prefill()
            y = torch.empty_like(x)
            res = {"config": cfg.name, "T": T}
            for name in paths:
                fn = (lambda: forward_moe_prefill(tiled, pw, sc, x, y)) if name == "gemm" else (lambda: forward_moe(tiled, sc, x, y))
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                ts = timed_calls(fn, 7, flush)
                us = statistics.median(ts)
                U = int(torch.unique(sc.topk_indices(T)).numel())
                alg = configs.algorithmic_bytes(cfg, T, U)
                ops = configs.int8_ops(cfg, T)
                t_hbm = alg / (hbm_peak * 1e9) * 1e6
                t_i8 = ops / (i8_peak_tops * 1e12) * 1e6 if i8_peak_tops else 0.0
                res[name] = {"us_per_layer_call": us, "us_stats": pct(ts), "tokens_per_s": T / (us * 1e-6),
                             "int8_tops": ops / (us * 1e-6) / 1e12, "hbm_gbs": alg / (us * 1e-6) / 1e9,
                             "frac": max(t_hbm, t_i8) / us, "bound": "hbm" if t_hbm >= t_i8 else "tensor"}
                res.update(distinct_experts=U, algorithmic_bytes=alg, int8_ops=ops, roofline_us={"hbm": t_hbm, "int8": t_i8})
            res["device_status"] = sc.status()
            out.append(res)
            del sc, x, y
        del tiled, pw
        torch.cuda.empty_cache()
    return {"how": "one layer, one call per sample, L2 flushed (256 MB written) before every sample, CUDA events on the launching "
                   "stream, median of 7; gemm = chimere_b200_moe_forward_prefill (tcgen05 grouped GEMM for experts with >= 8 tokens), "
                   "gemv = chimere_b200_moe_forward; frac = max(algorithmic bytes / measured HBM peak, int8 operations / measured "
                   "int8 tensor peak) / time",
            "results": out}


def run_expert_parallel(args, cfg, dev, rank, world, local, dist, hbm_peak, peak_kind):
    """N > 1: the same layer with its experts sharded over the ranks (E/N each, contiguous), router and shared
    expert replicated, T tokens per rank (weak scaling).  Dispatch and combine either by the kernels themselves (peer
    stores over NVLink, the default) or by NCCL all-to-all (--ep-exchange nccl)."""
    import torch
    from chimere_b200 import abi, configs, formats
    from chimere_b200.ep import ExpertParallelMoE
    T, L, K, W = args.tokens, args.layers, args.steps, args.warmup
    lib = abi.load()

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

    def build(cfg_, n_layers, tokens, seed0):
        eps = []
        for i in range(n_layers):
            full = configs.make_layer(cfg_, device=dev, seed=seed0 + i)        # same weights on every rank, then sharded
            eps.append(ExpertParallelMoE(full, max_tokens=tokens, rank=rank, world=world, device=dev, prefill=tokens * cfg_.top_k > 1024))
            del full
        return eps

    def exchange_mode(eps, tokens):
        """peer stores when asked for and the batch is decode-size; else the fixed-size NCCL exchange; else exact splits."""
        if tokens * cfg.top_k <= 1024 and args.ep_exchange == "peer":
            try:
                for e in eps:
                    e.enable_peer_exchange()
                return "peer"
            except Exception as exc:   # no IPC between these processes: the collective path still works
                print(f"[bench] peer exchange not available ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
        return "padded" if tokens * cfg.top_k <= 1024 else "exact"

    def graph_or_eager(step):
        note, graph = "eager launches", None
        try:
            step(); step()
            torch.cuda.synchronize(); dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            torch.cuda.synchronize()
            note = "CUDA graph replay of one step"
        except Exception as exc:
            graph = None
            note = f"eager launches (graph capture failed: {type(exc).__name__})"
            print(f"[bench] graph capture failed: {exc}", file=sys.stderr)
            torch.cuda.synchronize()
        return (graph.replay if graph is not None else step), note

    def received_pairs(eps, tokens):
        """Routed pairs every owner rank received in the last call of each layer: (mean, max) over ranks, averaged over layers."""
        k_, e_loc = cfg.top_k, cfg.E // world
        tot = torch.zeros(world, device=dev)
        for e in eps:
            idx = e.ws_home.topk_idx(tokens, k_).reshape(-1).to(torch.int64)
            tot += torch.bincount(torch.div(idx, e_loc, rounding_mode="floor"), minlength=world).to(tot.dtype)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        tot /= len(eps)
        return float(tot.mean().item()), float(tot.max().item())

    # ---- headline: the decode layer, T tokens per rank, L layers per step ----
    layers = build(cfg, L, T, 1000)
    xs = [configs.make_input(cfg, T, device=dev, seed=31 * (rank + 1) + i) for i in range(L)]
    ys = [torch.empty_like(x) for x in xs]
    mode = exchange_mode(layers, T)
    fwd = {"peer": lambda ep, x, y: ep.forward_peer(x, y), "padded": lambda ep, x, y: ep.forward_padded(x, y),
           "exact": lambda ep, x, y: ep.forward(x, y)}

    def step():
        for ep, x, y in zip(layers, xs, ys):
            fwd[mode](ep, x, y)

    run_step, timing_note = graph_or_eager(step) if mode != "exact" else (step, "eager launches")
    sampler = ClockSampler(local)
    secs = timed(run_step, K, W)
    clocks = sampler.stop()
    value = world * T * L * K / secs

    hx = [x.cpu().pin_memory() for x in xs]
    hy = [torch.empty(T, cfg.H).pin_memory() for _ in xs]

    def e2e_step():
        for ep, a, b, x, y in zip(layers, hx, hy, xs, ys):
            x.copy_(a, non_blocking=True)
            fwd[mode](ep, x, y)
            b.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    e2e_secs = timed(e2e_step, K, W)
    rows_mean, rows_max = received_pairs(layers, T)
    status = max(int(e.ws_home.arena[e.ws_home.ws.status - e.ws_home.arena.data_ptr():][:4].view(torch.int32).item()) for e in layers)
    del layers, xs, ys, run_step
    torch.cuda.empty_cache()

    # ---- secondary: the expert-parallel stack (Q4_0 experts, Zipf-biased routing, RMSNorm between the layers) ----
    stack = None
    if args.ep_stack_layers > 0:
        scfg = configs.QWEN_Q4_0_ZIPF
        stack = {"workload": f"{scfg.name}: {args.ep_stack_layers} layers with independent seeded weights, experts sharded {scfg.E // world} per GPU, "
                             "RMSNorm (unit weight, eps 1e-6) between the layers; tokens split evenly over the ranks", "results": []}
        for total_tokens in (64, 8192):
            tr = total_tokens // world
            if tr * world != total_tokens or tr < 1:
                continue
            eps = build(scfg, args.ep_stack_layers, tr, 4000)
            smode = exchange_mode(eps, tr)
            xa, xb = configs.make_input(scfg, tr, device=dev, seed=7 + rank), torch.empty(tr, scfg.H, device=dev)
            st = torch.cuda.current_stream(dev).cuda_stream

            def stack_step():
                h = xa
                for ep in eps:
                    fwd[smode](ep, h, xb)
                    abi.check(lib.chimere_b200_rmsnorm(xb.data_ptr(), xb.data_ptr(), tr, scfg.H, 1e-6, st), "rmsnorm")
                    h = xb

            run, note = graph_or_eager(stack_step) if smode != "exact" else (stack_step, "eager launches, one host synchronisation per layer for the split sizes")
            reps = 5 if smode != "exact" else 2
            s_secs = timed(run, reps, 2)
            r_mean, r_max = received_pairs(eps, tr)
            st_status = max(int(e.ws_home.arena[e.ws_home.ws.status - e.ws_home.arena.data_ptr():][:4].view(torch.int32).item()) for e in eps)
            stack["results"].append({"T_total": total_tokens, "T_per_rank": tr, "exchange": smode, "timing": note,
                                     "ms_per_stack": 1e3 * s_secs / reps, "tokens_per_s": total_tokens * reps / s_secs,
                                     "us_per_layer": 1e6 * s_secs / reps / args.ep_stack_layers,
                                     "pairs_received_per_rank_mean": r_mean, "pairs_received_per_rank_max": r_max,
                                     "imbalance": r_max / max(r_mean, 1e-9), "device_status": st_status})
            del eps, run
            torch.cuda.empty_cache()

    if rank == 0:
        b_gu = cfg.F * formats.row_bytes(cfg.type_gate_up, cfg.H)
        b_dn = cfg.H * formats.row_bytes(cfg.type_down, cfg.F)
        layer_us = secs / (K * L) * 1e6
        # per rank and layer call: every received pair's expert (upper bound on distinct experts: one per pair) + shared + router
        alg = min(rows_mean, cfg.E / world) * (2 * b_gu + b_dn) + (2 * b_gu + b_dn) + 4 * cfg.E * cfg.H + 8 * T * cfg.H
        ds = (cfg.H // 32 + 3) & ~3
        nvlink = (rows_mean * (cfg.H + 4 * ds + 12) + world * T * cfg.H * 4 if mode == "peer"
                  else world * T * cfg.top_k * (cfg.H + 4 * ds + 4 + 4 * cfg.H))
        exch = {"peer": "rows and partial sums written into the peers' buffers by the kernels (NVLink peer stores + flags), fixed-size slots, "
                        "owners return one partial sum per (home rank, token); no collective call, no host sync",
                "padded": "NCCL all-to-all, fixed size (padded to T*k rows per destination), no host sync",
                "exact": "NCCL all-to-all with exact split sizes, one host sync per layer call"}[mode]
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": 1e3 * secs / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "int8 block dots (dp4a), f32 accumulate", "data": "synthetic",
                "config": dict(workload_config(cfg, T, L), parallelism=f"ep{world}: {cfg.E // world} experts per GPU, router + shared expert replicated, "
                               f"{T} tokens per GPU", timing="CUDA events around K steps, max over ranks; " + timing_note,
                               exchange=exch, weight_layout="tiled"),
                "roofline": {"bound": "hbm", "kernel": "expert-parallel layer call (per rank)", "achieved": alg / (layer_us * 1e-6) / 1e9,
                             "peak": hbm_peak, "unit": "GB/s", "frac": alg / (layer_us * 1e-6) / 1e9 / hbm_peak, "peak_kind": peak_kind,
                             "traffic": None, "us_per_layer_call": layer_us,
                             "pairs_received_per_rank_mean": rows_mean, "pairs_received_per_rank_max": rows_max,
                             "nvlink_bytes_per_rank_per_call": nvlink},
                "cpu_baseline": None,
                "e2e": {"value": world * T * L * K / e2e_secs, "unit": UNIT, "h2d_bytes_per_step": L * T * cfg.H * 4,
                        "d2h_bytes_per_step": L * T * cfg.H * 4, "ms_per_step": 1e3 * e2e_secs / K},
                "gpu_launches": (10 if mode == "peer" else 9) * L * K, "clocks": clocks, "device_status": status, "ep_stack": stack}
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
    ap.add_argument("--prefill-tokens", default="512,2048,8192",
                    help="comma list of T for the prefill configuration in the secondary measurement ('' = none of them, 'none' = skip the secondary measurement)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="run only the int8 peak probe and the secondary measurement and print their JSON (used for profiling the grouped GEMM)")
    ap.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: dispatch / combine by the kernels' own peer stores (default) or by NCCL all-to-all")
    ap.add_argument("--ep-stack-layers", type=int, default=40,
                    help="N > 1: layers of the secondary expert-parallel stack measurement (0 = skip it)")
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
    hbm_peak, peak_kind = peaks()
    if args.prefill_only:
        i8 = measure_int8_peak(lib, dev)
        i8_tops = i8.get("m128_n256_k32", {}).get("tops")
        print(json.dumps({"int8_peak": i8, "secondary": measure_secondary(lib, dev, hbm_peak, i8_tops, [int(t) for t in args.prefill_tokens.split(",") if t])}))
        return 0
    cfg = configs.QWEN_IQ3S
    T, L, K, W = args.tokens, args.layers, args.steps, args.warmup
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

    def graph_of(fn):
        """The launches of fn() as one CUDA graph, so that the device time is not hidden behind the host's launch rate."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            fn()  # warm (also sets kernel attributes outside capture)
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                fn()
        return g

    def time_steps(run, k, w):
        """k timed repetitions of run() on `stream` after w warm-ups, bracketed by a synchronize on both sides.
        Returns (seconds for the k repetitions, per-repetition seconds); all device time, CUDA events on `stream`."""
        with torch.cuda.stream(stream):
            for _ in range(w):
                run()
            stream.synchronize()
            torch.cuda.synchronize()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(k + 1)]
            ev[0].record(stream)
            for i in range(k):
                run()
                ev[i + 1].record(stream)
            stream.synchronize()
            torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[k]) * 1e-3, [ev[i].elapsed_time(ev[i + 1]) * 1e-3 for i in range(k)]

    def distinct_experts(Tn):
        return [int(torch.unique(sc.topk_indices(Tn)).numel()) for sc in scratch]

    # ---- headline: graph replay of one step = L layer calls ----
    graph = graph_of(lambda: enqueue_layers(T))
    sampler = ClockSampler(local)
    secs, per_step = time_steps(graph.replay, K, W)
    clocks = sampler.stop()
    value = world * T * L * K / secs
    U = distinct_experts(T)
    layer_bytes = sum(configs.algorithmic_bytes(cfg, T, u) for u in U) / L
    layer_us = secs / (K * L) * 1e6
    layer_gbs = layer_bytes / (layer_us * 1e-6) / 1e9

    # ---- the three kernels of a layer call, each replayed alone over the rotating layers ----
    from chimere_b200 import formats
    b_gu = cfg.F * formats.row_bytes(cfg.type_gate_up, cfg.H)
    b_gu_sh = cfg.F_s * formats.row_bytes(cfg.type_gate_up, cfg.H)
    b_dn = cfg.H * formats.row_bytes(cfg.type_down, cfg.F)
    b_dn_sh = cfg.H * formats.row_bytes(cfg.type_down, cfg.F_s)
    xq_row = cfg.H // 32 * 36
    iq_row = max(cfg.F, cfg.F_s) // 32 * 36

    def stage_times(Tn, reps):
        """us per launch of the router, gate/up and down kernels at batch size Tn (the workspaces must hold the routing of
        a layer call at Tn), and the algorithmic bytes of the two GEMV launches."""
        def calls(entry, with_x=False, with_y=False):
            def run():
                for w, sc, x, y in zip(layers, scratch, xs, ys):
                    a = [C.byref(w.as_struct())] + ([x.data_ptr()] if with_x else []) + ([y.data_ptr()] if with_y else []) + [Tn, C.byref(sc.ws), sptr]
                    rc = entry(*a)
                    if rc:
                        raise RuntimeError(f"stage rc={rc}")
            return run
        Un = distinct_experts(Tn)
        pairs = Tn * cfg.top_k + Tn
        gu_b = sum(2 * (u * b_gu + b_gu_sh) + Tn * xq_row + pairs * (cfg.F // 32 * 36) for u in Un) / L
        dn_b = sum(u * b_dn + b_dn_sh + pairs * iq_row + Tn * cfg.H * 4 for u in Un) / L
        gu = time_steps(graph_of(calls(lib.chimere_b200_moe_gate_up)).replay, reps, 3)[0] / (reps * L)
        dn = time_steps(graph_of(calls(lib.chimere_b200_moe_down_combine, with_y=True)).replay, reps, 3)[0] / (reps * L)
        rt = time_steps(graph_of(calls(lib.chimere_b200_moe_route, with_x=True)).replay, reps, 3)[0] / (reps * L)
        return {"route_us": rt * 1e6, "gate_up_us": gu * 1e6, "down_us": dn * 1e6, "gate_up_bytes": gu_b, "down_bytes": dn_b,
                "gate_up_frac": gu_b / gu / 1e9 / hbm_peak, "down_frac": dn_b / dn / 1e9 / hbm_peak}

    stg = stage_times(T, max(5, K))
    gu_secs, dn_secs, rt_secs, gu_bytes, dn_bytes = stg["gate_up_us"] * 1e-6, stg["down_us"] * 1e-6, stg["route_us"] * 1e-6, stg["gate_up_bytes"], stg["down_bytes"]
    kname = "bulk_kernel<IQ3_S, gate_up>" if args.layout == "tiled" else "gate_up_kernel<IQ3_S>"
    traffic, traffic_src = captured_traffic(kname, f"{cfg.name} T={T}")
    roof = {"bound": "hbm", "kernel": kname, "achieved": gu_bytes / gu_secs / 1e9, "peak": hbm_peak,
            "unit": "GB/s", "frac": gu_bytes / gu_secs / 1e9 / hbm_peak, "peak_kind": peak_kind,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this shape, from the committed ncu capture
            # table (None when this kernel and shape have not been captured)
            "traffic": traffic, "traffic_source": traffic_src,
            "us_per_launch": gu_secs * 1e6, "algorithmic_bytes_per_launch": gu_bytes,
            "down_kernel": {"achieved": dn_bytes / dn_secs / 1e9, "frac": dn_bytes / dn_secs / 1e9 / hbm_peak,
                            "us_per_launch": dn_secs * 1e6, "algorithmic_bytes_per_launch": dn_bytes},
            "route_kernel": {"us_per_launch": rt_secs * 1e6},
            "layer": {"achieved": layer_gbs, "frac": layer_gbs / hbm_peak, "us_per_layer_call": layer_us,
                      "algorithmic_bytes_per_call": layer_bytes, "distinct_experts_mean": sum(U) / L}}

    # ---- sweep over T: the layer call and its three kernels (graph replay over the rotating layers) ----
    sweep = []
    if not args.no_sweep:
        for Tn in (1, 2, 4, 8):
            g = graph_of(lambda: enqueue_layers(Tn))
            s_ = time_steps(g.replay, max(5, K), 3)[0] / max(5, K)
            Un = distinct_experts(Tn)
            b = sum(configs.algorithmic_bytes(cfg, Tn, u) for u in Un) / L
            us = s_ / L * 1e6
            ent = {"T": Tn, "us_per_layer_call": us, "tokens_layers_per_s": Tn * L / s_,
                   "hbm_gbs": b / (us * 1e-6) / 1e9, "hbm_frac": b / (us * 1e-6) / 1e9 / hbm_peak,
                   "algorithmic_bytes_per_call": b, "distinct_experts_mean": sum(Un) / L}
            ent["kernels"] = stage_times(Tn, 5)
            sweep.append(ent)
            del g

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
    torch.cuda.synchronize()
    e2e_steps = []
    t0 = time.perf_counter()
    for _ in range(K):
        t1 = time.perf_counter()
        e2e_step()                       # every call ends with a stream synchronisation: the step is complete on return
        e2e_steps.append(time.perf_counter() - t1)
    torch.cuda.synchronize()
    e2e_secs = time.perf_counter() - t0
    e2e = {"value": world * T * L * K / e2e_secs, "unit": UNIT, "h2d_bytes_per_step": L * T * cfg.H * 4,
           "d2h_bytes_per_step": L * T * cfg.H * 4, "ms_per_step": 1e3 * e2e_secs / K,
           "ms_per_step_stats": pct([1e3 * t for t in e2e_steps]),
           "how": "chimere_b200_moe_forward_host per layer call: pinned host x copied in, layer (its last kernel stores y straight into the pinned host buffer), stream synchronised; host clock"}

    status = max(sc.status() for sc in scratch)
    secondary, i8 = None, None
    if args.prefill_tokens != "none" and args.layout == "tiled":
        del graph
        layers.clear(); scratch.clear(); xs.clear(); ys.clear(); host_calls.clear()
        torch.cuda.empty_cache()
        i8 = measure_int8_peak(lib, dev)
        secondary = measure_secondary(lib, dev, hbm_peak, i8.get("m128_n256_k32", {}).get("tops"), [int(t) for t in args.prefill_tokens.split(",") if t])

    cpu = None
    if not args.no_cpu_baseline:
        v, threads, dt = cpu_port_tokens_per_s(cfg, T, 2, min_seconds=10.0)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"T={T} tokens through 2 layers, repeated for {dt:.1f} s; CPU restatement in oracle/ with OpenMP"}
        # the reference's own default for its CPU expert path is four threads (moe_ffn.rs:1551, ggml_backend.rs:292-300)
        v4, t4, dt4 = cpu_port_tokens_per_s(cfg, T, 2, threads=4, min_seconds=6.0)
        cpu["threads4"] = {"value": v4, "cores": t4, "sample": f"the same sample with 4 threads for {dt4:.1f} s (the reference's default thread count for this path)"}

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": 1e3 * secs / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 block dots (dp4a), f32 accumulate", "data": "synthetic",
            "config": dict(workload_config(cfg, T, L), parallelism="single GPU",
                           timing="CUDA graph replay of one step, CUDA events on the launching stream",
                           weight_layout=args.layout),
            "ms_per_step_stats": pct([1e3 * t for t in per_step]),
            "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": 3 * L * K, "clocks": clocks,
            "sweep": sweep, "int8_peak": i8, "secondary": secondary, "device_status": status}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
