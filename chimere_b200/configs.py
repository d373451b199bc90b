"""The benchmark configurations of the MoE path as seeded synthetic layers.

Shapes, weight types, value distributions and routing variants follow the five configurations
the benchmark definition lists (Qwen3.5-35B-A3B-shaped layer with Q4_0 / IQ3_S+Q4_0 / Q8_0
experts, a Nemotron-H-style layer, and a 40-layer stack).  No real model weights are involved:
weights are drawn ~N(0, 0.02) and quantized with chimere_b200.formats, inputs ~N(0, 1).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import abi, formats
from .layer import MoeWeightsRaw

Q4_0, Q8_0, IQ3_S = formats.TYPE_Q4_0, formats.TYPE_Q8_0, formats.TYPE_IQ3_S


@dataclass(frozen=True)
class LayerConfig:
    name: str
    H: int
    E: int
    F: int
    F_s: int
    top_k: int
    type_gate_up: int
    type_down: int
    act: int = abi.ACT_SWIGLU
    route_mode: int = abi.ROUTE_SOFTMAX_RENORM
    route_scale: float = 1.0
    shared_gate: bool = True      # shared expert scaled by sigmoid(x . w_sg)
    zipf_bias: bool = False       # per-expert logit bias 2*log(rank^-1.1) over a seeded permutation
    seed: int = 0
    type_sh_gate_up: Optional[int] = None   # shared expert's weight types when they differ from the routed experts'
    type_sh_down: Optional[int] = None      # (the production files quantize the shared expert differently, moe_ffn.rs:1618-1705)


QWEN_Q4_0 = LayerConfig("qwen35-moe-q4_0", 2048, 256, 512, 512, 8, Q4_0, Q4_0, seed=0)
QWEN_IQ3S = LayerConfig("qwen35-moe-iq3s-q4_0", 2048, 256, 512, 512, 8, IQ3_S, Q4_0, seed=1)
QWEN_Q8_0 = LayerConfig("qwen35-moe-q8_0-zipf", 2048, 256, 512, 512, 8, Q8_0, Q8_0, zipf_bias=True, seed=2)
NEMOTRON_Q4_0 = LayerConfig("nemotron-h-moe-q4_0", 2688, 128, 1856, 3712, 6, Q4_0, Q4_0, act=abi.ACT_RELU2,
                            route_mode=abi.ROUTE_SIGMOID_NORM_SCALE, route_scale=2.5, shared_gate=False, seed=3)
QWEN_Q4_0_ZIPF = LayerConfig("qwen35-moe-q4_0-zipf", 2048, 256, 512, 512, 8, Q4_0, Q4_0, zipf_bias=True, seed=4)
# the production mix: IQ3_S routed experts, Q5_K shared expert (moe_ffn.rs:1597-1650); not one of the benchmark's five
QWEN_IQ3S_Q5K = LayerConfig("qwen35-moe-iq3s-q4_0-shared-q5k", 2048, 256, 512, 512, 8, IQ3_S, Q4_0, seed=5,
                            type_sh_gate_up=formats.TYPE_Q5_K, type_sh_down=formats.TYPE_Q5_K)
CONFIGS = [QWEN_Q4_0, QWEN_IQ3S, QWEN_Q8_0, NEMOTRON_Q4_0, QWEN_Q4_0_ZIPF]


def scaled(cfg: LayerConfig, **kw) -> LayerConfig:
    """A smaller copy of a configuration (tests)."""
    d = dict(cfg.__dict__)
    d.update(kw)
    return LayerConfig(**d)


def _quant_matrix_stack(qtype: int, n: int, rows: int, cols: int, gen: torch.Generator, device, chunk: int = 16) -> torch.Tensor:
    """n matrices [rows, cols] ~N(0, 0.02), quantized; returns u8 [n, rows*row_bytes]."""
    rb = formats.row_bytes(qtype, cols)
    if qtype in (formats.TYPE_Q4_K, formats.TYPE_Q5_K, formats.TYPE_Q6_K):   # no quantizer for these: seeded valid blocks
        seed = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=gen, device=device).item())
        return torch.from_numpy(formats.random_kquant_rows(qtype, n * rows, cols, seed=seed)).reshape(n, rows * rb).to(device)
    out = torch.empty(n, rows * rb, dtype=torch.uint8, device=device)
    for e0 in range(0, n, chunk):
        e1 = min(n, e0 + chunk)
        w = torch.randn((e1 - e0) * rows, cols, generator=gen, device=device, dtype=torch.float32) * 0.02
        out[e0:e1] = formats.quantize(qtype, w).reshape(e1 - e0, rows * rb)
    return out


def zipf_bias(E: int, gen: torch.Generator, device) -> torch.Tensor:
    """b_e = 2*log(rank_e^-1.1), ranks 1..E dealt to the experts by a seeded permutation."""
    perm = torch.randperm(E, generator=gen, device=device)
    rank = torch.empty(E, dtype=torch.float32, device=device)
    rank[perm] = torch.arange(1, E + 1, dtype=torch.float32, device=device)
    return (2.0 * (-1.1) * torch.log(rank)).contiguous()


def make_layer(cfg: LayerConfig, device="cpu", seed: Optional[int] = None) -> MoeWeightsRaw:
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(cfg.seed if seed is None else seed)
    dual = cfg.act == abi.ACT_SWIGLU
    router = (torch.randn(cfg.E, cfg.H, generator=gen, device=dev) * 0.02).contiguous()
    gate = _quant_matrix_stack(cfg.type_gate_up, cfg.E, cfg.F, cfg.H, gen, dev) if dual else None
    up = _quant_matrix_stack(cfg.type_gate_up, cfg.E, cfg.F, cfg.H, gen, dev)
    down = _quant_matrix_stack(cfg.type_down, cfg.E, cfg.H, cfg.F, gen, dev)
    kw = {}
    if cfg.F_s > 0:
        t_gu = cfg.type_gate_up if cfg.type_sh_gate_up is None else cfg.type_sh_gate_up
        t_dn = cfg.type_down if cfg.type_sh_down is None else cfg.type_sh_down
        kw["shexp_gate_raw"] = _quant_matrix_stack(t_gu, 1, cfg.F_s, cfg.H, gen, dev)[0] if dual else None
        kw["shexp_up_raw"] = _quant_matrix_stack(t_gu, 1, cfg.F_s, cfg.H, gen, dev)[0]
        kw["shexp_down_raw"] = _quant_matrix_stack(t_dn, 1, cfg.H, cfg.F_s, gen, dev)[0]
        kw["type_sh_gate"] = t_gu if dual else 0
        kw["type_sh_up"], kw["type_sh_down"] = t_gu, t_dn
        if cfg.shared_gate:
            kw["shexp_gate_proj"] = (torch.randn(cfg.H, generator=gen, device=dev) * 0.02).contiguous()
    if cfg.zipf_bias:
        kw["router_bias"] = zipf_bias(cfg.E, gen, dev)
    return MoeWeightsRaw(H=cfg.H, E=cfg.E, F=cfg.F, F_s=cfg.F_s, top_k=cfg.top_k,
                         type_gate=cfg.type_gate_up if dual else 0, type_up=cfg.type_gate_up, type_down=cfg.type_down,
                         router_weight=router, up_exps_raw=up, down_exps_raw=down, gate_exps_raw=gate,
                         route_mode=cfg.route_mode, route_scale=cfg.route_scale, act=cfg.act, **kw)


def make_input(cfg: LayerConfig, T: int, device="cpu", seed: Optional[int] = None) -> torch.Tensor:
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000003 * (cfg.seed if seed is None else seed) + T)
    return torch.randn(T, cfg.H, generator=gen, device=dev, dtype=torch.float32).contiguous()


def algorithmic_bytes(cfg: LayerConfig, T: int, distinct_experts: int) -> int:
    """Bytes one layer call must move at least: every selected expert's weights once, the shared
    expert, the router, w_sg, and x in / y out in fp32.  Intermediates are not counted."""
    n_mat = 3 if cfg.act == abi.ACT_SWIGLU else 2
    b_gu = cfg.F * formats.row_bytes(cfg.type_gate_up, cfg.H)
    b_dn = cfg.H * formats.row_bytes(cfg.type_down, cfg.F)
    b_exp = (n_mat - 1) * b_gu + b_dn
    b_sh = 0
    if cfg.F_s > 0:
        t_gu = cfg.type_gate_up if cfg.type_sh_gate_up is None else cfg.type_sh_gate_up
        t_dn = cfg.type_down if cfg.type_sh_down is None else cfg.type_sh_down
        b_sh = (n_mat - 1) * cfg.F_s * formats.row_bytes(t_gu, cfg.H) + cfg.H * formats.row_bytes(t_dn, cfg.F_s)
    return distinct_experts * b_exp + b_sh + 4 * cfg.E * cfg.H + (4 * cfg.H if cfg.shared_gate else 0) + 8 * T * cfg.H


def int8_ops(cfg: LayerConfig, T: int) -> int:
    n_mat = 3 if cfg.act == abi.ACT_SWIGLU else 2
    return 2 * T * (cfg.top_k * n_mat * cfg.F * cfg.H + n_mat * cfg.F_s * cfg.H)
