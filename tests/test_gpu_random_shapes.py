"""Seeded random layer shapes, weight types, routing variants and batch sizes through both whole-layer entries: router
logits, dispatch permutation and offsets bit for bit, output rows within the benchmark's tolerance of the CPU oracle.
Complements the fixed configurations: odd expert counts, top-k from 1 to 8, layers without a shared expert, K-quant
shared experts, batches on both sides of every kernel-selection threshold (4, 8, 32 tokens; the GEMM's 8 rows per expert)."""
import random

import numpy as np
import pytest
import torch

import oracle
from chimere_b200 import configs, formats
from chimere_b200.layer import MoeScratch, MoeWeightsPrefill, MoeWeightsTiled, forward_moe, forward_moe_prefill
from parity_util import check_rows, oracle_on_gpu_routing

pytestmark = pytest.mark.gpu


def _case(seed):
    rng = random.Random(seed)
    base = rng.choice([configs.QWEN_Q4_0, configs.QWEN_IQ3S, configs.QWEN_Q8_0, configs.NEMOTRON_Q4_0])
    H = rng.choice([256, 512, 1024, 2048])
    E = rng.choice([8, 16, 24, 64, 128, 256])
    k = min(rng.choice([1, 2, 4, 6, 8]), E)
    mult = 256 if configs.IQ3_S in (base.type_gate_up, base.type_down) else 64
    F, Fs = mult * rng.choice([1, 2, 3]), rng.choice([0, mult, 2 * mult])
    kw = dict(E=E, H=H, F=F, F_s=Fs, top_k=k, seed=rng.randrange(10 ** 6))
    if Fs and Fs % 256 == 0 and rng.random() < 0.3:
        kw.update(type_sh_gate_up=formats.TYPE_Q5_K, type_sh_down=rng.choice([formats.TYPE_Q4_K, formats.TYPE_Q5_K, formats.TYPE_Q6_K]))
    T = rng.choice([1, 2, 3, 4, 5, 8, 9, 17, 33, 70, 200])
    prefill = T >= 33 and rng.random() < 0.5
    return configs.scaled(base, **kw), T, prefill


@pytest.mark.parametrize("seed", range(24))
def test_random_layer(seed):
    cfg, T, prefill = _case(1000 + seed)
    raw = configs.make_layer(cfg, device="cuda")
    tiled = MoeWeightsTiled(raw)
    x = configs.make_input(cfg, T, device="cuda")
    sc = MoeScratch(tiled, T)
    y = forward_moe_prefill(tiled, MoeWeightsPrefill(raw), sc, x) if prefill else forward_moe(tiled, sc, x)
    torch.cuda.synchronize()
    assert sc.status() == 0
    idx = sc.topk_indices(T).cpu().numpy()
    o = oracle_on_gpu_routing(raw.to("cpu"), x.cpu().numpy(), idx)
    assert np.array_equal(sc.router_logits(T).cpu().numpy(), o["logits"]), cfg
    perm, offs = oracle.permute(idx, cfg.E)
    assert np.array_equal(sc.perm(T).cpu().numpy(), perm), cfg
    assert np.array_equal(sc.offsets().cpu().numpy(), offs), cfg
    check_rows(y.cpu().numpy(), o["y"])
