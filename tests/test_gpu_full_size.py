"""GPU parity at the benchmark's own sizes, for the batches that run on the tensor-core path.

  prefill configuration : 256 experts, all Q8_0, Zipf-skewed routing, T = 512 / 2048 / 8192
  Nemotron-H-style layer : 128 experts of width 1856 (ungated, squared ReLU), shared width 3712, T = 256, both entries
  CPU-runnable layer    : 256 experts, Q4_0, T = 16, through the prefill entry as well

For every token: router logits and Q8_1 bytes bit-exact against the CPU oracle, routing indices equal (an expf
near-tie between the host's and the GPU's exponential is the only accepted difference, and the oracle is then re-run
on the GPU's indices), the dispatch permutation and offsets bit-exact, and the fp32 output rows within max relative
error 1e-2 and cosine >= 0.9999."""
import numpy as np
import pytest
import torch

import oracle
from chimere_b200 import abi, configs
from chimere_b200.layer import MoeScratch, MoeWeightsPrefill, MoeWeightsTiled, forward_moe, forward_moe_prefill
from parity_util import check_rows, oracle_on_gpu_routing

pytestmark = pytest.mark.gpu

_cache = {}


def _weights(cfg):
    """(raw on the device, host copy, tiled32 form, GEMM form) of a configuration; one configuration is kept at a time
    (the prefill configuration alone is 0.9 GB per form)."""
    if _cache.get("cfg") != cfg.name:
        _cache.clear()
        torch.cuda.empty_cache()
        raw = configs.make_layer(cfg, device="cuda")
        _cache.update(cfg=cfg.name, raw=raw, host=raw.to("cpu"), tiled=MoeWeightsTiled(raw), pw=MoeWeightsPrefill(raw))
    return _cache["raw"], _cache["host"], _cache["tiled"], _cache["pw"]


def _check_layer_call(cfg, T, entry):
    raw, wh, tiled, pw = _weights(cfg)
    x = configs.make_input(cfg, T, device="cuda")
    sc = MoeScratch(tiled, T)
    y = forward_moe_prefill(tiled, pw, sc, x) if entry == "prefill" else forward_moe(tiled, sc, x)
    torch.cuda.synchronize()
    assert sc.status() == 0, "a bounded wait in a kernel ran out"
    idx = sc.topk_indices(T).cpu().numpy()
    xh = x.cpu().numpy()
    o = oracle_on_gpu_routing(wh, xh, idx)
    assert np.array_equal(sc.router_logits(T).cpu().numpy(), o["logits"]), "router logits must match the oracle bit for bit"
    assert np.array_equal(sc.x_q8(T).cpu().numpy(), o["x_q8"]), "Q8_1 bytes of the input"
    np.testing.assert_allclose(sc.topk_weights(T).cpu().numpy(), o["topk_w"], rtol=4e-6)
    perm, offs = oracle.permute(idx, cfg.E)
    assert np.array_equal(sc.perm(T).cpu().numpy(), perm), "dispatch permutation"
    assert np.array_equal(sc.offsets().cpu().numpy(), offs), "per-expert offsets"
    check_rows(y.cpu().numpy(), o["y"])
    return offs


@pytest.mark.parametrize("T", [512, 2048, 8192])
def test_prefill_configuration_full_size(T):
    offs = _check_layer_call(configs.QWEN_Q8_0, T, "prefill")
    counts = np.diff(offs)
    # the Zipf bias must have done its work: a few experts hold most pairs, so several token tiles per expert exist
    # and the persistent tile walk wraps many times
    assert counts.max() >= T // 2 and (counts >= 8).sum() >= 8


@pytest.mark.parametrize("entry", ["prefill", "decode"])
def test_nemotron_style_layer_T256(entry):
    _check_layer_call(configs.NEMOTRON_Q4_0, 256, entry)


def test_cpu_runnable_configuration_T16_prefill_entry():
    _check_layer_call(configs.QWEN_Q4_0, 16, "prefill")


def test_prefill_and_decode_entries_agree_on_integer_dots():
    """Both entries compute the same integer block dots; only the order of the fp32 additions differs."""
    cfg, T = configs.QWEN_Q4_0, 16
    raw, wh, tiled, pw = _weights(cfg)
    x = configs.make_input(cfg, T, device="cuda")
    sc = MoeScratch(tiled, T)
    y1 = forward_moe(tiled, sc, x).clone()
    y2 = forward_moe_prefill(tiled, pw, sc, x)
    torch.cuda.synchronize()
    assert (y1 - y2).abs().max() <= 2e-3 * y1.abs().max()
