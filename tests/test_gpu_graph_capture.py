"""The whole-layer entries inside a CUDA graph: no allocation, no host synchronisation, no device-to-host copy in them,
and the programmatic launch edges between the kernels are captured with the kernels.  A replay on new input contents must
give exactly what the eager call gives."""
import pytest
import torch

from chimere_b200 import configs, formats
from chimere_b200.layer import MoeScratch, MoeWeightsPrefill, MoeWeightsTiled, forward_moe, forward_moe_prefill

pytestmark = pytest.mark.gpu

CASES = [
    ("decode", configs.scaled(configs.QWEN_IQ3S, E=32, F=256, F_s=256, H=1024), 8),
    ("decode", configs.scaled(configs.NEMOTRON_Q4_0, E=16, F=128, F_s=256, H=512), 5),
    ("decode, Q5_K shared expert", configs.scaled(configs.QWEN_IQ3S, E=32, F=256, F_s=512, H=1024, type_sh_gate_up=formats.TYPE_Q5_K,
                                                  type_sh_down=formats.TYPE_Q5_K), 8),
    ("prefill", configs.scaled(configs.QWEN_Q8_0, E=16, F=128, F_s=128, H=512), 300),
]


@pytest.mark.parametrize("kind,cfg,T", CASES, ids=[c[0] + " " + c[1].name for c in CASES])
def test_layer_call_replays_from_a_graph(kind, cfg, T):
    raw = configs.make_layer(cfg, device="cuda")
    tiled = MoeWeightsTiled(raw)
    pw = MoeWeightsPrefill(raw) if kind == "prefill" else None
    sc = MoeScratch(tiled, T)
    if pw is not None:
        sc.enable_prefill()
    x, y = torch.empty(T, cfg.H, device="cuda"), torch.empty(T, cfg.H, device="cuda")
    call = (lambda: forward_moe_prefill(tiled, pw, sc, x, y)) if pw is not None else (lambda: forward_moe(tiled, sc, x, y))
    inputs = [configs.make_input(cfg, T, device="cuda", seed=s) for s in (1, 2, 3)]
    eager = []
    for xi in inputs:
        x.copy_(xi)
        call()
        eager.append(y.clone())
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        x.copy_(inputs[0])
        call()                                  # warm-up on the capture stream (function attributes are set on first use)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            call()
    torch.cuda.synchronize()
    for xi, want in zip(inputs, eager):
        x.copy_(xi)
        graph.replay()
        graph.replay()                          # twice in a row: counters and flags are back where they started
        torch.cuda.synchronize()
        assert torch.equal(y, want)
    assert sc.status() == 0
