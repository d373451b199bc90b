"""The tcgen05 block-scaled int8 GEMM primitive against an exact reference computed with torch on the
same GPU (float64 accumulation of the exact integer block dots)."""
import pytest
import torch

from chimere_b200 import abi

pytestmark = pytest.mark.gpu


def _pack(lib, q, sc):
    rows, cols = q.shape
    out = torch.zeros(lib.chimere_b200_mma128_bytes(rows, cols), dtype=torch.uint8, device="cuda")
    abi.check(lib.chimere_b200_pack_mma128(q.data_ptr(), sc.data_ptr(), out.data_ptr(), rows, cols, None), "pack_mma128")
    return out


def _run(rows, tokens, cols, unit_scales):
    lib = abi.load()
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + tokens)
    A = torch.randint(-127, 128, (rows, cols), generator=g, device="cuda", dtype=torch.int32).to(torch.int8)
    B = torch.randint(-127, 128, (tokens, cols), generator=g, device="cuda", dtype=torch.int32).to(torch.int8)
    nb = cols // 32
    if unit_scales:
        sa, sb = torch.ones(rows, nb, device="cuda"), torch.ones(tokens, nb, device="cuda")
    else:
        # weight-side scales as ggml has them: an f16 value (times a small odd factor, as IQ3_S sub-blocks do)
        sa = (torch.rand(rows, nb, generator=g, device="cuda") * 0.01 + 0.001).half().float() * (1 + 2 * torch.randint(0, 16, (rows, nb), generator=g, device="cuda"))
        sb = torch.rand(tokens, nb, generator=g, device="cuda") * 0.05 + 0.001
    pa, pb = _pack(lib, A, sa), _pack(lib, B, sb)
    out = torch.full((rows, tokens), float("nan"), device="cuda")
    items = torch.zeros(((rows + 127) // 128) * ((tokens + 127) // 128) * 32 + 256, dtype=torch.uint8, device="cuda")
    status = torch.zeros(64, dtype=torch.int32, device="cuda")
    abi.check(lib.chimere_b200_gemm_i8(pa.data_ptr(), pb.data_ptr(), rows, tokens, cols, out.data_ptr(), items.data_ptr(),
                                       status.data_ptr(), None), "gemm_i8")
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    Ab = A.reshape(rows, nb, 32).double()
    Bb = B.reshape(tokens, nb, 32).double()
    S = torch.einsum("rbk,tbk->rtb", Ab, Bb)                      # exact integer block dots
    ref = torch.einsum("rtb,rb,tb->rt", S, sa.double(), sb.double())
    return out, ref


@pytest.mark.parametrize("rows,tokens,cols", [(128, 128, 128), (256, 200, 512), (192, 37, 2048), (384, 20, 256), (128, 50, 96), (2048, 1100, 512)])
def test_integer_dots_exact_with_unit_scales(rows, tokens, cols):
    out, ref = _run(rows, tokens, cols, unit_scales=True)
    assert torch.equal(out.double(), ref), "unit scales: every output is an integer below 2^24 and must be exact"


@pytest.mark.parametrize("rows,tokens,cols", [(256, 200, 512), (512, 128, 2048), (256, 60, 1024), (256, 9, 160)])
def test_block_scaled_result(rows, tokens, cols):
    out, ref = _run(rows, tokens, cols, unit_scales=False)
    rel = (out.double() - ref).abs().max() / ref.abs().max()
    assert rel < 1e-5, float(rel)


# ---------------------------------------------------------------- the MoE layer on the GEMM path ----
import numpy as np  # noqa: E402

import oracle  # noqa: E402
from chimere_b200 import configs  # noqa: E402
from chimere_b200.layer import MoeScratch, MoeWeightsPrefill, MoeWeightsTiled, forward_moe, forward_moe_prefill  # noqa: E402

PREFILL_CASES = [
    (configs.scaled(configs.QWEN_Q8_0, E=16), 300),        # Zipf bias: a few experts get most tokens, the tail stays on the GEMV
    (configs.scaled(configs.QWEN_Q4_0, E=8), 200),
    (configs.scaled(configs.QWEN_IQ3S, E=8), 130),
    (configs.scaled(configs.NEMOTRON_Q4_0, E=8, F=1792, F_s=3712 - 128), 96),   # no gate matrix: 128-row tiles
    (configs.scaled(configs.NEMOTRON_Q4_0, E=8, name="nemotron-full-widths"), 160),  # F = 1856 = 14.5 row tiles: the last one is zero-padded
]


@pytest.mark.parametrize("cfg,T", PREFILL_CASES, ids=lambda v: getattr(v, "name", str(v)))
def test_prefill_forward_matches_oracle_and_gemv_path(cfg, T):
    raw = configs.make_layer(cfg, device="cuda")
    tiled, pw = MoeWeightsTiled(raw), MoeWeightsPrefill(raw)
    x = configs.make_input(cfg, T, device="cuda")
    sc = MoeScratch(tiled, T)
    y_gemv = forward_moe(tiled, sc, x).clone()
    y = forward_moe_prefill(tiled, pw, sc, x)
    torch.cuda.synchronize()
    assert sc.status() == 0
    o = oracle.moe_forward(raw.to("cpu"), x.cpu().numpy(), taps=False)
    for name, got in (("gemm", y), ("gemv", y_gemv)):
        g, ref = got.cpu().numpy().astype(np.float64), o["y"].astype(np.float64)
        rel = np.abs(g - ref).max(axis=1) / np.abs(ref).max(axis=1)
        cos = (g * ref).sum(1) / (np.linalg.norm(g, axis=1) * np.linalg.norm(ref, axis=1))
        assert rel.max() <= 1e-2 and cos.min() >= 0.9999, (name, rel.max(), cos.min())
    # the two GPU paths compute the same integer block dots; only fp32 summation order differs
    assert (y - y_gemv).abs().max() <= 2e-3 * y_gemv.abs().max()
