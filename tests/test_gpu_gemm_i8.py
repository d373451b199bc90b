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
        sa = torch.rand(rows, nb, generator=g, device="cuda") * 0.01 + 0.001
        sb = torch.rand(tokens, nb, generator=g, device="cuda") * 0.05 + 0.001
    pa, pb = _pack(lib, A, sa), _pack(lib, B, sb)
    out = torch.full((rows, tokens), float("nan"), device="cuda")
    items = torch.zeros(((rows + 127) // 128) * ((tokens + 127) // 128) * 32, dtype=torch.uint8, device="cuda")
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


@pytest.mark.parametrize("rows,tokens,cols", [(128, 128, 128), (256, 200, 512), (192, 37, 2048)])
def test_integer_dots_exact_with_unit_scales(rows, tokens, cols):
    out, ref = _run(rows, tokens, cols, unit_scales=True)
    assert torch.equal(out.double(), ref), "unit scales: every output is an integer below 2^24 and must be exact"


@pytest.mark.parametrize("rows,tokens,cols", [(256, 200, 512), (512, 128, 2048)])
def test_block_scaled_result(rows, tokens, cols):
    out, ref = _run(rows, tokens, cols, unit_scales=False)
    rel = (out.double() - ref).abs().max() / ref.abs().max()
    assert rel < 1e-5, float(rel)
