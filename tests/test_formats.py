"""Block formats: our quantizers against the gguf package, the IQ3_S codebook against the
reference's table, and the oracle's dequantizers against both."""
import os
import re

import numpy as np
import pytest
import torch

import oracle
from chimere_b200 import formats as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference tree: CHIMERE_REFERENCE_DIR, or a directory named "reference" beside the repository
REF_DIR = os.environ.get("CHIMERE_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
REF_LOADER = os.path.join(REF_DIR, "chimere-server", "src", "gguf_loader.rs")


def test_grid_matches_gguf_package():
    from gguf import quants
    quants.IQ3_S.init_grid()
    g = np.asarray(quants.IQ3_S.grid).reshape(512, 4)
    assert np.array_equal(g.astype(np.uint8), F.iq3s_grid())


@pytest.mark.skipif(not os.path.exists(REF_LOADER), reason="reference tree not mounted")
def test_grid_matches_reference_table():
    txt = open(REF_LOADER).read()
    body = txt[txt.index("const IQ3S_GRID: [u32; 512]"):]
    body = body[:body.index("];")]
    vals = [int(v, 16) for v in re.findall(r"0x([0-9a-fA-F]{8})", body)]
    assert len(vals) == 512
    g = F.iq3s_grid().astype(np.uint32)
    mine = g[:, 0] | (g[:, 1] << 8) | (g[:, 2] << 16) | (g[:, 3] << 24)
    assert np.array_equal(mine, np.array(vals, dtype=np.uint32))


@pytest.mark.parametrize("qtype,gname", [(F.TYPE_Q4_0, "Q4_0"), (F.TYPE_Q8_0, "Q8_0")])
def test_quantizers_match_gguf_bytes(qtype, gname):
    from gguf import quants
    from gguf.constants import GGMLQuantizationType as GT
    torch.manual_seed(5)
    w = torch.randn(48, 512) * 0.02
    mine = F.quantize(qtype, w).numpy()
    ref = quants.quantize(w.numpy(), getattr(GT, gname)).reshape(48, -1)
    assert np.array_equal(mine, ref)


def test_iq3s_encoder_roundtrip_and_gguf_dequant():
    from gguf import quants
    from gguf.constants import GGMLQuantizationType as GT
    torch.manual_seed(6)
    w = torch.randn(32, 1024) * 0.02
    enc = F.quantize_iq3_s(w)
    assert enc.shape == (32, 4 * 110)
    deq = F.dequantize(F.TYPE_IQ3_S, enc, 1024).numpy()
    ref = quants.dequantize(enc.numpy(), GT.IQ3_S).reshape(32, 1024)
    assert np.array_equal(deq, ref)
    rmse = float(np.sqrt(np.mean((deq - w.numpy()) ** 2)) / 0.02)
    assert rmse < 0.25, rmse  # 3.4 bits per weight: ~16 % of sigma


@pytest.mark.parametrize("qtype", [F.TYPE_Q4_0, F.TYPE_Q8_0, F.TYPE_IQ3_S])
def test_oracle_dequant_matches(qtype):
    torch.manual_seed(7)
    w = torch.randn(16, 512) * 0.02
    enc = F.quantize(qtype, w)
    a = oracle.dequant(qtype, enc.numpy(), 16 * 512).reshape(16, 512)
    b = F.dequantize(qtype, enc, 512).numpy()
    assert np.array_equal(a, b)


def test_known_q8_0_block():
    # src/gguf_loader.rs:1765-1790 of the reference: d = 1.0, qs = 0..31 dequantises to 0..31
    blk = np.zeros(34, np.uint8)
    blk[:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    blk[2:] = np.arange(32, dtype=np.uint8)
    out = oracle.dequant(F.TYPE_Q8_0, blk, 32)
    assert np.array_equal(out, np.arange(32, dtype=np.float32))


def test_q8_1_torch_matches_oracle_bytes():
    torch.manual_seed(8)
    x = torch.randn(4, 256)
    a = F.quantize_q8_1(x).numpy().reshape(4, 8, 36)
    b = oracle.quantize_q8_1(x.numpy()).reshape(4, 8, 36)
    assert np.array_equal(a[..., :2], b[..., :2]) and np.array_equal(a[..., 4:], b[..., 4:])
