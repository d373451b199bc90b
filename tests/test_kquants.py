"""K-quant super-blocks (Q4_K, Q5_K, Q6_K) of the plain GEMV entries: the CPU restatement against an independent
decoder, and the dot-product formula against plain dequantised arithmetic.

The layouts are the ones the reference reads (ffi/src/lib.rs:51-54,368-499 for Q5_K; src/gguf_loader.rs:855-927 for
Q6_K, :1274-1345 for Q4_K).  The independent decoder is the `gguf` Python package's dequantize()."""
import numpy as np
import pytest

import oracle
from chimere_b200 import formats

KTYPES = [formats.TYPE_Q4_K, formats.TYPE_Q5_K, formats.TYPE_Q6_K]


@pytest.mark.parametrize("qtype", KTYPES)
def test_block_sizes(qtype):
    assert formats.row_bytes(qtype, 2048) == 8 * {formats.TYPE_Q4_K: 144, formats.TYPE_Q5_K: 176, formats.TYPE_Q6_K: 210}[qtype]
    assert oracle.lib().orc_row_bytes(qtype, 2048) == formats.row_bytes(qtype, 2048)


@pytest.mark.parametrize("qtype", KTYPES)
def test_oracle_dequant_matches_independent_decoder(qtype):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    W = formats.random_kquant_rows(qtype, 6, 1024, seed=qtype)
    ours = oracle.dequant(qtype, W, 6 * 1024).reshape(6, 1024)
    gtype = {formats.TYPE_Q4_K: gguf.GGMLQuantizationType.Q4_K, formats.TYPE_Q5_K: gguf.GGMLQuantizationType.Q5_K,
             formats.TYPE_Q6_K: gguf.GGMLQuantizationType.Q6_K}[qtype]
    theirs = quants.dequantize(W, gtype)
    assert theirs.shape == (6, 1024)
    # both compute d*sc*q - dmin*m in f32 from the same integers; the products may be associated differently
    np.testing.assert_allclose(ours, theirs, rtol=2e-6, atol=1e-9)
    assert 0.005 < ours.std() < 0.08     # the random blocks look like weights


def _mins(qtype, W, cols):
    """dmin * m_j of every 32-weight sub-block, [rows, cols/32] (zeros for Q6_K); numpy restatement of the six-bit packing."""
    rows = W.shape[0]
    if qtype == formats.TYPE_Q6_K:
        return np.zeros((rows, cols // 32))
    blk = W.reshape(rows, cols // 256, formats.BLOCK_BYTES[qtype])
    dmin = blk[..., 2:4].copy().view(np.float16).astype(np.float64)[..., 0]
    sc = blk[..., 4:16].astype(np.int64)
    m = np.empty(blk.shape[:2] + (8,), np.int64)
    for j in range(8):
        m[..., j] = (sc[..., j + 4] & 63) if j < 4 else ((sc[..., j + 4] >> 4) | ((sc[..., j] >> 6) << 4))
    return (dmin[..., None] * m).reshape(rows, cols // 32)


@pytest.mark.parametrize("qtype", KTYPES)
def test_oracle_dot_is_the_dequantised_dot(qtype):
    """vec_dot semantics (ffi/src/lib.rs:385-499): sum over sub-blocks of d*d8*sc*dot - dmin*m*s8.  With the dequantised
    weights w = d*sc*q - dmin*m and the dequantised input xh = d8*q8 that is w . xh + sum_j dmin*m_j*(sum(xh_j) - s8_j):
    s8 is the f16 sum of the ORIGINAL inputs of the block, not of their quantised values."""
    rows, cols = 40, 2048
    W = formats.random_kquant_rows(qtype, rows, cols, seed=100 + qtype)
    x = np.random.default_rng(5).standard_normal(cols).astype(np.float32)
    xq = oracle.quantize_q8_1(x)
    y = oracle.gemv(qtype, W, xq, cols, rows)
    blocks = xq.reshape(cols // 32, 36)
    ds = blocks[:, 0:4].copy().view(np.float16).astype(np.float64)
    xh = blocks[:, 4:].view(np.int8).astype(np.float64) * ds[:, :1]
    ref = oracle.dequant(qtype, W, rows * cols).reshape(rows, cols).astype(np.float64) @ xh.reshape(cols)
    ref += _mins(qtype, W, cols) @ (xh.sum(1) - ds[:, 1])
    np.testing.assert_allclose(y, ref, rtol=0, atol=3e-5 * np.abs(ref).max())


# ---- the reference's own Q5_K checks (ffi/src/lib.rs:1050-1270), on blocks built the way its test helper builds them:
# every six-bit scale 1, every min 0, dmin 0, d = amax / 31, quants round(|v| / d) ----
def _ramp_block_q5k(values):
    values = np.asarray(values, np.float32)
    assert values.size == 256
    blk = np.zeros(176, np.uint8)
    amax = float(np.abs(values).max())
    d = amax / 31.0 if amax > 0 else 0.0
    blk[0:2] = np.array([d], np.float16).view(np.uint8)
    blk[4:8] = 1            # scales of sub-blocks 0..3
    blk[12:16] = 1          # low nibbles: scales of sub-blocks 4..7 (mins stay 0)
    q = np.clip(np.round(np.abs(values) / d), 0, 31).astype(np.uint8) if d > 0 else np.zeros(256, np.uint8)
    for j in range(8):
        sub = q[32 * j:32 * j + 32]
        qs = blk[48 + 32 * (j // 2):48 + 32 * (j // 2) + 32]
        qs |= ((sub & 15) << 4) if (j & 1) else (sub & 15)
        blk[16:48] |= ((sub >> 4) & 1) << j
    return blk


def test_q5k_dot_against_dequantised_dot_as_the_reference_tests_it():
    w = _ramp_block_q5k(np.arange(256) * 0.1)
    x = (1.0 - np.arange(256) * 0.005).astype(np.float32)
    y = oracle.gemv(formats.TYPE_Q5_K, w[None, :], oracle.quantize_q8_1(x), 256, 1)[0]
    ref = float(oracle.dequant(formats.TYPE_Q5_K, w, 256).astype(np.float64) @ x.astype(np.float64))
    assert abs(y - ref) / abs(ref) < 0.01          # the reference's bound (lib.rs:1195-1198)
    # and the decoder returns the ramp up to half a quantisation step
    np.testing.assert_allclose(oracle.dequant(formats.TYPE_Q5_K, w, 256), np.arange(256) * 0.1, atol=0.5 * 25.5 / 31 + 0.02)   # half a step + the f16 rounding of d


def test_q5k_zero_input_gives_zero():
    w = _ramp_block_q5k(np.ones(256))
    y = oracle.gemv(formats.TYPE_Q5_K, w[None, :], oracle.quantize_q8_1(np.zeros(256, np.float32)), 256, 1)[0]
    assert abs(y) < 1e-6                            # lib.rs:1211-1214


def test_q5k_matmul_rows_as_the_reference_tests_them():
    rows = np.stack([_ramp_block_q5k((r + 1) * np.arange(256) * 0.01) for r in range(4)])
    x = (1.0 / (1.0 + np.arange(256))).astype(np.float32)
    y = oracle.gemv(formats.TYPE_Q5_K, rows, oracle.quantize_q8_1(x), 256, 4)
    for r in range(4):
        ref = float(oracle.dequant(formats.TYPE_Q5_K, rows[r], 256).astype(np.float64) @ x.astype(np.float64))
        assert abs(y[r] - ref) / abs(ref) < 0.02    # lib.rs:1262-1266
