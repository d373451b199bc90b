"""ggml block formats on the MoE path: sizes, quantizers and a dequantizer, written with torch
ops so the same code builds small CPU fixtures for the tests and full-size layers on the GPU
for the benchmark.

Formats (sizes as in chimere-server/src/gguf_loader.rs:161-193 of the reference):
  Q4_0   18 B / 32 weights : f16 d, 16 bytes; low nibbles = elements 0..15, high = 16..31,
                              value = (nibble - 8) * d            (gguf_loader.rs:752-772)
  Q8_0   34 B / 32 weights : f16 d, 32 int8, value = q * d         (gguf_loader.rs:793-837)
  IQ3_S 110 B / 256 weights: f16 d, qs[64], qh[8], signs[32], scales[4]; value =
                              d * (1 + 2*scale4) * (+-grid byte)   (gguf_loader.rs:1022-1170)
  Q8_1   36 B / 32 values  : f16 d, f16 s, 32 int8 (activations; chimere_kernels.cu:1495-1523)

The Q4_0 and Q8_0 quantizers follow ggml's reference rounding (tests compare their bytes with
gguf.quants).  Neither the reference nor the gguf package has an IQ3_S *encoder*; the one here
is our own (nearest codebook entry per 4 weights through a 4096-entry table) -- any valid
encoding serves, because parity means identical bytes.
"""
from __future__ import annotations

import os
import re

import numpy as np
import torch

TYPE_Q4_0, TYPE_Q8_0, TYPE_IQ3_S = 2, 8, 21
# K-quant super-blocks: only the plain GEMV entries (chimere_mmvq_q4k / _q5k / _q6k) take them
TYPE_Q4_K, TYPE_Q5_K, TYPE_Q6_K = 12, 13, 14
TYPE_NAMES = {TYPE_Q4_0: "Q4_0", TYPE_Q8_0: "Q8_0", TYPE_IQ3_S: "IQ3_S", TYPE_Q4_K: "Q4_K", TYPE_Q5_K: "Q5_K", TYPE_Q6_K: "Q6_K"}
BLOCK_ELEMS = {TYPE_Q4_0: 32, TYPE_Q8_0: 32, TYPE_IQ3_S: 256, TYPE_Q4_K: 256, TYPE_Q5_K: 256, TYPE_Q6_K: 256}
BLOCK_BYTES = {TYPE_Q4_0: 18, TYPE_Q8_0: 34, TYPE_IQ3_S: 110, TYPE_Q4_K: 144, TYPE_Q5_K: 176, TYPE_Q6_K: 210}
Q8_1_BYTES = 36


def random_kquant_rows(qtype: int, rows: int, cols: int, seed: int = 0, scale: float = 0.02) -> np.ndarray:
    """Seeded rows of valid K-quant super-blocks with the quants, high bits and scales drawn at random and f16 super-block
    scales sized so that the weights come out zero-mean with a standard deviation near `scale`.  Stands in
    for a quantizer: the GEMV entries decode blocks, they never make them.  Returns u8 [rows, row_bytes]."""
    assert qtype in (TYPE_Q4_K, TYPE_Q5_K, TYPE_Q6_K) and cols % 256 == 0
    rng = np.random.default_rng(seed)
    nb, bb = rows * (cols // 256), BLOCK_BYTES[qtype]
    blk = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)
    if qtype == TYPE_Q6_K:       # weight = d * sc * q, sc int8, q in -32..31
        d = (scale / (64.0 * 18.0)) * rng.uniform(0.5, 1.5, nb)
        blk[:, 208:210] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
    else:
        # weight = d * sc_j * q - dmin * m_j with six-bit sc_j, m_j and q in 0..15 (Q4_K) or 0..31 (Q5_K).  m_j = sc_j and
        # dmin = d * qmax / 2 centre every sub-block on zero, as a quantizer's blocks of zero-mean weights are.
        qmax = 15.0 if qtype == TYPE_Q4_K else 31.0
        sc = rng.integers(1, 64, size=(nb, 8), dtype=np.uint8)
        packed = np.empty((nb, 12), np.uint8)
        packed[:, 0:4] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)          # scales of sub-blocks 0..3, top bits of 4..7
        packed[:, 4:8] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)          # mins: the same values
        packed[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((sc[:, 4:8] & 0x0F) << 4)
        blk[:, 4:16] = packed
        d = (scale / (32.0 * qmax * 0.29)) * rng.uniform(0.5, 1.5, nb)
        dmin = d * qmax * 0.5 * rng.uniform(0.9, 1.1, nb)
        blk[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
        blk[:, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(nb, 2)
    return blk.reshape(rows, cols // 256 * bb)


def row_bytes(qtype: int, ncols: int) -> int:
    assert ncols % BLOCK_ELEMS[qtype] == 0, (qtype, ncols)
    return ncols // BLOCK_ELEMS[qtype] * BLOCK_BYTES[qtype]


def _grid_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "iq3s_grid.inc")


_GRID = None
_NEAREST = None


def iq3s_grid() -> np.ndarray:
    """The 512-entry codebook as uint8 [512, 4], parsed from the generated include file."""
    global _GRID
    if _GRID is None:
        txt = open(_grid_path()).read()
        vals = [int(v, 16) for v in re.findall(r"0x([0-9a-fA-F]{8})u", txt)]
        assert len(vals) == 512
        u = np.array(vals, dtype=np.uint32)
        _GRID = np.stack([(u >> (8 * i)) & 0xFF for i in range(4)], axis=1).astype(np.uint8)
    return _GRID


def _nearest_table() -> np.ndarray:
    """For each of the 8^4 level combinations (l0 | l1<<3 | l2<<6 | l3<<9, level l = magnitude
    2l+1) the index of the nearest codebook entry."""
    global _NEAREST
    if _NEAREST is None:
        g = iq3s_grid().astype(np.float32)
        key = np.arange(4096)
        lat = np.stack([2 * ((key >> (3 * i)) & 7) + 1 for i in range(4)], axis=1).astype(np.float32)
        d2 = ((lat[:, None, :] - g[None, :, :]) ** 2).sum(-1)
        _NEAREST = d2.argmin(1).astype(np.int16)
    return _NEAREST


def _f16_bytes(d: torch.Tensor) -> torch.Tensor:
    """fp32 tensor [...] -> its f16 (round-to-nearest-even) little-endian bytes [..., 2]."""
    return d.to(torch.float16).contiguous().view(torch.uint8).reshape(*d.shape, 2)


def quantize_q4_0(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] fp32 -> uint8 [rows, cols/32*18].  ggml quantize_row_q4_0_ref: the element of
    largest magnitude maps to -8: d = max/-8, q = min(15, trunc(x/d + 8.5))."""
    rows, cols = w.shape
    x = w.reshape(rows, cols // 32, 32).float()
    ix = x.abs().argmax(dim=-1, keepdim=True)
    mx = torch.gather(x, -1, ix)
    d = mx / -8.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = torch.clamp((x * inv + 8.5).to(torch.int32), max=15).to(torch.uint8)
    packed = q[..., :16] | (q[..., 16:] << 4)
    out = torch.cat([_f16_bytes(d.squeeze(-1)), packed], dim=-1)
    return out.reshape(rows, cols // 32 * 18).contiguous()


def _roundf(x: torch.Tensor) -> torch.Tensor:
    """C roundf: halves away from zero (torch.round is half-to-even)."""
    return torch.sign(x) * torch.floor(x.abs() + 0.5)


def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] fp32 -> uint8 [rows, cols/32*34].  ggml quantize_row_q8_0_ref:
    d = amax/127, q = roundf(x * (1/d))."""
    rows, cols = w.shape
    x = w.reshape(rows, cols // 32, 32).float()
    d = x.abs().amax(dim=-1, keepdim=True) / 127.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = _roundf(x * inv).to(torch.int8).view(torch.uint8)
    out = torch.cat([_f16_bytes(d.squeeze(-1)), q], dim=-1)
    return out.reshape(rows, cols // 32 * 34).contiguous()


def quantize_iq3_s(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] fp32 (cols % 256 == 0) -> uint8 [rows, cols/256*110].  Our own encoder:
    per 32-weight sub-block the target step is amax/15; the super-block scale d = max step / 31
    (stored f16), sub-block scale nibble sc = round((step/d - 1)/2) in 0..15; each weight's level is
    round((|w|/(d*(1+2sc)) - 1)/2) in 0..7; each group of 4 levels goes to the nearest codebook
    entry; signs are stored verbatim."""
    rows, cols = w.shape
    dev = w.device
    nsb = cols // 256
    x = w.reshape(rows, nsb, 8, 32).float()
    step = x.abs().amax(dim=-1) / 15.0                                  # [rows, nsb, 8]
    d = (step.amax(dim=-1) / 31.0).to(torch.float16).float()            # [rows, nsb], as stored
    dsafe = torch.where(d > 0, d, torch.ones_like(d))
    sc = torch.clamp(torch.round((step / dsafe[..., None] - 1.0) / 2.0), 0, 15)
    db = dsafe[..., None] * (1.0 + 2.0 * sc)                            # [rows, nsb, 8]
    lvl = torch.clamp(torch.round((x.abs() / db[..., None] - 1.0) / 2.0), 0, 7).to(torch.int64)
    lv = lvl.reshape(rows, nsb, 8, 8, 4)
    key = lv[..., 0] | (lv[..., 1] << 3) | (lv[..., 2] << 6) | (lv[..., 3] << 9)
    nearest = torch.from_numpy(_nearest_table().astype(np.int64)).to(dev)
    gi = nearest[key]                                                    # [rows, nsb, 8 sub, 8 grp] 0..511
    qs = (gi & 0xFF).to(torch.uint8).reshape(rows, nsb, 64)
    bit = torch.arange(8, device=dev, dtype=torch.int64)
    qh = (((gi >> 8) & 1) << bit).sum(dim=-1).to(torch.uint8)           # [rows, nsb, 8]
    neg = (x < 0).to(torch.int64).reshape(rows, nsb, 8, 4, 8)           # sign byte g2 of sub-block: 8 weights
    signs = (neg << bit).sum(dim=-1).to(torch.uint8).reshape(rows, nsb, 32)
    sci = sc.to(torch.int64)
    scales = (sci[..., 0::2] | (sci[..., 1::2] << 4)).to(torch.uint8)   # [rows, nsb, 4]
    out = torch.cat([_f16_bytes(d), qs, qh, signs, scales], dim=-1)
    return out.reshape(rows, nsb * 110).contiguous()


QUANTIZERS = {TYPE_Q4_0: quantize_q4_0, TYPE_Q8_0: quantize_q8_0, TYPE_IQ3_S: quantize_iq3_s}


def quantize(qtype: int, w: torch.Tensor) -> torch.Tensor:
    return QUANTIZERS[qtype](w)


def dequantize(qtype: int, data: torch.Tensor, cols: int) -> torch.Tensor:
    """uint8 [rows, row_bytes] -> fp32 [rows, cols] (the reference's dequantisation rules)."""
    rows = data.shape[0]
    dev = data.device
    if qtype == TYPE_Q4_0:
        b = data.reshape(rows, cols // 32, 18)
        d = b[..., :2].contiguous().view(torch.float16).float()
        q = b[..., 2:]
        lo = (q & 0x0F).to(torch.float32) - 8.0
        hi = (q >> 4).to(torch.float32) - 8.0
        return (torch.cat([lo, hi], dim=-1) * d).reshape(rows, cols)
    if qtype == TYPE_Q8_0:
        b = data.reshape(rows, cols // 32, 34)
        d = b[..., :2].contiguous().view(torch.float16).float()
        return (b[..., 2:].contiguous().view(torch.int8).float() * d).reshape(rows, cols)
    b = data.reshape(rows, cols // 256, 110)
    d = b[..., :2].contiguous().view(torch.float16).float()            # [rows, nsb, 1]
    qs = b[..., 2:66].to(torch.int64).reshape(rows, -1, 8, 8)
    qh = b[..., 66:74].to(torch.int64)
    bit = torch.arange(8, device=dev, dtype=torch.int64)
    gi = qs | (((qh[..., None] >> bit) & 1) << 8)
    grid = torch.from_numpy(iq3s_grid().astype(np.float32)).to(dev)
    mag = grid[gi]                                                       # [rows, nsb, 8, 8, 4]
    sg = b[..., 74:106].to(torch.int64).reshape(rows, -1, 8, 4)
    neg = ((sg[..., None] >> bit) & 1).reshape(rows, -1, 8, 8, 4)
    sc = b[..., 106:110].to(torch.int64)
    nib = torch.stack([sc & 0x0F, sc >> 4], dim=-1).reshape(rows, -1, 8).float()
    db = d * (1.0 + 2.0 * nib)                                           # [rows, nsb, 8]
    val = torch.where(neg == 1, -mag, mag) * db[..., None, None]
    return val.reshape(rows, cols)


def quantize_q8_1(x: torch.Tensor) -> torch.Tensor:
    """fp32 [rows, n] -> uint8 [rows, n/32*36], ggml-compatible dialect (d = amax/127,
    q = roundf(x/d), s = sum of the raw values; chimere_kernels.cu:1495-1523).  The s field is
    summed in torch's order, so only d and q are meant to be compared bit for bit."""
    rows, n = x.shape
    xb = x.reshape(rows, n // 32, 32).float()
    amax = xb.abs().amax(dim=-1, keepdim=True)
    d = amax / 127.0
    q = torch.where(amax == 0, torch.zeros_like(xb), _roundf(xb / torch.where(d == 0, torch.ones_like(d), d)))
    q = q.to(torch.int8).view(torch.uint8)
    out = torch.cat([_f16_bytes(d.squeeze(-1)), _f16_bytes(xb.sum(-1)), q], dim=-1)
    return out.reshape(rows, n // 32 * 36).contiguous()
