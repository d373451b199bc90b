"""Pins the CPU oracle on the known-answer values the reference's own tests hold for this path.
Each case names the reference test it comes from (paths relative to chimere-server/)."""
import json
import os

import numpy as np
import pytest

import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def logits_of(probs):
    return np.log(np.asarray(probs, dtype=np.float32))


def test_topk_known_probs():
    # src/moe_forward.rs:321-404 and src/raw_forward.rs:1856-1904: probs [0.05,0.60,0.10,0.25], k=2
    idx, w, p = oracle.topk_softmax(logits_of([0.05, 0.60, 0.10, 0.25]), 2)
    assert idx.tolist() == [1, 3]
    assert abs(float(w.sum()) - 1.0) < 1e-6
    assert abs(float(w[0] / w[1]) - 2.4) < 1e-5
    np.testing.assert_allclose(p, [0.05, 0.60, 0.10, 0.25], rtol=1e-6)


def test_topk_k1_weight_is_one():
    idx, w, _ = oracle.topk_softmax(logits_of([0.05, 0.60, 0.10, 0.25]), 1)
    assert idx.tolist() == [1] and w[0] == 1.0


def test_topk_uniform_ties_go_to_lowest_index():
    # src/raw_forward.rs:1880-1904: four equal probabilities, k=2 -> 0.5 each; strict '>' scan => ids 0,1
    idx, w, p = oracle.topk_softmax(np.zeros(4, np.float32), 2)
    assert idx.tolist() == [0, 1]
    assert w.tolist() == [0.5, 0.5]
    assert p.tolist() == [0.25] * 4


def test_topk_k_equals_E():
    idx, w, _ = oracle.topk_softmax(np.array([0.3, -1.0, 2.0], np.float32), 3)
    assert idx.tolist() == [2, 0, 1] and abs(float(w.sum()) - 1) < 1e-6


def test_softmax_sums_to_one_256():
    # src/raw_forward.rs:1822-1854
    rng = np.random.default_rng(0)
    _, _, p = oracle.topk_softmax(rng.normal(0, 0.9, 256).astype(np.float32), 8)
    assert abs(float(p.astype(np.float64).sum()) - 1.0) < 1e-5


def test_swiglu_values():
    # src/expert.rs:356-411: silu(1) = sigmoid(1) ~ 0.7311, silu(0) = 0
    L = oracle.lib()
    assert abs(L.orc_swiglu(1.0, 1.0) - 0.7310586) < 1e-6
    assert L.orc_swiglu(0.0, 5.0) == 0.0
    assert L.orc_relu2(-3.0) == 0.0 and L.orc_relu2(3.0) == 9.0


def test_q8_1_known_values():
    # ffi/src/lib.rs:965-1044: input 1..32 -> d = 32/127; zeros -> all zero; negatives -> q <= 0
    x = np.arange(1, 33, dtype=np.float32)
    blk = oracle.quantize_q8_1(x)
    d = np.frombuffer(blk[:2].tobytes(), np.float16)[0]
    assert d == np.float16(np.float32(32.0) / np.float32(127.0))
    q = blk[4:].view(np.int8)
    assert q[-1] == 127 and q[0] == 4   # 1 / (32/127) = 3.97 -> 4
    assert np.max(np.abs(q.astype(np.float32) * np.float32(32.0 / 127.0) - x)) < 0.3
    s = np.frombuffer(blk[2:4].tobytes(), np.float16)[0]
    assert s == np.float16(528.0)        # ggml dialect: s = sum of the raw values
    z = oracle.quantize_q8_1(np.zeros(32, np.float32))
    assert not z.any()
    n = oracle.quantize_q8_1(-x)
    assert (n[4:].view(np.int8) <= 0).all()
    # the reference's own dialect (chimere_kernels.cu:754-777) gives the same q bytes here
    own = oracle.quantize_q8_1(x, own_dialect=True)
    assert np.array_equal(own[4:], blk[4:])


def test_q8_1_dialects_agree_on_random_q():
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, 32 * 64).astype(np.float32)
    a = oracle.quantize_q8_1(x).reshape(-1, 36)[:, 4:].view(np.int8)
    b = oracle.quantize_q8_1(x, own_dialect=True).reshape(-1, 36)[:, 4:].view(np.int8)
    # x/d vs x*(1/d) may differ in the last ulp exactly at a rounding boundary: at most a handful of +-1
    assert np.abs(a.astype(int) - b.astype(int)).max() <= 1
    assert (a != b).mean() < 1e-3


def test_dot_and_sigmoid_gate_known_values():
    # src/scratch_pool.rs:412-491: dot(1..2048, ones) = 2 098 176; 1*sigmoid(0)+2 = 2.5; 3*sigmoid(2)+1
    a = np.arange(1, 2049, dtype=np.float32)
    L = oracle.lib()
    assert L.orc_dot_strided256(a.ctypes.data, np.ones(2048, np.float32).ctypes.data, 2048) == 2098176.0
    out = oracle.sigmoid_gate_add(np.array([1.0, 3.0]), 0.0, np.array([2.0, 1.0]))
    assert out[0] == 2.5
    out2 = oracle.sigmoid_gate_add(np.array([3.0]), 2.0, np.array([1.0]))
    assert abs(out2[0] - (3.0 / (1.0 + np.exp(-2.0)) + 1.0)) < 1e-6


def test_weighted_combine_order():
    y = np.array([[1.0, 2.0], [10.0, 20.0]], np.float32)
    out = oracle.weighted_combine(y, np.array([0.25, 0.75], np.float32))
    assert out.tolist() == [7.75, 15.5]


def test_permutation_is_stable_counting_sort():
    idx = np.array([[2, 0], [0, 1], [2, 1]], np.int32)
    perm, offs = oracle.permute(idx, 4)
    assert offs.tolist() == [0, 2, 4, 6, 6]
    assert perm.tolist() == [1, 2, 3, 5, 0, 4]


def test_f16_roundtrip_all_halves():
    L = oracle.lib()
    for h in list(range(0, 0x7C00, 7)) + [0x7BFF, 0x0001, 0x03FF, 0x0400]:
        assert L.orc_f32_to_f16(L.orc_f16_to_f32(h)) == h
    vals = np.random.default_rng(2).normal(0, 1, 2000).astype(np.float32) * np.float32(10.0) ** np.random.default_rng(3).integers(-8, 5, 2000)
    for v in vals:
        assert L.orc_f32_to_f16(float(v)) == int(np.float16(v).view(np.uint16))


def test_iq3s_synthetic_fixture_dot_matches_dequant():
    # Fixture of src/kernels/fused_gate_up.rs:388-411: weight byte i = i % 251, Q8_1 blocks with
    # d bits 0x1000, s = 0, qs[j] = j % 5.  The integer path must equal dequantise-then-dot.
    cols, rows = 2048, 8
    W = (np.arange(rows * cols // 256 * 110) % 251).astype(np.uint8)
    q8 = np.zeros(cols // 32 * 36, np.uint8).reshape(-1, 36)
    q8[:, 1] = 0x10
    q8[:, 4:] = (np.arange(32) % 5).astype(np.uint8)
    y = oracle.gemv(21, W, q8.reshape(-1), cols, rows)
    deq = oracle.dequant(21, W, rows * cols).reshape(rows, cols).astype(np.float64)
    dx = float(np.frombuffer(bytes([0x00, 0x10]), np.float16)[0])
    xv = np.tile(np.arange(32) % 5, cols // 32).astype(np.float64) * dx
    ref = deq @ xv
    finite = np.isfinite(ref)
    assert finite.any()
    np.testing.assert_allclose(y[finite], ref[finite], rtol=2e-5)


def test_committed_golden_vectors():
    """tests/golden/*.json were produced by tests/golden/make_golden.py from this oracle at a pinned
    state; they guard the oracle itself against silent drift."""
    path = os.path.join(GOLDEN, "oracle_small_layer.json")
    if not os.path.exists(path):
        pytest.skip("golden file not generated yet")
    import torch
    from chimere_b200 import configs
    g = json.load(open(path))
    for case in g["cases"]:
        cfg = configs.scaled(getattr(configs, case["config"]), **case["overrides"])
        w = configs.make_layer(cfg)
        x = configs.make_input(cfg, case["T"])
        o = oracle.moe_forward(w, x.numpy())
        assert o["topk_idx"].tolist() == case["topk_idx"]
        np.testing.assert_allclose(o["y"][:, :8], np.array(case["y_head"], np.float32), rtol=1e-5, atol=1e-7)
        assert int(o["x_q8"].astype(np.int64).sum()) == case["x_q8_checksum"]
