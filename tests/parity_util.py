"""Comparison helpers shared by the GPU parity tests.

Bars (from the benchmark definition): fp32 layer outputs within max relative error 1e-2 and cosine >= 0.9999
per token row; routing indices equal to the oracle's."""
import numpy as np

import oracle
from chimere_b200 import abi

REL_TOL = 1e-2      # max |y - ref| / max |ref| per token row
COS_TOL = 0.9999


def check_rows(y, ref):
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    for t in range(ref.shape[0]):
        scale = np.abs(ref[t]).max()
        rel = np.abs(y[t] - ref[t]).max() / max(scale, 1e-30)
        cos = float(y[t] @ ref[t] / (np.linalg.norm(y[t]) * np.linalg.norm(ref[t]) + 1e-30))
        assert rel <= REL_TOL, (t, rel)
        assert cos >= COS_TOL, (t, cos)


def near_tie_ok(idx_gpu, idx_cpu, logits, route_mode=abi.ROUTE_SOFTMAX_RENORM):
    """Where GPU and CPU routing differ, the probabilities involved must be within a few ulp of one
    another (the host's expf and the GPU's expf differ in the last place)."""
    for t in np.nonzero((idx_gpu != idx_cpu).any(axis=1))[0]:
        k = idx_cpu.shape[1]
        _, _, p = (oracle.topk_softmax(logits[t], k) if route_mode == abi.ROUTE_SOFTMAX_RENORM else oracle.topk_sigmoid(logits[t], k, 1.0))
        a, b = p[idx_gpu[t]], p[idx_cpu[t]]
        ok = np.abs(a - b) <= 4 * np.spacing(np.maximum(a, b))
        if not ok.all():
            return False
    return True


def oracle_on_gpu_routing(wh, x, idx_gpu, taps=True):
    """The oracle's layer output for comparison with the GPU's.  Routing must agree; where the GPU's indices
    differ from the oracle's own they may do so only at an expf near-tie, and the oracle is then run again
    with the GPU's indices forced, so that the rest of the layer is still checked."""
    o = oracle.moe_forward(wh, x, taps=True)
    if not np.array_equal(idx_gpu, o["topk_idx"]):
        assert near_tie_ok(idx_gpu, o["topk_idx"], o["logits"], wh.route_mode), "routing differs from the oracle beyond an expf near-tie"
        o = oracle.moe_forward(wh, x, taps=taps, forced_idx=idx_gpu)
        assert np.array_equal(idx_gpu, o["topk_idx"]) if taps else True
    return o
