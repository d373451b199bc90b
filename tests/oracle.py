"""ctypes loader for the CPU oracle (oracle/libmoe_oracle.so).  Test infrastructure: imported by
tests, the smoke check and the benchmark's CPU-baseline leg only."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB_PATH = os.path.join(ORACLE_DIR, "libmoe_oracle.so")
REF_CUBIN = os.path.join(ORACLE_DIR, "_ref", "chimere_kernels.cubin")
REF_FUSED_OPS_CUBIN = os.path.join(ORACLE_DIR, "_ref", "fused_ops_kernels.cubin")

_lib = None


def build(force: bool = False) -> str:
    """make decides whether the oracle is stale (it depends on the C file, the codebook and the ABI header)."""
    if force and os.path.exists(LIB_PATH):
        os.unlink(LIB_PATH)
    r = subprocess.run(["make", "-C", ORACLE_DIR, "libmoe_oracle.so"], capture_output=True, text=True)
    if r.returncode != 0 and not os.path.exists(LIB_PATH):
        raise RuntimeError("building the CPU oracle failed:\n" + r.stdout + r.stderr)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        L.orc_f32_to_f16.restype, L.orc_f32_to_f16.argtypes = C.c_uint16, [C.c_float]
        L.orc_f16_to_f32.restype, L.orc_f16_to_f32.argtypes = C.c_float, [C.c_uint16]
        L.orc_dot_strided256.restype = C.c_float
        L.orc_dot_strided256.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.orc_swiglu.restype, L.orc_swiglu.argtypes = C.c_float, [C.c_float, C.c_float]
        L.orc_relu2.restype, L.orc_relu2.argtypes = C.c_float, [C.c_float]
        L.orc_row_bytes.restype, L.orc_row_bytes.argtypes = C.c_int64, [C.c_int, C.c_int]
        L.orc_dequant.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        L.orc_moe_forward_ex.restype = C.c_int
        L.orc_moe_forward_ex.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int] + [C.c_void_p] * 7
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def router_logits(W, bias, x):
    W, x = f32(W), f32(x)
    E, H = W.shape
    out = np.empty(E, np.float32)
    b = None if bias is None else f32(bias)
    lib().orc_router_logits(_p(W), _p(b), _p(x), C.c_int(E), C.c_int(H), _p(out))
    return out


def topk_softmax(logits, k):
    logits = f32(logits)
    E = logits.shape[0]
    idx, w, probs = np.empty(k, np.int32), np.empty(k, np.float32), np.empty(E, np.float32)
    lib().orc_topk_softmax(_p(logits), C.c_int(E), C.c_int(k), _p(idx), _p(w), _p(probs))
    return idx, w, probs


def topk_sigmoid(logits, k, scale):
    logits = f32(logits)
    E = logits.shape[0]
    idx, w, probs = np.empty(k, np.int32), np.empty(k, np.float32), np.empty(E, np.float32)
    lib().orc_topk_sigmoid(_p(logits), C.c_int(E), C.c_int(k), C.c_float(scale), _p(idx), _p(w), _p(probs))
    return idx, w, probs


def quantize_q8_1(x, own_dialect=False):
    x = f32(x).reshape(-1)
    out = np.zeros(x.size // 32 * 36, np.uint8)
    fn = lib().orc_quantize_q8_1_own if own_dialect else lib().orc_quantize_q8_1
    fn(_p(x), _p(out), C.c_int(x.size))
    return out


def block_sumi(qtype, W, xq8, ncols, nrows):
    W, xq8 = np.ascontiguousarray(W, np.uint8), np.ascontiguousarray(xq8, np.uint8)
    out = np.empty((nrows, ncols // 32), np.int32)
    lib().orc_block_sumi(C.c_int(qtype), _p(W), _p(xq8), _p(out), C.c_int(ncols), C.c_int(nrows))
    return out


def gemv(qtype, W, xq8, ncols, nrows):
    W, xq8 = np.ascontiguousarray(W, np.uint8), np.ascontiguousarray(xq8, np.uint8)
    out = np.empty(nrows, np.float32)
    lib().orc_gemv(C.c_int(qtype), _p(W), _p(xq8), _p(out), C.c_int(ncols), C.c_int(nrows))
    return out


def dequant(qtype, W, n):
    W = np.ascontiguousarray(W, np.uint8)
    out = np.empty(n, np.float32)
    lib().orc_dequant(C.c_int(qtype), _p(W), _p(out), C.c_int64(n))
    return out


def permute(idx, E):
    idx = np.ascontiguousarray(idx, np.int32)
    T, k = idx.shape
    perm, offs = np.empty(T * k, np.int32), np.empty(E + 1, np.int32)
    lib().orc_permute(_p(idx), C.c_int(T), C.c_int(k), C.c_int(E), _p(perm), _p(offs))
    return perm, offs


def weighted_combine(y, w):
    y, w = f32(y), f32(w)
    k, H = y.shape
    out = np.empty(H, np.float32)
    lib().orc_weighted_combine(_p(y), _p(w), _p(out), C.c_int(H), C.c_int(k))
    return out


def sigmoid_gate_add(sh, logit, routed):
    sh, routed = f32(sh), f32(routed)
    out = np.empty_like(sh)
    lib().orc_sigmoid_gate_add(_p(sh), C.c_float(logit), _p(routed), _p(out), C.c_int(sh.size))
    return out


def rmsnorm(x, eps=1e-6):
    x = f32(x)
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(y), C.c_int(x.shape[0]), C.c_int(x.shape[1]), C.c_float(eps))
    return y


def add_residual_rmsnorm(hidden, residual, weight, eps=1e-6):
    """Returns (updated residual, normed) for rows [T, n]."""
    hidden, weight = f32(hidden), f32(weight)
    res = f32(residual).copy()
    normed = np.empty_like(res)
    lib().orc_add_residual_rmsnorm(_p(hidden), _p(res), _p(weight), _p(normed), C.c_int(res.shape[0]), C.c_int(res.shape[1]), C.c_float(eps))
    return res, normed


def moe_forward(weights, x, taps=True, forced_idx=None):
    """weights: chimere_b200.layer.MoeWeightsRaw on the CPU; x: [T, H] array.  Returns dict.
    forced_idx [T, k] (optional): route with these expert ids instead of the oracle's own top-k."""
    st = weights.as_struct()
    x = f32(x)
    T, H = x.shape
    k, E = weights.top_k, weights.E
    Fmax = max(weights.F, weights.F_s)
    y = np.empty((T, H), np.float32)
    out = {"y": y}
    if taps:
        out.update(topk_idx=np.empty((T, k), np.int32), topk_w=np.empty((T, k), np.float32),
                   logits=np.empty((T, E), np.float32), x_q8=np.empty((T, H // 32 * 36), np.uint8),
                   inter_q8=np.zeros((T, k + 1, Fmax // 32 * 36), np.uint8), sh_logit=np.zeros(T, np.float32))
    forced = None if forced_idx is None else np.ascontiguousarray(forced_idx, np.int32).reshape(T, k)
    rc = lib().orc_moe_forward_ex(C.byref(st), _p(x), _p(y), C.c_int(T), _p(forced),
                                  _p(out.get("topk_idx")), _p(out.get("topk_w")), _p(out.get("logits")),
                                  _p(out.get("x_q8")), _p(out.get("inter_q8")), _p(out.get("sh_logit")))
    assert rc == 0
    return out
