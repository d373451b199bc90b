"""Runs the reference's own CUDA kernels (chimere-server/kernels/chimere_kernels.cu, compiled
unchanged for sm_100a into oracle/_ref/chimere_kernels.cubin by oracle/Makefile) through the
CUDA driver API, on torch device buffers.  Used by the GPU tests as the second, stronger oracle:
same GPU, same expf, so routing weights can be compared bit for bit.  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os

import torch

from oracle import REF_CUBIN, REF_FUSED_OPS_CUBIN

_cuda = None
_modules = {}
_funcs = {}


def available() -> bool:
    return os.path.exists(REF_CUBIN) and torch.cuda.is_available()


def fused_ops_available() -> bool:
    return os.path.exists(REF_FUSED_OPS_CUBIN) and torch.cuda.is_available()


def _drv():
    global _cuda
    if _cuda is None:
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # primary context current on this thread
        _cuda = C.CDLL("libcuda.so.1")
    return _cuda


def _module(path: str):
    if path not in _modules:
        drv = _drv()
        mod = C.c_void_p()
        data = open(path, "rb").read()
        rc = drv.cuModuleLoadData(C.byref(mod), data)
        assert rc == 0, f"cuModuleLoadData({os.path.basename(path)}) failed: {rc}"
        _modules[path] = mod
    return _modules[path]


def _func(name: str, cubin: str = REF_CUBIN):
    if (cubin, name) not in _funcs:
        drv = _drv()
        f = C.c_void_p()
        rc = drv.cuModuleGetFunction(C.byref(f), _module(cubin), name.encode())
        assert rc == 0, f"cuModuleGetFunction({name}) failed: {rc}"
        _funcs[(cubin, name)] = f
    return _funcs[(cubin, name)]


def _launch(name, grid, block, smem, args, cubin: str = REF_CUBIN):
    """args: list of ctypes values (c_void_p for pointers, c_int for ints)."""
    drv = _drv()
    f = _func(name, cubin)
    arr = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = drv.cuLaunchKernel(f, grid[0], grid[1], grid[2], block[0], block[1], block[2], smem, stream, arr, None)
    assert rc == 0, f"cuLaunchKernel({name}) failed: {rc}"


def _dp(t: torch.Tensor):
    assert t.is_cuda and t.is_contiguous()
    return C.c_void_p(t.data_ptr())


def f32_gemv(A: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """f32_gemv_kernel (chimere_kernels.cu:706-741), launched as src/kernels/elementwise.rs:599-630 does:
    grid (rows), block 256, dynamic shared = cols * 4."""
    rows, cols = A.shape
    y = torch.empty(rows, dtype=torch.float32, device=A.device)
    _launch("f32_gemv_kernel", (rows, 1, 1), (256, 1, 1), cols * 4, [_dp(A), _dp(x), _dp(y), C.c_int(rows), C.c_int(cols)])
    return y


def topk_softmax(logits: torch.Tensor, k: int):
    """topk_softmax (chimere_kernels.cu:1150-1223), launched as src/kernels/topk_softmax.rs:126-135:
    grid 1, block max(256, next pow2 of E), shared E*4 bytes (at least 32 floats for the warp maxima)."""
    E = logits.numel()
    assert E <= 256
    idx = torch.empty(k, dtype=torch.int32, device=logits.device)
    w = torch.empty(k, dtype=torch.float32, device=logits.device)
    _launch("topk_softmax", (1, 1, 1), (256, 1, 1), max(E, 32) * 4, [_dp(logits), _dp(idx), _dp(w), C.c_int(E), C.c_int(k)])
    return idx, w


def ggml_quantize_q8_1(x: torch.Tensor) -> torch.Tensor:
    """ggml_quantize_q8_1 (chimere_kernels.cu:1495-1523): grid ncols/32, block 32."""
    n = x.numel()
    out = torch.zeros(n // 32 * 36, dtype=torch.uint8, device=x.device)
    _launch("ggml_quantize_q8_1", (n // 32, 1, 1), (32, 1, 1), 0, [_dp(x), _dp(out), C.c_int(n)])
    return out


def gemv_iq3s_q8(weights: torch.Tensor, q8: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """gemv_iq3s_q8 (chimere_kernels.cu:874-925): grid rows, block 128, shared 16 bytes (4 warp sums);
    the f32 `input` argument is unused by the kernel body."""
    y = torch.empty(rows, dtype=torch.float32, device=weights.device)
    dummy = torch.zeros(1, dtype=torch.float32, device=weights.device)
    _launch("gemv_iq3s_q8", (rows, 1, 1), (128, 1, 1), 16, [_dp(weights), _dp(dummy), _dp(y), C.c_int(cols), _dp(q8)])
    return y


def silu_mul_batched(gate: torch.Tensor, up: torch.Tensor, ffn: int, top_k: int) -> torch.Tensor:
    """silu_mul_batched_kernel (chimere_kernels.cu:1533-1547)."""
    out = torch.empty_like(gate)
    _launch("silu_mul_batched_kernel", ((ffn + 255) // 256, top_k, 1), (256, 1, 1), 0,
            [_dp(gate), _dp(up), _dp(out), C.c_int(ffn), C.c_int(top_k)])
    return out


def weighted_combine(outs: torch.Tensor, w: torch.Tensor, H: int, k: int) -> torch.Tensor:
    """weighted_combine_kernel (chimere_kernels.cu:1551-1565)."""
    y = torch.empty(H, dtype=torch.float32, device=outs.device)
    _launch("weighted_combine_kernel", ((H + 255) // 256, 1, 1), (256, 1, 1), 0, [_dp(outs), _dp(w), _dp(y), C.c_int(H), C.c_int(k)])
    return y


def dequant_iq3s(data: torch.Tensor, n_blocks: int) -> torch.Tensor:
    """dequant_iq3s (chimere_kernels.cu:203-290)."""
    out = torch.empty(n_blocks * 256, dtype=torch.float32, device=data.device)
    _launch("dequant_iq3s", ((n_blocks + 255) // 256, 1, 1), (256, 1, 1), 0, [_dp(data), _dp(out), C.c_int(n_blocks)])
    return out


def fused_moe_iq3s(hidden: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor,
                   weights: torch.Tensor, hidden_size: int, expert_ffn: int, bytes_gate: int, bytes_up: int, bytes_down: int) -> torch.Tensor:
    """fused_moe_iq3s (chimere_kernels.cu:1093-1143), the reference's whole-layer kernel for one token: one CTA per
    selected expert dequantises its IQ3_S gate / up / down matrices on the fly (fp32 input, no activation
    quantisation), applies SwiGLU and adds weight * down row sums into `output` with atomicAdd.  Launched as
    src/kernels/fused_moe.rs:379-386 does: grid = top_k, block 256, shared (hidden + 3 * ffn) * 4 bytes; the output
    must start at zero."""
    k = ids.numel()
    out = torch.zeros(hidden_size, dtype=torch.float32, device=hidden.device)
    _launch("fused_moe_iq3s", (k, 1, 1), (256, 1, 1), (hidden_size + 3 * expert_ffn) * 4,
            [_dp(hidden), _dp(gate), _dp(up), _dp(down), _dp(ids), _dp(weights), _dp(out), C.c_int(hidden_size), C.c_int(expert_ffn),
             C.c_int(bytes_gate), C.c_int(bytes_up), C.c_int(bytes_down)])
    return out


def fused_add_residual_rmsnorm(hidden: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """fused_add_residual_rmsnorm (src/kernels/fused_ops.rs:91-140, the source the reference compiles with NVRTC), one row,
    launched as its wrapper does (:667-669): grid 1, block 256, 1 KiB of shared memory.  Updates `residual` in place and
    returns the normalised row."""
    n = hidden.numel()
    normed = torch.empty_like(hidden)
    _launch("fused_add_residual_rmsnorm", (1, 1, 1), (256, 1, 1), 256 * 4,
            [_dp(hidden), _dp(residual), _dp(weight), _dp(normed), C.c_int(n), C.c_float(eps)], cubin=REF_FUSED_OPS_CUBIN)
    return normed
