"""Host-side mirror of the reference's MoE operator interface, over the C ABI.

  MoeWeightsRaw   <- struct MoeWeightsRaw, chimere-server/src/qwen35_model/compute_graph.rs:1000-1049
                     (router_weight, shexp_gate_proj, {gate,up,down}_exps_raw with per-expert byte
                     strides, shexp_{gate,up,down}_raw)
  MoeScratch      <- GgmlGpuBuffers::with_moe, src/kernels/ggml_gpu.rs:358-406 (scratch allocated once)
  forward_moe     <- forward_moe_cudarc_with_cache, src/qwen35_model/moe_ffn.rs:1081-1768

PyTorch is used only to own device memory and streams; every computation happens inside the
CUDA library.  Tensors may live on the CPU too: the same struct, filled with host pointers, is
what the test-suite hands to its CPU oracle.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional

import torch

from . import abi
from .formats import row_bytes


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


@dataclass
class MoeWeightsRaw:
    """One layer's weights as raw ggml bytes (uint8 tensors) plus the fp32 router tensors."""
    H: int
    E: int
    F: int
    F_s: int
    top_k: int
    type_gate: int
    type_up: int
    type_down: int
    router_weight: torch.Tensor                     # f32 [E, H]
    up_exps_raw: torch.Tensor                       # u8  [E, F * row_bytes(H)]
    down_exps_raw: torch.Tensor                     # u8  [E, H * row_bytes(F)]
    gate_exps_raw: Optional[torch.Tensor] = None    # u8  [E, F * row_bytes(H)]; None for relu^2 experts
    shexp_gate_proj: Optional[torch.Tensor] = None  # f32 [H]
    shexp_gate_raw: Optional[torch.Tensor] = None
    shexp_up_raw: Optional[torch.Tensor] = None
    shexp_down_raw: Optional[torch.Tensor] = None
    router_bias: Optional[torch.Tensor] = None      # f32 [E]
    route_mode: int = abi.ROUTE_SOFTMAX_RENORM
    route_scale: float = 1.0
    act: int = abi.ACT_SWIGLU
    type_sh_gate: int = 0
    type_sh_up: int = 0
    type_sh_down: int = 0
    _struct: Optional[abi.MoeLayer] = field(default=None, repr=False)

    @property
    def expert_bytes_up(self) -> int:
        return self.F * row_bytes(self.type_up, self.H)

    @property
    def expert_bytes_gate(self) -> int:
        return self.F * row_bytes(self.type_gate, self.H)

    @property
    def expert_bytes_down(self) -> int:
        return self.H * row_bytes(self.type_down, self.F)

    def tensors(self):
        return [self.router_weight, self.up_exps_raw, self.down_exps_raw, self.gate_exps_raw, self.shexp_gate_proj,
                self.shexp_gate_raw, self.shexp_up_raw, self.shexp_down_raw, self.router_bias]

    def to(self, device) -> "MoeWeightsRaw":
        kw = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in self.__dict__.items() if k != "_struct"}
        return MoeWeightsRaw(**kw)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors() if t is not None)

    def as_struct(self) -> abi.MoeLayer:
        """struct chimere_moe_layer pointing at this object's tensors (device or host)."""
        if self._struct is None:
            for t in self.tensors():
                assert t is None or t.is_contiguous()
            s = abi.MoeLayer()
            s.H, s.E, s.F, s.F_s, s.top_k = self.H, self.E, self.F, self.F_s, self.top_k
            s.route_mode, s.act, s.route_scale = self.route_mode, self.act, self.route_scale
            s.type_gate, s.type_up, s.type_down = self.type_gate, self.type_up, self.type_down
            s.type_sh_gate, s.type_sh_up, s.type_sh_down = self.type_sh_gate, self.type_sh_up, self.type_sh_down
            s.router_w, s.router_bias, s.shexp_gate_w = _ptr(self.router_weight), _ptr(self.router_bias), _ptr(self.shexp_gate_proj)
            s.gate_exps, s.up_exps, s.down_exps = _ptr(self.gate_exps_raw), _ptr(self.up_exps_raw), _ptr(self.down_exps_raw)
            s.stride_gate = self.expert_bytes_gate if self.gate_exps_raw is not None else 0
            s.stride_up, s.stride_down = self.expert_bytes_up, self.expert_bytes_down
            s.sh_gate, s.sh_up, s.sh_down = _ptr(self.shexp_gate_raw), _ptr(self.shexp_up_raw), _ptr(self.shexp_down_raw)
            self._struct = s
        return self._struct


def formats_kquant_types():
    from . import formats
    return (formats.TYPE_Q4_K, formats.TYPE_Q5_K, formats.TYPE_Q6_K)


class MoeWeightsTiled:
    """The layer after the one-time load-side rewrite into the library's tiled32 layout
    (chimere_b200_moe_pack).  Router tensors are shared with the raw object; the expert matrices live
    in `arena`.  Offers the same attributes and as_struct() as MoeWeightsRaw."""

    def __init__(self, raw: MoeWeightsRaw, keep_raw: bool = True):
        lib = abi.load()
        assert raw.router_weight.is_cuda, "packing runs on the device"
        self.raw = raw
        for a in ("H", "E", "F", "F_s", "top_k", "type_gate", "type_up", "type_down", "route_mode", "route_scale", "act"):
            setattr(self, a, getattr(raw, a))
        rs = raw.as_struct()
        nbytes = lib.chimere_b200_moe_pack_bytes(C.byref(rs))
        if nbytes == 0:
            raise RuntimeError("chimere_b200_moe_pack_bytes rejected the layer description")
        self.arena = torch.empty(nbytes, dtype=torch.uint8, device=raw.router_weight.device)
        self._struct = abi.MoeLayer()
        stream = torch.cuda.current_stream(self.arena.device).cuda_stream
        abi.check(lib.chimere_b200_moe_pack(C.byref(rs), self.arena.data_ptr(), nbytes, C.byref(self._struct), stream),
                  "chimere_b200_moe_pack")
        self._keep = [raw.router_weight, raw.router_bias, raw.shexp_gate_proj]
        if raw.F_s > 0 and raw.type_sh_up in formats_kquant_types():   # a K-quant shared expert stays in its raw blocks
            self._keep += [raw.shexp_gate_raw, raw.shexp_up_raw, raw.shexp_down_raw]
        if not keep_raw:
            torch.cuda.current_stream(self.arena.device).synchronize()
            self.raw = None

    def as_struct(self) -> abi.MoeLayer:
        return self._struct

    def weight_bytes(self) -> int:
        return self.arena.numel() + sum(t.numel() * t.element_size() for t in self._keep if t is not None)


class MoeWeightsPrefill:
    """The GEMM copy of a layer's expert matrices (chimere_b200_moe_pack_prefill): int8 values and f32 block scales in
    the tensor-core operand order.  Built from the raw ggml form; used together with the tiled32 form."""

    def __init__(self, raw: MoeWeightsRaw):
        lib = abi.load()
        rs = raw.as_struct()
        nbytes = lib.chimere_b200_moe_pack_prefill_bytes(C.byref(rs))
        if nbytes == 0:
            raise RuntimeError("chimere_b200_moe_pack_prefill_bytes rejected the layer (needs H % 128 == 0 and, for gated experts, F % 64 == 0)")
        self.arena = torch.zeros(nbytes, dtype=torch.uint8, device=raw.router_weight.device)
        self.struct = abi.PrefillWeights()
        stream = torch.cuda.current_stream(self.arena.device).cuda_stream
        abi.check(lib.chimere_b200_moe_pack_prefill(C.byref(rs), self.arena.data_ptr(), nbytes, C.byref(self.struct), stream),
                  "chimere_b200_moe_pack_prefill")


class MoeScratch:
    """Device scratch for one stream, allocated once (the library itself never allocates)."""

    def __init__(self, w, max_T: int, device="cuda"):
        lib = abi.load()
        self.w, self.max_T, self.device = w, max_T, torch.device(device)
        nbytes = lib.chimere_b200_moe_workspace_bytes(C.byref(w.as_struct()), max_T)
        if nbytes == 0:
            raise RuntimeError("chimere_b200_moe_workspace_bytes rejected the layer description")
        self.arena = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.ws = abi.MoeWorkspace()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        abi.check(lib.chimere_b200_moe_workspace_init(C.byref(self.ws), self.arena.data_ptr(), nbytes,
                                                       C.byref(w.as_struct()), max_T, stream), "workspace_init")
        self.prefill = None
        self.x_dev = torch.empty(max_T, w.H, dtype=torch.float32, device=self.device)
        self.y_dev = torch.empty(max_T, w.H, dtype=torch.float32, device=self.device)

    def enable_prefill(self) -> None:
        """Adds the scratch of the GEMM path (token tiles) to this workspace."""
        lib = abi.load()
        n = lib.chimere_b200_moe_prefill_bytes(C.byref(self.w.as_struct()), self.max_T)
        if n == 0:
            raise RuntimeError("chimere_b200_moe_prefill_bytes rejected the layer")
        self.prefill = torch.zeros(n, dtype=torch.uint8, device=self.device)
        self.ws.prefill_arena, self.ws.prefill_bytes = self.prefill.data_ptr(), n

    # ---- parity taps: views into the arena -------------------------------------------------
    def _view(self, ptr: int, nbytes: int) -> torch.Tensor:
        off = ptr - self.arena.data_ptr()
        return self.arena[off:off + nbytes]

    def topk_indices(self, T: int) -> torch.Tensor:
        return self._view(self.ws.topk_idx, T * self.w.top_k * 4).view(torch.int32).reshape(T, self.w.top_k)

    def topk_weights(self, T: int) -> torch.Tensor:
        return self._view(self.ws.topk_w, T * self.w.top_k * 4).view(torch.float32).reshape(T, self.w.top_k)

    def router_logits(self, T: int) -> torch.Tensor:
        return self._view(self.ws.router_logits, T * self.w.E * 4).view(torch.float32).reshape(T, self.w.E)

    def sh_gate_logit(self, T: int) -> torch.Tensor:
        return self._view(self.ws.sh_gate_logit, T * 4).view(torch.float32)

    def x_q8(self, T: int) -> torch.Tensor:
        rb = self.w.H // 32 * 36
        return self._view(self.ws.x_q8, T * rb).reshape(T, rb)

    def perm(self, T: int) -> torch.Tensor:
        return self._view(self.ws.perm, T * self.w.top_k * 4).view(torch.int32)

    def offsets(self) -> torch.Tensor:
        return self._view(self.ws.offsets, (self.w.E + 1) * 4).view(torch.int32)

    def inter_q8(self, T: int) -> torch.Tensor:
        """[T*k + T, Fmax/32*36]: rows t*k+j = routed slot j of token t, rows T*k+t = shared expert."""
        rb = (max(self.w.F, self.w.F_s) // 32 * 36 + 15) & ~15   # rows start on 16-byte boundaries
        n = T * self.w.top_k + (T if self.w.F_s > 0 else 0)
        return self._view(self.ws.inter_q8, n * rb).reshape(n, rb)

    def status(self) -> int:
        return int(self._view(self.ws.status, 4).view(torch.int32).item())


def forward_moe(w, scratch: MoeScratch, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = MoE(x) for x [T, H] f32 on the device; all launches go to torch's current stream."""
    lib = abi.load()
    T = x.shape[0]
    assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == w.H
    if out is None:
        out = torch.empty_like(x)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    abi.check(lib.chimere_b200_moe_forward(C.byref(w.as_struct()), x.data_ptr(), out.data_ptr(), T,
                                            C.byref(scratch.ws), stream), "chimere_b200_moe_forward")
    return out


def forward_moe_prefill(w, pw: MoeWeightsPrefill, scratch: MoeScratch, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = MoE(x) with the large experts on the tensor-core GEMM (w: tiled32 layer, pw: its GEMM copy)."""
    lib = abi.load()
    if scratch.prefill is None:
        scratch.enable_prefill()
    if out is None:
        out = torch.empty_like(x)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    abi.check(lib.chimere_b200_moe_forward_prefill(C.byref(w.as_struct()), C.byref(pw.struct), x.data_ptr(), out.data_ptr(), x.shape[0],
                                                   C.byref(scratch.ws), stream), "chimere_b200_moe_forward_prefill")
    return out


def forward_moe_host(w, scratch: MoeScratch, x_host: torch.Tensor, y_host: torch.Tensor) -> torch.Tensor:
    """Same with (pinned) host tensors: copy in, layer, copy out, wait -- one C call."""
    lib = abi.load()
    T = x_host.shape[0]
    assert not x_host.is_cuda and not y_host.is_cuda and x_host.is_contiguous() and y_host.is_contiguous()
    stream = torch.cuda.current_stream(scratch.device).cuda_stream
    abi.check(lib.chimere_b200_moe_forward_host(C.byref(w.as_struct()), x_host.data_ptr(), y_host.data_ptr(), T,
                                                 scratch.x_dev.data_ptr(), scratch.y_dev.data_ptr(),
                                                 C.byref(scratch.ws), stream), "chimere_b200_moe_forward_host")
    return y_host


def route_only(w, scratch: MoeScratch, x: torch.Tensor) -> None:
    lib = abi.load()
    stream = torch.cuda.current_stream(x.device).cuda_stream
    abi.check(lib.chimere_b200_moe_route(C.byref(w.as_struct()), x.data_ptr(), x.shape[0], C.byref(scratch.ws), stream),
              "chimere_b200_moe_route")


def forward_moe_residual_norm(w, scratch: MoeScratch, hidden: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                              out: Optional[torch.Tensor] = None, pw: Optional[MoeWeightsPrefill] = None) -> torch.Tensor:
    """residual += hidden; y = MoE(rmsnorm(residual) * norm_weight): the half-layer as the reference's forward runs it
    (fused_add_residual_rmsnorm + forward_moe_cudarc_with_cache, compute_graph.rs:2063-2069).  `residual` is updated in place."""
    lib = abi.load()
    T = hidden.shape[0]
    if out is None:
        out = torch.empty_like(hidden)
    if pw is not None and scratch.prefill is None:
        scratch.enable_prefill()
    stream = torch.cuda.current_stream(hidden.device).cuda_stream
    abi.check(lib.chimere_b200_moe_forward_residual_norm(C.byref(w.as_struct()), C.byref(pw.struct) if pw is not None else None, hidden.data_ptr(),
                                                         residual.data_ptr(), norm_weight.data_ptr(), eps, out.data_ptr(), T,
                                                         C.byref(scratch.ws), stream), "chimere_b200_moe_forward_residual_norm")
    return out


def routing_trace(w, scratch: MoeScratch, T: int, trace: Optional[torch.Tensor] = None, expert_load: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The expert ids of the last routing in `scratch` as uint8 [T, top_k] (the drafter tooling's layout); `expert_load`
    (int32 [E], optional) accumulates the pairs per expert."""
    lib = abi.load()
    if trace is None:
        trace = torch.empty(T, w.top_k, dtype=torch.uint8, device=scratch.device)
    stream = torch.cuda.current_stream(scratch.device).cuda_stream
    abi.check(lib.chimere_b200_moe_routing_trace(C.byref(w.as_struct()), T, C.byref(scratch.ws), trace.data_ptr(),
                                                 None if expert_load is None else expert_load.data_ptr(), stream), "chimere_b200_moe_routing_trace")
    return trace
