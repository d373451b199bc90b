"""GGUF ingestion for the MoE path: the tensors of one layer as a MoeWeightsRaw.

Host-side mirror of what the reference does when it builds its per-layer weight structs (compute_graph.rs:992-999,
1400-1500 on top of gguf_loader.rs:286-455): find blk.{L}.ffn_gate_inp, ffn_{gate,up,down}_exps, ffn_{gate,up,down}_shexp
and ffn_gate_inp_shexp, check their shapes against each other and upload the bytes as they lie in the file.  The file is
parsed by the C-ABI reader of the library (chimere_b200_gguf_*); nothing here touches the GPU kernels.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from . import abi, formats
from .layer import MoeWeightsRaw

LAYER_TYPES = (formats.TYPE_Q4_0, formats.TYPE_Q8_0, formats.TYPE_IQ3_S)
KQUANT_TYPES = (formats.TYPE_Q4_K, formats.TYPE_Q5_K, formats.TYPE_Q6_K)


class GgufFile:
    """An open GGUF file: tensor directory, integer / string metadata, raw tensor reads."""

    def __init__(self, path: str):
        self._lib = abi.load()
        self._h = C.c_void_p()
        abi.check(self._lib.chimere_b200_gguf_open(str(path).encode(), C.byref(self._h)), f"gguf_open({path})")

    def close(self) -> None:
        if self._h:
            self._lib.chimere_b200_gguf_close(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensor_names(self) -> List[str]:
        n = self._lib.chimere_b200_gguf_n_tensors(self._h)
        buf = C.create_string_buffer(256)
        out = []
        for i in range(n):
            self._lib.chimere_b200_gguf_tensor_name(self._h, i, buf, 256)
            out.append(buf.value.decode())
        return out

    def find(self, name: str) -> Optional[abi.GgufTensor]:
        t = abi.GgufTensor()
        rc = self._lib.chimere_b200_gguf_find(self._h, name.encode(), C.byref(t))
        if rc == -11:
            return None
        abi.check(rc, f"gguf_find({name})")
        return t

    def meta_int(self, key: str) -> Optional[int]:
        v = C.c_uint64()
        rc = self._lib.chimere_b200_gguf_meta_u64(self._h, key.encode(), C.byref(v))
        return None if rc == -11 else (abi.check(rc, key) or v.value)

    def meta_str(self, key: str) -> Optional[str]:
        buf = C.create_string_buffer(512)
        rc = self._lib.chimere_b200_gguf_meta_str(self._h, key.encode(), buf, 512)
        return None if rc < 0 else buf.value.decode()

    def read(self, t: abi.GgufTensor, device="cpu", pin: bool = True) -> torch.Tensor:
        """The tensor's bytes as a uint8 tensor on `device` (through a pinned host buffer when that is a GPU)."""
        dev = torch.device(device)
        host = torch.empty(t.nbytes, dtype=torch.uint8, pin_memory=(pin and dev.type == "cuda"))
        abi.check(self._lib.chimere_b200_gguf_read(self._h, C.byref(t), host.data_ptr(), t.nbytes), "gguf_read")
        return host.to(dev, non_blocking=False) if dev.type == "cuda" else host

    def moe_layer_info(self, layer: int) -> abi.GgufMoeLayer:
        info = abi.GgufMoeLayer()
        abi.check(self._lib.chimere_b200_gguf_moe_layer(self._h, layer, C.byref(info)), f"gguf_moe_layer({layer})")
        return info


def load_moe_layer(g: GgufFile, layer: int, device="cuda", top_k: Optional[int] = None, route_mode: int = abi.ROUTE_SOFTMAX_RENORM,
                   route_scale: float = 1.0, act: Optional[int] = None, with_shared: bool = True) -> MoeWeightsRaw:
    """Layer `layer`'s MoE tensors as raw ggml bytes on `device`.

    top_k defaults to the file's `<arch>.expert_used_count`.  Experts without a gate tensor are taken as ungated
    (squared ReLU) unless `act` says otherwise.  The routed experts must be Q4_0, Q8_0 or IQ3_S; the shared expert
    either one of those or K-quant throughout (the production files keep it in Q5_K: the whole-layer entries then run it
    as plain GEMVs on the raw blocks behind the routed part).  with_shared=False leaves it out.
    """
    info = g.moe_layer_info(layer)
    if top_k is None:
        arch = g.meta_str("general.architecture")
        top_k = g.meta_int(f"{arch}.expert_used_count") if arch else None
        if top_k is None:
            raise ValueError("top_k not given and the file has no <arch>.expert_used_count")
    if info.up_exps.ggml_type not in LAYER_TYPES or info.down_exps.ggml_type not in LAYER_TYPES:
        raise ValueError(f"routed experts of ggml type {info.up_exps.ggml_type}/{info.down_exps.ggml_type} are not on this path")
    dual = bool(info.has_gate)
    kw = {}
    shared = bool(info.has_shared) and with_shared
    if shared:
        sh = (info.sh_up, info.sh_down) + ((info.sh_gate,) if info.has_shared_gate else ())
        if not (all(t.ggml_type in LAYER_TYPES for t in sh) or all(t.ggml_type in KQUANT_TYPES for t in sh)):
            raise ValueError(f"shared expert of ggml types {[t.ggml_type for t in sh]}: neither all Q4_0/Q8_0/IQ3_S nor all K-quant; "
                             "load with with_shared=False")
        kw["shexp_up_raw"] = g.read(info.sh_up, device)
        kw["shexp_down_raw"] = g.read(info.sh_down, device)
        kw["type_sh_up"], kw["type_sh_down"] = info.sh_up.ggml_type, info.sh_down.ggml_type
        if info.has_shared_gate:
            kw["shexp_gate_raw"] = g.read(info.sh_gate, device)
            kw["type_sh_gate"] = info.sh_gate.ggml_type
        if info.has_shared_gate_proj:
            kw["shexp_gate_proj"] = g.read(info.sh_gate_proj, device).view(torch.float32)
    E = info.E
    return MoeWeightsRaw(
        H=info.H, E=E, F=info.F, F_s=info.F_s if shared else 0, top_k=int(top_k),
        type_gate=info.gate_exps.ggml_type if dual else 0, type_up=info.up_exps.ggml_type, type_down=info.down_exps.ggml_type,
        router_weight=g.read(info.router, device).view(torch.float32).view(E, info.H),
        up_exps_raw=g.read(info.up_exps, device).view(E, -1), down_exps_raw=g.read(info.down_exps, device).view(E, -1),
        gate_exps_raw=g.read(info.gate_exps, device).view(E, -1) if dual else None,
        route_mode=route_mode, route_scale=route_scale,
        act=act if act is not None else (abi.ACT_SWIGLU if dual else abi.ACT_RELU2), **kw)
