"""ctypes view of include/chimere_b200_moe.h: the structs and every exported entry point.

The library is loaded from this package's directory.  There is no fallback: if the shared
object is missing the import of the library handle raises, naming the build command.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libchimere_b200_moe.so")

TYPE_Q4_0, TYPE_Q8_0, TYPE_IQ3_S = 2, 8, 21
ROUTE_SOFTMAX_RENORM, ROUTE_SIGMOID_NORM_SCALE = 0, 1
ACT_SWIGLU, ACT_RELU2 = 0, 1
LAYOUT_GGML, LAYOUT_TILED32 = 0, 1


class MoeLayer(C.Structure):
    """struct chimere_moe_layer"""
    _fields_ = [
        ("H", C.c_int32), ("E", C.c_int32), ("F", C.c_int32), ("F_s", C.c_int32), ("top_k", C.c_int32),
        ("route_mode", C.c_int32), ("act", C.c_int32), ("route_scale", C.c_float),
        ("type_gate", C.c_int32), ("type_up", C.c_int32), ("type_down", C.c_int32),
        ("type_sh_gate", C.c_int32), ("type_sh_up", C.c_int32), ("type_sh_down", C.c_int32),
        ("layout", C.c_int32), ("reserved", C.c_int32),
        ("router_w", C.c_void_p), ("router_bias", C.c_void_p), ("shexp_gate_w", C.c_void_p),
        ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
        ("stride_gate", C.c_int64), ("stride_up", C.c_int64), ("stride_down", C.c_int64),
        ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p),
    ]


class MoeWorkspace(C.Structure):
    """struct chimere_moe_workspace"""
    _fields_ = [
        ("max_T", C.c_int32), ("reserved0", C.c_int32),
        ("topk_idx", C.c_void_p), ("topk_w", C.c_void_p), ("router_logits", C.c_void_p),
        ("sh_gate_logit", C.c_void_p), ("x_q8", C.c_void_p), ("perm", C.c_void_p), ("offsets", C.c_void_p),
        ("group_list", C.c_void_p), ("counters", C.c_void_p), ("inter_q8", C.c_void_p), ("pair_out", C.c_void_p),
        ("x_q", C.c_void_p), ("x_d", C.c_void_p), ("inter_q", C.c_void_p), ("inter_d", C.c_void_p),
        ("prefill_arena", C.c_void_p), ("prefill_bytes", C.c_size_t), ("status", C.c_void_p),
    ]


class PrefillWeights(C.Structure):
    """struct chimere_moe_prefill_weights"""
    _fields_ = [("gu_exps", C.c_void_p), ("stride_gu", C.c_int64), ("down_exps", C.c_void_p), ("stride_down", C.c_int64),
                ("sh_gu", C.c_void_p), ("sh_down", C.c_void_p), ("rows_per_gu_tile", C.c_int32), ("reserved", C.c_int32)]


_P = C.c_void_p
_LAYER_P, _WS_P = C.POINTER(MoeLayer), C.POINTER(MoeWorkspace)

# name -> (restype, argtypes); exactly the declarations of include/chimere_b200_moe.h
class GgufTensor(C.Structure):
    """struct chimere_gguf_tensor"""
    _fields_ = [("ggml_type", C.c_int32), ("n_dims", C.c_int32), ("dims", C.c_int64 * 4), ("file_offset", C.c_int64),
                ("nbytes", C.c_int64)]


class GgufMoeLayer(C.Structure):
    """struct chimere_gguf_moe_layer"""
    _fields_ = [(n, GgufTensor) for n in ("router", "gate_exps", "up_exps", "down_exps", "sh_gate", "sh_up", "sh_down", "sh_gate_proj")] + \
               [(n, C.c_int32) for n in ("has_gate", "has_shared", "has_shared_gate", "has_shared_gate_proj", "H", "E", "F", "F_s")]


PROTOTYPES = {
    "chimere_b200_moe_workspace_bytes": (C.c_size_t, [_LAYER_P, C.c_int]),
    "chimere_b200_moe_workspace_init": (C.c_int, [_WS_P, _P, C.c_size_t, _LAYER_P, C.c_int, _P]),
    "chimere_b200_moe_pack_bytes": (C.c_size_t, [_LAYER_P]),
    "chimere_b200_moe_pack": (C.c_int, [_LAYER_P, _P, C.c_size_t, _LAYER_P, _P]),
    "chimere_b200_packed_matrix_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "chimere_b200_pack_matrix": (C.c_int, [C.c_int, _P, _P, C.c_int, C.c_int, _P]),
    "chimere_b200_block_sumi_tiled": (C.c_int, [C.c_int, _P, _P, _P, C.c_int, C.c_int, _P]),
    "chimere_b200_moe_forward": (C.c_int, [_LAYER_P, _P, _P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_forward_host": (C.c_int, [_LAYER_P, _P, _P, C.c_int, _P, _P, _WS_P, _P]),
    "chimere_b200_moe_route": (C.c_int, [_LAYER_P, _P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_route_noalloc": (C.c_int, [_LAYER_P, _P, C.c_int, _P, _P, _P]),
    "chimere_b200_moe_gate_up": (C.c_int, [_LAYER_P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_down_combine": (C.c_int, [_LAYER_P, _P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_route_home": (C.c_int, [_LAYER_P, _P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_shared_expert": (C.c_int, [_LAYER_P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_experts": (C.c_int, [_LAYER_P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_experts_packed": (C.c_int, [_LAYER_P, C.c_int, _P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_ep_pack": (C.c_int, [_LAYER_P, C.c_int, _WS_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "chimere_b200_moe_ep_finish": (C.c_int, [_LAYER_P, _P, _P, C.c_int, _WS_P, _P, _P]),
    "chimere_b200_moe_ep_pack_p2p": (C.c_int, [_LAYER_P, C.c_int, _WS_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "chimere_b200_moe_ep_wait": (C.c_int, [_P, C.c_int, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_experts_packed_p2p": (C.c_int, [_LAYER_P, C.c_int, _P, C.c_int, _P, C.c_int, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_ep_return_p2p": (C.c_int, [_LAYER_P, _WS_P, _P, C.c_int, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "chimere_b200_moe_ep_finish_p2p": (C.c_int, [_LAYER_P, _P, _P, C.c_int, C.c_int, _WS_P, _P, _P, _P]),
    "chimere_b200_moe_permute": (C.c_int, [_LAYER_P, C.c_int, _WS_P, _P]),
    "chimere_b200_block_sumi": (C.c_int, [C.c_int, _P, _P, _P, C.c_int, C.c_int, _P]),
    "chimere_b200_mma128_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "chimere_b200_pack_mma128": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, _P]),
    "chimere_b200_gemm_i8": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P, _P]),
    "chimere_b200_mma_i8_probe": (C.c_int, [C.c_int, C.c_int, C.c_int, _P, _P]),
    "chimere_b200_moe_pack_prefill_bytes": (C.c_size_t, [_LAYER_P]),
    "chimere_b200_moe_pack_prefill": (C.c_int, [_LAYER_P, _P, C.c_size_t, C.POINTER(PrefillWeights), _P]),
    "chimere_b200_moe_prefill_bytes": (C.c_size_t, [_LAYER_P, C.c_int]),
    "chimere_b200_moe_forward_prefill": (C.c_int, [_LAYER_P, C.POINTER(PrefillWeights), _P, _P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_forward_residual_norm": (C.c_int, [_LAYER_P, C.POINTER(PrefillWeights), _P, _P, _P, C.c_float, _P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_routing_trace": (C.c_int, [_LAYER_P, C.c_int, _WS_P, _P, _P, _P]),
    "chimere_b200_moe_experts_prefill": (C.c_int, [_LAYER_P, C.POINTER(PrefillWeights), C.c_int, _WS_P, _P]),
    "chimere_b200_moe_shared_expert_prefill": (C.c_int, [_LAYER_P, C.POINTER(PrefillWeights), C.c_int, _WS_P, _P]),
    "chimere_b200_moe_experts_packed_prefill": (C.c_int, [_LAYER_P, C.POINTER(PrefillWeights), C.c_int, _P, C.c_int, _WS_P, _P]),
    "chimere_b200_moe_ep_pack_sorted": (C.c_int, [_LAYER_P, C.c_int, _WS_P, _P, _P, C.c_int, C.c_int, _P]),
    "chimere_b200_rmsnorm": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_float, _P]),
    "chimere_b200_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(_P)]),
    "chimere_b200_gguf_close": (None, [_P]),
    "chimere_b200_gguf_n_tensors": (C.c_int64, [_P]),
    "chimere_b200_gguf_tensor_name": (C.c_int, [_P, C.c_int64, C.c_char_p, C.c_int]),
    "chimere_b200_gguf_find": (C.c_int, [_P, C.c_char_p, C.POINTER(GgufTensor)]),
    "chimere_b200_gguf_read": (C.c_int, [_P, C.POINTER(GgufTensor), _P, C.c_int64]),
    "chimere_b200_gguf_meta_u64": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_uint64)]),
    "chimere_b200_gguf_meta_str": (C.c_int, [_P, C.c_char_p, C.c_char_p, C.c_int]),
    "chimere_b200_gguf_moe_layer": (C.c_int, [_P, C.c_int, C.POINTER(GgufMoeLayer)]),
    "chimere_b200_abi_version": (C.c_int, []),
    "chimere_b200_built_for_sm": (C.c_int, []),
    "chimere_quantize_q8_1": (None, [_P, _P, C.c_int64, C.c_int64, _P]),
    "chimere_quantize_q8_1_batched": (None, [_P, _P, C.c_int64, C.c_int64, C.c_int, _P]),
    "chimere_mmvq_iq3s": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "chimere_mmvq_q8_0": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "chimere_mmvq_q4_0": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "chimere_mmvq_iq3s_f32": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P]),
    "chimere_mmvq_q8_0_f32": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P]),
    "chimere_mmvq_q4_0_f32": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P]),
    "chimere_mmvq_q5k": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "chimere_mmvq_q4k": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "chimere_mmvq_q6k": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "chimere_mmvq_q5k_f32": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P]),
    "chimere_mmvq_q4k_f32": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P]),
    "chimere_mmvq_q6k_f32": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P]),
    "chimere_mmvq_iq3s_batched": (None, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int, _P]),
    "chimere_mmvq_q4_0_batched": (None, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int, _P]),
    "chimere_mmvq_q8_0_batched": (None, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int, _P]),
    "chimere_q8_1_block_bytes": (C.c_int, []),
    "chimere_q8_1_block_elems": (C.c_int, []),
    "chimere_matrix_row_padding": (C.c_int, []),
}

_lib = None


def load() -> C.CDLL:
    """The library handle with argument types set.  Raises if the library has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m chimere_b200.build` (needs nvcc); "
                               "there is no CPU or PyTorch fallback for this path")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


ERRORS = {-1: "null pointer", -2: "bad dimension", -3: "unsupported weight type", -4: "workspace too small",
          -5: "misaligned arena", -6: "entry not available", -7: "larger than the built-in scratch",
          -8: "first call on this device was made during stream capture", -9: "file I/O", -10: "not a GGUF v2/v3 file or truncated",
          -11: "no such tensor or key"}


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = ERRORS.get(rc, f"CUDA error {-(rc + 100)}" if rc <= -100 else "error")
        raise RuntimeError(f"{what} failed: {rc} ({msg})")
