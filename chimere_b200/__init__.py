"""chimere_b200: the quantized MoE feed-forward path of chimere, written for B200 (sm_100a).

The computation lives in libchimere_b200_moe.so (CUDA, built in-tree by chimere_b200.build) and
is reached through the C ABI of include/chimere_b200_moe.h; this package is the thin host side.
"""
from . import abi, formats  # noqa: F401
from .layer import MoeScratch, MoeWeightsPrefill, MoeWeightsRaw, MoeWeightsTiled, forward_moe_prefill, forward_moe, forward_moe_host, route_only  # noqa: F401
