"""Routing traces in the drafter tooling's wire format.

The reference's target daemon (chimere-dflash/extract/target_daemon.cpp:18-23) captures the "ffn_moe_topk-{L}" tensor of
selected layers during an evaluation and serves it as
    [n_layers: u16 LE][n_tokens: u16 LE][data: uint8[n_layers][n_tokens][8]]
(the payload of its CMD_GET_ROUTING response).  RoutingTrace collects the per-layer byte planes that
chimere_b200_moe_routing_trace writes and produces / parses that payload."""
from __future__ import annotations

import struct
from typing import List

import numpy as np


class RoutingTrace:
    def __init__(self, n_tokens: int, top_k: int = 8):
        self.n_tokens, self.top_k = n_tokens, top_k
        self.layers: List[np.ndarray] = []

    def add_layer(self, ids_u8) -> None:
        """ids_u8: [n_tokens, top_k] uint8 (a torch tensor on any device or an array)."""
        a = ids_u8.cpu().numpy() if hasattr(ids_u8, "cpu") else np.asarray(ids_u8)
        a = np.ascontiguousarray(a, dtype=np.uint8)
        assert a.shape == (self.n_tokens, self.top_k), a.shape
        self.layers.append(a)

    def payload(self) -> bytes:
        """The CMD_GET_ROUTING response payload.  The tooling stores eight ids per token; layers with a smaller top_k are
        padded with zeros on the right."""
        data = np.zeros((len(self.layers), self.n_tokens, 8), np.uint8)
        for i, a in enumerate(self.layers):
            data[i, :, :self.top_k] = a
        return struct.pack("<HH", len(self.layers), self.n_tokens) + data.tobytes()

    @staticmethod
    def parse(payload: bytes) -> np.ndarray:
        """uint8 [n_layers, n_tokens, 8] from a payload."""
        n_layers, n_tokens = struct.unpack_from("<HH", payload, 0)
        data = np.frombuffer(payload, np.uint8, n_layers * n_tokens * 8, 4)
        return data.reshape(n_layers, n_tokens, 8)
