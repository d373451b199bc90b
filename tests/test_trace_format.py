"""The routing-trace wire format (CPU): header, byte order and padding of the payload the drafter tooling expects
(chimere-dflash/extract/target_daemon.cpp:18-23: [n_layers:u16][n_tokens:u16][uint8[n_layers][n_tokens][8]])."""
import struct

import numpy as np

from chimere_b200.trace import RoutingTrace


def test_payload_layout_roundtrip():
    rng = np.random.default_rng(0)
    tr = RoutingTrace(n_tokens=5, top_k=8)
    layers = [rng.integers(0, 256, (5, 8)).astype(np.uint8) for _ in range(3)]
    for a in layers:
        tr.add_layer(a)
    p = tr.payload()
    assert len(p) == 4 + 3 * 5 * 8
    assert struct.unpack_from("<HH", p) == (3, 5)
    assert p[4:4 + 8] == layers[0][0].tobytes()              # layer 0, token 0, slots in order
    assert np.array_equal(RoutingTrace.parse(p), np.stack(layers))


def test_smaller_top_k_is_padded_to_eight_slots():
    tr = RoutingTrace(n_tokens=2, top_k=6)
    tr.add_layer(np.arange(12, dtype=np.uint8).reshape(2, 6))
    d = RoutingTrace.parse(tr.payload())
    assert d.shape == (1, 2, 8)
    assert d[0, 0].tolist() == [0, 1, 2, 3, 4, 5, 0, 0]
