"""Writes tests/golden/oracle_small_layer.json: routing indices, the head of every output row and a
checksum of the Q8_1 bytes for a few small seeded layers, computed by the CPU oracle
(oracle/moe_oracle.c).  The reference cannot be imported here (Rust + an un-vendored ggml), so these
vectors pin the oracle against silent drift; the known-answer values of the reference's own tests are
checked separately in tests/test_oracle_golden.py.

    python tests/golden/make_golden.py
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import numpy as np  # noqa: E402

import oracle  # noqa: E402
from chimere_b200 import configs  # noqa: E402

CASES = [
    {"config": "QWEN_Q4_0", "overrides": {"E": 16, "H": 256, "F": 64, "F_s": 64}, "T": 5},
    {"config": "QWEN_IQ3S", "overrides": {"E": 16, "H": 256, "F": 64, "F_s": 64}, "T": 3},
    {"config": "QWEN_Q8_0", "overrides": {"E": 16, "H": 256, "F": 64, "F_s": 64}, "T": 4},
    {"config": "NEMOTRON_Q4_0", "overrides": {"E": 8, "H": 256, "F": 64, "F_s": 128}, "T": 2},
]

if __name__ == "__main__":
    out = {"generator": "tests/golden/make_golden.py", "cases": []}
    for case in CASES:
        cfg = configs.scaled(getattr(configs, case["config"]), **case["overrides"])
        w = configs.make_layer(cfg)
        x = configs.make_input(cfg, case["T"])
        o = oracle.moe_forward(w, x.numpy())
        out["cases"].append(dict(case, topk_idx=o["topk_idx"].tolist(), y_head=np.asarray(o["y"][:, :8], np.float64).tolist(),
                                 x_q8_checksum=int(o["x_q8"].astype(np.int64).sum())))
    with open(os.path.join(HERE, "oracle_small_layer.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", len(out["cases"]), "cases")
