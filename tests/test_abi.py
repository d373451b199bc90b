"""The C-ABI library builds, loads, exports every symbol the header declares, and rejects bad
arguments on the host (no GPU needed: argument errors are found before anything is launched)."""
import ctypes as C
import os
import re

import pytest

from chimere_b200 import abi, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "chimere_b200_moe.h")


@pytest.fixture(scope="module")
def lib():
    build.build()
    return abi.load()


def declared_functions():
    txt = open(HEADER).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(chimere_[a-z0-9_]+)\s*\(", txt)))


def test_header_symbols_exported(lib):
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(abi.PROTOTYPES), "ctypes prototypes and header disagree"


def test_constants(lib):
    # ffi/ggml_cuda_gemv.cu:196-209 of the reference
    assert lib.chimere_q8_1_block_bytes() == 36
    assert lib.chimere_q8_1_block_elems() == 32
    assert lib.chimere_matrix_row_padding() == 512
    assert lib.chimere_b200_built_for_sm() == 100


def test_struct_sizes():
    assert C.sizeof(abi.MoeLayer) == 160
    assert C.sizeof(abi.MoeWorkspace) == 8 + 18 * 8


def _layer(**kw):
    s = abi.MoeLayer()
    s.H, s.E, s.F, s.F_s, s.top_k = 2048, 256, 512, 512, 8
    s.route_scale = 1.0
    s.type_gate = s.type_up = s.type_sh_gate = s.type_sh_up = abi.TYPE_IQ3_S
    s.type_down = s.type_sh_down = abi.TYPE_Q4_0
    for f in ("router_w", "gate_exps", "up_exps", "down_exps", "sh_gate", "sh_up", "sh_down"):
        setattr(s, f, 256)  # non-null placeholders: never dereferenced on the host
    for k, v in kw.items():
        setattr(s, k, v)
    return s


def test_workspace_bytes_and_argument_errors(lib):
    good = _layer()
    n = lib.chimere_b200_moe_workspace_bytes(C.byref(good), 8)
    assert n > 72 * 2048 * 4  # at least the pair_out rows of 8 tokens
    assert lib.chimere_b200_moe_workspace_bytes(C.byref(good), 0) == 0
    assert lib.chimere_b200_moe_workspace_bytes(C.byref(_layer(E=257)), 8) == 0
    assert lib.chimere_b200_moe_workspace_bytes(C.byref(_layer(top_k=9)), 8) == 0
    assert lib.chimere_b200_moe_workspace_bytes(C.byref(_layer(H=2080)), 8) == 0      # IQ3_S needs H % 256 == 0
    assert lib.chimere_b200_moe_workspace_bytes(C.byref(_layer(type_up=12)), 8) == 0  # Q4_K is not on this path
    ws = abi.MoeWorkspace()
    assert lib.chimere_b200_moe_workspace_init(C.byref(ws), None, n, C.byref(good), 8, None) == -1
    assert lib.chimere_b200_moe_workspace_init(C.byref(ws), 4096 + 8, n, C.byref(good), 8, None) == -5
    assert lib.chimere_b200_moe_workspace_init(C.byref(ws), 4096, 16, C.byref(good), 8, None) == -4
    # forward with an uninitialised workspace / bad T
    assert lib.chimere_b200_moe_forward(C.byref(good), 256, 256, 1, C.byref(ws), None) == -1
    assert lib.chimere_b200_moe_forward(C.byref(good), None, 256, 1, C.byref(ws), None) == -1
    assert lib.chimere_b200_block_sumi(99, 256, 256, 256, 2048, 1, None) == -3
    assert lib.chimere_b200_block_sumi(abi.TYPE_IQ3_S, 256, 256, 256, 2080, 1, None) == -2


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(abi, "_lib", None)
    monkeypatch.setattr(abi, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        abi.load()
