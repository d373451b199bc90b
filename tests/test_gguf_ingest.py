"""GGUF ingestion of the MoE tensors: a file written with the `gguf` package's writer is read back through the library's
C-ABI reader and must give the layer's bytes unchanged (gguf_loader.rs:286-455, compute_graph.rs:992-999, 1400-1500)."""
import numpy as np
import pytest
import torch

from chimere_b200 import abi, configs, formats
from chimere_b200.gguf_io import GgufFile, load_moe_layer

gguf = pytest.importorskip("gguf")


def _write(path, layers, arch="qwen35moe", extra_first=True):
    """layers: {index: MoeWeightsRaw (host)}; tensors in GGUF order (innermost dimension first on disk)."""
    w = gguf.GGUFWriter(str(path), arch)
    first = next(iter(layers.values()))
    w.add_uint32(f"{arch}.expert_count", first.E)
    w.add_uint32(f"{arch}.expert_used_count", first.top_k)
    w.add_uint32(f"{arch}.expert_feed_forward_length", first.F)
    w.add_string("general.name", "synthetic layer for the ingestion test")
    w.add_array("tokenizer.dummy", ["a", "bb", "ccc"])          # arrays and strings must be skipped correctly
    w.add_array("some.ints", [1, 2, 3, 4, 5])
    if extra_first:
        w.add_tensor("token_embd.weight", np.arange(24, dtype=np.float32).reshape(3, 8))
    qt = {formats.TYPE_Q4_0: gguf.GGMLQuantizationType.Q4_0, formats.TYPE_Q8_0: gguf.GGMLQuantizationType.Q8_0,
          formats.TYPE_IQ3_S: gguf.GGMLQuantizationType.IQ3_S, formats.TYPE_Q5_K: gguf.GGMLQuantizationType.Q5_K}

    def quant(name, raw, qtype, shape_elems):
        # raw_shape is the byte shape: innermost = bytes of one row
        rows = int(np.prod(shape_elems[:-1]))
        arr = raw.numpy().reshape(*shape_elems[:-1], -1)
        assert arr.shape[-1] == formats.row_bytes(qtype, shape_elems[-1]) and arr.size // arr.shape[-1] == rows
        w.add_tensor(name, arr, raw_dtype=qt[qtype])

    for il, L in layers.items():
        p = f"blk.{il}."
        w.add_tensor(p + "ffn_gate_inp.weight", L.router_weight.numpy())
        if L.gate_exps_raw is not None:
            quant(p + "ffn_gate_exps.weight", L.gate_exps_raw, L.type_gate, (L.E, L.F, L.H))
        quant(p + "ffn_up_exps.weight", L.up_exps_raw, L.type_up, (L.E, L.F, L.H))
        quant(p + "ffn_down_exps.weight", L.down_exps_raw, L.type_down, (L.E, L.H, L.F))
        if L.F_s:
            if L.shexp_gate_raw is not None:
                quant(p + "ffn_gate_shexp.weight", L.shexp_gate_raw, L.type_sh_gate, (L.F_s, L.H))
            quant(p + "ffn_up_shexp.weight", L.shexp_up_raw, L.type_sh_up, (L.F_s, L.H))
            quant(p + "ffn_down_shexp.weight", L.shexp_down_raw, L.type_sh_down, (L.H, L.F_s))
            if L.shexp_gate_proj is not None:
                w.add_tensor(p + "ffn_gate_inp_shexp.weight", L.shexp_gate_proj.numpy())
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def _same(a, b):
    assert (a is None) == (b is None)
    if a is not None:
        assert a.dtype == b.dtype and torch.equal(a.reshape(-1), b.reshape(-1))


@pytest.mark.parametrize("cfg", [configs.scaled(configs.QWEN_IQ3S, E=8, F=256, F_s=256, H=512),
                                 configs.scaled(configs.NEMOTRON_Q4_0, E=6, F=64, F_s=128, H=256),
                                 configs.scaled(configs.QWEN_Q8_0, E=4, F=64, F_s=0, H=128, zipf_bias=False)])
def test_round_trip_through_a_gguf_file(tmp_path, cfg):
    layers = {0: configs.make_layer(cfg, seed=11), 3: configs.make_layer(cfg, seed=12)}
    path = tmp_path / "layer.gguf"
    _write(path, layers)
    with GgufFile(path) as g:
        names = g.tensor_names()
        assert "token_embd.weight" in names and "blk.3.ffn_up_exps.weight" in names
        assert g.meta_int("qwen35moe.expert_count") == cfg.E and g.meta_str("general.architecture") == "qwen35moe"
        assert g.meta_int("no.such.key") is None and g.find("blk.9.ffn_up_exps.weight") is None
        emb = g.read(g.find("token_embd.weight")).view(torch.float32)
        assert torch.equal(emb, torch.arange(24, dtype=torch.float32))
        for il, want in layers.items():
            got = load_moe_layer(g, il, device="cpu", route_mode=cfg.route_mode, route_scale=cfg.route_scale)
            assert (got.H, got.E, got.F, got.F_s, got.top_k) == (cfg.H, cfg.E, cfg.F, cfg.F_s, cfg.top_k)
            assert (got.type_gate, got.type_up, got.type_down, got.act) == (want.type_gate, want.type_up, want.type_down, want.act)
            for name in ("router_weight", "gate_exps_raw", "up_exps_raw", "down_exps_raw", "shexp_gate_raw", "shexp_up_raw",
                         "shexp_down_raw", "shexp_gate_proj"):
                _same(getattr(got, name), getattr(want, name))
        with pytest.raises(RuntimeError):
            g.moe_layer_info(1)          # no such layer


def test_kquant_shared_expert_loads_as_raw_blocks(tmp_path):
    cfg = configs.scaled(configs.QWEN_Q4_0, E=4, F=256, F_s=256, H=256)
    L = configs.make_layer(cfg, seed=5)
    for name, rows, cols in (("shexp_gate_raw", cfg.F_s, cfg.H), ("shexp_up_raw", cfg.F_s, cfg.H), ("shexp_down_raw", cfg.H, cfg.F_s)):
        setattr(L, name, torch.from_numpy(formats.random_kquant_rows(formats.TYPE_Q5_K, rows, cols, seed=rows)).reshape(-1))
    L.type_sh_gate = L.type_sh_up = L.type_sh_down = formats.TYPE_Q5_K
    path = tmp_path / "q5k.gguf"
    _write(path, {0: L})
    with GgufFile(path) as g:
        info = g.moe_layer_info(0)
        assert info.sh_up.ggml_type == formats.TYPE_Q5_K and info.sh_up.nbytes == cfg.F_s * formats.row_bytes(formats.TYPE_Q5_K, cfg.H)
        full = load_moe_layer(g, 0, device="cpu")
        assert full.F_s == cfg.F_s and full.type_sh_up == formats.TYPE_Q5_K and torch.equal(full.shexp_up_raw, L.shexp_up_raw)
        routed = load_moe_layer(g, 0, device="cpu", with_shared=False)
        assert routed.F_s == 0 and torch.equal(routed.up_exps_raw.reshape(-1), L.up_exps_raw.reshape(-1))
        assert torch.equal(g.read(info.sh_down), L.shexp_down_raw)


def test_malformed_files_are_refused(tmp_path):
    lib = abi.load()
    import ctypes as C
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    h = C.c_void_p()
    assert lib.chimere_b200_gguf_open(str(bad).encode(), C.byref(h)) == -10
    assert lib.chimere_b200_gguf_open(str(tmp_path / "missing.gguf").encode(), C.byref(h)) == -9
    cfg = configs.scaled(configs.QWEN_Q8_0, E=4, F=64, F_s=0, H=128, zipf_bias=False)
    good = tmp_path / "good.gguf"
    _write(good, {0: configs.make_layer(cfg, seed=1)})
    data = good.read_bytes()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(data[: len(data) - 1000])        # tensor data truncated
    assert lib.chimere_b200_gguf_open(str(cut).encode(), C.byref(h)) == -10
    cut.write_bytes(data[:60])                       # header truncated
    assert lib.chimere_b200_gguf_open(str(cut).encode(), C.byref(h)) == -10
