"""GPU parity: the CUDA library, called through its C ABI, against the CPU oracle and against
the reference's own kernels (oracle/_ref cubin) on identical inputs.

Bars (from the benchmark definition): routing indices, dispatch permutation, Q8_1 bytes and
per-block integer dots bit-exact; fp32 layer outputs within max relative error 1e-2 and
cosine >= 0.9999 per token row."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import refkernels
from chimere_b200 import abi, configs, formats
from chimere_b200.layer import MoeScratch, MoeWeightsTiled, forward_moe, forward_moe_host, route_only
from parity_util import COS_TOL, check_rows, near_tie_ok, oracle_on_gpu_routing  # noqa: F401

pytestmark = pytest.mark.gpu

_layers = {}


def layer_pair(cfg, layout="ggml"):
    """(device weights, host copy) of a configuration, generated once per session on the GPU;
    layout "tiled" returns the packed form of the same weights."""
    if cfg not in _layers:
        wd = configs.make_layer(cfg, device="cuda")
        _layers[cfg] = (wd, wd.to("cpu"))
    wd, wh = _layers[cfg]
    if layout == "tiled":
        key = (cfg, "tiled")
        if key not in _layers:
            _layers[key] = MoeWeightsTiled(wd)
        return _layers[key], wh
    return wd, wh


LAYOUTS = ["ggml", "tiled"]


SMALL = [
    configs.scaled(configs.QWEN_Q4_0, E=32),
    configs.scaled(configs.QWEN_IQ3S, E=32),
    configs.scaled(configs.QWEN_Q8_0, E=32),
    configs.scaled(configs.NEMOTRON_Q4_0, E=16),
    configs.scaled(configs.QWEN_IQ3S, E=8, H=256, F=64, F_s=64, top_k=2, name="tiny"),
    # the shared expert quantized differently from the routed ones (as the production files do): every stage then
    # runs two kernel instances, one per weight type
    configs.scaled(configs.QWEN_IQ3S, E=16, type_sh_gate_up=configs.Q8_0, type_sh_down=configs.Q8_0, name="iq3s+q4_0, shared q8_0"),
    configs.scaled(configs.QWEN_Q4_0, E=16, F_s=1024, type_sh_gate_up=configs.IQ3_S, type_sh_down=configs.Q8_0, name="q4_0, shared iq3s/q8_0"),
]


@pytest.mark.parametrize("cfg", SMALL, ids=lambda c: c.name)
@pytest.mark.parametrize("T", [1, 3, 8, 9, 40])
@pytest.mark.parametrize("layout", LAYOUTS)
def test_forward_small(cfg, T, layout):
    wd, wh = layer_pair(cfg, layout)
    x = configs.make_input(cfg, T, device="cuda")
    sc = MoeScratch(wd, T)
    y = forward_moe(wd, sc, x)
    torch.cuda.synchronize()
    assert sc.status() == 0
    idx = sc.topk_indices(T).cpu().numpy()
    o = oracle_on_gpu_routing(wh, x.cpu().numpy(), idx)
    logits = sc.router_logits(T).cpu().numpy()
    assert np.array_equal(logits, o["logits"]), "router logits must match the oracle bit for bit"
    assert np.array_equal(sc.x_q8(T).cpu().numpy(), o["x_q8"]), "Q8_1 bytes of the input"
    np.testing.assert_allclose(sc.topk_weights(T).cpu().numpy(), o["topk_w"], rtol=2e-6)
    perm, offs = oracle.permute(idx, cfg.E)
    assert np.array_equal(sc.perm(T).cpu().numpy(), perm)
    assert np.array_equal(sc.offsets().cpu().numpy(), offs)
    check_rows(y.cpu().numpy(), o["y"])
    # intermediates: Q8_1 scale and q within one step (float summation order differs)
    k = cfg.top_k
    iq = sc.inter_q8(T).cpu().numpy()
    nbF, nbS = cfg.F // 32, cfg.F_s // 32
    for t in range(T):
        for j in range(k + (1 if cfg.F_s else 0)):
            row = iq[t * k + j] if j < k else iq[T * k + t]
            nb = nbF if j < k else nbS
            a = row[:nb * 36].reshape(nb, 36)[:, 4:].view(np.int8).astype(int)
            b = o["inter_q8"][t, j][:nb * 36].reshape(nb, 36)[:, 4:].view(np.int8).astype(int)
            assert np.abs(a - b).max() <= 1


FULL = [(configs.QWEN_Q4_0, 16), (configs.QWEN_IQ3S, 1), (configs.QWEN_IQ3S, 2), (configs.QWEN_IQ3S, 4),
        (configs.QWEN_IQ3S, 8), (configs.NEMOTRON_Q4_0, 1)]


@pytest.mark.parametrize("cfg,T", FULL, ids=lambda v: getattr(v, "name", str(v)))
@pytest.mark.parametrize("layout", LAYOUTS)
def test_forward_full_size(cfg, T, layout):
    wd, wh = layer_pair(cfg, layout)
    x = configs.make_input(cfg, T, device="cuda")
    sc = MoeScratch(wd, T)
    y = forward_moe(wd, sc, x)
    y2 = forward_moe(wd, sc, x)
    torch.cuda.synchronize()
    assert sc.status() == 0
    assert torch.equal(y, y2), "two runs on the same input must agree bit for bit"
    idx = sc.topk_indices(T).cpu().numpy()
    o = oracle_on_gpu_routing(wh, x.cpu().numpy(), idx)
    check_rows(y.cpu().numpy(), o["y"])


@pytest.mark.parametrize("T", [16, 75, 2048])   # > 32: the large-batch router (token tiles in registers, ragged last tile)
def test_routing_bit_exact_against_reference_kernels(T):
    if not refkernels.available():
        pytest.skip("oracle/_ref cubin not built")
    cfg = configs.QWEN_Q4_0
    wd, _ = layer_pair(cfg)
    x = configs.make_input(cfg, T, device="cuda")
    sc = MoeScratch(wd, T)
    route_only(wd, sc, x)
    torch.cuda.synchronize()
    for t in (range(T) if T <= 128 else list(range(0, T, 37)) + [T - 1]):
        ref_logits = refkernels.f32_gemv(wd.router_weight, x[t])
        assert torch.equal(ref_logits, sc.router_logits(T)[t])
        ridx, rw = refkernels.topk_softmax(ref_logits, cfg.top_k)
        assert torch.equal(ridx, sc.topk_indices(T)[t])
        assert torch.equal(rw, sc.topk_weights(T)[t]), "weights must be bit-identical on the same GPU"
        q = refkernels.ggml_quantize_q8_1(x[t])
        assert torch.equal(q, sc.x_q8(T)[t])
        # shared-expert gate logit: same kernel shape as a one-row GEMV
        g = refkernels.f32_gemv(wd.shexp_gate_proj[None, :].contiguous(), x[t])
        assert torch.equal(g[0], sc.sh_gate_logit(T)[t])
    # the dispatch permutation of those indices: stable counting sort by expert
    perm, offs = oracle.permute(sc.topk_indices(T).cpu().numpy(), cfg.E)
    assert np.array_equal(sc.perm(T).cpu().numpy(), perm)
    assert np.array_equal(sc.offsets().cpu().numpy(), offs)


def test_routing_ties_and_zipf_bias():
    cfg = configs.scaled(configs.QWEN_Q8_0, E=64)
    wd, wh = layer_pair(cfg)
    T = 24
    x = torch.zeros(T, cfg.H, device="cuda")       # all logits = bias only -> deterministic order, no ties
    sc = MoeScratch(wd, T)
    route_only(wd, sc, x)
    torch.cuda.synchronize()
    order = torch.argsort(wd.router_bias, descending=True)[:cfg.top_k].to(torch.int32)
    assert torch.equal(sc.topk_indices(T)[0], order)
    # exact ties: zero router -> uniform probabilities -> experts 0..k-1 in order
    w0 = configs.make_layer(configs.scaled(configs.QWEN_Q4_0, E=16, name="ties"), device="cuda")
    w0.router_weight.zero_()
    sc0 = MoeScratch(w0, 4)
    route_only(w0, sc0, configs.make_input(cfg, 4, device="cuda"))
    torch.cuda.synchronize()
    assert sc0.topk_indices(4).cpu().tolist() == [list(range(8))] * 4
    assert sc0.topk_weights(4).cpu().tolist() == [[0.125] * 8] * 4


@pytest.mark.parametrize("qtype", [formats.TYPE_Q4_0, formats.TYPE_Q8_0, formats.TYPE_IQ3_S])
def test_block_sumi_bit_exact(qtype):
    lib = abi.load()
    torch.manual_seed(11)
    rows, cols = 96, 2048
    W = formats.quantize(qtype, torch.randn(rows, cols) * 0.02)
    xq = formats.quantize_q8_1(torch.randn(1, cols))
    ref = oracle.block_sumi(qtype, W.numpy(), xq.numpy(), cols, rows)
    Wd, xd = W.cuda(), xq.cuda()
    out = torch.empty(rows, cols // 32, dtype=torch.int32, device="cuda")
    abi.check(lib.chimere_b200_block_sumi(qtype, Wd.data_ptr(), xd.data_ptr(), out.data_ptr(), cols, rows, None), "sumi")
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), ref)
    # the packed (tiled32) form of the same matrix must give the same integers: the rewrite is lossless
    nbytes = lib.chimere_b200_packed_matrix_bytes(qtype, rows, cols)
    assert nbytes > 0
    packed = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    abi.check(lib.chimere_b200_pack_matrix(qtype, Wd.data_ptr(), packed.data_ptr(), rows, cols, None), "pack")
    out2 = torch.full((rows, cols // 32), -1, dtype=torch.int32, device="cuda")
    abi.check(lib.chimere_b200_block_sumi_tiled(qtype, packed.data_ptr(), xd.data_ptr(), out2.data_ptr(), cols, rows, None), "sumi tiled")
    torch.cuda.synchronize()
    assert np.array_equal(out2.cpu().numpy(), ref)


def _mmvq(name):
    return getattr(abi.load(), name)


@pytest.mark.parametrize("qtype,fn", [(formats.TYPE_Q4_0, "chimere_mmvq_q4_0"), (formats.TYPE_Q8_0, "chimere_mmvq_q8_0"),
                                      (formats.TYPE_IQ3_S, "chimere_mmvq_iq3s")])
@pytest.mark.parametrize("rows", [512, 77])
def test_legacy_mmvq(qtype, fn, rows):
    lib = abi.load()
    torch.manual_seed(12)
    cols = 2048
    W = formats.quantize(qtype, torch.randn(rows, cols) * 0.02)
    x = torch.randn(cols)
    xd = x.cuda()
    pad = 2048
    xq = torch.zeros(pad // 32 * 36, dtype=torch.uint8, device="cuda")
    lib.chimere_quantize_q8_1(xd.data_ptr(), xq.data_ptr(), cols, pad, None)
    y = torch.empty(rows, device="cuda")
    _mmvq(fn)(W.cuda().data_ptr(), xq.data_ptr(), y.data_ptr(), cols, rows, pad // 32, None)
    torch.cuda.synchronize()
    ref_q = oracle.quantize_q8_1(x.numpy())
    assert np.array_equal(xq.cpu().numpy()[:ref_q.size], ref_q)
    ref = oracle.gemv(qtype, W.numpy(), ref_q, cols, rows)
    np.testing.assert_allclose(y.cpu().numpy(), ref, rtol=1e-4, atol=1e-6)


def test_legacy_quantize_padding_and_batch():
    lib = abi.load()
    torch.manual_seed(13)
    ncols, pad, batch = 96, 512, 3   # rows padded to 512 elements as the reference's buffers are (ggml_gpu.rs:52-57)
    x = torch.randn(batch, ncols, device="cuda")
    out = torch.full((batch, pad // 32 * 36), 0xAB, dtype=torch.uint8, device="cuda")
    lib.chimere_quantize_q8_1_batched(x.data_ptr(), out.data_ptr(), ncols, pad, batch, None)
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    for b in range(batch):
        ref = oracle.quantize_q8_1(x[b].cpu().numpy())
        assert np.array_equal(o[b, :ref.size], ref)
        assert not o[b, ref.size:].any(), "blocks past ncols must be zero"


def test_iq3s_batched_synthetic_fixture():
    """The byte fixture of the reference's fused gate/up test (src/kernels/fused_gate_up.rs:388-443):
    weights byte i = i % 251 (second matrix +37), Q8_1 blocks d = 0x1000, qs[j] = j % 5, 4 experts,
    ids [1, 3].  Ours vs the CPU oracle and vs the reference's gemv_iq3s_q8 kernel."""
    lib = abi.load()
    cols, ffn, n_exp = 2048, 512, 4
    stride = ffn * cols // 256 * 110
    base = (np.arange(n_exp * stride) % 251).astype(np.uint8)
    q8 = np.zeros((cols // 32, 36), np.uint8)
    q8[:, 1] = 0x10
    q8[:, 4:] = (np.arange(32) % 5).astype(np.uint8)
    ids = [1, 3]
    for data in (base, (base.astype(np.int32) + 37).astype(np.uint8)):
        Wd = torch.from_numpy(data).cuda()
        qd = torch.from_numpy(q8.reshape(-1)).cuda()
        idd = torch.tensor(ids, dtype=torch.int32, device="cuda")
        y = torch.empty(len(ids) * ffn, device="cuda")
        lib.chimere_mmvq_iq3s_batched(Wd.data_ptr(), qd.data_ptr(), y.data_ptr(), idd.data_ptr(), cols, ffn, cols // 32,
                                      stride, 0, len(ids), None)
        torch.cuda.synchronize()
        got = y.cpu().numpy().reshape(len(ids), ffn)
        for s, e in enumerate(ids):
            ref = oracle.gemv(21, data[e * stride:(e + 1) * stride], q8.reshape(-1), cols, ffn)
            ok = np.isfinite(ref)
            np.testing.assert_allclose(got[s][ok], ref[ok], rtol=5e-3, atol=1e-4)   # the reference test's tolerance
            if refkernels.available():
                r = refkernels.gemv_iq3s_q8(Wd[e * stride:(e + 1) * stride].contiguous(), qd, ffn, cols).cpu().numpy()
                np.testing.assert_allclose(got[s][ok], r[ok], rtol=5e-3, atol=1e-4)


def test_reference_dequant_kernel_agrees_with_oracle():
    if not refkernels.available():
        pytest.skip("oracle/_ref cubin not built")
    torch.manual_seed(14)
    W = formats.quantize_iq3_s(torch.randn(8, 1024) * 0.02)
    ref = refkernels.dequant_iq3s(W.cuda().reshape(-1), 32).cpu().numpy()
    assert np.array_equal(ref, oracle.dequant(21, W.numpy(), 8 * 1024))


def test_host_entry_and_rmsnorm():
    cfg = SMALL[1]
    wd, wh = layer_pair(cfg)
    T = 5
    x = configs.make_input(cfg, T).pin_memory()
    y = torch.empty_like(x).pin_memory()
    sc = MoeScratch(wd, 8)
    forward_moe_host(wd, sc, x, y)
    o = oracle.moe_forward(wh, x.numpy(), taps=False)
    check_rows(y.numpy(), o["y"])
    # the same call again with new contents in the same host buffers
    first = y.clone()
    for rep in range(3):
        x.copy_(configs.make_input(cfg, T, seed=50 + rep))
        forward_moe_host(wd, sc, x, y)
        check_rows(y.numpy(), oracle.moe_forward(wh, x.numpy(), taps=False)["y"])
        assert not torch.equal(y, first)
    # pageable result buffer: the staged copy; bit-identical to the direct store into pinned memory
    y_pageable = torch.empty(T, cfg.H)
    forward_moe_host(wd, sc, x, y_pageable)
    assert torch.equal(y_pageable, y)
    lib = abi.load()
    yd = y.cuda()
    out = torch.empty_like(yd)
    abi.check(lib.chimere_b200_rmsnorm(yd.data_ptr(), out.data_ptr(), T, cfg.H, 1e-6, None), "rmsnorm")
    torch.cuda.synchronize()
    np.testing.assert_allclose(out.cpu().numpy(), oracle.rmsnorm(y.numpy()), rtol=1e-5, atol=1e-7)


def test_full_size_properties_decode_sweep():
    """Properties at the benchmark's full size that need no oracle run: rows of y depend only on
    their own token (batch of 8 == eight batches of 1), and routing weights sum to 1."""
    cfg = configs.QWEN_IQ3S
    wd, _ = layer_pair(cfg, "tiled")
    x = configs.make_input(cfg, 8, device="cuda")
    sc = MoeScratch(wd, 8)
    y8 = forward_moe(wd, sc, x).clone()
    w8 = sc.topk_weights(8).clone()
    for t in range(8):
        y1 = forward_moe(wd, sc, x[t:t + 1].contiguous())
        assert torch.equal(y1[0], y8[t])
    torch.cuda.synchronize()
    np.testing.assert_allclose(w8.sum(1).cpu().numpy(), np.ones(8), rtol=1e-6)


@pytest.mark.parametrize("qtype,fn", [(formats.TYPE_Q4_0, "chimere_mmvq_q4_0_f32"), (formats.TYPE_Q8_0, "chimere_mmvq_q8_0_f32"),
                                      (formats.TYPE_IQ3_S, "chimere_mmvq_iq3s_f32")])
def test_legacy_mmvq_from_f32_input(qtype, fn):
    """The fused quantize + GEMV entries (ffi/ggml_cuda_gemv.cu:322-352): the scratch must hold the Q8_1 row padded to
    512 elements, the output the GEMV of that row."""
    lib = abi.load()
    torch.manual_seed(15)
    rows, cols, pad = 200, 768, 1024           # 768 columns: padded to the next multiple of 512
    W = formats.quantize(qtype, torch.randn(rows, cols) * 0.02)
    x = torch.randn(cols)
    xd = x.cuda()
    scratch = torch.full((pad // 32 * 36,), 0xCD, dtype=torch.uint8, device="cuda")
    y = torch.empty(rows, device="cuda")
    getattr(lib, fn)(W.cuda().data_ptr(), xd.data_ptr(), y.data_ptr(), cols, rows, pad, scratch.data_ptr(), None)
    torch.cuda.synchronize()
    ref_q = oracle.quantize_q8_1(x.numpy())
    got_q = scratch.cpu().numpy()
    assert np.array_equal(got_q[:ref_q.size], ref_q)
    assert not got_q[ref_q.size:].any(), "blocks past ncols must be zero"
    ref = oracle.gemv(qtype, W.numpy(), ref_q, cols, rows)
    np.testing.assert_allclose(y.cpu().numpy(), ref, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("layout", LAYOUTS)
def test_whole_layer_against_reference_fused_kernel(layout):
    """The one whole-layer kernel of the reference that runs here: fused_moe_iq3s (chimere_kernels.cu:1093-1143), one
    token, gate / up / down all IQ3_S, routed experts only.  It multiplies dequantised weights with the fp32
    activations; the path built here (like the reference's production path, moe_ffn.rs:1185-1373) rounds the input
    and the intermediates to Q8_1 first.  That rounding alone moves an output by about 1 % of the largest one
    (two 8-bit roundings per output, measured 1.2e-2), so against this kernel the bar is 2.5e-2 and cosine >= 0.9999;
    the CPU oracle, which restates the Q8_1 path, must sit within the benchmark's own 1e-2 of the GPU result, and as
    far from the fused kernel as the GPU result does."""
    if not refkernels.available():
        pytest.skip("oracle/_ref cubin not built")
    cfg = configs.scaled(configs.QWEN_IQ3S, type_down=configs.IQ3_S, F_s=0, name="qwen35-moe-iq3s-all")
    wd, wh = layer_pair(cfg, layout)
    raw, _ = layer_pair(cfg)
    for seed in (1, 2, 3):
        x = configs.make_input(cfg, 1, device="cuda", seed=seed)
        sc = MoeScratch(wd, 1)
        y = forward_moe(wd, sc, x)
        torch.cuda.synchronize()
        ids, wts = sc.topk_indices(1)[0].contiguous(), sc.topk_weights(1)[0].contiguous()
        ref = refkernels.fused_moe_iq3s(x[0].contiguous(), raw.gate_exps_raw, raw.up_exps_raw, raw.down_exps_raw, ids, wts,
                                        cfg.H, cfg.F, raw.expert_bytes_gate, raw.expert_bytes_up, raw.expert_bytes_down)
        torch.cuda.synchronize()
        yg, yr = y.cpu().numpy()[0].astype(np.float64), ref.cpu().numpy().astype(np.float64)
        o = oracle_on_gpu_routing(wh, x.cpu().numpy(), sc.topk_indices(1).cpu().numpy())
        yo = o["y"][0].astype(np.float64)
        rel = lambda a, b: np.abs(a - b).max() / np.abs(b).max()
        cos = lambda a, b: float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))
        assert rel(yg, yr) <= 2.5e-2 and cos(yg, yr) >= COS_TOL, (rel(yg, yr), cos(yg, yr))
        check_rows(yg[None, :], yo[None, :])                      # the Q8_1 path itself: the benchmark's bar
        assert abs(rel(yo, yr) - rel(yg, yr)) <= 5e-3              # the distance to the fused kernel is the rounding, not the GPU code


def test_fused_residual_rmsnorm_then_layer():
    """residual += hidden, RMSNorm with a weight, then the layer, in one call.  The prologue must equal the reference's
    fused_add_residual_rmsnorm kernel bit for bit (it is run here from the source the reference hands to NVRTC), and the
    layer output must be what the plain entry gives on the normalised rows."""
    from chimere_b200.layer import forward_moe_residual_norm
    cfg = SMALL[1]
    wd, wh = layer_pair(cfg, "tiled")
    T, eps = 5, 1e-6
    g = torch.Generator(device="cuda").manual_seed(21)
    hidden = torch.randn(T, cfg.H, generator=g, device="cuda")
    residual = torch.randn(T, cfg.H, generator=g, device="cuda")
    weight = 1.0 + 0.1 * torch.randn(cfg.H, generator=g, device="cuda")
    res_ref, normed_ref = oracle.add_residual_rmsnorm(hidden.cpu().numpy(), residual.cpu().numpy(), weight.cpu().numpy(), eps)
    sc = MoeScratch(wd, 8)
    res_gpu = residual.clone()
    y = forward_moe_residual_norm(wd, sc, hidden, res_gpu, weight, eps)
    torch.cuda.synchronize()
    assert np.array_equal(res_gpu.cpu().numpy(), res_ref), "residual rows after the add"
    if refkernels.fused_ops_available():
        for t in range(T):
            r = residual[t].clone()
            n = refkernels.fused_add_residual_rmsnorm(hidden[t].contiguous(), r, weight, eps)
            torch.cuda.synchronize()
            assert torch.equal(r, res_gpu[t])
            assert np.array_equal(n.cpu().numpy(), normed_ref[t]), "oracle restatement vs the reference kernel"
    normed = torch.from_numpy(normed_ref).cuda()
    y_plain = forward_moe(wd, MoeScratch(wd, 8), normed)
    torch.cuda.synchronize()
    # the same kernels on the same rows (the prologue's rows equal the oracle's up to the GPU's sqrt / division rounding)
    np.testing.assert_allclose(y.cpu().numpy(), y_plain.cpu().numpy(), rtol=1e-4, atol=1e-6)
    check_rows(y.cpu().numpy(), oracle.moe_forward(wh, normed_ref, taps=False)["y"])


def test_routing_trace_layout_and_load():
    from chimere_b200.layer import routing_trace
    from chimere_b200.trace import RoutingTrace
    cfg = configs.QWEN_Q8_0     # Zipf-biased: a skewed load histogram
    wd, _ = layer_pair(cfg)
    T = 40
    sc = MoeScratch(wd, T)
    load = torch.zeros(cfg.E, dtype=torch.int32, device="cuda")
    tr = RoutingTrace(T, cfg.top_k)
    idx_layers = []
    for layer_seed in (5, 6):
        x = configs.make_input(cfg, T, device="cuda", seed=layer_seed)
        route_only(wd, sc, x)
        tr.add_layer(routing_trace(wd, sc, T, expert_load=load))
        idx_layers.append(sc.topk_indices(T).cpu().numpy().copy())
    torch.cuda.synchronize()
    data = RoutingTrace.parse(tr.payload())
    assert data.shape == (2, T, 8)
    for i, idx in enumerate(idx_layers):
        assert np.array_equal(data[i], idx.astype(np.uint8))
    ref_load = np.bincount(np.concatenate([i.reshape(-1) for i in idx_layers]), minlength=cfg.E)
    assert np.array_equal(load.cpu().numpy(), ref_load)


@pytest.mark.parametrize("qtype,fn", [(formats.TYPE_Q4_K, "chimere_mmvq_q4k"), (formats.TYPE_Q5_K, "chimere_mmvq_q5k"),
                                      (formats.TYPE_Q6_K, "chimere_mmvq_q6k")])
@pytest.mark.parametrize("rows,cols", [(512, 2048), (2048, 512), (77, 256)])
def test_legacy_mmvq_kquants(qtype, fn, rows, cols):
    """The K-quant GEMV entries (ffi/ggml_cuda_gemv.cu:118-172) at the shared expert's shapes (F_s x H, H x F_s) and a ragged
    one, with the f32-input forms beside them (:302-321, :353-391)."""
    lib = abi.load()
    W = formats.random_kquant_rows(qtype, rows, cols, seed=rows + qtype)
    x = np.random.default_rng(rows).standard_normal(cols).astype(np.float32)
    ref_q = oracle.quantize_q8_1(x)
    ref = oracle.gemv(qtype, W, ref_q, cols, rows)
    Wd, xd = torch.from_numpy(W).cuda(), torch.from_numpy(x).cuda()
    pad = (cols + 511) // 512 * 512
    xq = torch.zeros(pad // 32 * 36, dtype=torch.uint8, device="cuda")
    lib.chimere_quantize_q8_1(xd.data_ptr(), xq.data_ptr(), cols, pad, None)
    y = torch.empty(rows, device="cuda")
    getattr(lib, fn)(Wd.data_ptr(), xq.data_ptr(), y.data_ptr(), cols, rows, pad // 32, None)
    scratch = torch.full((pad // 32 * 36,), 0xCD, dtype=torch.uint8, device="cuda")
    y2 = torch.empty(rows, device="cuda")
    getattr(lib, fn + "_f32")(Wd.data_ptr(), xd.data_ptr(), y2.data_ptr(), cols, rows, pad, scratch.data_ptr(), None)
    torch.cuda.synchronize()
    assert np.array_equal(xq.cpu().numpy()[:ref_q.size], ref_q)
    assert np.array_equal(scratch.cpu().numpy()[:ref_q.size], ref_q)
    # same integer dots and scales; only the order of the fp32 additions differs
    tol = 2e-5 * np.abs(ref).max()
    np.testing.assert_allclose(y.cpu().numpy(), ref, rtol=0, atol=tol)
    assert torch.equal(y, y2)


def test_layer_loaded_from_a_gguf_file_gives_the_same_output(tmp_path):
    """File -> C-ABI reader -> pinned buffer -> device -> pack -> layer call, against the same layer built in memory."""
    pytest.importorskip("gguf")
    from chimere_b200.gguf_io import GgufFile, load_moe_layer
    from test_gguf_ingest import _write
    cfg = configs.scaled(configs.QWEN_IQ3S, E=16, F=256, F_s=256, H=512)
    host = configs.make_layer(cfg, seed=21)
    path = tmp_path / "layer.gguf"
    _write(path, {2: host})
    with GgufFile(path) as g:
        loaded = load_moe_layer(g, 2, device="cuda")
    x = configs.make_input(cfg, 8, device="cuda")
    outs = []
    for raw in (host.to("cuda"), loaded):
        tiled = MoeWeightsTiled(raw)
        sc = MoeScratch(tiled, 8)
        outs.append(forward_moe(tiled, sc, x).clone())
        assert sc.status() == 0
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("sh_types", [(formats.TYPE_Q5_K, formats.TYPE_Q5_K), (formats.TYPE_Q4_K, formats.TYPE_Q6_K)])
@pytest.mark.parametrize("T,entry", [(1, "decode"), (8, "decode"), (40, "decode"), (333, "decode"), (96, "prefill"), (600, "prefill")])
def test_layer_with_kquant_shared_expert(sh_types, T, entry):
    """The production mix: IQ3_S / Q4_0 routed experts with the shared expert in K-quant super-blocks (moe_ffn.rs:1597-1730).
    The whole-layer entries run the routed part as usual and the shared expert as GEMVs on the raw blocks."""
    from chimere_b200.layer import MoeWeightsPrefill, forward_moe_prefill
    cfg = configs.scaled(configs.QWEN_IQ3S, E=32, F=256, F_s=512, H=1024, type_sh_gate_up=sh_types[0], type_sh_down=sh_types[1], seed=31)
    raw = configs.make_layer(cfg, device="cuda")
    wh = raw.to("cpu")
    tiled = MoeWeightsTiled(raw)
    x = configs.make_input(cfg, T, device="cuda")
    sc = MoeScratch(tiled, T)
    y = forward_moe_prefill(tiled, MoeWeightsPrefill(raw), sc, x) if entry == "prefill" else forward_moe(tiled, sc, x)
    torch.cuda.synchronize()
    assert sc.status() == 0
    idx = sc.topk_indices(T).cpu().numpy()
    o = oracle_on_gpu_routing(wh, x.cpu().numpy(), idx)
    assert np.array_equal(sc.x_q8(T).cpu().numpy(), o["x_q8"])
    np.testing.assert_allclose(sc.sh_gate_logit(T).cpu().numpy(), o["sh_logit"], rtol=1e-5, atol=1e-6)
    check_rows(y.cpu().numpy(), o["y"])
    # the shared expert must have arrived: the same layer without it differs
    routed_only = configs.make_layer(configs.scaled(cfg, F_s=0), device="cuda")
    t2 = MoeWeightsTiled(routed_only)
    y2 = forward_moe(t2, MoeScratch(t2, T), x)
    assert (y - y2).abs().max() > 1e-3 * y.abs().max()


def test_kquant_shared_layer_through_the_host_and_residual_norm_entries():
    """The other whole-layer entries on a layer with a Q5_K shared expert: host buffers (staged copy back, because the
    shared expert's last step adds into y) and the fused residual-add + RMSNorm prologue."""
    from chimere_b200.layer import forward_moe_residual_norm
    cfg = configs.scaled(configs.QWEN_IQ3S, E=32, F=256, F_s=512, H=1024, type_sh_gate_up=formats.TYPE_Q5_K, type_sh_down=formats.TYPE_Q5_K, seed=33)
    raw = configs.make_layer(cfg, device="cuda")
    tiled = MoeWeightsTiled(raw)
    T = 6
    x = configs.make_input(cfg, T, device="cuda")
    sc = MoeScratch(tiled, 8)
    y = forward_moe(tiled, sc, x).clone()
    xh, yh = x.cpu().pin_memory(), torch.empty(T, cfg.H).pin_memory()
    forward_moe_host(tiled, sc, xh, yh)
    assert torch.equal(yh, y.cpu())
    # residual + norm prologue: hidden = 0, residual = x', unit weight -> the layer sees rmsnorm(x')
    resid = (x * 3.0).clone()
    y2 = forward_moe_residual_norm(tiled, sc, torch.zeros_like(x), resid, torch.ones(cfg.H, device="cuda"), 1e-6)
    lib = abi.load()
    normed = torch.empty_like(x)
    abi.check(lib.chimere_b200_rmsnorm((x * 3.0).contiguous().data_ptr(), normed.data_ptr(), T, cfg.H, 1e-6, None), "rmsnorm")
    y3 = forward_moe(tiled, MoeScratch(tiled, 8), normed)
    torch.cuda.synchronize()
    assert sc.status() == 0
    assert (y2 - y3).abs().max() <= 2e-5 * y3.abs().max()
    # the step-wise entries refuse such a layer
    assert lib.chimere_b200_moe_route(C.byref(tiled.as_struct()), x.data_ptr(), T, C.byref(sc.ws), None) == -6
