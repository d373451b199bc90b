"""The routing entry that allocates nothing (chimere_b200_moe_route_noalloc).

Hosts that gave every byte of device memory to their own pool at start-up, or that call from a place
where cudaMalloc is off limits, still need routing; for them the scratch is a fixed array inside the
library.  This test calls that entry through the C ABI twice in a row on different inputs -- the array
keeps the previous call's contents, so the second call proves the entry clears what it must -- and
expects exactly the indices and weights of the ordinary entry (integer routing is bit-exact, and the
weights come from the same kernel, so they are compared bit for bit too).  It is collected last so that
a run stopping at the first failure has already run every other test."""
import ctypes as C

import pytest
import torch

from chimere_b200 import abi, configs
from chimere_b200.layer import MoeScratch, route_only

pytestmark = pytest.mark.gpu


def _route_noalloc(lib, w, x, idx, wts):
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.chimere_b200_moe_route_noalloc(C.byref(w.as_struct()), x.data_ptr(), x.shape[0], idx.data_ptr(), wts.data_ptr(), stream)
    abi.check(rc, "chimere_b200_moe_route_noalloc")


def test_noalloc_routing_matches_ordinary_entry_twice():
    lib = abi.load()
    cfg = configs.scaled(configs.QWEN_Q4_0, E=64, F=64, F_s=64)
    w = configs.make_layer(cfg, device="cuda")
    sc = MoeScratch(w, 64)
    for T, seed in ((40, 1), (7, 2)):           # two calls in a row, the second smaller than the first
        x = configs.make_input(cfg, T, device="cuda", seed=seed)
        idx = torch.full((T, cfg.top_k), -1, dtype=torch.int32, device="cuda")
        wts = torch.full((T, cfg.top_k), -1.0, dtype=torch.float32, device="cuda")
        _route_noalloc(lib, w, x, idx, wts)
        route_only(w, sc, x)
        torch.cuda.synchronize()
        assert torch.equal(idx, sc.topk_indices(T))
        assert torch.equal(wts, sc.topk_weights(T))


@pytest.mark.parametrize("H,E,k,T", [(4096, 256, 8, 64),     # every stated limit at once: the scratch regions at their full size
                                     (2688, 128, 6, 40),     # H > 2048 with more than 32 tokens: the wide-row router kernel
                                     (4096, 256, 8, 8)])     # the decode-size kernel at the widest row
def test_noalloc_at_its_limits(H, E, k, T):
    """The built-in scratch is sized for T = 64, H = 4096, E = 256, top_k = 8.  Routing at exactly those sizes (and on the
    kernel variants that smaller cases never reach) must still equal the ordinary entry's, twice in a row."""
    lib = abi.load()
    mode = abi.ROUTE_SIGMOID_NORM_SCALE if E == 128 else abi.ROUTE_SOFTMAX_RENORM
    cfg = configs.scaled(configs.QWEN_Q4_0, H=H, E=E, top_k=k, F=64, F_s=64, route_mode=mode, route_scale=2.5 if E == 128 else 1.0,
                         name=f"limits-{H}-{E}-{k}")
    w = configs.make_layer(cfg, device="cuda")
    sc = MoeScratch(w, T)
    for seed in (3, 4):
        x = configs.make_input(cfg, T, device="cuda", seed=seed)
        idx = torch.full((T, k), -1, dtype=torch.int32, device="cuda")
        wts = torch.full((T, k), -1.0, dtype=torch.float32, device="cuda")
        _route_noalloc(lib, w, x, idx, wts)
        route_only(w, sc, x)
        torch.cuda.synchronize()
        assert torch.equal(idx, sc.topk_indices(T))
        assert torch.equal(wts, sc.topk_weights(T))


def test_noalloc_rejects_sizes_beyond_its_scratch():
    """Everything larger than the built-in scratch answers -7 before anything is launched: T > 64, H > 4096, E > 256."""
    lib = abi.load()
    cfg = configs.scaled(configs.QWEN_Q4_0, E=16, F=64, F_s=64)
    w = configs.make_layer(cfg, device="cuda")
    x = configs.make_input(cfg, 65, device="cuda")
    idx = torch.empty(65, cfg.top_k, dtype=torch.int32, device="cuda")
    wts = torch.empty(65, cfg.top_k, dtype=torch.float32, device="cuda")
    rc = lib.chimere_b200_moe_route_noalloc(C.byref(w.as_struct()), x.data_ptr(), 65, idx.data_ptr(), wts.data_ptr(), None)
    assert rc == -7
    # the same layer described with sizes beyond the limits (rejected on the host: the pointers are never followed)
    for field, value in (("H", 4096 + 32), ("E", 257)):
        st = abi.MoeLayer.from_buffer_copy(w.as_struct())
        setattr(st, field, value)
        rc = lib.chimere_b200_moe_route_noalloc(C.byref(st), x.data_ptr(), 8, idx.data_ptr(), wts.data_ptr(), None)
        assert rc == -7, (field, rc)
    st = abi.MoeLayer.from_buffer_copy(w.as_struct())
    st.H = 100                                   # not a multiple of 32: a malformed description, not a size limit
    assert lib.chimere_b200_moe_route_noalloc(C.byref(st), x.data_ptr(), 8, idx.data_ptr(), wts.data_ptr(), None) == -2
