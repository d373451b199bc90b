"""Expert parallelism for the MoE layer: experts sharded over the ranks of one node in contiguous
ranges, router and shared expert replicated, tokens sharded (every rank routes its own tokens).

The reference has no multi-GPU code (no collective library is linked, chimere-server/Cargo.toml:7-26);
this is the design of its benchmark configuration "expert-parallel stack": one all-to-all before the
expert products (dispatch: the Q8_1 planes of every (token, expert) pair go to the expert's owner;
quantisation happens once on the home rank, so results are bit-identical to the single-GPU path) and
one after (combine: the pairs' fp32 expert rows come home, where they are weighted and added in slot
order together with the shared expert).  torch.distributed (NCCL over NVLink on GPUs, gloo in the CPU
tests) carries the exchanges; all arithmetic is in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from . import abi
from .layer import MoeScratch, MoeWeightsPrefill, MoeWeightsRaw, MoeWeightsTiled


# ------------------------------------------------------------------ exchange plan (pure torch) ----
@dataclass
class DispatchPlan:
    order: torch.Tensor        # [P] pair ids (t*k + j) sorted by destination rank, stable
    send_counts: torch.Tensor  # [G] int64 pairs going to each rank
    local_ids: torch.Tensor    # [P] int32 expert id within the owner's shard, in send order


def plan_dispatch(topk_idx: torch.Tensor, experts_per_rank: int, world: int) -> DispatchPlan:
    """Pairs in row-major (token, slot) order -> send order grouped by owner rank (stable).  Host-side statement of the
    exchange plan, used by the CPU tests of the collective plumbing; the GPU path takes the order from the dispatch kernel's
    permutation instead (ExpertParallelMoE.forward)."""
    flat = topk_idx.reshape(-1).to(torch.int64)
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    order = torch.sort(dest, stable=True).indices
    send_counts = torch.bincount(dest, minlength=world)
    local_ids = (flat[order] - dest[order] * experts_per_rank).to(torch.int32)
    return DispatchPlan(order, send_counts, local_ids)


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts, group=group)
    return recv


def all_to_all_rows(send: torch.Tensor, send_counts: List[int], recv_counts: List[int], out: Optional[torch.Tensor] = None,
                    group=None) -> torch.Tensor:
    """Rows of `send` (grouped by destination) -> rows grouped by source, into `out[:sum(recv_counts)]`."""
    n = sum(recv_counts)
    if out is None:
        out = torch.empty((n,) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_to_all_single(out[:n], send.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return out[:n]


# ------------------------------------------------------------------ the layer on GPUs --------------
class ExpertParallelMoE:
    """One MoE layer on `world` GPUs.  `full_raw` is the whole layer (same on every rank, e.g. seeded);
    only this rank's expert range is kept on the device after construction."""

    def __init__(self, full_raw: MoeWeightsRaw, max_tokens: int, rank: int, world: int, device, group=None, prefill: bool = False):
        assert full_raw.E % world == 0
        self.rank, self.world, self.group = rank, world, group
        self.k, self.E, self.H = full_raw.top_k, full_raw.E, full_raw.H
        self.E_loc = full_raw.E // world
        lo, hi = rank * self.E_loc, (rank + 1) * self.E_loc
        dev = torch.device(device)
        sl = lambda t: None if t is None else t[lo:hi].contiguous().to(dev)
        mv = lambda t: None if t is None else t.contiguous().to(dev)
        local = MoeWeightsRaw(
            H=full_raw.H, E=self.E_loc, F=full_raw.F, F_s=full_raw.F_s, top_k=min(full_raw.top_k, self.E_loc),
            type_gate=full_raw.type_gate, type_up=full_raw.type_up, type_down=full_raw.type_down,
            router_weight=mv(full_raw.router_weight[lo:hi]), up_exps_raw=sl(full_raw.up_exps_raw), down_exps_raw=sl(full_raw.down_exps_raw),
            gate_exps_raw=sl(full_raw.gate_exps_raw), shexp_gate_proj=mv(full_raw.shexp_gate_proj),
            shexp_gate_raw=mv(full_raw.shexp_gate_raw), shexp_up_raw=mv(full_raw.shexp_up_raw), shexp_down_raw=mv(full_raw.shexp_down_raw),
            route_mode=full_raw.route_mode, route_scale=full_raw.route_scale, act=full_raw.act,
            type_sh_gate=full_raw.type_sh_gate, type_sh_up=full_raw.type_sh_up, type_sh_down=full_raw.type_sh_down)
        # prefill-size batches: the local shard's copy for the grouped GEMM (built from the raw blocks before they are dropped)
        self.pw_owner = MoeWeightsPrefill(local) if prefill else None
        self.packed = MoeWeightsTiled(local, keep_raw=False)
        self.router_weight = mv(full_raw.router_weight)
        self.router_bias = mv(full_raw.router_bias)
        # home view: the whole router, the shared expert; expert pointers are the local shard's (never used for routed pairs here)
        self.home = abi.MoeLayer.from_buffer_copy(self.packed.as_struct())
        self.home.E, self.home.top_k = self.E, self.k
        self.home.router_w = self.router_weight.data_ptr()
        self.home.router_bias = None if self.router_bias is None else self.router_bias.data_ptr()
        # owner view: the local shard as a layer of E_loc experts, one expert per row, no shared expert
        self.owner = abi.MoeLayer.from_buffer_copy(self.packed.as_struct())
        self.owner.E, self.owner.top_k, self.owner.F_s = self.E_loc, 1, 0
        self.max_tokens = max_tokens
        self.max_rows = max_tokens * self.k * world   # worst case: every pair of every rank lands here
        self.ws_home = _Scratch(self.home, full_raw, max_tokens, dev, prefill=prefill and full_raw.F_s > 0)
        self.ws_owner = _Scratch(self.owner, full_raw, self.max_rows, dev, prefill=prefill)
        self.rows_pair = torch.empty(max_tokens * self.k, self.H, dtype=torch.float32, device=dev)
        self.back = torch.empty(max_tokens * self.k, self.H, dtype=torch.float32, device=dev)
        self.lib = abi.load()
        self.last_recv_rows = 0

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Exact split sizes (prefill-size batches).  The routing kernel's dispatch has sorted the pairs by expert, which
        groups them by owner rank; a kernel packs the rows in that order, the per-rank counts are differences of the
        dispatch offsets (the one value the host needs: the split sizes of the collectives), one all-to-all carries the
        packed rows, the owner's experts run on them in place, one all-to-all carries the per-pair rows back."""
        lib, T, k, H, G = self.lib, x.shape[0], self.k, self.H, self.world
        assert T <= self.max_tokens and x.is_contiguous()
        if out is None:
            out = torch.empty_like(x)
        dev = x.device
        st = torch.cuda.current_stream(dev).cuda_stream
        if not hasattr(self, "_exact"):
            ds = self.ws_home.dstride
            rb = (H + 4 * ds + 4 + 15) & ~15
            self._exact = dict(rb=rb, send=torch.empty(self.max_tokens * k, rb, dtype=torch.uint8, device=dev),
                               recv=torch.empty(self.max_rows, rb, dtype=torch.uint8, device=dev),
                               slot=torch.zeros(self.max_tokens * k, dtype=torch.int32, device=dev),
                               bounds=torch.arange(0, self.E + 1, self.E_loc, device=dev))
        ex = self._exact
        rb = ex["rb"]
        abi.check(lib.chimere_b200_moe_route_home(C.byref(self.home), x.data_ptr(), T, C.byref(self.ws_home.ws), st), "route_home")
        abi.check(lib.chimere_b200_moe_ep_pack_sorted(C.byref(self.home), T, C.byref(self.ws_home.ws), ex["send"].data_ptr(), ex["slot"].data_ptr(),
                                                      self.E_loc, rb, st), "ep_pack_sorted")
        # the shared expert needs nothing from other ranks: enqueue it before the exchanges (on the grouped GEMM when the
        # batch fills token tiles)
        if self.pw_owner is not None and self.ws_home.prefill is not None and T >= 128:
            abi.check(lib.chimere_b200_moe_shared_expert_prefill(C.byref(self.home), C.byref(self.pw_owner.struct), T, C.byref(self.ws_home.ws), st),
                      "shared_expert_prefill")
        else:
            abi.check(lib.chimere_b200_moe_shared_expert(C.byref(self.home), T, C.byref(self.ws_home.ws), st), "shared_expert")
        send_counts_t = self.ws_home.offsets(self.E)[ex["bounds"]].diff().to(torch.int64)
        recv_counts_t = exchange_counts(send_counts_t, self.group)
        send_counts, recv_counts = send_counts_t.tolist(), recv_counts_t.tolist()   # host sync: split sizes
        n = sum(recv_counts)
        assert n <= self.max_rows
        self.last_recv_rows = n
        all_to_all_rows(ex["send"][:T * k], send_counts, recv_counts, ex["recv"], self.group)   # (a rank may receive nothing)
        if self.pw_owner is not None and n >= 512:   # many rows per expert: the grouped GEMM
            abi.check(lib.chimere_b200_moe_experts_packed_prefill(C.byref(self.owner), C.byref(self.pw_owner.struct), n, ex["recv"].data_ptr(), rb,
                                                                  C.byref(self.ws_owner.ws), st), "experts_packed_prefill")
        else:
            abi.check(lib.chimere_b200_moe_experts_packed(C.byref(self.owner), n, ex["recv"].data_ptr(), rb, C.byref(self.ws_owner.ws), st), "experts")
        # combine: the pairs' expert rows come home in send order; the finish kernel finds a pair's row through its slot
        back = all_to_all_rows(self.ws_owner.pair_out(self.max_rows)[:n], recv_counts, send_counts, self.back, self.group)
        abi.check(lib.chimere_b200_moe_ep_finish(C.byref(self.home), back.data_ptr(), ex["slot"].data_ptr(), T, C.byref(self.ws_home.ws),
                                                 out.data_ptr(), st), "ep_finish")
        return out

    # ---- decode-size batches: fixed-size exchange, no host synchronisation, CUDA-graph capturable ----
    def forward_padded(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """Same result as forward().  Every rank sends every other rank room for all of its T*k pairs (rows that are
        not there carry expert id -1 and cost the owner nothing), so no counts have to reach the host.  Meant for
        small T; the padding grows with world * T * k rows."""
        lib, T, k, H, G = self.lib, x.shape[0], self.k, self.H, self.world
        assert T == self.max_tokens, "the padded path works on a fixed batch size"
        C_ = T * k                                   # capacity per destination
        dev = x.device
        st = torch.cuda.current_stream(dev).cuda_stream
        if not hasattr(self, "_pad"):
            ds = self.ws_home.dstride
            rb = (H + 4 * ds + 4 + 15) & ~15
            self._pad = dict(ds=ds, rb=rb,
                             send=torch.empty(G * C_, rb, dtype=torch.uint8, device=dev), recv=torch.empty(G * C_, rb, dtype=torch.uint8, device=dev),
                             back=torch.empty(G * C_, H, dtype=torch.float32, device=dev),
                             slot=torch.zeros(T * k, dtype=torch.int32, device=dev))
        pd = self._pad
        rb, send, recv, back, slot = pd["rb"], pd["send"], pd["recv"], pd["back"], pd["slot"]
        n = G * C_
        abi.check(lib.chimere_b200_moe_route_home(C.byref(self.home), x.data_ptr(), T, C.byref(self.ws_home.ws), st), "route_home")
        abi.check(lib.chimere_b200_moe_ep_pack(C.byref(self.home), T, C.byref(self.ws_home.ws), send.data_ptr(), slot.data_ptr(),
                                               self.E_loc, G, C_, rb, st), "ep_pack")
        # the shared expert needs nothing from other ranks: it runs while the dispatch is in flight (the exchange is
        # enqueued on the communicator's stream; this stream joins it only after the shared expert's kernels)
        work = dist.all_to_all_single(recv, send, group=self.group, async_op=True)
        abi.check(lib.chimere_b200_moe_shared_expert(C.byref(self.home), T, C.byref(self.ws_home.ws), st), "shared_expert")
        work.wait()
        abi.check(lib.chimere_b200_moe_experts_packed(C.byref(self.owner), n, recv.data_ptr(), rb, C.byref(self.ws_owner.ws), st), "experts")
        dist.all_to_all_single(back, self.ws_owner.pair_out(n), group=self.group)
        abi.check(lib.chimere_b200_moe_ep_finish(C.byref(self.home), back.data_ptr(), slot.data_ptr(), T, C.byref(self.ws_home.ws),
                                                 out.data_ptr(), st), "ep_finish")
        self.last_recv_rows = n
        return out


    # ---- decode-size batches: the exchange done by the kernels themselves (peer stores over NVLink) ----
    def enable_peer_exchange(self) -> None:
        """Sets up the buffers the peers write into (one device allocation per rank, shared with the other ranks of the node
        through CUDA IPC) for batches of exactly `max_tokens` tokens.  Collective: every rank must call it."""
        T, k, H, G = self.max_tokens, self.k, self.H, self.world
        cap = T * k
        ds = self.ws_home.dstride
        rb = (H + 4 * ds + 12 + 15) & ~15
        recv_bytes = (G * cap * rb + 255) & ~255
        back_bytes = (G * T * H * 4 + 255) & ~255
        self._peer = PeerRegion(recv_bytes + back_bytes + 512, self.rank, G, self.group)
        dev = self.rows_pair.device
        ptrs = lambda off: torch.tensor([b + off for b in self._peer.bases], dtype=torch.int64, device=dev)
        self._p2p = dict(cap=cap, rb=rb, recv=self._peer.bases[self.rank], back=self._peer.bases[self.rank] + recv_bytes,
                         flags_in=self._peer.bases[self.rank] + recv_bytes + back_bytes, flags_back=self._peer.bases[self.rank] + recv_bytes + back_bytes + 256,
                         peer_recv=ptrs(0), peer_back=ptrs(recv_bytes), peer_flags_in=ptrs(recv_bytes + back_bytes),
                         peer_flags_back=ptrs(recv_bytes + back_bytes + 256),
                         ctr=torch.zeros(3 * 64, dtype=torch.int32, device=dev),
                         side=torch.cuda.Stream(device=dev), fork=torch.cuda.Event(), join=torch.cuda.Event())
        self.overlap_shared = os.environ.get("CHIMERE_EP_SERIAL_SHARED", "") == "" and self.home.F_s > 0

    def forward_peer(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """The layer with both exchanges done by peer stores and flags instead of collectives: no NCCL call, no host
        synchronisation, capturable in a CUDA graph.  The owners return one partial sum per (home rank, token), so the result
        equals forward() up to the order of those fp32 additions."""
        lib, T, G = self.lib, x.shape[0], self.world
        assert T == self.max_tokens and hasattr(self, "_p2p"), "call enable_peer_exchange() first; the batch size is fixed"
        pp = self._p2p
        st = torch.cuda.current_stream(x.device).cuda_stream
        ctr = pp["ctr"].data_ptr()
        abi.check(lib.chimere_b200_moe_route_home(C.byref(self.home), x.data_ptr(), T, C.byref(self.ws_home.ws), st), "route_home")
        # The shared expert needs nothing from other ranks and nothing the exchange writes: it runs on a second stream beside
        # the pack -> wait -> experts -> return chain (the fork and the join are captured with the rest in a CUDA graph).
        main = torch.cuda.current_stream(x.device)
        if self.overlap_shared:
            pp["fork"].record(main)
            pp["side"].wait_event(pp["fork"])
            abi.check(lib.chimere_b200_moe_shared_expert(C.byref(self.home), T, C.byref(self.ws_home.ws), pp["side"].cuda_stream), "shared_expert")
            pp["join"].record(pp["side"])
        abi.check(lib.chimere_b200_moe_ep_pack_p2p(C.byref(self.home), T, C.byref(self.ws_home.ws), pp["peer_recv"].data_ptr(),
                                                   pp["peer_flags_in"].data_ptr(), ctr, self.rank, self.E_loc, G, pp["cap"], pp["rb"], st), "ep_pack_p2p")
        if not self.overlap_shared:
            abi.check(lib.chimere_b200_moe_shared_expert(C.byref(self.home), T, C.byref(self.ws_home.ws), st), "shared_expert")
        n = G * pp["cap"]
        abi.check(lib.chimere_b200_moe_experts_packed_p2p(C.byref(self.owner), n, pp["recv"], pp["rb"], pp["flags_in"], G, pp["cap"],
                                                          C.byref(self.ws_owner.ws), st), "experts")
        abi.check(lib.chimere_b200_moe_ep_return_p2p(C.byref(self.owner), C.byref(self.ws_owner.ws), pp["recv"], pp["rb"], pp["peer_back"].data_ptr(),
                                                     pp["peer_flags_back"].data_ptr(), ctr + 256, self.rank, G, T, pp["cap"], st), "ep_return_p2p")
        if self.overlap_shared:
            main.wait_event(pp["join"])
        abi.check(lib.chimere_b200_moe_ep_finish_p2p(C.byref(self.home), pp["back"], pp["flags_back"], G, T, C.byref(self.ws_home.ws), out.data_ptr(),
                                                     ctr + 512, st), "ep_finish_p2p")
        self.last_recv_rows = n
        return out


class PeerRegion:
    """One zeroed device allocation per rank that every rank of the node can address: allocated with cudaMalloc, exported with
    CUDA IPC, the handles exchanged through the process group.  bases[r] is rank r's region as seen from this process (this
    rank's own pointer for r == rank).  Peer access is plain load / store over NVLink; nothing here uses multicast."""

    def __init__(self, nbytes: int, rank: int, world: int, group=None):
        from cuda.bindings import runtime as rt
        self._rt, self.nbytes = rt, nbytes
        err, ptr = rt.cudaMalloc(nbytes)
        if err != rt.cudaError_t.cudaSuccess:
            raise RuntimeError(f"cudaMalloc({nbytes}) failed: {err}")
        self.ptr = int(ptr)
        (err,) = rt.cudaMemset(self.ptr, 0, nbytes)
        assert err == rt.cudaError_t.cudaSuccess, err
        torch.cuda.synchronize()
        self.bases = [0] * world
        self.bases[rank] = self.ptr
        self._opened = []
        if world > 1:
            err, handle = rt.cudaIpcGetMemHandle(self.ptr)
            assert err == rt.cudaError_t.cudaSuccess, err
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle.reserved), group=group)
            for r in range(world):
                if r == rank:
                    continue
                h = rt.cudaIpcMemHandle_t()
                h.reserved = handles[r]
                err, p = rt.cudaIpcOpenMemHandle(h, rt.cudaIpcMemLazyEnablePeerAccess)
                if err != rt.cudaError_t.cudaSuccess:
                    raise RuntimeError(f"cudaIpcOpenMemHandle(rank {r}) failed: {err}")
                self.bases[r] = int(p)
                self._opened.append(int(p))
            dist.barrier(group=group)   # every region is zeroed and mapped before anyone writes into a peer


class _Scratch:
    """Workspace of one layer view plus typed views of the buffers the exchanges touch."""

    def __init__(self, struct: abi.MoeLayer, dims: MoeWeightsRaw, max_T: int, dev, prefill: bool = False):
        lib = abi.load()
        self.H = struct.H
        self.dstride = (struct.H // 32 + 3) & ~3
        nbytes = lib.chimere_b200_moe_workspace_bytes(C.byref(struct), max_T)
        if nbytes == 0:
            raise RuntimeError("workspace_bytes rejected the layer view")
        self.arena = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self.ws = abi.MoeWorkspace()
        st = torch.cuda.current_stream(dev).cuda_stream
        abi.check(lib.chimere_b200_moe_workspace_init(C.byref(self.ws), self.arena.data_ptr(), nbytes, C.byref(struct), max_T, st), "workspace_init")
        self.prefill = None
        if prefill:
            n = lib.chimere_b200_moe_prefill_bytes(C.byref(struct), max_T)
            if n == 0:
                raise RuntimeError("prefill_bytes rejected the layer view")
            self.prefill = torch.zeros(n, dtype=torch.uint8, device=dev)
            self.ws.prefill_arena, self.ws.prefill_bytes = self.prefill.data_ptr(), n

    def _view(self, ptr, nbytes):
        off = ptr - self.arena.data_ptr()
        return self.arena[off:off + nbytes]

    def topk_idx(self, T, k):
        return self._view(self.ws.topk_idx, T * k * 4).view(torch.int32).reshape(T, k)

    def offsets(self, E):
        return self._view(self.ws.offsets, (E + 1) * 4).view(torch.int32)

    def x_q(self, T):
        return self._view(self.ws.x_q, T * self.H).view(torch.int8).reshape(T, self.H)

    def x_d(self, T):
        return self._view(self.ws.x_d, T * self.dstride * 4).view(torch.float32).reshape(T, self.dstride)

    def pair_out(self, n):
        return self._view(self.ws.pair_out, n * self.H * 4).view(torch.float32).reshape(n, self.H)
