"""Host logic of the expert-parallel exchange on CPU: two gloo ranks build their dispatch plans, trade
counts and rows, "compute" a function of (row, expert id) on the owner, send the rows home and put them
back in (token, slot) order.  The result must equal the same function applied locally."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    from chimere_b200.ep import all_to_all_rows, exchange_counts, plan_dispatch
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(100 + rank)
        T, k, E, H = 5 + rank, 3, 8, 16
        E_loc = E // world
        idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32)
        x = torch.randn(T, H)
        plan = plan_dispatch(idx, E_loc, world)
        recv_counts = exchange_counts(plan.send_counts).tolist()
        send_counts = plan.send_counts.tolist()
        assert sum(send_counts) == T * k
        tok = torch.div(plan.order, k, rounding_mode="floor")
        rows = all_to_all_rows(x[tok], send_counts, recv_counts)
        ids = all_to_all_rows(plan.local_ids, send_counts, recv_counts)
        assert rows.shape[0] == sum(recv_counts)
        assert ids.numel() == 0 or (int(ids.max()) < E_loc and int(ids.min()) >= 0)
        owner_out = rows * (ids.to(torch.float32)[:, None] + rank * E_loc + 1.0)   # stands in for the expert products
        back = all_to_all_rows(owner_out, recv_counts, send_counts)
        got = torch.empty(T * k, H)
        got.index_copy_(0, plan.order, back)
        want = x.repeat_interleave(k, dim=0) * (idx.reshape(-1).to(torch.float32)[:, None] + 1.0)
        results[rank] = bool(torch.equal(got, want))
    finally:
        dist.destroy_process_group()


def test_exchange_round_trip_two_ranks():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_plan_is_stable_and_complete():
    from chimere_b200.ep import plan_dispatch
    idx = torch.tensor([[5, 0, 2], [1, 7, 3]], dtype=torch.int32)
    plan = plan_dispatch(idx, 4, 2)
    assert plan.send_counts.tolist() == [4, 2]
    assert plan.order.tolist() == [1, 2, 3, 5, 0, 4]          # rank 0 gets experts 0,2,1,3 (pair order kept), rank 1 gets 5,7
    assert plan.local_ids.tolist() == [0, 2, 1, 3, 1, 3]
