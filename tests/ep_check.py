"""Run under torchrun on >= 2 GPUs: the expert-parallel layer must reproduce the single-GPU layer bit for
bit on every rank's own tokens (same kernels, same Q8_1 bytes, same combine order)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from chimere_b200 import configs  # noqa: E402
from chimere_b200.ep import ExpertParallelMoE  # noqa: E402
from chimere_b200.layer import MoeScratch, MoeWeightsTiled, forward_moe  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    for cfg, T in ((configs.scaled(configs.QWEN_IQ3S, E=32), 8), (configs.scaled(configs.QWEN_Q4_0_ZIPF, E=64), 40),
                   (configs.scaled(configs.NEMOTRON_Q4_0, E=16), 3)):
        full = configs.make_layer(cfg, device=dev)                     # same seed on every rank
        ep = ExpertParallelMoE(full, max_tokens=T, rank=rank, world=world, device=dev)
        x = configs.make_input(cfg, T, device=dev, seed=50 + rank)     # this rank's tokens
        y_ep = ep.forward(x).clone()
        y_ep2 = ep.forward_padded(x, torch.empty_like(x)).clone()     # fixed-size exchange, workspaces reused
        packed = MoeWeightsTiled(full)
        y_ref = forward_moe(packed, MoeScratch(packed, T, device=dev), x)
        torch.cuda.synchronize()
        same = bool(torch.equal(y_ep, y_ref)) and bool(torch.equal(y_ep2, y_ref))
        print(f"rank {rank} {cfg.name} T={T}: {'bit-exact' if same else 'MISMATCH'} (rows received {ep.last_recv_rows})", flush=True)
        ok = ok and same
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
