"""Rank body of tests/test_shard_gloo.py (run as a script, one process per rank)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from hbsattn_b200.shard import kv_head_range, shard_by_kv_heads
from oracle import oracle_forward


def _worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    cu_q, cu_k = [0, 48, 112], [0, 80, 131]
    hq, hk, d = 6, 3, 16
    q = torch.randn(cu_q[-1], hq, d, generator=g)
    k = torch.randn(cu_k[-1], hk, d, generator=g)
    v = torch.randn(cu_k[-1], hk, d, generator=g)
    mask = torch.rand(hk, 4, 5, generator=g) < 0.6
    qs, ks, vs, ms, q_slice = shard_by_kv_heads(q, k, v, mask, rank, world)
    mine = oracle_forward(qs, ks, vs, cu_q, cu_k, ms, 32, 32, True, None)
    parts = [torch.empty(cu_q[-1], (kv_head_range(hk, r, world)[1] - kv_head_range(hk, r, world)[0]) * (hq // hk), d)
             for r in range(world)]
    dist.all_gather(parts, mine.contiguous()) if len({p.shape for p in parts}) == 1 else None
    if len({p.shape for p in parts}) != 1:                      # uneven shards: gather through object lists
        objs = [None] * world
        dist.all_gather_object(objs, mine)
        parts = objs
    t = torch.tensor([1.0 + rank, 10.0 * (rank + 1)], dtype=torch.float64)
    tmax, wsum = t[:1].clone(), t[1:].clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(wsum, op=dist.ReduceOp.SUM)
    if rank == 0:
        full = oracle_forward(q, k, v, cu_q, cu_k, mask, 32, 32, True, None)
        got = torch.cat(parts, dim=1)
        torch.save({"err": (full - got).abs().max().item(), "tmax": tmax.item(), "wsum": wsum.item()}, out_path)
    dist.barrier()
    dist.destroy_process_group()



if __name__ == "__main__":
    _worker(int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4])
