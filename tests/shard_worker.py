"""Rank body of tests/test_shard_gloo.py (run as a script, one process per rank)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from hbsattn_b200.shard import dense_mask_of_csr, pack_units, plan_units, unit_flops, unpack_output
from oracle import oracle_block_decisions, oracle_forward


def _worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    cu_q, cu_k = [0, 48, 112, 144], [0, 80, 131, 150]
    hq, hk, d, qbs, kbs, causal = 6, 3, 16, 32, 16, True
    q = torch.randn(cu_q[-1], hq, d, generator=g)
    k = torch.randn(cu_k[-1], hk, d, generator=g)
    v = torch.randn(cu_k[-1], hk, d, generator=g)
    mask = torch.rand(hk, 5, 11, generator=g) < 0.6
    # every rank derives the same plan from the same decisions
    dec = oracle_block_decisions(cu_q, cu_k, mask, qbs, kbs, causal)
    flops = unit_flops(dec, cu_q, cu_k, qbs, kbs, d, hq // hk)
    plan = plan_units(flops, world)
    mine = pack_units(plan[rank], q, k, v, cu_q, cu_k, mask, qbs, kbs)
    # the oracle takes a dense mask: expand this rank's CSR rows (the GPU path consumes the CSR form directly)
    dense = dense_mask_of_csr(mine.csr_row_ptr, mine.csr_col_idx, 1, mine.num_q_block, mine.num_k_block)
    out = oracle_forward(mine.q, mine.k, mine.v, mine.cu_q_seqlens.tolist(), mine.cu_k_seqlens.tolist(), dense, qbs, kbs, causal, None)
    parts = [None] * world
    dist.all_gather_object(parts, (plan[rank], mine.q_rows, out))
    t = torch.tensor([1.0 + rank, 10.0 * (rank + 1)], dtype=torch.float64)
    tmax, wsum = t[:1].clone(), t[1:].clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(wsum, op=dist.ReduceOp.SUM)
    if rank == 0:
        full = oracle_forward(q, k, v, cu_q, cu_k, mask, qbs, kbs, causal, None)
        got = torch.full_like(full, float("nan"))
        seen = []
        for units, rows, o in parts:
            mine.units, mine.q_rows = units, rows           # reuse the container for unpacking the other rank's part
            unpack_output(mine, o, got)
            seen += list(units)
        torch.save({"err": (full - got).abs().max().item(), "tmax": tmax.item(), "wsum": wsum.item(),
                    "units": sorted(seen), "all_units": sorted((b, h) for b in range(len(cu_q) - 1) for h in range(hk))}, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    _worker(int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4])
