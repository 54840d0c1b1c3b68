"""The (sample, kv-head) unit planner and packer of hbsattn_b200/shard.py, without a GPU.

* the longest-processing-time plan assigns every unit exactly once and balances the FLOPs of skewed varlen
  workloads (draws shaped like the heterogeneous-block and the unequal-length benchmark configurations) within 5 %;
* two CPU ranks (gloo): each packs its units into one varlen problem with a CSR block mask and computes it with the
  oracle (the GPU kernels are not involved here - this checks the partition, the packing and the gather only); the
  gathered result must equal the unsharded one, and the reduction bench.py uses for timings (max of times, sum of
  work) must agree."""
import os
import socket
import subprocess
import sys

import numpy as np
import torch

from hbsattn_b200.shard import csr_of_mask, dense_mask_of_csr, kv_head_range, plan_imbalance, plan_units, unit_flops
from oracle import oracle_block_decisions


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_kv_head_ranges_cover_everything():
    for hk in (1, 3, 8, 32):
        for world in (1, 2, 4, 8):
            ranges = [kv_head_range(hk, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == hk
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1


def _draw(seed, batch, q_range, k_range, hk, qbs, kbs, causal, p_keep):
    rng = np.random.default_rng(seed)
    q_lens = (rng.integers(q_range[0], q_range[1] + 1, size=batch) // 16) * 16
    k_lens = q_lens if k_range is None else rng.integers(k_range[0], k_range[1] + 1, size=batch)
    cu_q = [0] + [int(x) for x in np.cumsum(q_lens)]
    cu_k = [0] + [int(x) for x in np.cumsum(k_lens)]
    nqb = sum((int(n) + qbs - 1) // qbs for n in q_lens)
    nkb = sum((int(n) + kbs - 1) // kbs for n in k_lens)
    mask = torch.rand(hk, nqb, nkb, generator=torch.Generator().manual_seed(seed)) < p_keep
    dec = oracle_block_decisions(cu_q, cu_k, mask, qbs, kbs, causal)
    return cu_q, cu_k, dec


def test_plan_balances_skewed_workloads():
    cases = [
        ("varlen 1024-16384, 80x48, non-causal", _draw(3, 8, (1024, 16384), None, 8, 80, 48, False, 0.3), 80, 48, 4),
        ("q 128-512, k 16384-32768, 16x128, causal", _draw(5, 16, (128, 512), (16384, 32768), 8, 16, 128, True, 0.2), 16, 128, 8),
    ]
    for name, (cu_q, cu_k, dec), qbs, kbs, group in cases:
        flops = unit_flops(dec, cu_q, cu_k, qbs, kbs, 128, group)
        assert flops.shape == (len(cu_q) - 1, dec.shape[0]) and (flops > 0).all()
        assert flops.max() / flops.min() > 3.0, "the draw is supposed to be skewed"
        for world in (2, 4, 8):
            plan = plan_units(flops, world)
            flat = sorted(u for units in plan for u in units)
            assert flat == sorted((b, h) for b in range(flops.shape[0]) for h in range(flops.shape[1])), name
            assert plan_imbalance(plan, flops) <= 1.05, (name, world, plan_imbalance(plan, flops))
        # a plain split by kv-head ranges would not do: all samples of a head land on one rank, heads cost the same
        # on average, but a split by samples is off by the length skew
        by_sample = [[(b, h) for h in range(flops.shape[1])] for b in range(flops.shape[0])]
        assert plan_imbalance(by_sample, flops) > 1.3


def test_csr_round_trip():
    mask = torch.rand(3, 7, 9, generator=torch.Generator().manual_seed(1)) < 0.4
    row_ptr, col_idx = csr_of_mask(mask)
    assert row_ptr.dtype == torch.int32 and col_idx.dtype == torch.int32 and row_ptr.numel() == 3 * 7 + 1
    assert int(row_ptr[-1]) == int(mask.sum())
    assert torch.equal(dense_mask_of_csr(row_ptr, col_idx, 3, 7, 9), mask)


def test_two_rank_shard_and_gather(tmp_path):
    out = str(tmp_path / "res.pt")
    port = _free_port()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "shard_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(port), out]) for r in range(2)]
    for pr in procs:
        assert pr.wait(timeout=240) == 0
    res = torch.load(out)
    assert res["units"] == res["all_units"]
    assert res["err"] <= 1e-6
    assert res["tmax"] == 2.0 and res["wsum"] == 30.0
