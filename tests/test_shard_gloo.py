"""Two CPU ranks (gloo): each takes its kv-head shard, computes it with the oracle (the GPU kernels are
not involved here - this checks the partition and the gather only), the gathered result must equal the
unsharded one, and the timing reduction used by bench.py (max of times, sum of work) must agree."""
import os
import socket

import subprocess
import sys

import torch

from hbsattn_b200.shard import kv_head_range


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


def test_two_rank_shard_and_gather(tmp_path):
    out = str(tmp_path / "res.pt")
    port = _free_port()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "shard_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(port), out]) for r in range(2)]
    for pr in procs:
        assert pr.wait(timeout=240) == 0
    res = torch.load(out)
    assert res["err"] <= 1e-6
    assert res["tmax"] == 2.0 and res["wsum"] == 30.0
