"""Rows whose maximum jumps between K/V tiles: the kernel runs a tile's exponentials against the reference of
the previous tiles and must notice (from the packed P) when that reference is stale, rescale O and redo the
tile.  Scores here grow from k-block to k-block by far more than the 2^8 slack, in both directions of the
key order, with and without rows that have no reference at first (bottom-right causal, q_len > k_len)."""
import numpy as np
import pytest
import torch

from helpers import make_problem
from oracle import error_stats, oracle_forward

pytestmark = pytest.mark.gpu


def _run(pr, dtype):
    import hbsattn_b200 as hb
    out = hb.HBSAttention(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"], None)
    torch.cuda.synchronize()
    assert hb.last_status()[0] == 0
    want = oracle_forward(pr["q"].cpu().float(), pr["k"].cpu().float(), pr["v"].cpu().float(), pr["cu_q_list"],
                          pr["cu_k_list"], pr["mask"].cpu(), pr["qbs"], pr["kbs"], pr["causal"], None)
    assert torch.isfinite(out).all()
    st = error_stats(want, out)
    assert st["max_abs"] <= 2e-2 and st["mean_abs"] <= 1e-3, f"max-abs {st['max_abs']:.3e} mean-abs {st['mean_abs']:.3e}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("growing", [True, False])
@pytest.mark.parametrize("causal,q_lens,k_lens", [(False, [256, 384], [512, 640]), (True, [384, 512], [384, 512]),
                                                  (True, [512, 300], [256, 200])])
def test_maximum_jumps_between_tiles(dtype, growing, causal, q_lens, k_lens):
    dev = torch.device("cuda:0")
    pr = make_problem(31, q_lens, k_lens, 4, 2, 128, 128, 64, causal, dtype, 1.0, force=None, device=dev)
    # keys of k-block j scaled by a factor that changes the row maxima by ~10-60 in the log2 domain per block
    k = pr["k"].float()
    tok = 0
    for b in range(len(k_lens)):
        nblk = (k_lens[b] + 63) // 64
        for j in range(nblk):
            f = 1.0 + 2.5 * (j if growing else nblk - 1 - j)
            k[tok + j * 64: tok + min((j + 1) * 64, k_lens[b])] *= f
        tok += k_lens[b]
    pr["k"] = k.to(dtype)
    _run(pr, dtype)
