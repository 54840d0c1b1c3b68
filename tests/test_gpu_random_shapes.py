"""Seeded random problem shapes through both CUDA kernel families, against the fp32 oracle.

Every draw picks batch, ragged q/k lengths (cu_q != cu_k, bottom-right alignment, samples where q is longer than k),
GQA ratio, head dimension (any multiple of 8 up to 256 for the tensor-core kernel), heterogeneous block sizes (multiples
of 16, not only powers of two), causal or not, mask density, dtype and an explicit or default softmax scale - the axes
of test/test_accuracy.py:17-29 drawn jointly instead of as a grid, at sizes the oracle finishes in well under a second.
Checked per draw: oracle tolerance (max-abs <= 2e-2 for outputs up to 2 in magnitude, mean-abs <= 1e-3) for both families, agreement of the two
independently written kernels, the valid/skip bitmap bit for bit against the oracle's, and exact zeros where the oracle
has rows without keys."""
import numpy as np
import pytest
import torch

from oracle import error_stats, oracle_block_decisions, oracle_forward
from helpers import make_lengths, make_problem

pytestmark = pytest.mark.gpu

N_DRAWS = 200


def draw(seed):
    rng = np.random.default_rng(1000003 * seed + 17)
    batch = int(rng.integers(1, 6))
    qbs = int(rng.choice([16, 32, 48, 64, 80, 128, 144]))
    kbs = int(rng.choice([16, 32, 48, 64, 80, 128, 144, 256]))
    hk = int(rng.choice([1, 2, 3]))
    group = int(rng.choice([1, 2, 3, 4, 8]))
    d = int(rng.choice([16, 24, 32, 40, 64, 72, 96, 128, 160, 256]))
    causal = bool(rng.integers(0, 2))
    same = bool(rng.integers(0, 3) == 0)
    q_lens = make_lengths(rng, batch, 1, 700)
    k_lens = q_lens if same else make_lengths(rng, batch, 1, 900)
    dtype = torch.bfloat16 if rng.integers(0, 2) else torch.float16
    p_keep = float(rng.choice([0.15, 0.4, 0.8, 1.0]))
    force = [None, "first", "diag"][int(rng.integers(0, 3))]
    scale = None if rng.integers(0, 2) else float(rng.uniform(0.05, 0.4))
    return dict(batch=batch, qbs=qbs, kbs=kbs, hq=hk * group, hk=hk, d=d, causal=causal, q_lens=q_lens, k_lens=k_lens,
                dtype=dtype, p_keep=p_keep, force=force, scale=scale)


@pytest.mark.parametrize("seed", range(N_DRAWS))
def test_random_shape(seed):
    import hbsattn_b200 as hb
    c = draw(seed)
    pr = make_problem(seed, c["q_lens"], c["k_lens"], c["hq"], c["hk"], c["d"], c["qbs"], c["kbs"], c["causal"], c["dtype"],
                      c["p_keep"], c["force"])
    gold = oracle_forward(pr["q"].float(), pr["k"].float(), pr["v"].float(), pr["cu_q_list"], pr["cu_k_list"], pr["mask"],
                          c["qbs"], c["kbs"], c["causal"], c["scale"])
    # 2e-2 / 1e-3 are stated for outputs of order one; a sharp softmax (large explicit scale, few keys) returns single V
    # rows, and from 4 upwards one bf16 step of the OUTPUT is 0.031 already - both bounds grow with the largest output
    grow = max(1.0, gold.abs().max().item() / 2.0)
    tol, tol_mean = 2e-2 * grow, 1e-3 * grow
    outs = {}
    for family in ("sm100", "generic"):
        hb.set_kernel_family(family)
        try:
            out = hb.HBSAttention(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], c["qbs"], c["kbs"], c["causal"],
                                  c["scale"])
            assert hb.last_status()[0] == 0, (family, c)
        finally:
            hb.set_kernel_family("auto")
        assert torch.isfinite(out).all(), (family, c)
        st = error_stats(gold, out)
        assert st["max_abs"] <= tol and st["mean_abs"] <= tol_mean, (family, st, c)
        outs[family] = out
    assert (outs["sm100"].float() - outs["generic"].float()).abs().max().item() <= 2.0 * tol, c
    # rows the oracle leaves without keys are exact zeros in both kernels
    dead = (gold.abs().sum(dim=-1) == 0)
    if dead.any():
        assert outs["sm100"][dead].abs().max().item() == 0.0 and outs["generic"][dead].abs().max().item() == 0.0, c
    # the valid/skip decision, bit for bit
    bitmap, counts = hb.block_decisions(pr["q"], pr["k"], pr["cu_q"], pr["cu_k"], pr["mask"], c["qbs"], c["kbs"], c["causal"])
    want = oracle_block_decisions(pr["cu_q_list"], pr["cu_k_list"], pr["mask"].cpu(), c["qbs"], c["kbs"], c["causal"])
    assert torch.equal(bitmap.cpu().bool(), torch.as_tensor(want).bool()), c
