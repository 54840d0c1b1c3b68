"""LSE output of the forward (natural-log sum of exponentials per row) against the fp32 oracle, for the
tensor-core and the generic kernel family, including rows that see no key (-inf)."""
import numpy as np
import pytest
import torch

from helpers import make_lengths, make_problem
from oracle import oracle_forward

pytestmark = pytest.mark.gpu

CASES = [
    # dtype, hq, hk, d, qbs, kbs, causal
    (torch.bfloat16, 8, 2, 128, 128, 128, True),
    (torch.float16, 4, 4, 64, 64, 64, False),
    (torch.bfloat16, 8, 1, 128, 80, 48, False),
    (torch.float32, 4, 2, 32, 32, 16, True),        # generic kernel
]


@pytest.mark.parametrize("dtype,hq,hk,d,qbs,kbs,causal", CASES)
def test_lse_matches_oracle(dtype, hq, hk, d, qbs, kbs, causal):
    import hbsattn_b200 as hb
    dev = torch.device("cuda:0")
    lens = make_lengths(np.random.default_rng(21), 3, 90, 700)
    pr = make_problem(21, lens, lens, hq, hk, d, qbs, kbs, causal, dtype, 0.4, force=None, device=dev)
    out, lse = hb.HBSAttention_with_lse(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], qbs, kbs, causal, None)
    ref_out = hb.HBSAttention(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], qbs, kbs, causal, None)
    torch.cuda.synchronize()
    assert torch.equal(out, ref_out), "asking for the LSE must not change the output"
    want_out, want_lse = oracle_forward(pr["q"].cpu().float(), pr["k"].cpu().float(), pr["v"].cpu().float(),
                                        pr["cu_q_list"], pr["cu_k_list"], pr["mask"].cpu(), qbs, kbs, causal, None,
                                        return_lse=True)
    got = lse.cpu()
    dead = torch.isinf(want_lse) & (want_lse < 0)
    assert torch.equal(torch.isinf(got) & (got < 0), dead), "rows without keys must be -inf, and only those"
    err = (got[~dead] - want_lse[~dead]).abs()
    # scores come from 16-bit inputs multiplied exactly and summed in fp32; the exponentials are approximate (ex2)
    assert err.max().item() <= 2e-3, f"lse max-abs error {err.max().item():.3e}"


def test_no_lse_written_when_null():
    """The default path passes lse = NULL: the forward must not write anywhere else."""
    import hbsattn_b200 as hb
    dev = torch.device("cuda:0")
    pr = make_problem(5, [200, 130], [200, 130], 4, 2, 64, 64, 64, True, torch.bfloat16, 0.6, force="diag", device=dev)
    guard = torch.full((pr["q"].shape[0], 4), 7.0, dtype=torch.float32, device=dev)
    hb.HBSAttention(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], 64, 64, True, None)
    torch.cuda.synchronize()
    assert bool((guard == 7.0).all())
