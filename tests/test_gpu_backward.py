"""Backward of the operator (dq, dk, dv over the active block pairs) against torch.autograd through the fp32 oracle.

The reference has no backward (hbsattn/hbsa_interface.py:30-32); the check is the mathematics of its forward
(hbsattn/reference.py:23-107, restated by the oracle) differentiated by autograd in fp32 on the same inputs.
Tolerance: every gradient within 2e-2 of the oracle's gradient relative to that gradient's largest magnitude, and
within 1e-2 on average relative to its mean magnitude (the inputs, the forward output that enters delta, and the
gradients themselves are rounded to the 16-bit dtype); 1e-4 / 1e-5 for fp32 inputs.  Rows that see no key get zeros."""
import numpy as np
import pytest
import torch

from helpers import make_lengths, make_problem
from oracle import oracle_forward

pytestmark = pytest.mark.gpu

CASES = [
    # name, batch, q range, k range, hq, hk, d, qbs, kbs, causal, dtype
    ("mha_128x128_causal", 3, (100, 500), None, 2, 2, 128, 128, 128, True, torch.bfloat16),
    ("gqa4_80x48", 3, (100, 400), None, 8, 2, 64, 80, 48, False, torch.bfloat16),
    ("gqa2_16x128_bottom_right", 3, (64, 200), (300, 900), 4, 2, 64, 16, 128, True, torch.float16),
    ("fp32_32x16_d18", 4, (30, 120), (20, 150), 4, 2, 18, 32, 16, True, torch.float32),
    ("q_longer_than_k", 2, (200, 300), (40, 120), 2, 1, 32, 64, 64, True, torch.float32),
]


def _oracle_grads(pr, d_out):
    q, k, v = (pr[n].float().detach().clone().requires_grad_(True) for n in ("q", "k", "v"))
    out = oracle_forward(q, k, v, pr["cu_q_list"], pr["cu_k_list"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"], None)
    out.backward(d_out.float())
    return q.grad, k.grad, v.grad


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_backward_matches_autograd_of_the_oracle(case):
    import hbsattn_b200 as hb
    name, batch, qr, kr, hq, hk, d, qbs, kbs, causal, dtype = case
    rng = np.random.default_rng(len(name))
    q_lens = make_lengths(rng, batch, *qr)
    k_lens = q_lens if kr is None else make_lengths(rng, batch, *kr)
    pr = make_problem(51, q_lens, k_lens, hq, hk, d, qbs, kbs, causal, dtype, 0.5, "first" if not causal else None)
    g = torch.Generator(device="cpu").manual_seed(7)
    d_out = torch.randn(pr["q"].shape, generator=g).to(dtype).cuda()
    q, k, v = (pr[n].detach().clone().requires_grad_(True) for n in ("q", "k", "v"))
    out = hb.HBSAttention(q, k, v, pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"], None)
    out.backward(d_out)
    assert hb.last_status()[0] == 0
    want = _oracle_grads(pr, d_out)
    rel_max, rel_mean = (1e-4, 1e-5) if dtype == torch.float32 else (2e-2, 1e-2)
    for nm, got, ref in zip(("dq", "dk", "dv"), (q.grad, k.grad, v.grad), want):
        assert got.dtype == dtype and got.shape == ref.shape and torch.isfinite(got).all(), nm
        err = (got.float() - ref).abs()
        assert err.max().item() <= rel_max * ref.abs().max().item(), (nm, err.max().item(), ref.abs().max().item())
        assert err.mean().item() <= rel_mean * ref.abs().mean().item(), (nm, err.mean().item(), ref.abs().mean().item())


def test_backward_of_rows_without_keys_is_zero():
    import hbsattn_b200 as hb
    pr = make_problem(52, [256, 128], [64, 128], 2, 2, 64, 64, 64, True, torch.bfloat16, 1.0, None)
    q = pr["q"].detach().clone().requires_grad_(True)
    out = hb.HBSAttention(q, pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], 64, 64, True, None)
    out.float().sum().backward()
    # sample 0 has q_len 256 > k_len 64: its first 192 rows see no key (bottom-right alignment)
    assert q.grad[:192].abs().max().item() == 0.0
    assert q.grad[192:256].abs().max().item() > 0.0


def test_attention_backward_function_with_lse():
    import hbsattn_b200 as hb
    pr = make_problem(53, [200, 300], [200, 300], 4, 2, 128, 128, 128, True, torch.bfloat16, 0.6, "diag")
    out, lse = hb.HBSAttention_with_lse(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], 128, 128, True)
    d_out = torch.ones_like(out)
    dq, dk, dv = hb.attention_backward(pr["q"], pr["k"], pr["v"], out, lse, d_out, pr["cu_q"], pr["cu_k"], pr["mask"], 128, 128, True)
    want = _oracle_grads(pr, d_out)
    for got, ref in zip((dq, dk, dv), want):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
