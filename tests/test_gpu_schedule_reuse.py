"""One schedule, several attention launches (layers / decode steps that share a mask): every launch must equal
the full forward on the same inputs, bit for bit, for the tensor-core and the generic kernel family."""
import numpy as np
import pytest
import torch

from helpers import make_lengths, make_problem

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,headdim", [(torch.bfloat16, 128), (torch.float16, 64), (torch.float32, 32)])
def test_schedule_reused_over_three_calls(dtype, headdim):
    import hbsattn_b200 as hb
    dev = torch.device("cuda:0")
    lens = make_lengths(np.random.default_rng(11), 3, 150, 900)
    pr = make_problem(11, lens, lens, 8, 2, headdim, 128, 64, True, dtype, 0.4, force="diag", device=dev)
    sched = hb.build_schedule(pr["q"], pr["k"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], True)
    g = torch.Generator(device="cpu").manual_seed(5)
    for step in range(3):
        q = torch.randn(pr["q"].shape, generator=g).to(dtype).to(dev)
        k = torch.randn(pr["k"].shape, generator=g).to(dtype).to(dev)
        v = torch.randn(pr["v"].shape, generator=g).to(dtype).to(dev)
        scale = None if step != 1 else 0.17
        got = hb.attention_with_schedule(q, k, v, sched, scale)
        want = hb.HBSAttention(q, k, v, pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], True, scale)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"launch {step} on the reused schedule differs from the full forward"
        assert hb.last_status()[0] == 0


def test_schedule_rejects_other_head_count():
    import hbsattn_b200 as hb
    dev = torch.device("cuda:0")
    lens = [256, 128]
    pr = make_problem(3, lens, lens, 4, 2, 64, 64, 64, False, torch.bfloat16, 0.5, force="first", device=dev)
    sched = hb.build_schedule(pr["q"], pr["k"], pr["cu_q"], pr["cu_k"], pr["mask"], 64, 64, False)
    k4 = torch.randn(pr["k"].shape[0], 4, 64, device=dev, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        hb.attention_with_schedule(pr["q"], k4, k4, sched)
