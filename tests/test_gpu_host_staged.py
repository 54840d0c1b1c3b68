"""HostStagedAttention: forwards from pinned host tensors, pipelined over two device slots, against the
direct device call on the same inputs."""
import numpy as np
import pytest
import torch

from helpers import make_lengths, make_problem

pytestmark = pytest.mark.gpu


def _host(t):
    return t.cpu().pin_memory()


def test_host_staged_matches_device_call_over_reused_slots():
    import hbsattn_b200 as hb
    dev = torch.device("cuda:0")
    staged = hb.HostStagedAttention(dev)
    problems, outs = [], []
    for i in range(5):                       # 5 submits over 2 slots: every slot is reused
        causal = bool(i & 1)
        lens = make_lengths(np.random.default_rng(100 + i), 3, 100, 700)
        pr = make_problem(100 + i, lens, lens, 4, 2, 128, 128, 64 if i % 2 else 128, causal, torch.bfloat16, 0.4,
                          force="first", device=dev)
        problems.append(pr)
        o, ticket = staged.submit(_host(pr["q"]), _host(pr["k"]), _host(pr["v"]), _host(pr["cu_q"]), _host(pr["cu_k"]),
                                  _host(pr["mask"]), pr["qbs"], pr["kbs"], causal, None)
        assert ticket == i
        outs.append(o)
    staged.wait()
    for pr, o in zip(problems, outs):
        ref = hb.HBSAttention(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"],
                              pr["causal"], None)
        torch.cuda.synchronize()
        assert torch.equal(o, ref.cpu()), "the staged forward must be bit-identical to the device call"


def test_host_staged_done_event_and_given_output():
    import hbsattn_b200 as hb
    dev = torch.device("cuda:0")
    lens = make_lengths(np.random.default_rng(7), 2, 64, 300)
    pr = make_problem(7, lens, lens, 8, 2, 64, 64, 64, True, torch.float16, 0.5, force="first", device=dev)
    staged = hb.HostStagedAttention(dev)
    out = torch.zeros(pr["q"].shape, dtype=pr["q"].dtype).pin_memory()
    o, ticket = staged.submit(_host(pr["q"]), _host(pr["k"]), _host(pr["v"]), _host(pr["cu_q"]), _host(pr["cu_k"]),
                              _host(pr["mask"]), pr["qbs"], pr["kbs"], True, 0.2, out=out)
    assert o is out
    staged.done_event(ticket).synchronize()
    ref = hb.HBSAttention(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], True, 0.2)
    torch.cuda.synchronize()
    assert torch.equal(out, ref.cpu())
    with pytest.raises(ValueError):
        staged.done_event(ticket + 1)
