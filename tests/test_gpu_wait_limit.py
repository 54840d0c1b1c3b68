"""The give-up path of the tensor-core kernel: every wait inside it has a clock budget, and when one runs out the
kernel sets HBSA_STATUS_WAIT_LIMIT, all of its warps leave, tensor memory is given back and the call returns.

It is exercised in the one form that puts nothing at risk: a debug switch makes the kernel's loader warp publish
no work at all, so no copy and no tensor-core instruction is ever issued and the other warps simply wait until a
(here: very short) budget is spent.  The next forward with the default budget must then be correct, which also shows
that tensor memory was released."""
import pytest
import torch

from helpers import make_problem
from oracle import error_stats, oracle_forward

pytestmark = pytest.mark.gpu


def test_wait_limit_is_reported_and_the_gpu_stays_usable():
    import hbsattn_b200 as hb
    from hbsattn_b200 import _lib
    lib = _lib.load()
    pr = make_problem(41, [256, 384], [256, 384], 4, 2, 128, 128, 128, True, torch.bfloat16, 0.6, "diag")
    args = (pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"], None)
    hb.set_kernel_family("sm100")
    try:
        lib.hbsa_debug_set_wait_budget(2_000_000, 1)          # about one millisecond of SM clocks; the loader stays silent
        with pytest.raises(RuntimeError, match="device status 2"):
            hb.HBSAttention(*args)
        assert hb.last_status()[0] == _lib.HBSA_STATUS_WAIT_LIMIT
        lib.hbsa_debug_set_wait_budget(0, 0)                   # defaults again
        out = hb.HBSAttention(*args)
        assert hb.last_status()[0] == 0
    finally:
        lib.hbsa_debug_set_wait_budget(0, 0)
        hb.set_kernel_family("auto")
    gold = oracle_forward(pr["q"].float(), pr["k"].float(), pr["v"].float(), pr["cu_q_list"], pr["cu_k_list"], pr["mask"],
                          pr["qbs"], pr["kbs"], pr["causal"], None)
    st = error_stats(gold, out)
    assert st["max_abs"] <= 2e-2 and st["mean_abs"] <= 1e-3, st
