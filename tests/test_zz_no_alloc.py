"""hbsa_forward_static_scratch: the forward for hosts that cannot give the library scratch memory
(a server that owns all device memory in its own arena, a plug-in callback that may not call
cudaMalloc).  It must produce what hbsa_forward produces, call after call, while every call reuses
the same built-in scratch array and therefore starts from the previous call's leftovers.

Collected last on purpose (file name), and self-contained: it passes alone in a fresh process and
after the rest of the suite."""
import ctypes

import pytest
import torch

from helpers import make_problem


def _args(lib_mod, pr, out, workspace):
    from hbsattn_b200.hbsa_interface import make_args
    a = make_args(pr["q"], pr["k"], pr["v"], out, pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"],
                  None, pr["num_q_block"], pr["num_k_block"], workspace, lib_mod.HBSA_IMPL_AUTO)
    return a


@pytest.mark.gpu
def test_static_scratch_matches_forward_twice_in_a_row():
    from hbsattn_b200 import _lib
    from hbsattn_b200.hbsa_interface import alloc_workspace, read_status
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    # Two different problems, so that the second call really starts from foreign leftovers.
    problems = [
        make_problem(31, [300, 520, 77], [300, 520, 77], 8, 2, 128, 128, 128, True, torch.bfloat16, 0.5, "diag"),
        make_problem(32, [200, 333], [450, 900], 4, 4, 64, 32, 48, False, torch.bfloat16, 0.4, "first"),
    ]
    for pr in problems:
        want = torch.empty_like(pr["q"])
        ws = alloc_workspace(pr["k"].shape[1], pr["num_q_block"], pr["num_k_block"], pr["cu_q"].numel() - 1, dev)
        a = _args(_lib, pr, want, ws)
        assert lib.hbsa_forward(ctypes.byref(a), stream) == 0, _lib.last_error()
        assert read_status(ws)[0] == 0
        for call in range(2):
            got = torch.full_like(pr["q"], float("nan"))
            b = _args(_lib, pr, got, ws)
            b.workspace, b.workspace_bytes = None, 0            # the entry point must not need them
            rc = lib.hbsa_forward_static_scratch(ctypes.byref(b), stream)
            assert rc == 0, _lib.last_error()
            torch.cuda.synchronize()
            assert torch.isfinite(got).all(), f"call {call}: rows were left unwritten"
            # same kernels on the same inputs: the suite's tolerance (max-abs 2e-2), in practice bit-equal
            assert (got.float() - want.float()).abs().max().item() <= 2e-2, f"call {call}"


def test_static_scratch_rejects_oversized_problem():
    """Refused on the host before any CUDA call, with the needed size in the message."""
    from hbsattn_b200 import _lib
    lib = _lib.load()
    a = _lib.ForwardArgs()
    a.struct_bytes = ctypes.sizeof(_lib.ForwardArgs)
    a.nhead_k, a.num_q_block, a.num_k_block, a.batch = 64, 1 << 16, 1 << 16, 8     # 4M rows
    need = lib.hbsa_workspace_bytes(64, 1 << 16, 1 << 16, 8)
    assert need > _lib.STATIC_SCRATCH_BYTES
    assert lib.hbsa_forward_static_scratch(ctypes.byref(a), None) == -5
    msg = _lib.last_error()
    assert str(need) in msg and str(_lib.STATIC_SCRATCH_BYTES) in msg
