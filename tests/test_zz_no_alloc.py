"""hbsa_forward_static_scratch: the forward for hosts that cannot give the library scratch memory
(a server that owns all device memory in its own arena, a plug-in callback that may not call
cudaMalloc).  It must produce what hbsa_forward produces, call after call, while every call reuses
the same built-in scratch array and therefore starts from the previous call's leftovers - of a
larger problem, of a smaller one, or of a call that ended with an error status.

Collected last on purpose (file name), and self-contained: it passes alone in a fresh process and
after the rest of the suite."""
import ctypes

import pytest
import torch

from helpers import make_problem


def _args(lib_mod, pr, out, workspace, num_k_block=None):
    from hbsattn_b200.hbsa_interface import make_args
    a = make_args(pr["q"], pr["k"], pr["v"], out, pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"],
                  None, pr["num_q_block"], pr["num_k_block"] if num_k_block is None else num_k_block, workspace, lib_mod.HBSA_IMPL_AUTO)
    return a


def _static_status(lib, stream):
    st = (ctypes.c_int32 * 16)()
    assert lib.hbsa_static_scratch_status(ctypes.cast(st, ctypes.c_void_p), stream) == 0
    return list(st)


@pytest.mark.gpu
def test_static_scratch_matches_forward_twice_in_a_row():
    from hbsattn_b200 import _lib
    from hbsattn_b200.hbsa_interface import alloc_workspace, read_status
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    # Different problems in a row, so that every call starts from foreign leftovers: a mid-sized one, a larger
    # one on the other kernel geometry, and a much smaller one (fewer rows, fewer CTAs than the call before it).
    problems = [
        make_problem(31, [300, 520, 77], [300, 520, 77], 8, 2, 128, 128, 128, True, torch.bfloat16, 0.5, "diag"),
        make_problem(32, [200, 333, 1500, 800], [450, 900, 1500, 700], 4, 4, 64, 32, 48, False, torch.bfloat16, 0.4, "first"),
        make_problem(33, [130], [90], 2, 1, 128, 128, 128, True, torch.bfloat16, 1.0, None),
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
            assert _static_status(lib, stream)[0] == 0
            # the same kernels on the same inputs in the same order per row: not a bit may differ
            assert torch.equal(got, want), f"call {call}: max-abs difference {(got.float() - want.float()).abs().max().item()}"


@pytest.mark.gpu
def test_static_scratch_reports_a_device_status():
    """A block count that contradicts cu_seqlens is found on the device: nothing is computed, the output is zeros,
    and the status is readable although the caller holds no workspace pointer.  The next call is unaffected."""
    from hbsattn_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    pr = make_problem(34, [256, 300], [256, 300], 4, 2, 128, 128, 128, True, torch.bfloat16, 0.6, "diag")
    wide = torch.zeros(pr["mask"].shape[0], pr["mask"].shape[1], pr["mask"].shape[2] + 1, dtype=torch.bool, device=dev)
    wide[:, :, :-1] = pr["mask"]
    bad = dict(pr, mask=wide)
    got = torch.full_like(pr["q"], float("nan"))
    a = _args(_lib, bad, got, torch.empty(1, dtype=torch.uint8, device=dev), num_k_block=pr["num_k_block"] + 1)
    a.workspace, a.workspace_bytes = None, 0
    assert lib.hbsa_forward_static_scratch(ctypes.byref(a), stream) == 0, _lib.last_error()
    st = _static_status(lib, stream)
    assert st[0] == _lib.HBSA_STATUS_BLOCK_COUNT_MISMATCH and st[1] == pr["num_q_block"] and st[2] == pr["num_k_block"]
    assert (got == 0).all()
    good = torch.full_like(pr["q"], float("nan"))
    b = _args(_lib, pr, good, torch.empty(1, dtype=torch.uint8, device=dev))
    b.workspace, b.workspace_bytes = None, 0
    assert lib.hbsa_forward_static_scratch(ctypes.byref(b), stream) == 0, _lib.last_error()
    assert _static_status(lib, stream)[0] == 0
    assert torch.isfinite(good).all()


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
