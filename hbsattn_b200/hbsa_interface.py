"""Operator API of the block-sparse attention forward.

Same callable, same positional arguments, same assertions and exception types as the
reference's ``hbsattn/hbsa_interface.py:6-35``; the body hands raw pointers, strides and sizes
to ``hbsa_forward`` of the C ABI, which builds the block metadata and the work schedule on the
device and runs the sm_100a attention kernel on torch's current stream.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.HBSA_DTYPE_BF16, torch.float16: _lib.HBSA_DTYPE_F16, torch.float32: _lib.HBSA_DTYPE_F32}
_IMPLS = {"auto": _lib.HBSA_IMPL_AUTO, "generic": _lib.HBSA_IMPL_GENERIC, "sm100": _lib.HBSA_IMPL_SM100}

_state = {"impl": os.environ.get("HBSATTN_B200_IMPL", "auto"), "last_workspace": None}


def set_kernel_family(name: str) -> None:
    """``'auto'`` (default), ``'sm100'`` (tcgen05 kernel, error if ineligible) or ``'generic'``."""
    if name not in _IMPLS:
        raise ValueError(f"Invalid kernel family: {name}")
    _state["impl"] = name


def _validate_default() -> bool:
    return os.environ.get("HBSATTN_B200_VALIDATE", "1") != "0"


def read_status(workspace: torch.Tensor):
    """Synchronises and returns the 16 device status words of a forward's workspace."""
    lib = _lib.load()
    out = (ctypes.c_int32 * _lib.STATUS_WORDS)()
    with torch.cuda.device(workspace.device):
        stream = torch.cuda.current_stream(workspace.device).cuda_stream
        rc = lib.hbsa_read_status(workspace.data_ptr(), ctypes.cast(out, ctypes.c_void_p), stream)
    if rc != 0:
        raise RuntimeError(f"hbsa_read_status failed ({rc}): {_lib.last_error()}")
    return list(out)


def last_workspace():
    """Workspace tensor of the most recent forward of this process (its first 16 int32 words are the device status)."""
    return _state["last_workspace"]


def last_status():
    """Status words of the most recent forward on this process (synchronises)."""
    ws = _state["last_workspace"]
    return read_status(ws) if ws is not None else [0] * _lib.STATUS_WORDS


def make_args(q, k, v, out, cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size, k_block_size, causal,
              softmax_scale, num_q_block, num_k_block, workspace, impl, lse=None, csr=None):
    """``block_mask``: the dense bool mask, or None when ``csr = (row_ptr, col_idx)`` (int32 device tensors) is given."""
    a = _lib.ForwardArgs()
    a.struct_bytes = ctypes.sizeof(_lib.ForwardArgs)
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.o = out.data_ptr() if out is not None else None
    for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("o_stride", out if out is not None else q)):
        arr = getattr(a, name)
        for i in range(3):
            arr[i] = t.stride(i)
    a.cu_q_seqlens = cu_q_seqlens.data_ptr()
    a.cu_k_seqlens = cu_k_seqlens.data_ptr()
    if block_mask is not None:
        a.block_mask = block_mask.data_ptr()
        for i in range(3):
            a.mask_stride[i] = block_mask.stride(i)      # bool: one byte per element
    if csr is not None:
        a.csr_row_ptr, a.csr_col_idx = csr[0].data_ptr(), csr[1].data_ptr()
    a.total_q, a.total_k = q.shape[0], k.shape[0]
    a.nhead_q, a.nhead_k, a.headdim = q.shape[1], k.shape[1], q.shape[2]
    a.batch = cu_q_seqlens.numel() - 1
    a.num_q_block, a.num_k_block = int(num_q_block), int(num_k_block)
    a.q_block_size, a.k_block_size = int(q_block_size), int(k_block_size)
    a.causal = 1 if causal else 0
    a.use_default_scale = 1 if softmax_scale is None else 0
    a.softmax_scale = 0.0 if softmax_scale is None else float(softmax_scale)
    a.dtype = _DTYPES[q.dtype]
    a.impl = impl
    a.workspace = workspace.data_ptr()
    a.workspace_bytes = workspace.numel()
    a.lse = lse.data_ptr() if lse is not None else None
    return a


def _prepare(q, k, v, cu_q_seqlens, cu_k_seqlens, block_mask):
    if not (q.is_cuda and k.is_cuda and v.is_cuda and block_mask.is_cuda and cu_q_seqlens.is_cuda and cu_k_seqlens.is_cuda):
        raise RuntimeError("hbsattn_b200 runs on CUDA tensors only (sm_100a); there is no CPU path")
    assert q.ndim == 3 and k.ndim == 3 and v.ndim == 3, "q, k, v must be (seqlen, nhead, headdim)"
    assert q.dtype == k.dtype == v.dtype and q.dtype in _DTYPES, "q, k, v must share a dtype of bfloat16, float16 or float32"
    assert k.shape == v.shape and q.shape[2] == k.shape[2], "k and v must have the same shape and q's headdim"
    assert len(cu_q_seqlens) == len(cu_k_seqlens) and cu_q_seqlens.ndim == 1 and cu_k_seqlens.ndim == 1, \
        "cu_q_seqlens and cu_k_seqlens must be 1D tensors of same length"
    if cu_q_seqlens.dtype != torch.int32:
        cu_q_seqlens = cu_q_seqlens.to(torch.int32)
    if cu_k_seqlens.dtype != torch.int32:
        cu_k_seqlens = cu_k_seqlens.to(torch.int32)
    return cu_q_seqlens.contiguous(), cu_k_seqlens.contiguous()


def alloc_workspace(nhead_k, num_q_block, num_k_block, batch, device) -> torch.Tensor:
    nbytes = _lib.load().hbsa_workspace_bytes(nhead_k, num_q_block, num_k_block, batch)
    return torch.empty(nbytes, dtype=torch.uint8, device=device)     # torch's CUDA allocations are 512-byte aligned


class _HBSAttentionFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size, k_block_size, causal,
                softmax_scale, tile_mode='auto', num_q_block=None, cu_q_block=None, q_block_to_batch=None,
                cu_num_q_block=None, num_k_block=None, cu_k_block=None, k_block_to_batch=None, cu_num_k_block=None):
        """``q``: (total_q, nhead_q, headdim); ``k``, ``v``: (total_k, nhead_k, headdim), packed varlen.
        ``block_mask``: bool (nhead_k, num_q_block, num_k_block) over global block indices.
        The eight trailing arguments are the outputs of ``calculate_blocks`` for q and k; they are
        accepted for compatibility (``test/test_accuracy.py:72``) - only the two block counts are used,
        the tables themselves are rebuilt on the device from ``cu_*_seqlens``.  When they are given the call
        does not synchronise: should the counts contradict ``cu_*_seqlens`` the device notices, computes
        nothing and returns zeros, and ``last_status()`` reports ``HBSA_STATUS_BLOCK_COUNT_MISMATCH``.
        Returns a contiguous (total_q, nhead_q, headdim) tensor in ``q``'s dtype.
        """
        have_meta = not (num_q_block is None or cu_q_block is None or q_block_to_batch is None or cu_num_q_block is None
                         or num_k_block is None or cu_k_block is None or k_block_to_batch is None or cu_num_k_block is None)
        assert block_mask.dtype == torch.bool, "block_mask must be a boolean tensor"
        assert block_mask.ndim == 3, "block_mask must have shape (nheads_k, num_q_block, num_k_block)"
        if have_meta:
            assert block_mask.shape == (k.shape[1], num_q_block, num_k_block), \
                f"block_mask must be a boolean tensor of shape (nheads_k, num_q_block, num_k_block) = ({k.shape[1]}, {num_q_block}, {num_k_block})"
        else:
            assert block_mask.shape[0] == k.shape[1], \
                f"block_mask must be a boolean tensor of shape (nheads_k, num_q_block, num_k_block); nheads_k = {k.shape[1]}"
            num_q_block, num_k_block = block_mask.shape[1], block_mask.shape[2]

        if tile_mode == 'auto':
            pass
        elif tile_mode == 'fix':
            assert (q_block_size & (q_block_size - 1) == 0) and (k_block_size & (k_block_size - 1) == 0), \
                "q_block_size and k_block_size must be powers of 2"
        else:
            raise ValueError(f"Invalid tile mode: {tile_mode}")

        assert q.shape[1] % k.shape[1] == 0, "nhead_q must be divisible by nhead_k (for GQA)"
        assert q_block_size % 16 == 0 and k_block_size % 16 == 0 and q_block_size > 0 and k_block_size > 0, \
            "q_block_size and k_block_size must be integer multiples of 16."

        cu_q32, cu_k32 = _prepare(q, k, v, cu_q_seqlens, cu_k_seqlens, block_mask)
        lib = _lib.load()
        dev = q.device
        want_grad = any(ctx.needs_input_grad[:3])
        with torch.cuda.device(dev):
            out = torch.empty(q.shape, dtype=q.dtype, device=dev)
            if q.shape[0] == 0:
                return out
            ws = alloc_workspace(k.shape[1], num_q_block, num_k_block, cu_q32.numel() - 1, dev)
            # the backward starts from the log-sum-exp of every row: keep it when a gradient is wanted
            lse = torch.empty((q.shape[0], q.shape[1]), dtype=torch.float32, device=dev) if want_grad else None
            args = make_args(q, k, v, out, cu_q32, cu_k32, block_mask, q_block_size, k_block_size, causal, softmax_scale,
                             num_q_block, num_k_block, ws, _IMPLS[_state["impl"]], lse=lse)
            if want_grad:
                ctx.save_for_backward(q, k, v, out, lse, cu_q32, cu_k32, block_mask)
                ctx.hbsa = (int(q_block_size), int(k_block_size), bool(causal), softmax_scale, int(num_q_block), int(num_k_block))
            stream = torch.cuda.current_stream(dev).cuda_stream
            rc = lib.hbsa_forward(ctypes.byref(args), stream)
            if rc != 0:
                raise RuntimeError(f"hbsa_forward failed ({rc}): {_lib.last_error()}")
            _state["last_workspace"] = ws
            if not have_meta and _validate_default():
                # The reference computes the block tables here (one host sync) and asserts the mask
                # shape against them (hbsa_interface.py:14-20); the device did the same check.
                status = read_status(ws)
                assert status[0] != _lib.HBSA_STATUS_BLOCK_COUNT_MISMATCH, \
                    f"block_mask must be a boolean tensor of shape (nheads_k, num_q_block, num_k_block) = ({k.shape[1]}, {status[1]}, {status[2]})"
                if status[0] != _lib.HBSA_STATUS_OK:
                    raise RuntimeError(f"hbsa_forward: device status {status[0]} (work item {status[3]})")
        return out

    @staticmethod
    def backward(ctx, do):
        """dq, dk, dv over the active block pairs (``hbsa_backward`` of the C ABI).  The reference raises
        ``NotImplementedError`` here (``hbsattn/hbsa_interface.py:30-32``)."""
        q, k, v, out, lse, cu_q32, cu_k32, block_mask = ctx.saved_tensors
        qbs, kbs, causal, softmax_scale, nqb, nkb = ctx.hbsa
        dq, dk, dv = attention_backward(q, k, v, out, lse, do, cu_q32, cu_k32, block_mask, qbs, kbs, causal, softmax_scale, nqb, nkb)
        return (dq, dk, dv) + (None,) * 16


HBSAttention = _HBSAttentionFunction.apply


def attention_backward(q, k, v, out, lse, d_out, cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size, k_block_size, causal,
                       softmax_scale=None, num_q_block=None, num_k_block=None):
    """Gradients of ``HBSAttention`` with respect to q, k and v, given the forward's output and ``lse``
    (``HBSAttention_with_lse``): returns ``(dq, dk, dv)`` in the dtype and shapes of q, k, v."""
    assert lse is not None and lse.dtype == torch.float32 and lse.shape == (q.shape[0], q.shape[1]), "lse must be float32 [total_q, nhead_q]"
    assert d_out.shape == q.shape, "the output gradient must have the shape of q"
    cu_q32, cu_k32 = _prepare(q, k, v, cu_q_seqlens, cu_k_seqlens, block_mask)
    if d_out.dtype != q.dtype:
        d_out = d_out.to(q.dtype)
    nqb = block_mask.shape[1] if num_q_block is None else num_q_block
    nkb = block_mask.shape[2] if num_k_block is None else num_k_block
    lib = _lib.load()
    dev = q.device
    with torch.cuda.device(dev):
        dq = torch.empty(q.shape, dtype=q.dtype, device=dev)
        dk = torch.empty(k.shape, dtype=k.dtype, device=dev)
        dv = torch.empty(v.shape, dtype=v.dtype, device=dev)
        if q.shape[0] == 0 or k.shape[0] == 0:
            return dq.zero_(), dk.zero_(), dv.zero_()
        ws = alloc_workspace(k.shape[1], nqb, nkb, cu_q32.numel() - 1, dev)
        b = _lib.BackwardArgs()
        b.struct_bytes = ctypes.sizeof(_lib.BackwardArgs)
        b.fwd = make_args(q, k, v, out, cu_q32, cu_k32, block_mask, q_block_size, k_block_size, causal, softmax_scale, nqb, nkb, ws,
                          _lib.HBSA_IMPL_AUTO, lse=lse.contiguous())
        b.d_o = d_out.data_ptr()
        for i in range(3):
            b.do_stride[i] = d_out.stride(i)
        b.dq, b.dk, b.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        nbytes = lib.hbsa_backward_workspace_bytes(q.shape[0], k.shape[0], q.shape[1], k.shape[1], q.shape[2])
        gws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        b.grad_workspace, b.grad_workspace_bytes = gws.data_ptr(), nbytes
        rc = lib.hbsa_backward(ctypes.byref(b), torch.cuda.current_stream(dev).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"hbsa_backward failed ({rc}): {_lib.last_error()}")
        _state["last_workspace"] = ws
        gws.record_stream(torch.cuda.current_stream(dev))
    return dq, dk, dv


def block_decisions(q, k, cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size, k_block_size, causal):
    """The valid/skip decision of every (kv-head, q-block, k-block) pair as the forward takes it:
    returns ``(decisions bool [nhead_k, num_q_block, num_k_block], counts int32 [nhead_k, num_q_block])``."""
    cu_q32, cu_k32 = _prepare(q, k, k, cu_q_seqlens, cu_k_seqlens, block_mask)
    lib = _lib.load()
    dev = q.device
    nhk, nqb, nkb = block_mask.shape
    with torch.cuda.device(dev):
        ws = alloc_workspace(nhk, nqb, nkb, cu_q32.numel() - 1, dev)
        args = make_args(q, k, k, None, cu_q32, cu_k32, block_mask, q_block_size, k_block_size, causal, 1.0,
                         nqb, nkb, ws, _lib.HBSA_IMPL_AUTO)
        dec = torch.empty((nhk, nqb, nkb), dtype=torch.uint8, device=dev)
        counts = torch.empty((nhk, nqb), dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = lib.hbsa_block_decisions(ctypes.byref(args), dec.data_ptr(), counts.data_ptr(), stream)
        if rc != 0:
            raise RuntimeError(f"hbsa_block_decisions failed ({rc}): {_lib.last_error()}")
        _state["last_workspace"] = ws
    return dec.bool(), counts


def _check_csr(row_ptr, col_idx, nhead_k, num_q_block):
    assert row_ptr.is_cuda and col_idx.is_cuda, "the CSR block mask must live on the device"
    assert row_ptr.dtype == torch.int32 and col_idx.dtype == torch.int32, "csr_row_ptr and csr_col_idx must be int32"
    assert row_ptr.ndim == 1 and row_ptr.numel() == nhead_k * num_q_block + 1, \
        f"csr_row_ptr must have nheads_k * num_q_block + 1 = {nhead_k * num_q_block + 1} entries"
    return row_ptr.contiguous(), col_idx.contiguous()


def HBSAttention_csr(q, k, v, cu_q_seqlens, cu_k_seqlens, csr_row_ptr, csr_col_idx, num_q_block, num_k_block,
                     q_block_size, k_block_size, causal, softmax_scale=None):
    """``HBSAttention`` with the block mask in CSR form: row ``hk * num_q_block + qb`` of ``csr_row_ptr`` (int32
    ``[nhead_k * num_q_block + 1]``) owns the global k-block indices ``csr_col_idx[row_ptr[r]:row_ptr[r + 1]]`` (int32,
    ascending) that q-block ``qb`` of kv-head ``hk`` attends to.  The reference takes dense masks only; this form
    holds nothing but the active pairs, which is what lets ``hbsattn_b200.shard.pack_units`` put units of different
    kv-heads into one call.  ``num_q_block`` / ``num_k_block`` are the block counts ``calculate_blocks`` returns."""
    assert q.shape[1] % k.shape[1] == 0, "nhead_q must be divisible by nhead_k (for GQA)"
    assert q_block_size % 16 == 0 and k_block_size % 16 == 0 and q_block_size > 0 and k_block_size > 0, \
        "q_block_size and k_block_size must be integer multiples of 16."
    cu_q32, cu_k32 = _prepare(q, k, v, cu_q_seqlens, cu_k_seqlens, csr_row_ptr)
    row_ptr, col_idx = _check_csr(csr_row_ptr, csr_col_idx, k.shape[1], num_q_block)
    lib = _lib.load()
    dev = q.device
    with torch.cuda.device(dev):
        out = torch.empty(q.shape, dtype=q.dtype, device=dev)
        if q.shape[0] == 0:
            return out
        ws = alloc_workspace(k.shape[1], num_q_block, num_k_block, cu_q32.numel() - 1, dev)
        args = make_args(q, k, v, out, cu_q32, cu_k32, None, q_block_size, k_block_size, causal, softmax_scale,
                         num_q_block, num_k_block, ws, _IMPLS[_state["impl"]], csr=(row_ptr, col_idx))
        rc = lib.hbsa_forward(ctypes.byref(args), torch.cuda.current_stream(dev).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"hbsa_forward failed ({rc}): {_lib.last_error()}")
        _state["last_workspace"] = ws
        if _validate_default():
            status = read_status(ws)
            assert status[0] != _lib.HBSA_STATUS_BLOCK_COUNT_MISMATCH, \
                f"num_q_block / num_k_block must be ({status[1]}, {status[2]}) for these cu_seqlens and block sizes"
            if status[0] != _lib.HBSA_STATUS_OK:
                raise RuntimeError(f"hbsa_forward: device status {status[0]} (work item {status[3]})")
    return out


def block_decisions_csr(q, k, cu_q_seqlens, cu_k_seqlens, csr_row_ptr, csr_col_idx, num_q_block, num_k_block,
                        q_block_size, k_block_size, causal, want_bitmap=True):
    """``block_decisions`` for a CSR block mask (see ``HBSAttention_csr``).  With ``want_bitmap=False`` only the counts
    are computed and the first element of the result is None (the dense bitmap of a packed long-context problem can be
    far larger than the problem itself)."""
    cu_q32, cu_k32 = _prepare(q, k, k, cu_q_seqlens, cu_k_seqlens, csr_row_ptr)
    nhk = k.shape[1]
    row_ptr, col_idx = _check_csr(csr_row_ptr, csr_col_idx, nhk, num_q_block)
    lib = _lib.load()
    dev = q.device
    with torch.cuda.device(dev):
        ws = alloc_workspace(nhk, num_q_block, num_k_block, cu_q32.numel() - 1, dev)
        args = make_args(q, k, k, None, cu_q32, cu_k32, None, q_block_size, k_block_size, causal, 1.0,
                         num_q_block, num_k_block, ws, _lib.HBSA_IMPL_AUTO, csr=(row_ptr, col_idx))
        dec = torch.empty((nhk, num_q_block, num_k_block), dtype=torch.uint8, device=dev) if want_bitmap else None
        counts = torch.empty((nhk, num_q_block), dtype=torch.int32, device=dev)
        rc = lib.hbsa_block_decisions(ctypes.byref(args), dec.data_ptr() if want_bitmap else None, counts.data_ptr(),
                                      torch.cuda.current_stream(dev).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"hbsa_block_decisions failed ({rc}): {_lib.last_error()}")
        _state["last_workspace"] = ws
    return (dec.bool() if want_bitmap else None), counts


class MaskSchedule:
    """The work schedule of one (cu_q_seqlens, cu_k_seqlens, block_mask, block sizes, causal) layout, built once
    on the device by ``build_schedule`` and reused by ``attention_with_schedule`` for every call that shares the
    layout (the layers of a model, the steps of a decode loop).  The reference's callers reuse the outputs of
    ``calculate_blocks`` the same way (``test/test_speedup.py:100-102,152``); here the reusable part also holds the
    active k-block counts and the ordered work-item table, so a reused call launches the attention kernel alone.

    The tensors the schedule was built from must stay alive and unchanged while it is in use, and calls that share
    a schedule must not overlap on the GPU (the kernel's work cursor lives in the schedule)."""

    def __init__(self, workspace, cu_q32, cu_k32, block_mask, q_block_size, k_block_size, causal):
        self.workspace = workspace
        self.cu_q_seqlens, self.cu_k_seqlens, self.block_mask = cu_q32, cu_k32, block_mask
        self.q_block_size, self.k_block_size, self.causal = int(q_block_size), int(k_block_size), bool(causal)
        self.nhead_k, self.num_q_block, self.num_k_block = block_mask.shape


def build_schedule(q, k, cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size, k_block_size, causal) -> MaskSchedule:
    """``q`` and ``k`` only say which shapes, dtype and device the later calls will have; they are not read."""
    assert block_mask.dtype == torch.bool and block_mask.ndim == 3, "block_mask must be a boolean tensor of shape (nheads_k, num_q_block, num_k_block)"
    assert block_mask.shape[0] == k.shape[1], f"block_mask must have nheads_k = {k.shape[1]} planes"
    assert q_block_size % 16 == 0 and k_block_size % 16 == 0 and q_block_size > 0 and k_block_size > 0, \
        "q_block_size and k_block_size must be integer multiples of 16."
    cu_q32, cu_k32 = _prepare(q, k, k, cu_q_seqlens, cu_k_seqlens, block_mask)
    lib = _lib.load()
    dev = q.device
    nhk, nqb, nkb = block_mask.shape
    with torch.cuda.device(dev):
        ws = alloc_workspace(nhk, nqb, nkb, cu_q32.numel() - 1, dev)
        args = make_args(q, k, k, None, cu_q32, cu_k32, block_mask, q_block_size, k_block_size, causal, None, nqb, nkb, ws,
                         _IMPLS[_state["impl"]])
        rc = lib.hbsa_build_schedule(ctypes.byref(args), torch.cuda.current_stream(dev).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"hbsa_build_schedule failed ({rc}): {_lib.last_error()}")
        _state["last_workspace"] = ws
    return MaskSchedule(ws, cu_q32, cu_k32, block_mask, q_block_size, k_block_size, causal)


def attention_with_schedule(q, k, v, schedule: MaskSchedule, softmax_scale=None):
    """``HBSAttention`` for a layout whose schedule is already on the device: one kernel launch."""
    assert q.shape[1] % k.shape[1] == 0, "nhead_q must be divisible by nhead_k (for GQA)"
    assert k.shape[1] == schedule.nhead_k, "k has a different number of heads than the schedule's block_mask"
    s = schedule
    _prepare(q, k, v, s.cu_q_seqlens, s.cu_k_seqlens, s.block_mask)
    lib = _lib.load()
    dev = q.device
    with torch.cuda.device(dev):
        out = torch.empty(q.shape, dtype=q.dtype, device=dev)
        if q.shape[0] == 0:
            return out
        args = make_args(q, k, v, out, s.cu_q_seqlens, s.cu_k_seqlens, s.block_mask, s.q_block_size, s.k_block_size, s.causal,
                         softmax_scale, s.num_q_block, s.num_k_block, s.workspace, _IMPLS[_state["impl"]])
        rc = lib.hbsa_attention(ctypes.byref(args), torch.cuda.current_stream(dev).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"hbsa_attention failed ({rc}): {_lib.last_error()}")
        _state["last_workspace"] = s.workspace
    return out


def HBSAttention_with_lse(q, k, v, cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size, k_block_size, causal,
                          softmax_scale=None):
    """``HBSAttention`` that also returns the natural-log sum of exponentials of every row's allowed scaled
    scores: ``(out, lse)`` with ``lse`` float32 ``[total_q, nhead_q]``, ``-inf`` for rows that see no key.
    The reference has no such output (its kernels keep ``log(l)`` without the row maximum,
    ``fwd_triton_auto_tile_size.py:249``, and drop it); it is what a backward pass starts from."""
    assert block_mask.dtype == torch.bool, "block_mask must be a boolean tensor"
    assert block_mask.ndim == 3 and block_mask.shape[0] == k.shape[1], \
        f"block_mask must be a boolean tensor of shape (nheads_k, num_q_block, num_k_block); nheads_k = {k.shape[1]}"
    assert q.shape[1] % k.shape[1] == 0, "nhead_q must be divisible by nhead_k (for GQA)"
    assert q_block_size % 16 == 0 and k_block_size % 16 == 0 and q_block_size > 0 and k_block_size > 0, \
        "q_block_size and k_block_size must be integer multiples of 16."
    cu_q32, cu_k32 = _prepare(q, k, v, cu_q_seqlens, cu_k_seqlens, block_mask)
    lib = _lib.load()
    dev = q.device
    nhk, nqb, nkb = block_mask.shape
    with torch.cuda.device(dev):
        out = torch.empty(q.shape, dtype=q.dtype, device=dev)
        lse = torch.empty((q.shape[0], q.shape[1]), dtype=torch.float32, device=dev)
        if q.shape[0] == 0:
            return out, lse
        ws = alloc_workspace(nhk, nqb, nkb, cu_q32.numel() - 1, dev)
        args = make_args(q, k, v, out, cu_q32, cu_k32, block_mask, q_block_size, k_block_size, causal, softmax_scale,
                         nqb, nkb, ws, _IMPLS[_state["impl"]], lse=lse)
        rc = lib.hbsa_forward(ctypes.byref(args), torch.cuda.current_stream(dev).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"hbsa_forward failed ({rc}): {_lib.last_error()}")
        _state["last_workspace"] = ws
        if _validate_default():
            status = read_status(ws)
            assert status[0] != _lib.HBSA_STATUS_BLOCK_COUNT_MISMATCH, \
                f"block_mask must be a boolean tensor of shape (nheads_k, num_q_block, num_k_block) = ({k.shape[1]}, {status[1]}, {status[2]})"
            if status[0] != _lib.HBSA_STATUS_OK:
                raise RuntimeError(f"hbsa_forward: device status {status[0]} (work item {status[3]})")
    return out, lse
