"""Forward for callers whose tensors live in (pinned) host memory.

The reference's callers keep q, k, v and the mask on the device (``test/test_speedup.py:88-115``).
A host that stages every batch through PCIe pays 3-4x the attention time in copies, and
the copy in and the copy out use opposite directions of the link, so consecutive batches can
overlap: while batch i is copied out, batch i + 1 is copied in.  ``HostStagedAttention`` keeps
two device slots and three streams (copy in, compute, copy out) and chains them with events;
every call is still one ``HBSAttention`` forward on the device tensors of its slot.

No result is cached and nothing is skipped: per call the inputs are copied in, the schedule is
built, the attention kernel runs and the output is copied out.
"""
from __future__ import annotations

import torch

from . import _lib
from .hbsa_interface import HBSAttention, last_workspace, read_status
from .utils import calculate_blocks


class HostStagedAttention:
    """``submit(...)`` enqueues one forward from host tensors into a host output tensor and returns
    without waiting; ``wait()`` blocks until everything submitted so far has landed in its output.

    All host tensors should be pinned; a host tensor must not be reused as an input of a later
    ``submit`` or read as an output before ``wait()`` (or ``done_event(ticket).synchronize()``).
    """

    def __init__(self, device=None, slots: int = 2):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("HostStagedAttention needs a CUDA device; there is no CPU path")
        self.slots = int(slots)
        with torch.cuda.device(self.device):
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self._dev = [dict() for _ in range(self.slots)]     # per slot: name -> device tensor
        self._ev_in = [None] * self.slots                   # inputs of the slot have landed
        self._ev_run = [None] * self.slots                  # the forward of the slot has run
        self._ev_out = [None] * self.slots                  # the output of the slot has been copied out
        self._count = 0

    def _buf(self, slot: int, name: str, like: torch.Tensor) -> torch.Tensor:
        t = self._dev[slot].get(name)
        if t is None or t.shape != like.shape or t.dtype != like.dtype:
            t = torch.empty(like.shape, dtype=like.dtype, device=self.device)
            self._dev[slot][name] = t
        return t

    def submit(self, q, k, v, cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size, k_block_size, causal,
               softmax_scale=None, out=None, tile_mode="auto"):
        """Arguments as ``HBSAttention`` but on the host.  Returns ``(out, ticket)``; ``out`` is the
        (pinned) host tensor the result is written to (allocated if not given)."""
        slot = self._count % self.slots
        if out is None:
            out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
        host = {"q": q, "k": k, "v": v, "cu_q": cu_q_seqlens, "cu_k": cu_k_seqlens, "mask": block_mask}
        with torch.cuda.device(self.device):
            # The caller's stream may have produced the host data through earlier GPU work.
            self.s_in.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.s_in):
                if self._ev_run[slot] is not None:
                    self.s_in.wait_event(self._ev_run[slot])      # the previous forward of this slot has read its inputs
                dev = {}
                for name, h in host.items():
                    d = self._buf(slot, name, h)
                    d.copy_(h, non_blocking=True)
                    dev[name] = d
                self._ev_in[slot] = torch.cuda.Event()
                self._ev_in[slot].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self._ev_in[slot])
                if self._ev_out[slot] is not None:
                    self.s_run.wait_event(self._ev_out[slot])     # the slot's previous output has left the device
                # block counts on the host: no device read-back on this path
                meta_q = calculate_blocks(cu_q_seqlens, q_block_size)
                meta_k = calculate_blocks(cu_k_seqlens, k_block_size)
                o = HBSAttention(dev["q"], dev["k"], dev["v"], dev["cu_q"], dev["cu_k"], dev["mask"], q_block_size,
                                 k_block_size, causal, softmax_scale, tile_mode, *meta_q, *meta_k)
                self._dev[slot]["out"] = o                         # keeps the tensor alive until the slot is reused
                self._dev[slot]["workspace"] = last_workspace()    # holds the device status words of this forward
                self._ev_run[slot] = torch.cuda.Event()
                self._ev_run[slot].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self._ev_run[slot])
                o.record_stream(self.s_out)
                out.copy_(o, non_blocking=True)
                self._ev_out[slot] = torch.cuda.Event()
                self._ev_out[slot].record(self.s_out)
        self._count += 1
        return out, self._count - 1

    def done_event(self, ticket: int) -> torch.cuda.Event:
        """Event that fires when the output of ``ticket`` is in host memory (valid until its slot is reused)."""
        if not (self._count - self.slots <= ticket < self._count):
            raise ValueError("ticket is too old or not submitted yet")
        return self._ev_out[ticket % self.slots]

    def wait(self) -> None:
        """Blocks until every submitted forward has landed, then reads the device status words of the last forward
        of every slot: a forward that gave up (``HBSA_STATUS_WAIT_LIMIT``) or found the block counts inconsistent
        with ``cu_*_seqlens`` raises here instead of handing back zeros silently."""
        with torch.cuda.device(self.device):
            self.s_out.synchronize()
            self.s_run.synchronize()
            self.s_in.synchronize()
            for slot in self._dev:
                ws = slot.get("workspace")
                if ws is not None:
                    status = read_status(ws)
                    if status[0] != _lib.HBSA_STATUS_OK:
                        raise RuntimeError(f"HostStagedAttention: device status {status[0]} (detail {status[1:4]})")
