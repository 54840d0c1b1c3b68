"""Block metadata of a packed varlen batch - same name, arguments and return value as the
reference's ``hbsattn/utils.py:7-50`` (``calculate_blocks``), built by two CUDA kernels through
the C ABI instead of a dozen torch launches."""
from __future__ import annotations

import torch

from . import _lib


def _calculate_blocks_host(cu_seqlen: torch.Tensor, block_size: int):
    """Host arithmetic for a ``cu_seqlen`` that lives in CPU memory (mask construction and
    shard planning happen on the host; the attention itself never runs there)."""
    cu = cu_seqlen.to(torch.int64)
    lens = cu[1:] - cu[:-1]
    nblk = torch.clamp((lens + (block_size - 1)) // block_size, min=0)
    cu_num_block = torch.zeros(nblk.numel() + 1, dtype=cu_seqlen.dtype)
    cu_num_block[1:] = nblk.cumsum(0).to(cu_seqlen.dtype)
    num_block = int(cu_num_block[-1])
    block_to_batch = torch.repeat_interleave(torch.arange(nblk.numel()), nblk).to(torch.int32)
    first = cu_num_block[:-1].to(torch.int64)[block_to_batch.long()]
    idx_in_sample = torch.arange(num_block) - first
    b = block_to_batch.long()
    ends = torch.minimum(cu[b] + (idx_in_sample + 1) * block_size, cu[b + 1]) - cu[0]
    cu_block = torch.zeros(num_block + 1, dtype=torch.int32)
    cu_block[1:] = ends.to(torch.int32)
    return num_block, cu_block, block_to_batch, cu_num_block


def calculate_blocks(cu_seqlen: torch.Tensor, block_size: int):
    """Returns ``(num_block, cu_block, block_to_batch, cu_num_block)``.

    * ``num_block``      python int, total number of blocks (costs one device-to-host read,
                         as in the reference at ``utils.py:27``)
    * ``cu_block``       int32 ``[num_block+1]`` token offset of every block boundary
    * ``block_to_batch`` int32 ``[num_block]`` sample index of every block
    * ``cu_num_block``   ``[batch+1]`` first block index of every sample, in ``cu_seqlen``'s dtype
    """
    assert cu_seqlen.ndim == 1 and cu_seqlen.numel() >= 2, "cu_seqlen must be a 1D tensor of length batch + 1"
    block_size = int(block_size)
    assert block_size > 0, "block_size must be positive"
    if not cu_seqlen.is_cuda:
        return _calculate_blocks_host(cu_seqlen, block_size)
    lib = _lib.load()
    dev = cu_seqlen.device
    cu32 = cu_seqlen if cu_seqlen.dtype == torch.int32 else cu_seqlen.to(torch.int32)
    cu32 = cu32.contiguous()
    batch = cu32.numel() - 1
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        cu_num_block = torch.empty(batch + 1, dtype=torch.int32, device=dev)
        rc = lib.hbsa_calculate_blocks(cu32.data_ptr(), batch, block_size, 0, None, None, cu_num_block.data_ptr(), stream)
        if rc != 0:
            raise RuntimeError(f"hbsa_calculate_blocks failed ({rc}): {_lib.last_error()}")
        num_block = int(cu_num_block[-1].item())
        cu_block = torch.empty(num_block + 1, dtype=torch.int32, device=dev)
        block_to_batch = torch.empty(num_block, dtype=torch.int32, device=dev)
        if num_block > 0:
            rc = lib.hbsa_calculate_blocks(cu32.data_ptr(), batch, block_size, num_block, cu_block.data_ptr(),
                                           block_to_batch.data_ptr(), cu_num_block.data_ptr(), stream)
            if rc != 0:
                raise RuntimeError(f"hbsa_calculate_blocks failed ({rc}): {_lib.last_error()}")
        else:
            cu_block.zero_()
    if cu_num_block.dtype != cu_seqlen.dtype:
        cu_num_block = cu_num_block.to(cu_seqlen.dtype)
    return num_block, cu_block, block_to_batch, cu_num_block
