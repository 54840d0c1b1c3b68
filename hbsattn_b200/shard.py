"""Splitting one forward over several GPUs.

(sample, kv-head) units are independent in this operator - samples never attend across each other
(``hbsattn/reference.py:56-60``) and a kv-head touches only its own q-heads, k/v head and mask plane
(``fwd_triton_fix_tile_size.py:74,122``) - so a multi-GPU run needs no collective on the data path.
The split used here is by kv-head: every rank takes a contiguous range of kv-heads with the q-heads of
their groups, as zero-copy views (the kernels take strides), and the outputs are concatenated along the
head dimension.
"""
from __future__ import annotations

from typing import Tuple


def kv_head_range(nhead_k: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous kv-head range of `rank`; ranges differ by at most one head."""
    assert 0 <= rank < world_size and nhead_k >= 1
    base, extra = divmod(nhead_k, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_by_kv_heads(q, k, v, block_mask, rank: int, world_size: int):
    """Views of (q, k, v, block_mask) holding the kv-heads of `rank` and their q-heads, plus the
    q-head slice the rank's output occupies in the full result. Empty range -> (None,)*4 + slice."""
    nhead_q, nhead_k = q.shape[1], k.shape[1]
    assert nhead_q % nhead_k == 0, "nhead_q must be divisible by nhead_k (for GQA)"
    group = nhead_q // nhead_k
    h0, h1 = kv_head_range(nhead_k, rank, world_size)
    q_slice = slice(h0 * group, h1 * group)
    if h1 == h0:
        return None, None, None, None, q_slice
    return q[:, q_slice], k[:, h0:h1], v[:, h0:h1], block_mask[h0:h1], q_slice
