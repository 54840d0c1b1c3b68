"""Splitting one forward over several GPUs.

(sample, kv-head) units are independent in this operator - samples never attend across each other
(``hbsattn/reference.py:56-60``, ``fwd_triton_auto_tile_size.py:112-117``) and a kv-head touches only its own
q-heads, its k/v head and its mask plane (``fwd_triton_fix_tile_size.py:74,122``) - so a multi-GPU run needs no
collective on the data path: every rank computes whole units and the outputs are disjoint.

The split has two steps.

``plan_units``   assigns the units to ranks by longest processing time first on each unit's FLOPs over active
                 block pairs (varlen batches and causal masks make units differ by an order of magnitude).
``pack_units``   turns the units of one rank into ONE varlen problem: every unit becomes a sample of its own with
                 a single kv-head and the ``group`` q-heads that belong to it, and its mask plane becomes the rows of
                 a CSR block mask over the packed block indices.  A CSR mask holds only active pairs, so packing
                 units of different kv-heads side by side does not square the mask size the way a dense
                 ``(nhead_k, num_q_block, num_k_block)`` mask over global block indices would.

Both run on the host with numpy/torch arithmetic and take any device for the tensors they slice.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import numpy as np
import torch

Unit = Tuple[int, int]          # (sample, kv-head)


def unit_flops(decisions, cu_q_seqlens, cu_k_seqlens, q_block_size: int, k_block_size: int, headdim: int, group: int) -> np.ndarray:
    """FLOPs over active block pairs of every unit: float64 ``[batch, nhead_k]``.

    ``decisions``: bool ``[nhead_k, num_q_block, num_k_block]`` valid/skip decisions (``block_decisions`` of the
    package, or the oracle's).  A pair counts ``4 * rows(qb) * rows(kb) * headdim`` per q-head of the group."""
    dec = torch.as_tensor(decisions)
    cu_q = np.asarray(torch.as_tensor(cu_q_seqlens).cpu(), dtype=np.int64)
    cu_k = np.asarray(torch.as_tensor(cu_k_seqlens).cpu(), dtype=np.int64)
    batch = len(cu_q) - 1
    out = np.zeros((batch, dec.shape[0]), dtype=np.float64)
    nqb = (np.diff(cu_q) + q_block_size - 1) // q_block_size
    nkb = (np.diff(cu_k) + k_block_size - 1) // k_block_size
    cnq = np.concatenate([[0], np.cumsum(nqb)])
    cnk = np.concatenate([[0], np.cumsum(nkb)])
    for b in range(batch):
        rq = np.minimum(q_block_size, (cu_q[b + 1] - cu_q[b]) - np.arange(nqb[b]) * q_block_size).astype(np.float64)
        rk = np.minimum(k_block_size, (cu_k[b + 1] - cu_k[b]) - np.arange(nkb[b]) * k_block_size).astype(np.float64)
        plane = dec[:, cnq[b]:cnq[b + 1], cnk[b]:cnk[b + 1]].to(torch.float64)
        w = torch.as_tensor(np.outer(rq, rk), device=plane.device)
        out[b] = (plane * w).sum(dim=(1, 2)).cpu().numpy() * (4.0 * headdim * group)
    return out


def active_plane(mask_plane: torch.Tensor, q_len: int, k_len: int, q_block_size: int, k_block_size: int, causal: bool) -> torch.Tensor:
    """Valid/skip decision of one unit from its own mask plane ``[nqb, nkb]`` (bool, any device): the pair (qb, kb) is
    computed iff the mask has it and - under a causal mask aligned bottom-right - the first key of kb is not beyond
    what the last row of qb may see: ``kb * k_block_size <= min((qb + 1) * q_block_size, q_len) - 1 + (k_len - q_len)``.
    This is the block-level consequence of the element mask of ``hbsattn/reference.py:56-89``, the same rule the
    schedule kernel applies on the device."""
    if not causal:
        return mask_plane.clone()
    nqb, nkb = mask_plane.shape
    dev = mask_plane.device
    last_row = torch.clamp((torch.arange(nqb, device=dev) + 1) * q_block_size, max=q_len) - 1
    limit = last_row + (k_len - q_len)
    first_key = torch.arange(nkb, device=dev) * k_block_size
    return mask_plane & (first_key[None, :] <= limit[:, None])


def plane_flops(active: torch.Tensor, q_len: int, k_len: int, q_block_size: int, k_block_size: int, headdim: int, group: int) -> float:
    """FLOPs over the active pairs of one unit plane (``4 * rows(qb) * rows(kb) * headdim`` per pair and q-head)."""
    nqb, nkb = active.shape
    dev = active.device
    rq = torch.clamp(q_len - torch.arange(nqb, device=dev) * q_block_size, max=q_block_size).to(torch.float64)
    rk = torch.clamp(k_len - torch.arange(nkb, device=dev) * k_block_size, max=k_block_size).to(torch.float64)
    return float((active.to(torch.float64) * rq[:, None] * rk[None, :]).sum().item()) * 4.0 * headdim * group


def plan_units(flops: np.ndarray, world_size: int) -> List[List[Unit]]:
    """Longest-processing-time-first assignment of the ``[batch, nhead_k]`` units to ``world_size`` ranks.

    Units are taken from the most expensive to the cheapest (ties by (sample, kv-head)) and each goes to the rank
    with the least work so far (ties to the lowest rank), so every rank computes the same plan from the same
    ``flops``.  Returns the units of every rank in the order they were assigned."""
    assert world_size >= 1
    flops = np.asarray(flops, dtype=np.float64)
    batch, nhead_k = flops.shape
    order = sorted(((b, h) for b in range(batch) for h in range(nhead_k)), key=lambda u: (-flops[u[0], u[1]], u[0], u[1]))
    load = [0.0] * world_size
    plan: List[List[Unit]] = [[] for _ in range(world_size)]
    for u in order:
        r = min(range(world_size), key=lambda i: (load[i], i))
        plan[r].append(u)
        load[r] += float(flops[u[0], u[1]])
    return plan


def plan_imbalance(plan: Sequence[Sequence[Unit]], flops: np.ndarray) -> float:
    """max over ranks / mean over ranks of the planned FLOPs (1.0 = perfectly even)."""
    loads = [sum(float(flops[b, h]) for b, h in units) for units in plan]
    mean = sum(loads) / len(loads)
    return max(loads) / mean if mean > 0 else 1.0


@dataclass
class PackedUnits:
    """One rank's share as a single varlen problem (see ``pack_units``)."""
    units: List[Unit]
    q: torch.Tensor                 # [sum q_len, group, headdim]
    k: torch.Tensor                 # [sum k_len, 1, headdim]
    v: torch.Tensor
    cu_q_seqlens: torch.Tensor      # int32 [len(units) + 1]
    cu_k_seqlens: torch.Tensor
    csr_row_ptr: torch.Tensor       # int32 [num_q_block + 1]
    csr_col_idx: torch.Tensor       # int32 [nnz], packed k-block indices, ascending in every row
    num_q_block: int
    num_k_block: int
    q_block_size: int
    k_block_size: int
    q_rows: List[Tuple[int, int]] = field(default_factory=list)      # per unit: token range in the original q


def _blocks(length: int, bs: int) -> int:
    return (int(length) + bs - 1) // bs


def csr_of_plane(plane: torch.Tensor, col_base: int):
    """Row lengths and ascending column indices (+ ``col_base``) of a bool ``[rows, cols]`` mask plane."""
    nz = plane.nonzero()                      # row-major order: ascending columns inside every row
    counts = torch.bincount(nz[:, 0], minlength=plane.shape[0])
    return counts, (nz[:, 1] + col_base).to(torch.int32)


def pack_units(units: Sequence[Unit], q, k, v, cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size: int, k_block_size: int) -> PackedUnits:
    """Gathers the units ``(sample, kv-head)`` of one rank out of the full tensors into one packed problem.

    ``q``: ``[total_q, nhead_q, headdim]``, ``k``/``v``: ``[total_k, nhead_k, headdim]``, ``block_mask``: bool
    ``[nhead_k, num_q_block, num_k_block]`` over global block indices, as ``HBSAttention`` takes them.  The result
    has one sample per unit, ``nhead_k = 1`` and ``nhead_q = group``; entries of ``block_mask`` that pair blocks of
    different samples are dropped (the operator ignores them anyway)."""
    cu_q = [int(x) for x in torch.as_tensor(cu_q_seqlens).cpu()]
    cu_k = [int(x) for x in torch.as_tensor(cu_k_seqlens).cpu()]
    batch = len(cu_q) - 1
    group = q.shape[1] // k.shape[1]
    cnq, cnk = [0], [0]
    for b in range(batch):
        cnq.append(cnq[-1] + _blocks(cu_q[b + 1] - cu_q[b], q_block_size))
        cnk.append(cnk[-1] + _blocks(cu_k[b + 1] - cu_k[b], k_block_size))
    dev = q.device
    qs, ks, vs, counts, cols, rows = [], [], [], [], [], []
    new_cu_q, new_cu_k, kb_base = [0], [0], 0
    for (b, h) in units:
        qs.append(q[cu_q[b]:cu_q[b + 1], h * group:(h + 1) * group])
        ks.append(k[cu_k[b]:cu_k[b + 1], h:h + 1])
        vs.append(v[cu_k[b]:cu_k[b + 1], h:h + 1])
        c, idx = csr_of_plane(block_mask[h, cnq[b]:cnq[b + 1], cnk[b]:cnk[b + 1]], kb_base)
        counts.append(c)
        cols.append(idx)
        kb_base += cnk[b + 1] - cnk[b]
        new_cu_q.append(new_cu_q[-1] + cu_q[b + 1] - cu_q[b])
        new_cu_k.append(new_cu_k[-1] + cu_k[b + 1] - cu_k[b])
        rows.append((cu_q[b], cu_q[b + 1]))
    if not units:
        empty = q.new_zeros((0, group, q.shape[2]))
        z32 = torch.zeros(1, dtype=torch.int32, device=dev)
        return PackedUnits([], empty, k.new_zeros((0, 1, k.shape[2])), v.new_zeros((0, 1, v.shape[2])), z32, z32.clone(), z32.clone(),
                           torch.zeros(0, dtype=torch.int32, device=dev), 0, 0, q_block_size, k_block_size, [])
    all_counts = torch.cat(counts)
    row_ptr = torch.zeros(all_counts.numel() + 1, dtype=torch.int64, device=all_counts.device)
    row_ptr[1:] = torch.cumsum(all_counts, 0)
    assert int(row_ptr[-1]) < 2 ** 31, "CSR block masks are limited to 2^31 - 1 active pairs"
    return PackedUnits(
        units=list(units), q=torch.cat(qs).contiguous(), k=torch.cat(ks).contiguous(), v=torch.cat(vs).contiguous(),
        cu_q_seqlens=torch.tensor(new_cu_q, dtype=torch.int32, device=dev),
        cu_k_seqlens=torch.tensor(new_cu_k, dtype=torch.int32, device=dev),
        csr_row_ptr=row_ptr.to(torch.int32).to(dev), csr_col_idx=torch.cat(cols).to(dev),
        num_q_block=int(all_counts.numel()), num_k_block=int(kb_base), q_block_size=q_block_size, k_block_size=k_block_size, q_rows=rows)


def unpack_output(packed: PackedUnits, out_packed: torch.Tensor, out_full: torch.Tensor) -> None:
    """Writes a rank's packed output ``[sum q_len, group, headdim]`` into its places of the full ``[total_q, nhead_q, headdim]``."""
    group = out_packed.shape[1]
    pos = 0
    for (b, h), (r0, r1) in zip(packed.units, packed.q_rows):
        n = r1 - r0
        out_full[r0:r1, h * group:(h + 1) * group] = out_packed[pos:pos + n].to(out_full.device)
        pos += n


def dense_mask_of_csr(row_ptr, col_idx, nhead_k: int, num_q_block: int, num_k_block: int) -> torch.Tensor:
    """The dense bool ``[nhead_k, num_q_block, num_k_block]`` mask a CSR block mask stands for (small problems, tests)."""
    rp = torch.as_tensor(row_ptr).cpu().to(torch.int64)
    ci = torch.as_tensor(col_idx).cpu().to(torch.int64)
    mask = torch.zeros(nhead_k * num_q_block, num_k_block, dtype=torch.bool)
    rows = torch.repeat_interleave(torch.arange(nhead_k * num_q_block), rp[1:] - rp[:-1])
    mask[rows, ci] = True
    return mask.view(nhead_k, num_q_block, num_k_block)


def csr_of_mask(block_mask: torch.Tensor):
    """CSR form ``(row_ptr int32 [nhead_k * num_q_block + 1], col_idx int32 [nnz])`` of a dense block mask."""
    nhk, nqb, nkb = block_mask.shape
    counts, idx = csr_of_plane(block_mask.reshape(nhk * nqb, nkb), 0)
    row_ptr = torch.zeros(nhk * nqb + 1, dtype=torch.int64, device=block_mask.device)
    row_ptr[1:] = torch.cumsum(counts, 0)
    assert int(row_ptr[-1]) < 2 ** 31, "CSR block masks are limited to 2^31 - 1 active pairs"
    return row_ptr.to(torch.int32), idx


def kv_head_range(nhead_k: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous kv-head range of ``rank`` when a forward is split by kv-heads alone (ranges differ by at most
    one head).  The unit planner above balances better; this is the split to use when every rank must keep a
    zero-copy view ``q[:, h0 * group:h1 * group]``, ``k[:, h0:h1]``, ``block_mask[h0:h1]`` of shared tensors."""
    assert 0 <= rank < world_size and nhead_k >= 1
    base, extra = divmod(nhead_k, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)
