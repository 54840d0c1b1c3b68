"""CPU oracle for the heterogeneous block-sparse attention forward.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module;
it is the checker used by the tests, by the smoke check and by the CPU-baseline
leg of the benchmark.  It is a vectorised restatement, in fp32 torch ops, of the
reference's PyTorch implementations:

  * ``oracle_calculate_blocks``  follows ``hbsattn/utils.py:7-50``
  * ``oracle_forward``           follows ``hbsattn/reference.py:23-107``
                                 (``hbsattn_reference_v1_base``) and is also
                                 equal to ``reference.py:188-265`` (v3)
  * ``oracle_block_decisions``   is the block-level consequence of the element
                                 mask built at ``reference.py:56-89`` /
                                 ``:209-247``: a (kv-head, q-block, k-block)
                                 pair is *active* iff at least one (row, key)
                                 element of it survives all three masks.

Parity pin: ``tests/golden/make_golden.py`` imports the unmodified reference,
runs it on seeded inputs and stores inputs and outputs under ``tests/golden``;
``tests/test_oracle_golden.py`` checks this module against those fixtures.
The reference loops in pure Python over (row, key) pairs for the causal mask
(``reference.py:72-77``); here the same predicate is evaluated with broadcast
integer compares, which is what makes sizes beyond a few hundred tokens usable.
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = [
    "oracle_calculate_blocks",
    "oracle_block_decisions",
    "oracle_forward",
    "oracle_active_flops",
    "error_stats",
]


def _as_int_list(x):
    if isinstance(x, torch.Tensor):
        return [int(v) for v in x.detach().cpu().tolist()]
    return [int(v) for v in np.asarray(x).tolist()]


def oracle_calculate_blocks(cu_seqlen, block_size: int):
    """Block tables of a packed varlen batch (``hbsattn/utils.py:7-50``).

    Returns ``(num_block, cu_block[int32, nb+1], block_to_batch[int32, nb],
    cu_num_block[int64, B+1])`` as numpy arrays.  ``cu_block`` holds global
    token offsets into the packed tensor; the last block of every sample is
    ragged (``utils.py:33-35``).
    """
    cu = _as_int_list(cu_seqlen)
    bs = int(block_size)
    cu_block = [0]
    block_to_batch = []
    cu_num_block = [0]
    for b in range(len(cu) - 1):
        length = cu[b + 1] - cu[b]
        nblk = (length + bs - 1) // bs
        for i in range(nblk):
            cu_block.append(min(cu[b] + (i + 1) * bs, cu[b + 1]))
            block_to_batch.append(b)
        cu_num_block.append(cu_num_block[-1] + nblk)
    return (
        cu_num_block[-1],
        np.asarray(cu_block, dtype=np.int32),
        np.asarray(block_to_batch, dtype=np.int32),
        np.asarray(cu_num_block, dtype=np.int64),
    )


def oracle_block_decisions(cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size, k_block_size, causal):
    """Exact valid/skip decision per (kv-head, q-block, k-block) as a bool array.

    active = block_mask  AND  same sample  AND  (not causal  OR  the last row of
    the q-block may see the first key of the k-block), with the bottom-right
    alignment ``offset = k_len - q_len`` of ``reference.py:64-77``.
    """
    cu_q = _as_int_list(cu_q_seqlens)
    cu_k = _as_int_list(cu_k_seqlens)
    nqb, cqb, qb2b, _ = oracle_calculate_blocks(cu_q, q_block_size)
    nkb, ckb, kb2b, _ = oracle_calculate_blocks(cu_k, k_block_size)
    bm = block_mask.detach().cpu().numpy() if isinstance(block_mask, torch.Tensor) else np.asarray(block_mask)
    assert bm.shape[1:] == (nqb, nkb), (bm.shape, nqb, nkb)
    cu_q_a = np.asarray(cu_q, dtype=np.int64)
    cu_k_a = np.asarray(cu_k, dtype=np.int64)
    same = qb2b[:, None] == kb2b[None, :]
    if causal:
        b_of_q = qb2b.astype(np.int64)
        off = (cu_k_a[b_of_q + 1] - cu_k_a[b_of_q]) - (cu_q_a[b_of_q + 1] - cu_q_a[b_of_q])
        last_row = cqb[1:].astype(np.int64) - 1 - cu_q_a[b_of_q]          # in-sample index of the last q row
        b_of_k = kb2b.astype(np.int64)
        first_key = ckb[:-1].astype(np.int64) - cu_k_a[b_of_k]            # in-sample index of the first key
        reach = (last_row + off)[:, None] >= first_key[None, :]
        same = same & reach
    return bm.astype(bool) & same[None, :, :]


def oracle_forward(q, k, v, cu_q_seqlens, cu_k_seqlens, block_mask, q_block_size, k_block_size,
                   causal, softmax_scale=None, return_lse=False):
    """fp32 block-sparse attention forward with the reference's semantics.

    For every q-block (``reference.py:46``) the scores against the keys of the
    q-block's own sample are formed in fp32 (``:52-53``; restricting to the
    sample's keys is the ``in_batch_mask`` of ``:56-60``), the causal
    (``:64-77``) and block (``:80-87``) masks are applied with ``-inf``
    (``:89-92``), a softmax over keys follows (``:95``) with rows that see no
    key set to zero (``:98``), and the result is the fp32 product with V cast
    to ``q.dtype`` (``:100-101``).  GQA: q-head ``h`` uses kv-head
    ``h // (Hq // Hk)`` (``:52``, ``:82``).

    ``return_lse=True`` also returns the natural-log sum of exponentials of every row's
    allowed scaled scores, fp32 ``[total_q, nhead_q]``, ``-inf`` for rows that see no key.
    The reference keeps no correct LSE (its Triton kernels store ``log(l)`` without the
    row maximum, ``fwd_triton_auto_tile_size.py:249``); this is the quantity a backward
    pass needs.
    """
    cu_q = _as_int_list(cu_q_seqlens)
    cu_k = _as_int_list(cu_k_seqlens)
    assert len(cu_q) == len(cu_k)
    nhead_q, nhead_k, headdim = q.shape[1], k.shape[1], q.shape[2]
    assert nhead_q % nhead_k == 0
    g = nhead_q // nhead_k
    scale = float(softmax_scale) if softmax_scale is not None else headdim ** -0.5
    nqb, cqb, qb2b, _ = oracle_calculate_blocks(cu_q, q_block_size)
    nkb, ckb, kb2b, cnk = oracle_calculate_blocks(cu_k, k_block_size)
    assert tuple(block_mask.shape) == (nhead_k, nqb, nkb)
    dev = q.device
    out = torch.empty_like(q)
    lse = torch.full((q.shape[0], nhead_q), float("-inf"), dtype=torch.float32, device=dev)
    ckb_t = torch.as_tensor(ckb.astype(np.int64), device=dev)
    head_k_of_q = torch.arange(nhead_q, device=dev) // g
    for qb in range(nqb):
        b = int(qb2b[qb])
        q0, q1 = int(cqb[qb]), int(cqb[qb + 1])
        ks, ke = cu_k[b], cu_k[b + 1]
        kb0, kb1 = int(cnk[b]), int(cnk[b + 1])
        rows = q1 - q0
        if ke == ks:
            out[q0:q1] = 0
            continue
        qf = q[q0:q1].float()                                   # [m, Hq, d]
        kf = k[ks:ke].float().repeat_interleave(g, dim=1)       # [s, Hq, d]
        vf = v[ks:ke].float().repeat_interleave(g, dim=1)
        s = torch.einsum("mhd,shd->msh", qf, kf) * scale         # [m, s, Hq]
        key_in = torch.arange(ke - ks, device=dev)               # in-sample key index
        # block id of every key of the sample, relative to the sample's first k-block
        key_blk = torch.bucketize(key_in + ks, ckb_t[kb0 + 1:kb1 + 1], right=True)
        bm = block_mask[:, qb, kb0:kb1].to(dev)                  # [Hk, nkb_sample]
        allowed = bm[head_k_of_q][:, key_blk]                    # [Hq, s]
        allowed = allowed.transpose(0, 1).unsqueeze(0).expand(rows, -1, -1)
        if causal:
            off = (ke - ks) - (cu_q[b + 1] - cu_q[b])
            q_in = torch.arange(q0 - cu_q[b], q1 - cu_q[b], device=dev)
            cm = (q_in[:, None] + off) >= key_in[None, :]        # [m, s]
            allowed = allowed & cm.unsqueeze(-1)
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=1)
        p = torch.nan_to_num(p, nan=0.0)
        out[q0:q1] = torch.einsum("msh,shd->mhd", p, vf)
        if return_lse:
            lse[q0:q1] = torch.logsumexp(s, dim=1)               # [m, Hq]; -inf where nothing is allowed
    return (out, lse) if return_lse else out


def oracle_active_flops(cu_q_seqlens, cu_k_seqlens, decisions, q_block_size, k_block_size, nhead_q, headdim):
    """FLOPs over active block pairs: ``sum 4 * rows(qb) * rows(kb) * d`` per q-head,
    with true (ragged) row counts; a partly causal-masked pair counts in full."""
    _, cqb, _, _ = oracle_calculate_blocks(cu_q_seqlens, q_block_size)
    _, ckb, _, _ = oracle_calculate_blocks(cu_k_seqlens, k_block_size)
    rq = np.diff(cqb).astype(np.float64)
    rk = np.diff(ckb).astype(np.float64)
    dec = np.asarray(decisions, dtype=np.float64)               # [Hk, NQB, NKB]
    g = nhead_q // dec.shape[0]
    pair_rows = np.einsum("hqk,q,k->", dec, rq, rk)
    return 4.0 * pair_rows * headdim * g


def error_stats(golden: torch.Tensor, result: torch.Tensor) -> dict:
    """max/mean absolute and relative error, defined as in ``hbsattn/benchmark.py:19-27``."""
    gf, rf = golden.float().cpu(), result.float().cpu()
    abs_error = (gf - rf).abs()
    rel_error = abs_error / (1e-4 + torch.maximum(gf.abs(), rf.abs()))
    return {
        "max_abs": abs_error.max().item() if abs_error.numel() else 0.0,
        "mean_abs": abs_error.mean().item() if abs_error.numel() else 0.0,
        "max_rel": rel_error.max().item() if rel_error.numel() else 0.0,
        "mean_rel": rel_error.mean().item() if rel_error.numel() else 0.0,
    }
