"""Shared input builders for the GPU parity tests (seeded, shaped like the reference's own tests)."""
import numpy as np
import torch

from oracle import oracle_calculate_blocks


def make_lengths(rng, batch, lo, hi, round_to=1):
    lens = rng.integers(lo, hi + 1, size=batch)
    lens = np.maximum((lens // round_to) * round_to, round_to)
    return [int(x) for x in lens]


def cu_from(lens):
    out = [0]
    for n in lens:
        out.append(out[-1] + int(n))
    return out


def make_problem(seed, q_lens, k_lens, nhead_q, nhead_k, headdim, qbs, kbs, causal, dtype, p_keep,
                 force="first", device="cuda"):
    """q/k/v ~ N(0,1), Bernoulli(p_keep) block mask over global block indices.
    force: "first" = first in-sample k-block forced True (test/test_accuracy.py:52-60),
           "diag"  = the last causal-valid k-block of every q-block forced True, None = nothing."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    cu_q, cu_k = cu_from(q_lens), cu_from(k_lens)
    q = torch.randn(cu_q[-1], nhead_q, headdim, generator=g).to(dtype)
    k = torch.randn(cu_k[-1], nhead_k, headdim, generator=g).to(dtype)
    v = torch.randn(cu_k[-1], nhead_k, headdim, generator=g).to(dtype)
    nqb, cqb, qb2b, cnq = oracle_calculate_blocks(cu_q, qbs)
    nkb, ckb, kb2b, cnk = oracle_calculate_blocks(cu_k, kbs)
    mask = torch.rand(nhead_k, nqb, nkb, generator=g) < p_keep
    if force is not None:
        for i in range(nqb):
            b = int(qb2b[i])
            first, last = int(cnk[b]), int(cnk[b + 1]) - 1
            if last < first:
                continue
            if force == "first":
                mask[:, i, first] = True
            else:
                off = (cu_k[b + 1] - cu_k[b]) - (cu_q[b + 1] - cu_q[b])
                limit = int(cqb[i + 1]) - 1 - cu_q[b] + off
                if limit >= 0:
                    mask[:, i, min(last, first + limit // kbs)] = True
    dev = torch.device(device)
    return dict(
        q=q.to(dev), k=k.to(dev), v=v.to(dev),
        cu_q=torch.tensor(cu_q, dtype=torch.int32, device=dev),
        cu_k=torch.tensor(cu_k, dtype=torch.int32, device=dev),
        cu_q_list=cu_q, cu_k_list=cu_k, mask=mask.to(dev), qbs=qbs, kbs=kbs, causal=causal,
        num_q_block=nqb, num_k_block=nkb,
    )
