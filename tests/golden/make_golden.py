"""Generate the golden fixtures in this folder from the UNMODIFIED reference.

Run once, in a container where the reference checkout is available:

    HBSATTN_REFERENCE=/path/to/hbsattn-checkout python tests/golden/make_golden.py

It imports ``hbsattn.reference`` / ``hbsattn.utils`` from that checkout (CPU only,
nothing is copied), runs ``hbsattn_reference_v1_base`` and
``hbsattn_reference_v3_qkallfirst`` on seeded inputs, and stores inputs and
outputs as ``golden_cases.npz`` plus an index ``golden_cases.json``.

The cases are: the README / ``test/test_accuracy.py:33-38`` layouts
(``cu_q=[0,32,64,96,128,160]``, ``cu_k`` equal or ``[0,32,61,100,134,157]``), a
spread over the parameter grid of ``test/test_accuracy.py:17-29``, and edge cases
(a q-block with no active k-block, ``q_len > k_len``).

The per-block valid/skip decision of the reference is derived from the
reference's own outputs: with ``q = 0`` every allowed key of a row gets the same
probability, and with ``v[s, :, j] = [key s lies in k-block j]`` the output
column ``j`` is the probability mass the row puts on k-block ``j`` - non-zero
exactly when some (row, key) element of that block pair survives the masks.
"""
import json
import os
import sys

import numpy as np
import torch

REF = os.environ.get("HBSATTN_REFERENCE")
if not REF or not os.path.isfile(os.path.join(REF, "hbsattn", "reference.py")):
    sys.exit("set HBSATTN_REFERENCE to the checkout of the reference (the directory that holds hbsattn/reference.py)")
sys.path.insert(0, REF)
sys.dont_write_bytecode = True
from hbsattn.reference import hbsattn_reference_v1_base, hbsattn_reference_v3_qkallfirst  # noqa: E402
from hbsattn.utils import calculate_blocks  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
CU_Q = [0, 32, 64, 96, 128, 160]
CU_K_SAME = [0, 32, 64, 96, 128, 160]
CU_K_DIFF = [0, 32, 61, 100, 134, 157]


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16)


def store(arrs, name, t):
    if t.dtype == torch.bfloat16:
        arrs[name + ".bf16bits"] = bf16_bits(t)
    else:
        arrs[name] = t.numpy()


def reference_decisions(cu_q, cu_k, block_mask, qbs, kbs, causal, nhead_q):
    nhk, nqb, nkb = block_mask.shape
    cu_q_t = torch.tensor(cu_q, dtype=torch.int32)
    cu_k_t = torch.tensor(cu_k, dtype=torch.int32)
    _, cqb, _, _ = calculate_blocks(cu_q_t, qbs)
    _, ckb, _, _ = calculate_blocks(cu_k_t, kbs)
    q = torch.zeros(cu_q[-1], nhead_q, nkb)
    k = torch.zeros(cu_k[-1], nhk, nkb)
    v = torch.zeros(cu_k[-1], nhk, nkb)
    for j in range(nkb):
        v[int(ckb[j]):int(ckb[j + 1]), :, j] = 1.0
    out = hbsattn_reference_v1_base(q, k, v, cu_q_t, cu_k_t, block_mask, qbs, kbs, causal, 1.0)
    g = nhead_q // nhk
    dec = np.zeros((nhk, nqb, nkb), dtype=np.uint8)
    for i in range(nqb):
        blk = out[int(cqb[i]):int(cqb[i + 1])]                 # [rows, Hq, nkb]
        hit = (blk > 0).any(dim=0).view(nhk, g, nkb).any(dim=1)
        dec[:, i, :] = hit.numpy()
    return dec


def run_case(name, seed, cu_q, cu_k, nhq, nhk, d, qbs, kbs, causal, scale, dtype, p_keep, force_first, arrs, index,
             kill_row=None):
    torch.manual_seed(seed)
    cu_q_t = torch.tensor(cu_q, dtype=torch.int32)
    cu_k_t = torch.tensor(cu_k, dtype=torch.int32)
    q = torch.randn(cu_q[-1], nhq, d, dtype=dtype)
    k = torch.randn(cu_k[-1], nhk, d, dtype=dtype)
    v = torch.randn(cu_k[-1], nhk, d, dtype=dtype)
    nqb, cqb, qb2b, cnq = calculate_blocks(cu_q_t, qbs)
    nkb, ckb, kb2b, cnk = calculate_blocks(cu_k_t, kbs)
    mask = torch.rand(nhk, nqb, nkb) < p_keep
    if force_first:                                           # test/test_accuracy.py:52-60
        for i in range(nqb):
            first = int((kb2b == qb2b[i]).nonzero()[0])
            mask[:, i, first] = True
    if kill_row is not None:                                  # a q-block that attends to nothing
        mask[:, kill_row, :] = False
    gold32 = hbsattn_reference_v1_base(q.float(), k.float(), v.float(), cu_q_t, cu_k_t, mask, qbs, kbs, causal, scale)
    v1 = hbsattn_reference_v1_base(q, k, v, cu_q_t, cu_k_t, mask, qbs, kbs, causal, scale)
    v3 = hbsattn_reference_v3_qkallfirst(q, k, v, cu_q_t, cu_k_t, mask, qbs, kbs, causal, scale)
    dec = reference_decisions(cu_q, cu_k, mask, qbs, kbs, causal, nhq)
    store(arrs, f"{name}/q", q)
    store(arrs, f"{name}/k", k)
    store(arrs, f"{name}/v", v)
    arrs[f"{name}/mask"] = mask.numpy()
    arrs[f"{name}/gold32"] = gold32.numpy()
    store(arrs, f"{name}/v1", v1)
    store(arrs, f"{name}/v3", v3)
    arrs[f"{name}/decisions"] = dec
    arrs[f"{name}/cu_q_block"] = cqb.numpy()
    arrs[f"{name}/cu_k_block"] = ckb.numpy()
    arrs[f"{name}/q_block_to_batch"] = qb2b.numpy()
    arrs[f"{name}/k_block_to_batch"] = kb2b.numpy()
    arrs[f"{name}/cu_num_q_block"] = cnq.numpy()
    arrs[f"{name}/cu_num_k_block"] = cnk.numpy()
    index[name] = dict(seed=seed, cu_q=cu_q, cu_k=cu_k, nhead_q=nhq, nhead_k=nhk, headdim=d, q_block_size=qbs,
                       k_block_size=kbs, causal=causal, softmax_scale=scale,
                       dtype=str(dtype).replace("torch.", ""), num_q_block=int(nqb), num_k_block=int(nkb))
    print(name, "ok", tuple(gold32.shape), "active", int(dec.sum()))


def main():
    arrs, index = {}, {}
    bf, f32 = torch.bfloat16, torch.float32
    # Config 1 of the baseline: README toy, seed 0, no forcing of the mask.
    run_case("cfg1", 0, CU_Q, CU_K_DIFF, 8, 2, 32, 32, 16, True, None, bf, 0.7, False, arrs, index)
    grid = [
        # name, seed, cu_k, hq, hk, d, qbs, kbs, causal, scale, dtype
        ("g00", 1, CU_K_SAME, 2, 2, 16, 16, 16, False, None, bf),
        ("g01", 2, CU_K_SAME, 8, 2, 16, 32, 32, True, 0.333, bf),
        ("g02", 3, CU_K_DIFF, 2, 2, 16, 80, 16, True, None, bf),
        ("g03", 4, CU_K_DIFF, 8, 2, 18, 16, 32, True, 0.333, f32),
        ("g04", 5, CU_K_DIFF, 2, 2, 18, 80, 32, False, None, f32),
        ("g05", 6, CU_K_SAME, 8, 2, 18, 32, 16, True, None, bf),
        ("g06", 7, CU_K_DIFF, 8, 2, 16, 32, 16, False, 0.333, f32),
        ("g07", 8, CU_K_SAME, 2, 2, 16, 80, 32, True, None, f32),
        ("g08", 9, CU_K_DIFF, 2, 2, 16, 16, 16, True, None, bf),
        ("g09", 10, CU_K_DIFF, 8, 2, 18, 80, 16, True, 0.333, bf),
    ]
    for name, seed, cu_k, hq, hk, d, qbs, kbs, causal, scale, dt in grid:
        run_case(name, seed, CU_Q, cu_k, hq, hk, d, qbs, kbs, causal, scale, dt, 0.7, True, arrs, index)
    # Edge cases: q_len > k_len (rows with no causal-valid key), a dead q-block, ragged q and k tails,
    # a block size larger than a whole sample.
    run_case("e00", 20, [0, 48, 100, 131], [0, 17, 80, 96], 4, 2, 32, 32, 16, True, None, bf, 0.8, False, arrs, index)
    run_case("e01", 21, [0, 40, 90], [0, 70, 183], 4, 1, 64, 16, 48, True, None, bf, 0.6, False, arrs, index,
             kill_row=1)
    run_case("e02", 22, [0, 33, 71], [0, 50, 95], 2, 2, 16, 128, 128, False, 0.5, f32, 1.0, False, arrs, index)
    np.savez_compressed(os.path.join(HERE, "golden_cases.npz"), **arrs)
    with open(os.path.join(HERE, "golden_cases.json"), "w") as f:
        json.dump(index, f, indent=1, sort_keys=True)
    print("wrote", len(index), "cases")


if __name__ == "__main__":
    main()
