"""Block masks in CSR form (csr_row_ptr / csr_col_idx of the C ABI, HBSAttention_csr of the Python mirror) and the
unit packer built on them.

A CSR mask must give exactly what the dense mask it was made from gives: the same valid/skip decisions bit for
bit, and - because the schedule and therefore every row's sequence of K/V tiles is the same - the same output bit
for bit, for both kernel families.  Packing (sample, kv-head) units into one problem with one kv-head
(hbsattn_b200.shard) changes which rows share an M tile but not the arithmetic of any row, so the gathered output
of the packed problems equals the unsharded output bit for bit as well."""
import numpy as np
import pytest
import torch

from helpers import make_lengths, make_problem
from oracle import error_stats, oracle_block_decisions, oracle_forward

pytestmark = pytest.mark.gpu

CASES = [
    # name, q range, k range, hq, hk, d, qbs, kbs, causal, dtype
    ("mha_128x128_causal", (200, 900), None, 4, 4, 128, 128, 128, True, torch.bfloat16),
    ("gqa4_80x48", (100, 900), None, 8, 2, 128, 80, 48, False, torch.bfloat16),
    ("gqa8_16x128_bottom_right", (128, 512), (1000, 3000), 16, 2, 64, 16, 128, True, torch.float16),
    ("gqa2_64x256", (300, 900), (200, 1200), 4, 2, 128, 64, 256, True, torch.bfloat16),
    ("fp32_32x16_d18", (40, 200), (30, 220), 4, 2, 18, 32, 16, True, torch.float32),
]


def _problem(case, seed=21, batch=4):
    name, qr, kr, hq, hk, d, qbs, kbs, causal, dtype = case
    rng = np.random.default_rng(seed)
    q_lens = make_lengths(rng, batch, *qr)
    k_lens = q_lens if kr is None else make_lengths(rng, batch, *kr)
    return make_problem(seed, q_lens, k_lens, hq, hk, d, qbs, kbs, causal, dtype, 0.4, "first")


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_csr_equals_dense(case):
    import hbsattn_b200 as hb
    from hbsattn_b200.shard import csr_of_mask
    pr = _problem(case)
    row_ptr, col_idx = csr_of_mask(pr["mask"])
    nqb, nkb = pr["num_q_block"], pr["num_k_block"]
    dec_d, cnt_d = hb.block_decisions(pr["q"], pr["k"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"])
    dec_c, cnt_c = hb.block_decisions_csr(pr["q"], pr["k"], pr["cu_q"], pr["cu_k"], row_ptr, col_idx, nqb, nkb, pr["qbs"], pr["kbs"], pr["causal"])
    assert torch.equal(dec_d, dec_c) and torch.equal(cnt_d, cnt_c)
    want = oracle_block_decisions(pr["cu_q_list"], pr["cu_k_list"], pr["mask"].cpu(), pr["qbs"], pr["kbs"], pr["causal"])
    np.testing.assert_array_equal(dec_c.cpu().numpy(), want)
    families = ("generic",) if pr["q"].dtype == torch.float32 or pr["q"].shape[2] not in (64, 128) else ("sm100", "generic")
    for family in families:
        hb.set_kernel_family(family)
        try:
            dense = hb.HBSAttention(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"], None)
            csr = hb.HBSAttention_csr(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], row_ptr, col_idx, nqb, nkb, pr["qbs"], pr["kbs"], pr["causal"])
            assert hb.last_status()[0] == 0
        finally:
            hb.set_kernel_family("auto")
        assert torch.equal(dense, csr), family


def test_csr_ignores_other_samples_entries():
    """Entries that pair blocks of different samples are dropped, as for the dense mask (an all-True mask holds many)."""
    import hbsattn_b200 as hb
    from hbsattn_b200.shard import csr_of_mask
    pr = make_problem(5, [300, 200, 450], [310, 150, 500], 4, 2, 128, 64, 128, True, torch.bfloat16, 1.0, None)
    row_ptr, col_idx = csr_of_mask(torch.ones_like(pr["mask"]))
    out = hb.HBSAttention_csr(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], row_ptr, col_idx, pr["num_q_block"], pr["num_k_block"],
                              pr["qbs"], pr["kbs"], pr["causal"])
    gold = oracle_forward(pr["q"].float(), pr["k"].float(), pr["v"].float(), pr["cu_q_list"], pr["cu_k_list"], torch.ones_like(pr["mask"]),
                          pr["qbs"], pr["kbs"], pr["causal"], None)
    st = error_stats(gold, out)
    assert st["max_abs"] <= 2e-2 and st["mean_abs"] <= 1e-3, st


@pytest.mark.parametrize("case", CASES[:3], ids=[c[0] for c in CASES[:3]])
@pytest.mark.parametrize("world", [2, 3])
def test_packed_units_equal_unsharded(case, world):
    """The plan/pack/unpack path of a multi-GPU run, all "ranks" on this one GPU, one after the other."""
    import hbsattn_b200 as hb
    from hbsattn_b200.shard import pack_units, plan_units, unit_flops, unpack_output
    pr = _problem(case, seed=33, batch=5)
    hb.set_kernel_family("sm100")
    try:
        full = hb.HBSAttention(pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"], None)
        dec, _ = hb.block_decisions(pr["q"], pr["k"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"], pr["causal"])
        group = pr["q"].shape[1] // pr["k"].shape[1]
        flops = unit_flops(dec, pr["cu_q"], pr["cu_k"], pr["qbs"], pr["kbs"], pr["q"].shape[2], group)
        plan = plan_units(flops, world)
        assert sorted(u for units in plan for u in units) == sorted((b, h) for b in range(5) for h in range(pr["k"].shape[1]))
        got = torch.full_like(full, float("nan"))
        for units in plan:
            pk = pack_units(units, pr["q"], pr["k"], pr["v"], pr["cu_q"], pr["cu_k"], pr["mask"], pr["qbs"], pr["kbs"])
            out = hb.HBSAttention_csr(pk.q, pk.k, pk.v, pk.cu_q_seqlens, pk.cu_k_seqlens, pk.csr_row_ptr, pk.csr_col_idx,
                                      pk.num_q_block, pk.num_k_block, pr["qbs"], pr["kbs"], pr["causal"])
            assert hb.last_status()[0] == 0
            unpack_output(pk, out, got)
    finally:
        hb.set_kernel_family("auto")
    assert torch.equal(got, full)
