"""Parity at the benchmark's own sizes (BASELINE configurations 2, 3, 4 and 5, and a 16k-token cut of 4).

The whole output is compared with the generic CUDA-core kernel (a second, independently written
implementation), and randomly chosen (sample, kv-head) units - which are independent of each other,
so the slice is exact - are compared with the fp32 oracle.  Tolerances as everywhere: max-abs <= 2e-2,
mean-abs <= 1e-3; the decision counts must match the oracle's bitmap exactly on the sliced units."""
import numpy as np
import pytest
import torch

import bench
from oracle import error_stats, oracle_block_decisions, oracle_forward

pytestmark = pytest.mark.gpu


def _forward(hb, wl, family):
    w = wl["w"]
    hb.set_kernel_family(family)
    try:
        mq = hb.calculate_blocks(wl["cu_q_t"], w["qbs"])
        mk = hb.calculate_blocks(wl["cu_k_t"], w["kbs"])
        out = hb.HBSAttention(wl["q"], wl["k"], wl["v"], wl["cu_q_t"], wl["cu_k_t"], wl["mask"], w["qbs"], w["kbs"],
                              w["causal"], None, "auto", *mq, *mk)
        assert hb.last_status()[0] == 0
        return out
    finally:
        hb.set_kernel_family("auto")


@pytest.mark.parametrize("name", ["cfg2", "cfg3", "cfg5", "cfg4_16k", "cfg4"])
def test_benchmark_workload_parity(name):
    import hbsattn_b200 as hb
    dev = torch.device("cuda", torch.cuda.current_device())
    if name == "cfg4" and torch.cuda.get_device_properties(dev).total_memory < 40 * 2 ** 30:
        pytest.skip("the 65536-token workload holds 17 GB of q/k/v/o plus two outputs")
    torch.cuda.empty_cache()
    wl = bench.make_workload(name, 0, dev)
    w = wl["w"]
    out = _forward(hb, wl, "sm100")
    assert torch.isfinite(out).all()
    ref = _forward(hb, wl, "generic")
    diff = (out.float() - ref.float()).abs()
    assert diff.max().item() <= 2e-2 and diff.mean().item() <= 1e-3, (diff.max().item(), diff.mean().item())
    del ref, diff
    dec, counts = hb.block_decisions(wl["q"], wl["k"], wl["cu_q_t"], wl["cu_k_t"], wl["mask"], w["qbs"], w["kbs"], w["causal"])
    g = w["hq"] // w["hk"]
    rng = np.random.default_rng(1)
    for _ in range(3):
        s, h = int(rng.integers(w["batch"])), int(rng.integers(w["hk"]))
        q0, q1 = int(wl["cu_q"][s]), int(wl["cu_q"][s + 1])
        k0, k1 = int(wl["cu_k"][s]), int(wl["cu_k"][s + 1])
        qb0, qb1 = int(wl["cnq"][s]), int(wl["cnq"][s + 1])
        kb0, kb1 = int(wl["cnk"][s]), int(wl["cnk"][s + 1])
        msk = wl["mask"][h:h + 1, qb0:qb1, kb0:kb1]
        gold = oracle_forward(wl["q"][q0:q1, h * g:(h + 1) * g].float(), wl["k"][k0:k1, h:h + 1].float(),
                              wl["v"][k0:k1, h:h + 1].float(), [0, q1 - q0], [0, k1 - k0], msk, w["qbs"], w["kbs"], w["causal"], None)
        st = error_stats(gold, out[q0:q1, h * g:(h + 1) * g])
        assert st["max_abs"] <= 2e-2 and st["mean_abs"] <= 1e-3, (name, s, h, st)
        want = oracle_block_decisions([0, q1 - q0], [0, k1 - k0], msk.cpu(), w["qbs"], w["kbs"], w["causal"])
        np.testing.assert_array_equal(dec[h, qb0:qb1, kb0:kb1].cpu().numpy(), want[0])
