"""The shipped tensor-core kernel hands P to the P V product, and the S columns back to the next S product, without
the fences and completion waits a strictly conservative reading of the tcgen05 ordering rules would add: its MMA
thread does not execute tcgen05.fence::after_thread_sync after observing a barrier, and it issues S(t+1) of a lane
into the columns P(t) occupies right behind P V(t), relying on tcgen05.mma instructions of one thread executing in
issue order.  If either shortcut ever let a product read a stale or overwritten P, some output rows would be
silently wrong - within tolerance of nothing in particular.

So the check is bit-level: libhbsattn_b200_strict.so (hbsattn_b200/build.py --strict) is the same source with the
fences and the waits compiled in.  Five runs of the shipped library and one run of the strict library on the
headline workload and on a long-context workload must all produce bit-identical outputs."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STRICT = os.path.join(ROOT, "hbsattn_b200", "libhbsattn_b200_strict.so")
WORKER = os.path.join(ROOT, "tests", "fingerprint_worker.py")

pytestmark = pytest.mark.gpu


def _run(workload, repeats, out_path, library=None):
    env = dict(os.environ)
    env.pop("HBSATTN_B200_LIBRARY", None)
    if library is not None:
        env["HBSATTN_B200_LIBRARY"] = library
    res = subprocess.run([sys.executable, WORKER, workload, str(repeats), out_path], env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return torch.load(out_path)


@pytest.mark.parametrize("workload", ["cfg2", "cfg4_16k"])
def test_shipped_and_strict_builds_agree_bit_for_bit(workload, tmp_path):
    assert os.path.exists(STRICT), "build it with: python hbsattn_b200/build.py --strict"
    shipped = _run(workload, 5, str(tmp_path / "shipped.pt"))
    strict = _run(workload, 1, str(tmp_path / "strict.pt"), STRICT)
    assert strict["library"] == STRICT and shipped["library"] != STRICT
    ref = strict["prints"][0]
    for i, fp in enumerate(shipped["prints"]):
        bad = (fp != ref).nonzero().flatten()
        assert bad.numel() == 0, f"{workload}: run {i} of the shipped library differs from the strict build in {bad.numel()} tokens, first {bad[:8].tolist()}"
