import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on the B200 box)")


class GoldenCase:
    """One fixture produced by tests/golden/make_golden.py from the unmodified reference."""

    def __init__(self, name, meta, arrs):
        self.name = name
        self.meta = meta
        self._arrs = arrs
        for key, val in meta.items():
            setattr(self, key, val)
        self.torch_dtype = getattr(torch, meta["dtype"])

    def tensor(self, field):
        key = f"{self.name}/{field}"
        if key + ".bf16bits" in self._arrs:
            bits = torch.from_numpy(self._arrs[key + ".bf16bits"].astype(np.int16))
            return bits.view(torch.bfloat16)
        return torch.from_numpy(np.asarray(self._arrs[key]))

    def array(self, field):
        return np.asarray(self._arrs[f"{self.name}/{field}"])


def _load_golden():
    with open(os.path.join(GOLDEN_DIR, "golden_cases.json")) as f:
        index = json.load(f)
    arrs = np.load(os.path.join(GOLDEN_DIR, "golden_cases.npz"))
    return [GoldenCase(name, meta, arrs) for name, meta in sorted(index.items())]


GOLDEN_CASES = _load_golden()


@pytest.fixture(params=GOLDEN_CASES, ids=[c.name for c in GOLDEN_CASES])
def golden_case(request):
    return request.param
