"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, the
struct mirror matches, argument validation rejects bad calls before any launch, and the host
arithmetic of calculate_blocks equals the oracle.  No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import oracle_calculate_blocks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import importlib.util
    spec = importlib.util.spec_from_file_location("hbsattn_b200_build", os.path.join(ROOT, "hbsattn_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)          # by path: importing the package itself needs the library
    mod.build()
    from hbsattn_b200 import _lib
    return _lib.load()


def test_header_symbols_are_exported(lib):
    from hbsattn_b200 import _lib
    header = open(os.path.join(ROOT, "include", "hbsattn_b200.h")).read()
    declared = set(re.findall(r"\b(hbsa_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.hbsa_version() == 4


def test_struct_mirror_size(lib):
    from hbsattn_b200 import _lib
    # 5 size_t/pointers + 12 int64 strides + 3 pointers + 3 int64 + 16 int32/float + 2 pointers/size_t
    assert ctypes.sizeof(_lib.ForwardArgs) == 8 * 5 + 8 * 12 + 8 * 3 + 8 * 3 + 4 * 16 + 8 * 2 + 8 + 8 * 2


def test_workspace_bytes(lib):
    assert lib.hbsa_workspace_bytes(0, 1, 1, 1) == 0
    small = lib.hbsa_workspace_bytes(2, 5, 12, 5)
    big = lib.hbsa_workspace_bytes(32, 4096, 4096, 8)
    assert 0 < small < big and small % 256 == 0 and big % 256 == 0
    assert big < 12 * 1024 * 1024         # a few ints per (kv-head, q-block) row, independent of num_k_block


def _args(**over):
    from hbsattn_b200 import _lib
    a = _lib.ForwardArgs()
    a.struct_bytes = ctypes.sizeof(_lib.ForwardArgs)
    fake = 0x1000
    a.q = a.k = a.v = a.o = fake
    a.cu_q_seqlens = a.cu_k_seqlens = a.block_mask = a.workspace = fake
    a.total_q = a.total_k = 64
    a.nhead_q, a.nhead_k, a.headdim, a.batch = 4, 2, 128, 1
    a.num_q_block = a.num_k_block = 4
    a.q_block_size = a.k_block_size = 16
    a.use_default_scale = 1
    a.workspace_bytes = 1 << 20
    for i, s in enumerate((4 * 128, 128, 1)):
        a.q_stride[i] = a.o_stride[i] = s
    for i, s in enumerate((2 * 128, 128, 1)):
        a.k_stride[i] = a.v_stride[i] = s
    for key, val in over.items():
        setattr(a, key, val)
    return a


@pytest.mark.parametrize("over,code", [
    (dict(nhead_q=3), -2), (dict(q_block_size=24), -3), (dict(k_block_size=0), -3), (dict(dtype=9), -4),
    (dict(workspace_bytes=16), -5), (dict(q=None), -1), (dict(struct_bytes=8), -8), (dict(headdim=512), -2),
])
def test_argument_errors_before_launch(lib, over, code):
    from hbsattn_b200 import _lib
    a = _args(**over)
    assert lib.hbsa_select_impl(ctypes.byref(a)) == code
    assert lib.hbsa_forward(ctypes.byref(a), None) == code
    assert len(_lib.last_error()) > 0


def test_kernel_family_selection(lib):
    from hbsattn_b200 import _lib
    assert lib.hbsa_select_impl(ctypes.byref(_args())) == _lib.HBSA_IMPL_SM100
    assert lib.hbsa_select_impl(ctypes.byref(_args(dtype=_lib.HBSA_DTYPE_F32))) == _lib.HBSA_IMPL_GENERIC
    assert lib.hbsa_select_impl(ctypes.byref(_args(headdim=18))) == _lib.HBSA_IMPL_GENERIC
    assert lib.hbsa_select_impl(ctypes.byref(_args(use_default_scale=0, softmax_scale=-1.0))) == _lib.HBSA_IMPL_GENERIC
    assert lib.hbsa_select_impl(ctypes.byref(_args(headdim=18, impl=_lib.HBSA_IMPL_SM100))) == -6
    assert "headdim" in _lib.last_error()


@pytest.mark.parametrize("block_size", [16, 32, 80, 128])
def test_host_calculate_blocks_matches_oracle(block_size):
    import hbsattn_b200
    rng = np.random.default_rng(block_size)
    for batch in (1, 5, 64):
        lens = rng.integers(1, 500, size=batch)
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        nb, cu_block, b2b, cnb = hbsattn_b200.calculate_blocks(torch.from_numpy(cu), block_size)
        onb, ocu_block, ob2b, ocnb = oracle_calculate_blocks(cu, block_size)
        assert nb == onb and isinstance(nb, int)
        np.testing.assert_array_equal(cu_block.numpy(), ocu_block)
        np.testing.assert_array_equal(b2b.numpy(), ob2b)
        np.testing.assert_array_equal(cnb.numpy(), ocnb)
        assert cu_block.dtype == torch.int32 and b2b.dtype == torch.int32 and cnb.dtype == torch.int32


def test_operator_refuses_cpu_tensors():
    import hbsattn_b200
    q = torch.zeros(16, 2, 16)
    cu = torch.tensor([0, 16], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        hbsattn_b200.HBSAttention(q, q, q, cu, cu, torch.ones(2, 1, 1, dtype=torch.bool), 16, 16, True, None)


def test_module_alias():
    import hbsattn_b200
    hbsattn_b200.install_as_hbsattn()
    from hbsattn import HBSAttention
    from hbsattn.utils import calculate_blocks
    assert HBSAttention is hbsattn_b200.HBSAttention and calculate_blocks is hbsattn_b200.calculate_blocks
