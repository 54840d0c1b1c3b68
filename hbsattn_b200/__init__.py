"""hbsattn_b200 - B200 (sm_100a) heterogeneous block-sparse attention forward.

Drop-in for the forward path of the reference package: ``HBSAttention`` and
``calculate_blocks`` keep the reference's names, positional arguments and error behaviour
(``hbsattn/hbsa_interface.py``, ``hbsattn/utils.py``).  The work is done by hand-written CUDA
kernels behind a C ABI (``include/hbsattn_b200.h``); importing this package fails if the
compiled library is absent.
"""
from . import _lib as _lib_module

_lib_module.load()          # fail loudly at import time when the CUDA library is missing

from .hbsa_interface import (HBSAttention, HBSAttention_csr, attention_backward, HBSAttention_with_lse, MaskSchedule, attention_with_schedule,  # noqa: E402
                             block_decisions, block_decisions_csr, build_schedule, last_status, set_kernel_family)
from .utils import calculate_blocks  # noqa: E402
from .host_staged import HostStagedAttention  # noqa: E402

__all__ = ["HBSAttention", "calculate_blocks", "block_decisions", "last_status", "set_kernel_family",
           "HBSAttention_with_lse", "HBSAttention_csr", "block_decisions_csr", "attention_backward", "HostStagedAttention", "MaskSchedule", "build_schedule", "attention_with_schedule", "install_as_hbsattn"]


def install_as_hbsattn(reference_package_dir=None) -> None:
    """Registers this package's operator under the reference's module names, so that
    ``from hbsattn import HBSAttention`` and ``from hbsattn.utils import calculate_blocks``
    (reference README, test/test_accuracy.py:14-15) resolve to the B200 implementation.

    The reference's own scripts also import ``hbsattn.reference`` (its PyTorch implementations) and
    ``hbsattn.benchmark`` (test/test_accuracy.py:9-13, test/test_speedup.py).  Those are not part of the forward
    this package replaces; pass the directory of an installed reference package (the one that holds its
    ``reference.py``) as ``reference_package_dir`` and they keep resolving to the reference's files, while
    ``hbsattn.HBSAttention``, ``hbsattn.hbsa_interface`` and ``hbsattn.utils`` are the ones of this package."""
    import sys
    import types
    from . import hbsa_interface, utils
    alias = types.ModuleType("hbsattn")
    alias.__doc__ = "alias of hbsattn_b200 under the reference's package name"
    alias.__path__ = [reference_package_dir] if reference_package_dir else []
    alias.HBSAttention = HBSAttention
    alias.hbsa_interface = hbsa_interface
    alias.utils = utils
    sys.modules["hbsattn"] = alias
    sys.modules["hbsattn.utils"] = utils
    sys.modules["hbsattn.hbsa_interface"] = hbsa_interface
