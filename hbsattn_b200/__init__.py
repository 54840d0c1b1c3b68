"""hbsattn_b200 - B200 (sm_100a) heterogeneous block-sparse attention forward.

Drop-in for the forward path of the reference package: ``HBSAttention`` and
``calculate_blocks`` keep the reference's names, positional arguments and error behaviour
(``hbsattn/hbsa_interface.py``, ``hbsattn/utils.py``).  The work is done by hand-written CUDA
kernels behind a C ABI (``include/hbsattn_b200.h``); importing this package fails if the
compiled library is absent.
"""
from . import _lib as _lib_module

_lib_module.load()          # fail loudly at import time when the CUDA library is missing

from .hbsa_interface import (HBSAttention, HBSAttention_with_lse, MaskSchedule, attention_with_schedule, block_decisions,  # noqa: E402
                             build_schedule, last_status, set_kernel_family)
from .utils import calculate_blocks  # noqa: E402
from .host_staged import HostStagedAttention  # noqa: E402

__all__ = ["HBSAttention", "calculate_blocks", "block_decisions", "last_status", "set_kernel_family",
           "HBSAttention_with_lse", "HostStagedAttention", "MaskSchedule", "build_schedule", "attention_with_schedule", "install_as_hbsattn"]


def install_as_hbsattn() -> None:
    """Registers this package under the reference's module names so that
    ``from hbsattn import HBSAttention`` and ``from hbsattn.utils import calculate_blocks``
    (reference README, test/test_accuracy.py:14-15) resolve to the B200 implementation."""
    import sys
    from . import hbsa_interface, utils
    sys.modules.setdefault("hbsattn", sys.modules[__name__])
    sys.modules.setdefault("hbsattn.utils", utils)
    sys.modules.setdefault("hbsattn.hbsa_interface", hbsa_interface)
