"""Test infrastructure: CPU restatement of the reference's algorithm (see hbsa_oracle.py).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this package.
"""
from .hbsa_oracle import (  # noqa: F401
    oracle_calculate_blocks,
    oracle_block_decisions,
    oracle_forward,
    oracle_active_flops,
    error_stats,
)
