"""CPU oracle for the MoE-layer hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this.  Only the tests, the smoke check and
the CPU-baseline leg of the benchmark may call it, and only as the checker.
"""
from .moe_oracle import *  # noqa: F401,F403
from .seqmix_oracle import *  # noqa: F401,F403
