"""lewi_surge_b200: the MoE-layer hot path of Lewi Surge as hand-written sm_100a CUDA kernels.

`ops` mirrors the reference's operator interface (modal/moe_permute.py, modal/padded_gmm.py),
`layer` runs the whole layer forward/backward, `ep` shards experts across GPUs, `_lib` binds the C ABI
(include/lewi_moe.h).  There is no CPU path in this package.
"""
from . import _lib, ops, layer  # noqa: F401
from ._lib import LewiError  # noqa: F401

__all__ = ["ops", "layer", "LewiError"]
