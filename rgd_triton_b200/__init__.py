"""rgd_triton_b200 — the rgd_triton operator set as hand-written sm_100a CUDA.

``rgd_triton_b200.ops`` mirrors ``rgd_triton.ops`` (module API);
``rgd_triton_b200.functional`` holds the autograd functions and the ``*_fn``
entries; ``rgd_triton_b200.compat.install()`` registers both under the
``rgd_triton`` import names so existing code runs unchanged.
"""
from . import ops, functional  # noqa: F401
from .ops import (  # noqa: F401
    CachableModule, FlashAttention, L2Normalize, FusedL2Normalize2, FusedHeadLayerNorm,
    FusedRMSNorm, FusedRMSNorm2, RoPE, FusedLNRoPE,
)

__version__ = "0.1.0"
