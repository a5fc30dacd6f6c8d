"""Register this package under the reference's import names.

After ``install()``::

    from rgd_triton.ops import FusedRMSNorm
    from rgd_triton.triton.normalization.rmsnorm_cached import triton_rms_func_fn
    from rgd_triton.triton.flash_attn.flash_attn_triton_cached import flash_attn_func

resolve to the sm_100a implementations, so models and tests written against
the reference package run unchanged.  ``install()`` refuses to shadow a real
``rgd_triton`` that is already imported unless ``force=True``.
"""
from __future__ import annotations

import sys
import types

from . import functional as F_
from . import ops

# reference module path -> names it exports (and that we provide)
_LAYOUT = {
    "rgd_triton.triton.flash_attn.flash_attn_triton_cached": ("flash_attn_func", "FlashAttnFunc"),
    "rgd_triton.triton.normalization.l2normalize_cached": ("triton_norm_func_fn", "Norm_Func"),
    "rgd_triton.triton.normalization.fused_l2normalize_cached": ("triton_fused_norm_func_fn", "Fused_Norm_Func"),
    "rgd_triton.triton.normalization.head_layernorm_cached": ("triton_fused_ln_func_fn", "Fused_LNQK_Func"),
    "rgd_triton.triton.normalization.rmsnorm_cached": ("triton_rms_func_fn", "RMS_Func"),
    "rgd_triton.triton.normalization.fused_rmsnorm_cached": ("triton_fused_rms_func_fn", "Fused_RMS_Func"),
    "rgd_triton.triton.rope.head_rope_cached": ("triton_rope_fn", "CombinedRoPEFunc"),
    "rgd_triton.triton.rope.fused_ln_rope_cached": ("triton_fused_ln_rope_fn", "FusedRoPEFunc"),
}


def install(force: bool = False) -> None:
    """Make ``import rgd_triton...`` resolve to this package."""
    existing = sys.modules.get("rgd_triton")
    if existing is not None and not getattr(existing, "__rgd_b200__", False) and not force:
        raise RuntimeError("a different rgd_triton is already imported; pass force=True to shadow it")

    def pkg(name: str) -> types.ModuleType:
        m = types.ModuleType(name)
        m.__path__ = []          # mark as package
        m.__rgd_b200__ = True
        sys.modules[name] = m
        return m

    root = pkg("rgd_triton")
    tri = pkg("rgd_triton.triton")
    root.triton = tri
    root.ops = ops
    sys.modules["rgd_triton.ops"] = ops
    for sub in ("flash_attn", "normalization", "rope"):
        setattr(tri, sub, pkg(f"rgd_triton.triton.{sub}"))
    for path, names in _LAYOUT.items():
        m = types.ModuleType(path)
        m.__rgd_b200__ = True
        for n in names:
            setattr(m, n, getattr(F_, n))
        sys.modules[path] = m
        parent, leaf = path.rsplit(".", 1)
        setattr(sys.modules[parent], leaf, m)


def uninstall() -> None:
    for name in [n for n, m in sys.modules.items() if n.split(".")[0] == "rgd_triton"
                 and (getattr(m, "__rgd_b200__", False) or m is ops)]:
        del sys.modules[name]
