"""Module API of the operator set: the eight ``nn.Module`` s of the reference's
``rgd_triton/ops.py`` (lines 12-249) with the same class names, constructor and
``forward`` signatures, defaults, parameter names (``weight``, ``weight1``,
``weight2``) and ``enable_cache`` / ``.cache`` behaviour, backed by the sm_100a
CUDA library instead of Triton kernels.

``state_dict`` s interchange with the reference: only the two RMSNorm modules
own parameters, under the same names and initialised to ones.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import functional as F_


class _LaunchCache:
    """Named slots, one per kernel of an operator (``fwd``, ``bwd``, ...), plus
    the native launch-plan cache of the C library.

    A slot holds the launch key (shapes, strides, dtypes, device) that was last
    validated for that kernel; a call with the same key skips host-side
    validation, a call with a different key re-validates and replaces it.
    ``native()`` is the ``rgd_cache`` handle (created on first use) in which the
    library keeps the encoded TMA descriptors of the calls this module made.
    """

    def __init__(self, fields):
        for name in fields:
            setattr(self, name, None)
        self._native = None

    def native(self):
        if self._native is None:
            from . import _lib
            self._native = _lib.load().rgd_cache_create()
        return self._native

    def stats(self):
        """(hits, misses, entries) of the native descriptor cache."""
        import ctypes as C
        from . import _lib
        h, m, e = C.c_int64(0), C.c_int64(0), C.c_int64(0)
        if self._native is not None:
            _lib.load().rgd_cache_stats(self._native, C.byref(h), C.byref(m), C.byref(e))
        return h.value, m.value, e.value

    def __del__(self):
        native, self._native = getattr(self, "_native", None), None
        if native is not None:
            try:
                from . import _lib
                _lib.load().rgd_cache_destroy(native)
            except Exception:       # interpreter shutdown
                pass

    # the native handle belongs to this process and this object only
    # (the marshalled arguments kept under "_plan_*" hold raw pointers and "_tiles" the tile lists of
    # the last bias tensor: they stay behind too)
    def __getstate__(self):
        state = {k: v for k, v in vars(self).items() if not k.startswith("_plan_") and k != "_tiles"}
        state["_native"] = None
        return state

    def __deepcopy__(self, memo):
        new = _LaunchCache(())
        for k, v in vars(self).items():
            if not k.startswith("_plan_") and k != "_tiles":
                setattr(new, k, None if k == "_native" else v)
        return new

    def __repr__(self):
        slots = {k: v for k, v in vars(self).items() if not k.startswith("_")}
        return "LaunchCache(" + ", ".join(f"{k}={'set' if v is not None else None}" for k, v in slots.items()) + ")"


class CachableModule(nn.Module):
    """Base class holding the per-module launch cache (ops.py:12-24 of the
    reference).  ``enable_cache(False)`` sets ``.cache`` to ``None``;
    ``enable_cache(True)`` installs a fresh, empty cache."""

    def __init__(self, cache_fields=None):
        super().__init__()
        self._cache_fields = tuple(cache_fields or ())
        self.cache = self._make_cache()

    def _make_cache(self):
        return _LaunchCache(self._cache_fields)

    def enable_cache(self, enable=True):
        self.cache = self._make_cache() if enable else None


class FlashAttention(CachableModule):
    """softmax(q k^T * softmax_scale + bias) v.  q: (B, Tq, h, d); k, v:
    (B, Tk, h, d); bias 4-D with last dims (1, Tk) or (Tq, Tk)."""

    def __init__(self):
        super().__init__(cache_fields=("fwd", "bwd_odot", "bwd"))
        self._fn = F_.flash_attn_func

    def forward(self, q, k, v, bias=None, causal=False, softmax_scale=None):
        return self._fn(q=q, k=k, v=v, bias=bias, causal=causal, softmax_scale=softmax_scale,
                        kernel_cache=self.cache)


class L2Normalize(CachableModule):
    """x / max(||x||, eps) over the last dim of a [B, N, C] tensor."""

    def __init__(self):
        super().__init__(cache_fields=("fwd", "bwd"))
        self._fn = F_.triton_norm_func_fn

    def forward(self, x, eps=1e-6):
        return self._fn(x=x, norm_eps=eps, kernel_cache=self.cache)


class FusedL2Normalize2(CachableModule):
    """L2Normalize on two tensors (same batch, any lengths / widths) in one launch."""

    def __init__(self):
        super().__init__(cache_fields=("fwd", "bwd"))
        self._fn = F_.triton_fused_norm_func_fn

    def forward(self, x1, x2, eps=1e-6):
        return self._fn(x1=x1, x2=x2, norm_eps=eps, kernel_cache=self.cache)


class FusedHeadLayerNorm(CachableModule):
    """Non-affine LayerNorm over head_dim of query and key in one launch.
    ``heads_second=True`` means [B, H, N, d], ``False`` means [B, N, H, d]."""

    def __init__(self):
        super().__init__(cache_fields=("fwd", "bwd"))
        self._fn = F_.triton_fused_ln_func_fn

    def forward(self, query, key, heads_second=True, eps=1e-6):
        return self._fn(query=query, key=key, heads_second=heads_second, norm_eps=eps, kernel_cache=self.cache)


class FusedRMSNorm(CachableModule):
    """RMSNorm over the last dim of [B, N, C] times an affine weight."""

    def __init__(self, normalized_shape, eps=1e-6, elementwise_affine=True, device=None, dtype=None):
        super().__init__(cache_fields=("fwd", "bwd", "bwd_dw"))
        if not isinstance(normalized_shape, int):
            raise AssertionError("Fused RMSNorm only supports int dims")
        self.normalized_shape = (normalized_shape,)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if self.elementwise_affine:
            self.weight = nn.Parameter(torch.empty(self.normalized_shape, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
        self.reset_parameters()
        self._fn = F_.triton_rms_func_fn

    def reset_parameters(self) -> None:
        if self.elementwise_affine:
            nn.init.ones_(self.weight)

    def forward(self, x, weight=None):
        if self.elementwise_affine:
            weight = self.weight   # a passed-in weight is ignored, as in the reference
        elif weight is None:
            raise AssertionError("Must pass in a weight tensor if not using element-wise affine")
        return self._fn(x=x, w=weight, norm_eps=self.eps, kernel_cache=self.cache)


class FusedRMSNorm2(CachableModule):
    """Two RMSNorms (separate widths and weights, same batch) in one launch."""

    def __init__(self, normalized_shape, eps=1e-6, elementwise_affine=True, device=None, dtype=None):
        super().__init__(cache_fields=("fwd", "bwd", "bwd_dw"))
        if not (isinstance(normalized_shape, (tuple, list)) and len(normalized_shape) == 2):
            raise AssertionError("Fused RMSNorm2 requires 2 int dims")
        self.normalized_shape1 = (normalized_shape[0],)
        self.normalized_shape2 = (normalized_shape[1],)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if self.elementwise_affine:
            self.weight1 = nn.Parameter(torch.empty(self.normalized_shape1, device=device, dtype=dtype))
            self.weight2 = nn.Parameter(torch.empty(self.normalized_shape2, device=device, dtype=dtype))
        else:
            self.register_parameter("weight1", None)
            self.register_parameter("weight2", None)
        self.reset_parameters()
        self._fn = F_.triton_fused_rms_func_fn

    def reset_parameters(self) -> None:
        if self.elementwise_affine:
            nn.init.ones_(self.weight1)
            nn.init.ones_(self.weight2)

    def forward(self, x1, x2, weight1=None, weight2=None):
        if self.elementwise_affine:
            weight1, weight2 = self.weight1, self.weight2
        elif weight1 is None or weight2 is None:
            raise AssertionError("Must pass in a weight tensor if not using element-wise affine")
        return self._fn(x1=x1, x2=x2, w1=weight1, w2=weight2, norm_eps=self.eps, kernel_cache=self.cache)


class RoPE(CachableModule):
    """Rotary embedding on the first R channels of the first ``seq_cutoff``
    tokens of query and key (one launch).  ``pos_emb`` is [2, P, R]: sin, cos.
    Out of place (the reference's module path rotated its inputs in place by
    accident; values are identical)."""

    def __init__(self):
        super().__init__(cache_fields=("fwd", "bwd"))
        self._fn = F_.triton_rope_fn

    def forward(self, query, key, pos_emb, seq_cutoff=None, heads_second=True):
        return self._fn(query=query, key=key, pos_emb=pos_emb, seq_cutoff=seq_cutoff, heads_second=heads_second,
                        kernel_cache=self.cache)


class FusedLNRoPE(CachableModule):
    """FusedHeadLayerNorm followed by RoPE in a single launch."""

    def __init__(self):
        super().__init__(cache_fields=("fwd", "bwd"))
        self._fn = F_.triton_fused_ln_rope_fn

    def forward(self, query, key, pos_emb, seq_cutoff=None, heads_second=True, eps=1e-6):
        return self._fn(query=query, key=key, pos_emb=pos_emb, seq_cutoff=seq_cutoff, heads_second=heads_second,
                        norm_eps=eps, kernel_cache=self.cache)


__all__ = [
    "CachableModule", "FlashAttention", "L2Normalize", "FusedL2Normalize2", "FusedHeadLayerNorm",
    "FusedRMSNorm", "FusedRMSNorm2", "RoPE", "FusedLNRoPE",
]
