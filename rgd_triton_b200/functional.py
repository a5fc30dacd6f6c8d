"""Autograd functions and functional entry points of the operator set.

Host-side mirror of the reference's ``*_Func`` autograd classes and ``*_fn``
entries (same names, argument order, defaults and error behaviour), with every
Triton launch replaced by one call into librgd_b200.so through the C ABI:

===========================  =======================================================
entry point here             reference entry it replaces
===========================  =======================================================
``triton_norm_func_fn``      normalization/l2normalize_cached.py:435-436
``triton_fused_norm_func_fn``  normalization/fused_l2normalize_cached.py:506-507
``triton_fused_ln_func_fn``  normalization/head_layernorm_cached.py:455-456
``triton_rms_func_fn``       normalization/rmsnorm_cached.py:628-629
``triton_fused_rms_func_fn``  normalization/fused_rmsnorm_cached.py:801-802
``triton_rope_fn``           rope/head_rope_cached.py:326-327
``triton_fused_ln_rope_fn``  rope/fused_ln_rope_cached.py:695-696
``flash_attn_func``          flash_attn/flash_attn_triton_cached.py:1131-1133
===========================  =======================================================

Differences from the reference, all deliberate:

* ``kernel_cache`` slots hold a validated launch key (shapes, strides, dtypes)
  instead of a compiled-kernel handle.  A call whose key differs re-validates
  and replaces the slot, so one module can be reused across shapes and dtypes
  (the reference silently mis-launches in that case).
* Row statistics are recomputed in the backward kernels, so nothing but the
  inputs is saved for backward (attention still saves O and LSE).
* ``triton_rope_fn`` is out of place unless ``in_place=True`` is passed by
  keyword; the reference's positional slip made the cached module path
  overwrite its inputs (rope/head_rope_cached.py:326-327 vs :279).
* RMSNorm's dweight is summed over batches in fp32 and rounded once.

Argument checks raise ``AssertionError`` explicitly (not ``assert``), so they
survive ``python -O``.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from ._lib import Bias, Heads, Rows

_FLOATS = (torch.float16, torch.bfloat16, torch.float32)


def _require(cond: bool, msg: str = "") -> None:
    if not cond:
        raise AssertionError(msg)


def _last_contig(t: torch.Tensor) -> torch.Tensor:
    """The kernels need a unit channel stride; anything else is copied, as in
    the reference.  Empty and single-channel tensors may report any stride."""
    if t.stride(-1) == 1:
        return t
    t = t.contiguous()
    if t.stride(-1) != 1:              # numel == 0 or a size-1 last dimension
        t = t.new_empty(t.shape).copy_(t)
    return t


def _i64(*vals) -> C.Array:
    return (C.c_int64 * len(vals))(*vals)


def _key(*tensors, extra=()) -> tuple:
    return tuple((tuple(t.shape), t.stride(), t.dtype, t.device.index) for t in tensors if t is not None) + tuple(extra)


def _cache_hit(cache, slot: str, key) -> bool:
    """True when `slot` of the module cache already holds this validated key."""
    return cache is not None and getattr(cache, slot, None) == key


def _cache_put(cache, slot: str, key) -> None:
    if cache is not None:
        setattr(cache, slot, key)


def _native_cache(cache):
    """The library's launch-plan cache behind a module cache (None without one)."""
    native = getattr(cache, "native", None)
    return native() if native is not None else None


# --------------------------------------------------------------------------
# Row L2 normalise
# --------------------------------------------------------------------------
def _check_rows(xs, what: str) -> None:
    for x in xs:
        _require(x.ndim == 3, f"{what}: expected [B, N, C] tensors, got {tuple(x.shape)}")
        _require(x.dtype in _FLOATS, "Only support fp16, bf16, and fp32")
        _require(x.stride(-1) == 1 or x.numel() == 0 or x.shape[-1] == 1,
                 f"{what}: last dimension must be contiguous")
        _lib.require_device(x)
    _require(all(x.dtype == xs[0].dtype for x in xs), "All tensors must have the same type")
    _require(all(x.shape[0] == xs[0].shape[0] for x in xs), f"{what}: batch sizes differ")


def _l2_launch(xs, dys, outs, eps: float, bwd: bool) -> None:
    lib = _lib.load()
    n = len(xs)
    xa = (Rows * n)(*[_lib.rows(t) for t in xs])
    oa = (Rows * n)(*[_lib.rows(t) for t in outs])
    N = _i64(*[t.shape[1] for t in xs])
    Cc = _i64(*[t.shape[2] for t in xs])
    B = xs[0].shape[0]
    dt = _lib.dtype_code(xs[0].dtype)
    with _lib.device_guard(xs[0]):
        if bwd:
            da = (Rows * n)(*[_lib.rows(t) for t in dys])
            code = lib.rgd_l2norm_bwd(n, xa, da, oa, N, Cc, B, float(eps), dt, _lib.stream_ptr())
        else:
            code = lib.rgd_l2norm_fwd(n, xa, oa, N, Cc, B, float(eps), dt, _lib.stream_ptr())
    _lib.check(code, "l2norm_bwd" if bwd else "l2norm_fwd")


class Norm_Func(torch.autograd.Function):
    """y = x / max(||x||_2, eps) over the last dim of [B, N, C] (l2normalize_cached.py:402-433)."""

    @staticmethod
    def forward(ctx, x, norm_eps=1e-6, use_ptx=False, kernel_cache=None):
        x = _last_contig(x)
        key = _key(x, extra=("l2", 1))
        if not _cache_hit(kernel_cache, "fwd", key):
            _check_rows([x], "L2Normalize")
            _cache_put(kernel_cache, "fwd", key)
        y = torch.empty_like(x)
        _l2_launch([x], None, [y], norm_eps, bwd=False)
        ctx.save_for_backward(x)
        ctx.norm_eps = norm_eps
        ctx.kernel_cache = kernel_cache
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = _last_contig(dy)
        key = _key(x, dy, extra=("l2", 1))
        if not _cache_hit(ctx.kernel_cache, "bwd", key):
            _check_rows([x, dy], "L2Normalize backward")
            _require(dy.shape == x.shape, "gradient shape mismatch")
            _cache_put(ctx.kernel_cache, "bwd", key)
        dx = torch.empty_like(x)
        _l2_launch([x], [dy], [dx], ctx.norm_eps, bwd=True)
        return dx, None, None, None


def triton_norm_func_fn(x, norm_eps=1e-6, use_ptx=False, kernel_cache=None):
    """L2-normalise the rows of x.  ``use_ptx`` is accepted and ignored."""
    return Norm_Func.apply(x, norm_eps, use_ptx, kernel_cache)


class Fused_Norm_Func(torch.autograd.Function):
    """Two L2 normalisations in one launch (fused_l2normalize_cached.py:464-503)."""

    @staticmethod
    def forward(ctx, x1, x2, norm_eps=1e-6, kernel_cache=None):
        x1, x2 = _last_contig(x1), _last_contig(x2)
        key = _key(x1, x2, extra=("l2", 2))
        if not _cache_hit(kernel_cache, "fwd", key):
            _check_rows([x1, x2], "FusedL2Normalize2")
            _cache_put(kernel_cache, "fwd", key)
        y1, y2 = torch.empty_like(x1), torch.empty_like(x2)
        _l2_launch([x1, x2], None, [y1, y2], norm_eps, bwd=False)
        ctx.save_for_backward(x1, x2)
        ctx.norm_eps = norm_eps
        ctx.kernel_cache = kernel_cache
        return y1, y2

    @staticmethod
    def backward(ctx, dy1, dy2):
        x1, x2 = ctx.saved_tensors
        dy1, dy2 = _last_contig(dy1), _last_contig(dy2)
        key = _key(x1, x2, dy1, dy2, extra=("l2", 2))
        if not _cache_hit(ctx.kernel_cache, "bwd", key):
            _check_rows([x1, x2, dy1, dy2], "FusedL2Normalize2 backward")
            _cache_put(ctx.kernel_cache, "bwd", key)
        dx1, dx2 = torch.empty_like(x1), torch.empty_like(x2)
        _l2_launch([x1, x2], [dy1, dy2], [dx1, dx2], ctx.norm_eps, bwd=True)
        return dx1, dx2, None, None


def triton_fused_norm_func_fn(x1, x2, norm_eps=1e-6, kernel_cache=None):
    return Fused_Norm_Func.apply(x1, x2, norm_eps, kernel_cache)


# --------------------------------------------------------------------------
# Row RMS norm with affine weight
# --------------------------------------------------------------------------
def _prep_weight(w: torch.Tensor, x: torch.Tensor):
    """Return (weight tensor, batch stride, per_batch) for the accepted weight
    forms [C], [1,1,C] (shared) and [B,1,C] (per batch) — rmsnorm_cached.py:582-589."""
    w = _last_contig(w)
    B, _, Cx = x.shape
    if w.ndim == 1:
        _require(w.shape[0] == Cx, f"weight has {w.shape[0]} channels, x has {Cx}")
        return w, 0, False
    _require(w.ndim == 3, f"weight must be [C] or [B|1, 1, C], got {tuple(w.shape)}")
    _require(w.shape[1] == 1, "sequence-dependent weights are not supported")
    _require(w.shape[2] == Cx, f"weight has {w.shape[2]} channels, x has {Cx}")
    if w.shape[0] == 1:
        return w, 0, False
    _require(w.shape[0] == B, "weight batch must be 1 or match x")
    return w, w.stride(0), True


def _rms_fwd(xs, ws, eps):
    lib = _lib.load()
    n = len(xs)
    preps = [_prep_weight(w, x) for w, x in zip(ws, xs)]
    _require(all(p[0].dtype == preps[0][0].dtype for p in preps), "weights must share one dtype")
    for p in preps:
        _require(p[0].dtype in _FLOATS, "Only support fp16, bf16, and fp32")
        _require(p[0].device == xs[0].device, "weight and input are on different devices")
    ys = [torch.empty_like(x) for x in xs]
    xa = (Rows * n)(*[_lib.rows(t) for t in xs])
    ya = (Rows * n)(*[_lib.rows(t) for t in ys])
    wp = (C.c_void_p * n)(*[p[0].data_ptr() for p in preps])
    wsb = _i64(*[p[1] for p in preps])
    N = _i64(*[t.shape[1] for t in xs])
    Cc = _i64(*[t.shape[2] for t in xs])
    with _lib.device_guard(xs[0]):
        code = lib.rgd_rmsnorm_fwd(n, xa, wp, wsb, ya, N, Cc, xs[0].shape[0], float(eps),
                                   _lib.dtype_code(xs[0].dtype), _lib.dtype_code(preps[0][0].dtype),
                                   _lib.stream_ptr())
    _lib.check(code, "rmsnorm_fwd")
    return ys, [p[0] for p in preps]


def _rms_bwd(xs, ws, dys, eps):
    lib = _lib.load()
    n = len(xs)
    preps = [_prep_weight(w, x) for w, x in zip(ws, xs)]
    B = xs[0].shape[0]
    dxs = [torch.empty_like(x) for x in xs]
    dws = []
    for (w, _, per_batch), x in zip(preps, xs):
        shape = (B, x.shape[2]) if per_batch else (x.shape[2],)
        dws.append(torch.empty(shape, dtype=w.dtype, device=w.device))
    N = _i64(*[t.shape[1] for t in xs])
    Cc = _i64(*[t.shape[2] for t in xs])
    with _lib.device_guard(xs[0]):
        nbytes = lib.rgd_rmsnorm_bwd_workspace_bytes(n, N, Cc, B)
        _require(nbytes >= 0, "rmsnorm_bwd: bad sizes")
        work = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=xs[0].device)
        xa = (Rows * n)(*[_lib.rows(t) for t in xs])
        da = (Rows * n)(*[_lib.rows(t) for t in dys])
        oa = (Rows * n)(*[_lib.rows(t) for t in dxs])
        wp = (C.c_void_p * n)(*[p[0].data_ptr() for p in preps])
        wsb = _i64(*[p[1] for p in preps])
        dwp = (C.c_void_p * n)(*[t.data_ptr() for t in dws])
        per = (C.c_int * n)(*[1 if p[2] else 0 for p in preps])
        code = lib.rgd_rmsnorm_bwd(n, xa, wp, wsb, da, oa, dwp, per, N, Cc, B, float(eps),
                                   _lib.dtype_code(xs[0].dtype), _lib.dtype_code(preps[0][0].dtype),
                                   work.data_ptr(), work.numel(), _lib.stream_ptr())
    _lib.check(code, "rmsnorm_bwd")
    return dxs, dws


class RMS_Func(torch.autograd.Function):
    """y = x * rsqrt(mean(x^2) + eps) * w  (rmsnorm_cached.py:572-625)."""

    @staticmethod
    def forward(ctx, x, w, norm_eps=1e-6, kernel_cache=None):
        x = _last_contig(x)
        key = _key(x, w, extra=("rms", 1))
        if not _cache_hit(kernel_cache, "fwd", key):
            _check_rows([x], "FusedRMSNorm")
            _cache_put(kernel_cache, "fwd", key)
        (y,), (wk,) = _rms_fwd([x], [w], norm_eps)
        ctx.save_for_backward(x, wk)
        ctx.wshape = w.shape
        ctx.norm_eps = norm_eps
        ctx.kernel_cache = kernel_cache
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = _last_contig(dy)
        key = _key(x, w, dy, extra=("rms", 1))
        if not _cache_hit(ctx.kernel_cache, "bwd", key):
            _check_rows([x, dy], "FusedRMSNorm backward")
            _cache_put(ctx.kernel_cache, "bwd", key)
            _cache_put(ctx.kernel_cache, "bwd_dw", key)
        (dx,), (dw,) = _rms_bwd([x], [w], [dy], ctx.norm_eps)
        return dx, dw.view(ctx.wshape), None, None


def triton_rms_func_fn(x, w, norm_eps=1e-6, kernel_cache=None):
    return RMS_Func.apply(x, w, norm_eps, kernel_cache)


class Fused_RMS_Func(torch.autograd.Function):
    """Two RMS norms with separate weights in one launch (fused_rmsnorm_cached.py:725-798)."""

    @staticmethod
    def forward(ctx, x1, x2, w1, w2, norm_eps=1e-6, kernel_cache=None):
        x1, x2 = _last_contig(x1), _last_contig(x2)
        key = _key(x1, x2, w1, w2, extra=("rms", 2))
        if not _cache_hit(kernel_cache, "fwd", key):
            _check_rows([x1, x2], "FusedRMSNorm2")
            _cache_put(kernel_cache, "fwd", key)
        (y1, y2), (wk1, wk2) = _rms_fwd([x1, x2], [w1, w2], norm_eps)
        ctx.save_for_backward(x1, x2, wk1, wk2)
        ctx.w1shape, ctx.w2shape = w1.shape, w2.shape
        ctx.norm_eps = norm_eps
        ctx.kernel_cache = kernel_cache
        return y1, y2

    @staticmethod
    def backward(ctx, dy1, dy2):
        x1, x2, w1, w2 = ctx.saved_tensors
        dy1, dy2 = _last_contig(dy1), _last_contig(dy2)
        key = _key(x1, x2, w1, w2, dy1, dy2, extra=("rms", 2))
        if not _cache_hit(ctx.kernel_cache, "bwd", key):
            _check_rows([x1, x2, dy1, dy2], "FusedRMSNorm2 backward")
            _cache_put(ctx.kernel_cache, "bwd", key)
            _cache_put(ctx.kernel_cache, "bwd_dw", key)
        (dx1, dx2), (dw1, dw2) = _rms_bwd([x1, x2], [w1, w2], [dy1, dy2], ctx.norm_eps)
        return dx1, dx2, dw1.view(ctx.w1shape), dw2.view(ctx.w2shape), None, None


def triton_fused_rms_func_fn(x1, x2, w1, w2, norm_eps=1e-6, kernel_cache=None):
    return Fused_RMS_Func.apply(x1, x2, w1, w2, norm_eps, kernel_cache)


# --------------------------------------------------------------------------
# Head operators: LayerNorm, RoPE, LayerNorm -> RoPE
# --------------------------------------------------------------------------
def _head_dims(q, k, heads_second: bool):
    if heads_second:
        bq, hq, nq, dq = q.shape
        bk, hk, nk, dk = k.shape
    else:
        bq, nq, hq, dq = q.shape
        bk, nk, hk, dk = k.shape
    _require((bq, hq, dq) == (bk, hk, dk), f"q and k must share (batch, heads, head_dim): {q.shape} vs {k.shape}")
    return bq, hq, nq, nk, dq


def _check_heads(ts, what: str, dmax: int) -> None:
    for t in ts:
        _require(t.ndim == 4, f"{what}: expected 4-D tensors, got {tuple(t.shape)}")
        _require(t.dtype in _FLOATS, "Only support fp16, bf16, and fp32")
        _require(t.stride(-1) == 1 or t.numel() == 0 or t.shape[-1] == 1,
                 f"{what}: last dimension must be contiguous")
        _lib.require_device(t)
    _require(all(t.dtype == ts[0].dtype for t in ts), "All tensors must have the same type")
    _require(ts[0].shape[-1] <= dmax, f"Only supports head dimensions up to {dmax}")


def _cutoffs(seq_cutoff, nq: int, nk: int):
    """seq_cutoff: None, an int, or a (q, k) pair (head_rope_cached.py:193-201)."""
    if seq_cutoff is None:
        return nq, nk
    if isinstance(seq_cutoff, (tuple, list)):
        return int(seq_cutoff[0]), int(seq_cutoff[1])
    return int(seq_cutoff), int(seq_cutoff)


def _prep_pos(pos_emb: torch.Tensor, x: torch.Tensor, nq: int, nk: int) -> torch.Tensor:
    _require(pos_emb.ndim == 3, f"pos_emb must be [2, P, R], got {tuple(pos_emb.shape)}")
    _require(pos_emb.shape[0] == 2, "pos_emb[0] is sin and pos_emb[1] is cos")
    _require(pos_emb.is_cuda and pos_emb.device == x.device, "pos_emb must be on the tensors' device")
    _require(pos_emb.dtype in _FLOATS, "Only support fp16, bf16, and fp32")
    _require(nq < pos_emb.shape[1] and nk < pos_emb.shape[1],
             "pos_emb must hold more positions than the longest sequence")
    pos_emb = _last_contig(pos_emb)
    # Arithmetic runs in the promoted type of x and the table: a table that is
    # neither x's type nor fp32 promotes to fp32 anyway.
    if pos_emb.dtype != x.dtype and pos_emb.dtype != torch.float32:
        pos_emb = pos_emb.float()
    return pos_emb


def _ln_launch(q, k, dqo, dko, qo, ko, heads_second, eps, bwd):
    lib = _lib.load()
    B, H, nq, nk, d = _head_dims(q, k, heads_second)
    hv = lambda t: C.byref(_lib.heads(t, heads_second))
    dt = _lib.dtype_code(q.dtype)
    with _lib.device_guard(q):
        if bwd:
            code = lib.rgd_headln_bwd(hv(q), hv(k), hv(dqo), hv(dko), hv(qo), hv(ko), B, H, nq, nk, d, float(eps), dt,
                                      _lib.stream_ptr())
        else:
            code = lib.rgd_headln_fwd(hv(q), hv(k), hv(qo), hv(ko), B, H, nq, nk, d, float(eps), dt,
                                      _lib.stream_ptr())
    _lib.check(code, "headln_bwd" if bwd else "headln_fwd")


class Fused_LNQK_Func(torch.autograd.Function):
    """Non-affine LayerNorm over head_dim of Q and K in one launch
    (head_layernorm_cached.py:416-453)."""

    @staticmethod
    def forward(ctx, q, k, heads_second=True, norm_eps=1e-6, kernel_cache=None):
        q, k = _last_contig(q), _last_contig(k)
        key = _key(q, k, extra=("ln", bool(heads_second)))
        if not _cache_hit(kernel_cache, "fwd", key):
            _check_heads([q, k], "FusedHeadLayerNorm", 256)
            _head_dims(q, k, heads_second)
            _cache_put(kernel_cache, "fwd", key)
        qo, ko = torch.empty_like(q), torch.empty_like(k)
        _ln_launch(q, k, None, None, qo, ko, heads_second, norm_eps, bwd=False)
        ctx.save_for_backward(q, k)
        ctx.heads_second, ctx.norm_eps, ctx.kernel_cache = heads_second, norm_eps, kernel_cache
        return qo, ko

    @staticmethod
    def backward(ctx, dqo, dko):
        q, k = ctx.saved_tensors
        dqo, dko = _last_contig(dqo), _last_contig(dko)
        key = _key(q, k, dqo, dko, extra=("ln", bool(ctx.heads_second)))
        if not _cache_hit(ctx.kernel_cache, "bwd", key):
            _check_heads([q, k, dqo, dko], "FusedHeadLayerNorm backward", 256)
            _require(dqo.shape == q.shape and dko.shape == k.shape, "gradient shape mismatch")
            _cache_put(ctx.kernel_cache, "bwd", key)
        dq, dk = torch.empty_like(dqo), torch.empty_like(dko)
        _ln_launch(q, k, dqo, dko, dq, dk, ctx.heads_second, ctx.norm_eps, bwd=True)
        return dq, dk, None, None, None


def triton_fused_ln_func_fn(query, key, heads_second=True, norm_eps=1e-6, kernel_cache=None):
    return Fused_LNQK_Func.apply(query, key, heads_second, norm_eps, kernel_cache)


def _rope_launch(q, k, pos, qo, ko, cuts, heads_second, transposed):
    lib = _lib.load()
    B, H, nq, nk, d = _head_dims(q, k, heads_second)
    hv = lambda t: C.byref(_lib.heads(t, heads_second))
    with _lib.device_guard(q):
        code = lib.rgd_rope(hv(q), hv(k), pos.data_ptr(), pos.stride(0), pos.stride(1), hv(qo), hv(ko),
                            B, H, nq, nk, d, pos.shape[1], pos.shape[2], cuts[0], cuts[1],
                            1 if transposed else 0, _lib.dtype_code(q.dtype), _lib.dtype_code(pos.dtype),
                            _lib.stream_ptr())
    _lib.check(code, "rope")


class CombinedRoPEFunc(torch.autograd.Function):
    """Interleaved-pair rotary embedding on the first R channels of the first
    `cutoff` tokens of Q and K, one launch (head_rope_cached.py:277-323).  The
    backward is the same kernel with the rotation inverted, applied to the
    upstream gradients."""

    @staticmethod
    def forward(ctx, q, k, pos_emb, seq_cutoff=None, heads_second=True, in_place=False, kernel_cache=None):
        q, k = _last_contig(q), _last_contig(k)
        key = _key(q, k, pos_emb, extra=("rope", bool(heads_second)))
        if not _cache_hit(kernel_cache, "fwd", key):
            _check_heads([q, k], "RoPE", 128)
            _cache_put(kernel_cache, "fwd", key)
        B, H, nq, nk, d = _head_dims(q, k, heads_second)
        pos = _prep_pos(pos_emb, q, nq, nk)
        cuts = _cutoffs(seq_cutoff, nq, nk)
        if in_place:
            qo, ko = q, k
            ctx.mark_dirty(q, k)
        else:
            qo, ko = torch.empty_like(q), torch.empty_like(k)
        _rope_launch(q, k, pos, qo, ko, cuts, heads_second, transposed=False)
        ctx.save_for_backward(pos)
        ctx.cuts, ctx.heads_second, ctx.kernel_cache = cuts, heads_second, kernel_cache
        return qo, ko

    @staticmethod
    def backward(ctx, dqo, dko):
        (pos,) = ctx.saved_tensors
        _require(not ctx.needs_input_grad[2], "CombinedRoPE does not support gradients in position embeddings")
        dqo, dko = _last_contig(dqo), _last_contig(dko)
        key = _key(dqo, dko, pos, extra=("rope", bool(ctx.heads_second)))
        if not _cache_hit(ctx.kernel_cache, "bwd", key):
            _check_heads([dqo, dko], "RoPE backward", 128)
            _cache_put(ctx.kernel_cache, "bwd", key)
        dq, dk = torch.empty_like(dqo), torch.empty_like(dko)
        _rope_launch(dqo, dko, pos, dq, dk, ctx.cuts, ctx.heads_second, transposed=True)
        return dq, dk, None, None, None, None, None


def triton_rope_fn(query, key, pos_emb, seq_cutoff=None, heads_second=True, fused_ln=False, kernel_cache=None,
                   in_place=False):
    """Rotary embedding on (query, key).  ``fused_ln`` is accepted for
    signature parity and ignored, as in the reference."""
    return CombinedRoPEFunc.apply(query, key, pos_emb, seq_cutoff, heads_second, in_place, kernel_cache)


def _lnrope_launch(q, k, dqo, dko, pos, qo, ko, cuts, heads_second, eps, bwd):
    lib = _lib.load()
    B, H, nq, nk, d = _head_dims(q, k, heads_second)
    hv = lambda t: C.byref(_lib.heads(t, heads_second))
    tail = (B, H, nq, nk, d, pos.shape[1], pos.shape[2], cuts[0], cuts[1], float(eps),
            _lib.dtype_code(q.dtype), _lib.dtype_code(pos.dtype), _lib.stream_ptr())
    with _lib.device_guard(q):
        if bwd:
            code = lib.rgd_lnrope_bwd(hv(q), hv(k), hv(dqo), hv(dko), pos.data_ptr(), pos.stride(0), pos.stride(1),
                                      hv(qo), hv(ko), *tail)
        else:
            code = lib.rgd_lnrope_fwd(hv(q), hv(k), pos.data_ptr(), pos.stride(0), pos.stride(1), hv(qo), hv(ko),
                                      *tail)
    _lib.check(code, "lnrope_bwd" if bwd else "lnrope_fwd")


class FusedRoPEFunc(torch.autograd.Function):
    """Head LayerNorm followed by rotary embedding in one launch; backward is
    inverse rotation then LayerNorm backward (fused_ln_rope_cached.py:649-692)."""

    @staticmethod
    def forward(ctx, q, k, pos_emb, seq_cutoff=None, heads_second=True, norm_eps=1e-6, kernel_cache=None):
        q, k = _last_contig(q), _last_contig(k)
        key = _key(q, k, pos_emb, extra=("lnrope", bool(heads_second)))
        if not _cache_hit(kernel_cache, "fwd", key):
            _check_heads([q, k], "FusedLNRoPE", 128)
            _cache_put(kernel_cache, "fwd", key)
        B, H, nq, nk, d = _head_dims(q, k, heads_second)
        pos = _prep_pos(pos_emb, q, nq, nk)
        cuts = _cutoffs(seq_cutoff, nq, nk)
        qo, ko = torch.empty_like(q), torch.empty_like(k)
        _lnrope_launch(q, k, None, None, pos, qo, ko, cuts, heads_second, norm_eps, bwd=False)
        ctx.save_for_backward(q, k, pos)
        ctx.cuts, ctx.heads_second, ctx.norm_eps, ctx.kernel_cache = cuts, heads_second, norm_eps, kernel_cache
        return qo, ko

    @staticmethod
    def backward(ctx, dqo, dko):
        q, k, pos = ctx.saved_tensors
        _require(not ctx.needs_input_grad[2], "CombinedRoPE does not support gradients in position embeddings")
        dqo, dko = _last_contig(dqo), _last_contig(dko)
        key = _key(q, k, dqo, dko, pos, extra=("lnrope", bool(ctx.heads_second)))
        if not _cache_hit(ctx.kernel_cache, "bwd", key):
            _check_heads([q, k, dqo, dko], "FusedLNRoPE backward", 128)
            _cache_put(ctx.kernel_cache, "bwd", key)
        dq, dk = torch.empty_like(dqo), torch.empty_like(dko)
        _lnrope_launch(q, k, dqo, dko, pos, dq, dk, ctx.cuts, ctx.heads_second, ctx.norm_eps, bwd=True)
        return dq, dk, None, None, None, None, None


def triton_fused_ln_rope_fn(query, key, pos_emb, seq_cutoff=None, heads_second=True, norm_eps=1e-6,
                            kernel_cache=None):
    return FusedRoPEFunc.apply(query, key, pos_emb, seq_cutoff, heads_second, norm_eps, kernel_cache)


# --------------------------------------------------------------------------
# FlashAttention
# --------------------------------------------------------------------------
def _attn_heads(t: torch.Tensor) -> Heads:
    # attention tensors are (batch, seqlen, nheads, headdim)
    return Heads(t.data_ptr(), t.stride(0), t.stride(2), t.stride(1))


def _prep_bias(bias, q, seqlen_q: int, seqlen_k: int):
    """Validate the bias and return (last-dim-contiguous bias, rgd_bias struct).
    Same rules as flash_attn_triton_cached.py:771-788."""
    if bias is None:
        return None, Bias(None, 0, 0, 0, _lib.RGD_BIAS_NONE, _lib.RGD_F32)
    batch, _, nheads, _ = q.shape
    _require(bias.dtype in (q.dtype, torch.float32), "bias must have q's dtype or float32")
    _require(bias.is_cuda and bias.device == q.device, "bias must be on q's device")
    _require(bias.dim() == 4, "bias must be 4-D")
    if bias.stride(-1) != 1:
        bias = bias.contiguous()
    if tuple(bias.shape[2:]) == (1, seqlen_k):
        kind = _lib.RGD_BIAS_VECTOR
    elif tuple(bias.shape[2:]) == (seqlen_q, seqlen_k):
        kind = _lib.RGD_BIAS_MATRIX
    else:
        raise RuntimeError("Last 2 dimensions of bias must be (1, seqlen_k) or (seqlen_q, seqlen_k)")
    full = bias.expand(batch, nheads, seqlen_q, seqlen_k)   # broadcast dims get stride 0
    sq = full.stride(2) if kind == _lib.RGD_BIAS_MATRIX else 0
    return bias, Bias(full.data_ptr(), full.stride(0), full.stride(1), sq, kind, _lib.dtype_code(full.dtype))


def _check_attn(q, k, v) -> None:
    _require(q.ndim == 4 and k.ndim == 4 and v.ndim == 4, "q, k, v must be (batch, seqlen, nheads, headdim)")
    batch, seqlen_q, nheads, d = q.shape
    seqlen_k = k.shape[1]
    _require(tuple(k.shape) == (batch, seqlen_k, nheads, d), f"k shape {tuple(k.shape)} does not match q")
    _require(tuple(v.shape) == (batch, seqlen_k, nheads, d), f"v shape {tuple(v.shape)} does not match k")
    _require(d <= 128, "FlashAttention only support head dimensions up to 128")
    _require(q.dtype == k.dtype == v.dtype, f"All tensors must have the same type {q.dtype=}, {k.dtype=}, {v.dtype=}")
    _require(q.dtype in (torch.float16, torch.bfloat16), "Only support fp16 and bf16")
    for t in (q, k, v):
        _lib.require_device(t)


class FlashAttnFunc(torch.autograd.Function):
    """softmax(Q K^T * scale + bias) V with O(T) memory
    (flash_attn_triton_cached.py:1079-1129).  Returns (o, lse)."""

    @staticmethod
    def forward(ctx, q, k, v, bias=None, causal=False, softmax_scale=None, kernel_cache=None):
        q, k, v = _last_contig(q), _last_contig(k), _last_contig(v)
        key = _key(q, k, v, bias, extra=("attn", bool(causal)))
        if not _cache_hit(kernel_cache, "fwd", key):
            _check_attn(q, k, v)
            _cache_put(kernel_cache, "fwd", key)
        lib = _lib.load()
        batch, seqlen_q, nheads, d = q.shape
        seqlen_k = k.shape[1]
        softmax_scale = softmax_scale or 1.0 / math.sqrt(d)
        bias_t, bias_s = _prep_bias(bias, q, seqlen_q, seqlen_k)
        o = torch.empty_like(q)
        lse = torch.empty((batch, nheads, lib.rgd_attn_lse_rows(seqlen_q)), device=q.device, dtype=torch.float32)
        with _lib.device_guard(q):
            code = lib.rgd_attn_fwd(C.byref(_attn_heads(q)), C.byref(_attn_heads(k)), C.byref(_attn_heads(v)),
                                    C.byref(bias_s), C.byref(_attn_heads(o)), lse.data_ptr(),
                                    batch, nheads, seqlen_q, seqlen_k, d, float(softmax_scale),
                                    1 if causal else 0, _lib.dtype_code(q.dtype), _native_cache(kernel_cache),
                                    _lib.stream_ptr())
        _lib.check(code, "attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse, bias_t)
        ctx.causal, ctx.softmax_scale, ctx.kernel_cache = causal, softmax_scale, kernel_cache
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, dlse):
        q, k, v, o, lse, bias = ctx.saved_tensors
        _require(not ctx.needs_input_grad[3], "FlashAttention does not support bias gradient yet")
        do = _last_contig(do)
        key = _key(q, k, v, do, bias, extra=("attn", bool(ctx.causal)))
        if not _cache_hit(ctx.kernel_cache, "bwd", key):
            _require(do.shape == q.shape and do.dtype == q.dtype, "dO must match q")
            _cache_put(ctx.kernel_cache, "bwd_odot", key)
            _cache_put(ctx.kernel_cache, "bwd", key)
        lib = _lib.load()
        batch, seqlen_q, nheads, d = q.shape
        seqlen_k = k.shape[1]
        _, bias_s = _prep_bias(bias, q, seqlen_q, seqlen_k)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dt = _lib.dtype_code(q.dtype)
        with _lib.device_guard(q):
            nbytes = lib.rgd_attn_bwd_workspace_bytes(batch, nheads, seqlen_q, seqlen_k, d, dt)
            _require(nbytes >= 0, "attn_bwd: bad sizes")
            work = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=q.device)
            hv = lambda t: C.byref(_attn_heads(t))
            code = lib.rgd_attn_bwd(hv(q), hv(k), hv(v), C.byref(bias_s), hv(o), lse.data_ptr(), hv(do),
                                    hv(dq), hv(dk), hv(dv), batch, nheads, seqlen_q, seqlen_k, d,
                                    float(ctx.softmax_scale), 1 if ctx.causal else 0, dt,
                                    work.data_ptr(), work.numel(), _native_cache(ctx.kernel_cache),
                                    _lib.stream_ptr())
        _lib.check(code, "attn_bwd")
        return dq, dk, dv, None, None, None, None


def flash_attn_func(q, k, v, bias=None, causal=False, softmax_scale=None, return_lse=False, kernel_cache=None):
    """q: (batch, seqlen_q, nheads, headdim); k, v: (batch, seqlen_k, nheads,
    headdim); bias: optional, 4-D, last two dims (1, seqlen_k) or (seqlen_q,
    seqlen_k), leading dims broadcastable to (batch, nheads)."""
    o, lse = FlashAttnFunc.apply(q, k, v, bias, causal, softmax_scale, kernel_cache)
    return (o, lse) if return_lse else o
