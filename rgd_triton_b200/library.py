"""The operator set as ``torch.library`` custom operators (namespace ``rgd_b200``).

The reference's entry points are ``torch.autograd.Function`` s around Triton
launches, which a tracing compiler has to break the graph at.  Here every
launch is also registered as a custom operator with a fake (shape-only)
implementation and an autograd formula, so ``torch.compile`` traces through the
modules of ``rgd_triton_b200.ops`` without graph breaks: while a compiler is
tracing, the functional entry points (``flash_attn_func``, ``triton_rms_func_fn``
...) route to these operators instead of the eager path.  The kernels, the C ABI
underneath and the results are the same; the per-module launch cache is not used
on this route (a compiled graph calls the operator directly).

    torch.ops.rgd_b200.l2norm(xs, eps) -> ys                (1 or 2 tensors)
    torch.ops.rgd_b200.rmsnorm(xs, ws, eps) -> ys
    torch.ops.rgd_b200.headln(q, k, heads_second, eps) -> (qo, ko)
    torch.ops.rgd_b200.rope(q, k, pos, cut_q, cut_k, heads_second, transposed) -> (qo, ko)
    torch.ops.rgd_b200.lnrope(q, k, pos, cut_q, cut_k, heads_second, eps) -> (qo, ko)
    torch.ops.rgd_b200.attn(q, k, v, bias, causal, softmax_scale) -> (o, lse)      (bias may require grad)

plus a ``*_bwd`` operator for each, which the autograd formulas call.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import functional as F_

Tensor = torch.Tensor
_op = torch.library.custom_op


def _like(ts):
    return [torch.empty_like(t) for t in ts]


# ----------------------------------------------------------------------------- L2 normalise
@_op("rgd_b200::l2norm", mutates_args=())
def l2norm(xs: List[Tensor], eps: float) -> List[Tensor]:
    return F_._l2_forward(list(xs), eps, None, "L2Normalize")[1]


@_op("rgd_b200::l2norm_bwd", mutates_args=())
def l2norm_bwd(xs: List[Tensor], dys: List[Tensor], eps: float) -> List[Tensor]:
    return F_._l2_backward([F_._last_contig(x) for x in xs], list(dys), eps, None, "L2Normalize")


l2norm.register_fake(lambda xs, eps: _like(xs))
l2norm_bwd.register_fake(lambda xs, dys, eps: _like(xs))


def _l2_setup(ctx, inputs, output):
    ctx.xs, ctx.eps = inputs[0], inputs[1]


def _l2_backward(ctx, dys):
    return torch.ops.rgd_b200.l2norm_bwd(ctx.xs, [d.contiguous() for d in dys], ctx.eps), None


l2norm.register_autograd(_l2_backward, setup_context=_l2_setup)


# ----------------------------------------------------------------------------- RMS norm
@_op("rgd_b200::rmsnorm", mutates_args=())
def rmsnorm(xs: List[Tensor], ws: List[Tensor], eps: float) -> List[Tensor]:
    return F_._rms_forward(list(xs), list(ws), eps, None, "FusedRMSNorm")[2]


@_op("rgd_b200::rmsnorm_bwd", mutates_args=())
def rmsnorm_bwd(xs: List[Tensor], ws: List[Tensor], dys: List[Tensor], eps: float) -> List[Tensor]:
    xs = [F_._last_contig(x) for x in xs]
    ws_c = [F_._last_contig(w) for w in ws]
    dxs, dws = F_._rms_backward(xs, ws_c, list(dys), eps, None, "FusedRMSNorm")
    return [*dxs, *[dw.view(w.shape) for dw, w in zip(dws, ws)]]


rmsnorm.register_fake(lambda xs, ws, eps: _like(xs))
rmsnorm_bwd.register_fake(lambda xs, ws, dys, eps: _like(xs) + _like(ws))


def _rms_setup(ctx, inputs, output):
    ctx.xs, ctx.ws, ctx.eps = inputs


def _rms_backward(ctx, dys):
    n = len(ctx.xs)
    g = torch.ops.rgd_b200.rmsnorm_bwd(ctx.xs, ctx.ws, [d.contiguous() for d in dys], ctx.eps)
    return g[:n], g[n:], None


rmsnorm.register_autograd(_rms_backward, setup_context=_rms_setup)


# ----------------------------------------------------------------------------- head LayerNorm
@_op("rgd_b200::headln", mutates_args=())
def headln(q: Tensor, k: Tensor, heads_second: bool, eps: float) -> Tuple[Tensor, Tensor]:
    return F_._ln_forward(q, k, heads_second, eps, None)[2:]


@_op("rgd_b200::headln_bwd", mutates_args=())
def headln_bwd(q: Tensor, k: Tensor, dqo: Tensor, dko: Tensor, heads_second: bool, eps: float) -> Tuple[Tensor, Tensor]:
    q, k, dqo, dko = (F_._last_contig(t) for t in (q, k, dqo, dko))
    F_._check_heads([q, k, dqo, dko], "FusedHeadLayerNorm backward", 256)
    dq, dk = torch.empty_like(dqo), torch.empty_like(dko)
    F_._ln_launch(None, q, k, dqo, dko, dq, dk, heads_second, eps, bwd=True)
    return dq, dk


headln.register_fake(lambda q, k, heads_second, eps: (torch.empty_like(q), torch.empty_like(k)))
headln_bwd.register_fake(lambda q, k, dqo, dko, heads_second, eps: (torch.empty_like(dqo), torch.empty_like(dko)))


def _headln_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0], inputs[1])
    ctx.hs, ctx.eps = inputs[2], inputs[3]


def _headln_backward(ctx, dqo, dko):
    q, k = ctx.saved_tensors
    dq, dk = torch.ops.rgd_b200.headln_bwd(q, k, dqo.contiguous(), dko.contiguous(), ctx.hs, ctx.eps)
    return dq, dk, None, None


headln.register_autograd(_headln_backward, setup_context=_headln_setup)


# ----------------------------------------------------------------------------- rotary, LayerNorm -> rotary
def _lens(q, k, heads_second):
    return (q.shape[2], k.shape[2]) if heads_second else (q.shape[1], k.shape[1])


@_op("rgd_b200::rope", mutates_args=())
def rope(q: Tensor, k: Tensor, pos: Tensor, cut_q: int, cut_k: int, heads_second: bool,
         transposed: bool) -> Tuple[Tensor, Tensor]:
    q, k = F_._last_contig(q), F_._last_contig(k)
    F_._check_heads([q, k], "RoPE", 128)
    pos = F_._prep_pos(pos, q, *_lens(q, k, heads_second))
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    F_._rope_launch(None, q, k, pos, qo, ko, (cut_q, cut_k), heads_second, transposed=transposed)
    return qo, ko


rope.register_fake(lambda q, k, pos, cut_q, cut_k, heads_second, transposed: (torch.empty_like(q), torch.empty_like(k)))


def _rope_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[2])
    ctx.args = inputs[3:]


def _rope_backward(ctx, dqo, dko):
    (pos,) = ctx.saved_tensors
    cut_q, cut_k, hs, transposed = ctx.args
    dq, dk = torch.ops.rgd_b200.rope(dqo.contiguous(), dko.contiguous(), pos, cut_q, cut_k, hs, not transposed)
    return dq, dk, None, None, None, None, None


rope.register_autograd(_rope_backward, setup_context=_rope_setup)


@_op("rgd_b200::lnrope", mutates_args=())
def lnrope(q: Tensor, k: Tensor, pos: Tensor, cut_q: int, cut_k: int, heads_second: bool,
           eps: float) -> Tuple[Tensor, Tensor]:
    return F_._lnrope_forward(q, k, pos, (cut_q, cut_k), heads_second, eps, None)[4:]


@_op("rgd_b200::lnrope_bwd", mutates_args=())
def lnrope_bwd(q: Tensor, k: Tensor, dqo: Tensor, dko: Tensor, pos: Tensor, cut_q: int, cut_k: int,
               heads_second: bool, eps: float) -> Tuple[Tensor, Tensor]:
    q, k, dqo, dko = (F_._last_contig(t) for t in (q, k, dqo, dko))
    F_._check_heads([q, k, dqo, dko], "FusedLNRoPE backward", 128)
    pos = F_._prep_pos(pos, q, *_lens(q, k, heads_second))
    dq, dk = torch.empty_like(dqo), torch.empty_like(dko)
    F_._lnrope_launch(None, q, k, dqo, dko, pos, dq, dk, (cut_q, cut_k), heads_second, eps, bwd=True)
    return dq, dk


lnrope.register_fake(lambda q, k, pos, cut_q, cut_k, heads_second, eps: (torch.empty_like(q), torch.empty_like(k)))
lnrope_bwd.register_fake(
    lambda q, k, dqo, dko, pos, cut_q, cut_k, heads_second, eps: (torch.empty_like(dqo), torch.empty_like(dko)))


def _lnrope_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0], inputs[1], inputs[2])
    ctx.args = inputs[3:]


def _lnrope_backward(ctx, dqo, dko):
    q, k, pos = ctx.saved_tensors
    dq, dk = torch.ops.rgd_b200.lnrope_bwd(q, k, dqo.contiguous(), dko.contiguous(), pos, *ctx.args)
    return dq, dk, None, None, None, None, None


lnrope.register_autograd(_lnrope_backward, setup_context=_lnrope_setup)


# ----------------------------------------------------------------------------- attention
@_op("rgd_b200::attn", mutates_args=())
def attn(q: Tensor, k: Tensor, v: Tensor, bias: Optional[Tensor], causal: bool,
         softmax_scale: float) -> Tuple[Tensor, Tensor]:
    _, _, _, o, lse, _, _, _ = F_._attn_forward(q, k, v, bias, causal, softmax_scale, None)
    return o, lse


@_op("rgd_b200::attn_bwd", mutates_args=())
def attn_bwd(q: Tensor, k: Tensor, v: Tensor, bias: Optional[Tensor], o: Tensor, lse: Tensor, do: Tensor,
             causal: bool, softmax_scale: float, want_dbias: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    dq, dk, dv, dbias = F_._attn_backward(q, k, v, bias, o, lse, do, causal, softmax_scale, None, want_dbias)
    return dq, dk, dv, (q.new_empty(0) if dbias is None else dbias)


def _attn_fake(q, k, v, bias, causal, softmax_scale):
    rows = (q.shape[1] + 63) // 64 * 64
    return torch.empty_like(q), q.new_empty((q.shape[0], q.shape[2], rows), dtype=torch.float32)


attn.register_fake(_attn_fake)
attn_bwd.register_fake(lambda q, k, v, bias, o, lse, do, causal, softmax_scale, want_dbias:
                       (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v),
                        torch.empty_like(bias) if want_dbias and bias is not None else q.new_empty(0)))


def _attn_setup(ctx, inputs, output):
    q, k, v, bias, causal, scale = inputs
    ctx.save_for_backward(q, k, v, bias, output[0], output[1])
    ctx.causal, ctx.scale = causal, scale
    ctx.bias_needs_grad = bias is not None and bias.requires_grad


def _attn_backward(ctx, do, dlse):
    q, k, v, bias, o, lse = ctx.saved_tensors
    dq, dk, dv, dbias = torch.ops.rgd_b200.attn_bwd(q, k, v, bias, o, lse, do.contiguous(), ctx.causal, ctx.scale,
                                                    ctx.bias_needs_grad)
    return dq, dk, dv, (dbias if ctx.bias_needs_grad else None), None, None


attn.register_autograd(_attn_backward, setup_context=_attn_setup)
