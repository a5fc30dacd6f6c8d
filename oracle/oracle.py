"""CPU oracle for the rgd_triton operator set.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch on the CPU, the arithmetic of the
reference's Triton kernels, one function per kernel, each citing the reference
lines it follows.  It is the checker the parity tests, ``smoke()`` and the
CPU-baseline leg of ``bench.py`` compare the CUDA library against; nothing in
the product package imports it, and it must never stand in for a kernel.

Parity pin: ``tests/golden/*.npz`` hold outputs of the reference itself, run
in this build's container under Triton's interpreter
(``TRITON_INTERPRET=1 python -O tests/golden/make_golden.py``) in fp32 and
fp16; ``tests/test_oracle_golden.py`` checks every function here against
them.  bf16 is not bit-faithful under the interpreter, so for bf16 the oracle
is these fp32 formulas rounded once (round-to-nearest-even) to bf16, which is
what the kernels' ``tl.store`` of an fp32 value does.

Conventions: all sums and intermediate values are fp32; "->T" is a single
rounding to the input dtype on store.  Inputs may be fp32 / fp16 / bf16 CPU
tensors.  Every function is pure.
"""
from __future__ import annotations

import math

import torch

# --------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------


def _f(x: torch.Tensor) -> torch.Tensor:
    return x.detach().to(torch.float32)


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance between two same-dtype tensors in units in the last place of
    that dtype (0 for bit-equal values; +0 and -0 count as equal)."""
    assert a.dtype == b.dtype and a.shape == b.shape
    if a.dtype == torch.float32:
        ia, ib = a.contiguous().view(torch.int32).to(torch.int64), b.contiguous().view(torch.int32).to(torch.int64)
        sign = 1 << 31
    else:
        ia, ib = a.contiguous().view(torch.int16).to(torch.int64), b.contiguous().view(torch.int16).to(torch.int64)
        sign = 1 << 15
    # map sign-magnitude bit patterns onto a monotone integer line
    ia = torch.where(ia < 0, -(ia + sign), ia)
    ib = torch.where(ib < 0, -(ib + sign), ib)
    return (ia - ib).abs()


# --------------------------------------------------------------------------
# RMSNorm  (rmsnorm_cached.py:54-101 forward, :198-236 backward)
# --------------------------------------------------------------------------


def _weight_view(w: torch.Tensor, B: int, C: int):
    """[C] / [1,1,C] -> shared weight; [B,1,C] -> per batch (rmsnorm_cached.py:582-589)."""
    wf = _f(w)
    if wf.ndim == 1 or wf.shape[0] == 1:
        return wf.reshape(1, 1, C).expand(B, 1, C), True
    return wf.reshape(B, 1, C), False


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = _f(x)
    B, N, C = xf.shape
    wf, _ = _weight_view(w, B, C)
    r = torch.rsqrt((xf * xf).sum(-1, keepdim=True) / C + eps)          # :75-76
    return ((xf * r) * wf).to(x.dtype)                                  # :97


def rmsnorm_bwd(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor, eps: float = 1e-6):
    """Returns (dx in x.dtype, dw in w.dtype and w's shape).  dw is summed
    over rows and (for a shared weight) batches in fp32 and rounded once."""
    xf, df = _f(x), _f(dy)
    B, N, C = xf.shape
    wf, shared = _weight_view(w, B, C)
    r = torch.rsqrt((xf * xf).sum(-1, keepdim=True) / C + eps)
    xh = xf * r                                                         # :211
    g = (xh * df * wf).sum(-1, keepdim=True) / C                        # :213, :229
    dx = ((df * wf - xh * g) * r).to(x.dtype)                           # :231
    dw = (xh * df).sum(dim=1, keepdim=True)                             # :237, per batch
    if shared:
        dw = dw.sum(dim=0)                                              # :611 (here in fp32)
    return dx, dw.reshape(w.shape).to(w.dtype)


# --------------------------------------------------------------------------
# L2 normalise  (l2normalize_cached.py:51-121 forward, :203-230 backward)
# --------------------------------------------------------------------------


def _l2_scale(xf: torch.Tensor, eps: float) -> torch.Tensor:
    length = torch.sqrt((xf * xf).sum(-1, keepdim=True))                # :72-73
    return torch.where(length < eps, torch.full_like(length, 1.0 / eps), 1.0 / length)   # :76-77


def l2norm_fwd(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = _f(x)
    return (xf * _l2_scale(xf, eps)).to(x.dtype)                        # :121


def l2norm_bwd(x: torch.Tensor, dy: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf, df = _f(x), _f(dy)
    rho = _l2_scale(xf, eps)          # the backward reuses the gated forward scale (:195)
    xh = xf * rho                                                       # :214
    g = (xh * df).sum(-1, keepdim=True)                                 # :216, :226
    return ((df - xh * g) * rho).to(x.dtype)                            # :228


# --------------------------------------------------------------------------
# Head LayerNorm  (head_layernorm_cached.py:79-99 forward, :184-199 backward)
# The channel axis is last for both layouts, so heads_second does not change
# the arithmetic.
# --------------------------------------------------------------------------


def _ln_stats(xf: torch.Tensor, eps: float):
    d = xf.shape[-1]
    mean = xf.sum(-1, keepdim=True) / d                                 # :85
    xs = xf - mean                                                      # :87
    var = (xs * xs).sum(-1, keepdim=True) / d                           # :88
    return xs, torch.rsqrt(var + eps)                                   # :89


def headln_fwd(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xs, rstd = _ln_stats(_f(x), eps)
    return (xs * rstd).to(x.dtype)                                      # :92


def _ln_bwd_f32(xf: torch.Tensor, df: torch.Tensor, eps: float) -> torch.Tensor:
    d = xf.shape[-1]
    xs, rstd = _ln_stats(xf, eps)
    xh = xs * rstd                                                      # :190
    a = (xh * df).sum(-1, keepdim=True) / d                             # :195
    b = df.sum(-1, keepdim=True) / d                                    # :196
    return (df - xh * a - b) * rstd                                     # :197


def headln_bwd(x: torch.Tensor, dy: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return _ln_bwd_f32(_f(x), _f(dy), eps).to(x.dtype)


# --------------------------------------------------------------------------
# Rotary embedding  (head_rope_cached.py:7-52 transform, :100-158 kernel body)
# --------------------------------------------------------------------------


def _rope_tables(pos_emb: torch.Tensor, n: int, d: int, heads_second: bool, dtype: torch.dtype):
    """sin / cos broadcast to the tensor layout, zero-padded from R to d channels."""
    R = pos_emb.shape[2]
    Rc = min(R, d)
    sin = torch.zeros(n, d, dtype=dtype)
    cos = torch.zeros(n, d, dtype=dtype)
    sin[:, :Rc] = pos_emb[0, :n, :Rc].to(dtype)
    cos[:, :Rc] = pos_emb[1, :n, :Rc].to(dtype)
    if heads_second:                      # [B, H, N, d]
        return sin[None, None], cos[None, None], Rc
    return sin[None, :, None], cos[None, :, None], Rc     # [B, N, H, d]


def _rotate_pairs(x: torch.Tensor, inverse: bool) -> torch.Tensor:
    """(x0, x1) -> (-x1, x0) per channel pair (:31-38); the inverse flips the sign."""
    d = x.shape[-1]
    if d % 2:
        x = torch.nn.functional.pad(x, (0, 1))
    xe, xo = x[..., 0::2], x[..., 1::2]
    rot = torch.stack((xo, -xe) if inverse else (-xo, xe), dim=-1).flatten(-2)
    return rot[..., :d]


def _rope_apply(x: torch.Tensor, pos_emb: torch.Tensor, cutoff: int, heads_second: bool, inverse: bool,
                compute_dtype: torch.dtype, fused: bool = False) -> torch.Tensor:
    """out = x*cos + rot(x)*sin on channels < R of tokens < cutoff, evaluated in
    `compute_dtype` (:46-51): one rounding per multiply and per add, or, with
    `fused`, rn(fma(rot, sin, rn(x*cos))) — the order the reference's compiled
    kernel uses for 16-bit types (rot*sin is exact in fp32 there)."""
    n = x.shape[2] if heads_second else x.shape[1]
    d = x.shape[-1]
    sin, cos, Rc = _rope_tables(pos_emb, n, d, heads_second, compute_dtype)
    xc = x.to(compute_dtype)
    if fused and compute_dtype in (torch.float16, torch.bfloat16):
        p1 = (xc * cos).double()
        out = (_rotate_pairs(xc, inverse).double() * sin.double() + p1).to(compute_dtype)   # exact sum, one rounding
    else:
        out = xc * cos + _rotate_pairs(xc, inverse) * sin
    tok = torch.arange(n)
    tok = tok[None, None, :, None] if heads_second else tok[None, :, None, None]
    mask = (tok < cutoff) & (torch.arange(d) < Rc)
    return torch.where(mask, out, xc)


def rope(x: torch.Tensor, pos_emb: torch.Tensor, cutoff: int | None = None, heads_second: bool = True,
         transposed: bool = False, mode: str = "compiled") -> torch.Tensor:
    """Stand-alone rotary.  The reference computes in the promoted dtype of x
    and the table without an fp32 upcast (head_rope_cached.py:127-142).  For a
    16-bit x with a table of the same type the result depends on how the
    expression is evaluated:
      mode="compiled"     rn(fma(rot, sin, rn(x*cos))): what the reference's
                          kernel does when compiled for a GPU (checked on B200:
                          bit-equal with its output for bf16, 99.999 % for fp16);
      mode="interpreted"  one rounding per operation: what Triton's interpreter
                          (the golden vectors) and torch eager do.
    The two differ by at most one unit in the last place of the larger product."""
    n = x.shape[2] if heads_second else x.shape[1]
    cutoff = n if cutoff is None else cutoff
    cd = torch.promote_types(x.dtype, pos_emb.dtype)
    return _rope_apply(x.detach(), pos_emb.detach(), cutoff, heads_second, transposed, cd,
                       fused=(mode == "compiled")).to(x.dtype)


# --------------------------------------------------------------------------
# Fused LayerNorm -> rotary  (fused_ln_rope_cached.py:54-114, :198-237, :349-375)
# --------------------------------------------------------------------------


def lnrope_fwd(x: torch.Tensor, pos_emb: torch.Tensor, cutoff: int | None = None, heads_second: bool = True,
               eps: float = 1e-6) -> torch.Tensor:
    n = x.shape[2] if heads_second else x.shape[1]
    cutoff = n if cutoff is None else cutoff
    xs, rstd = _ln_stats(_f(x), eps)
    y = xs * rstd
    return _rope_apply(y, _f(pos_emb), cutoff, heads_second, False, torch.float32).to(x.dtype)


def lnrope_bwd(x: torch.Tensor, dy: torch.Tensor, pos_emb: torch.Tensor, cutoff: int | None = None,
               heads_second: bool = True, eps: float = 1e-6) -> torch.Tensor:
    n = x.shape[2] if heads_second else x.shape[1]
    cutoff = n if cutoff is None else cutoff
    g = _rope_apply(_f(dy), _f(pos_emb), cutoff, heads_second, True, torch.float32)    # :349-360
    return _ln_bwd_f32(_f(x), g, eps).to(x.dtype)                                      # :363-372


# --------------------------------------------------------------------------
# Attention  (flash_attn_triton_cached.py:143-220 forward, :290 delta, :443-522 backward)
# Layout (batch, seqlen, nheads, headdim).  This is the exact (untiled) fp32
# evaluation of what the tiled kernels approximate; the kernels round P and dS
# to 16 bits before their second GEMMs, which is where their error comes from.
# --------------------------------------------------------------------------


def _scores(q, k, bias, causal: bool, scale: float) -> torch.Tensor:
    qf, kf = _f(q), _f(k)
    s = torch.einsum("bthd,bshd->bhts", qf, kf) * scale                 # :143-144, :173/:177
    if bias is not None:
        s = s + _f(bias)                                                # :173
    if causal:
        tq, tk = s.shape[-2:]
        keep = torch.arange(tq)[:, None] >= torch.arange(tk)[None, :]   # :150 (top-left aligned)
        s = s.masked_fill(~keep, float("-inf"))
    return s


def attn_fwd(q, k, v, bias=None, causal: bool = False, softmax_scale: float | None = None):
    """Returns (o in q.dtype, lse fp32 [B, H, Tq])."""
    scale = softmax_scale or 1.0 / math.sqrt(q.shape[-1])
    s = _scores(q, k, bias, causal, scale)
    lse = torch.logsumexp(s, dim=-1)                                    # :213-214
    p = torch.exp(s - lse[..., None])
    o = torch.einsum("bhts,bshd->bthd", p, _f(v))                       # :209, :218-220
    return o.to(q.dtype), lse


def attn_bwd(q, k, v, do, bias=None, causal: bool = False, softmax_scale: float | None = None):
    """Returns (dq, dk, dv) in q.dtype."""
    scale = softmax_scale or 1.0 / math.sqrt(q.shape[-1])
    s = _scores(q, k, bias, causal, scale)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])                                   # :476
    dof, vf = _f(do), _f(v)
    o = torch.einsum("bhts,bshd->bthd", p, vf)
    delta = (o * dof).sum(-1).permute(0, 2, 1)                          # :290, [B,H,Tq]
    dv = torch.einsum("bhts,bthd->bshd", p, dof)                        # :492
    dp = torch.einsum("bthd,bshd->bhts", dof, vf)                       # :500
    ds = p * (dp - delta[..., None]) * scale                            # :510
    dq = torch.einsum("bhts,bshd->bthd", ds, _f(k))                     # :522
    dk = torch.einsum("bhts,bthd->bshd", ds, _f(q))                     # :512
    return dq.to(q.dtype), dk.to(q.dtype), dv.to(q.dtype)


def attn_bwd_dbias(q, k, v, do, bias, causal: bool = False, softmax_scale: float | None = None):
    """Gradient of the additive bias in fp32, shaped like `bias`: the scores are
    q k^T * scale + bias (flash_attn_triton_cached.py:151-175), so
    d bias = dS / scale = P * (dP - delta), summed over the dimensions along which the
    bias is broadcast.  The reference does not produce it (:1107)."""
    scale = softmax_scale or 1.0 / math.sqrt(q.shape[-1])
    s = _scores(q, k, bias, causal, scale)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    dof, vf = _f(do), _f(v)
    o = torch.einsum("bhts,bshd->bthd", p, vf)
    delta = (o * dof).sum(-1).permute(0, 2, 1)
    dp = torch.einsum("bthd,bshd->bhts", dof, vf)
    ds = p * (dp - delta[..., None])
    dims = [i for i in range(4) if bias.shape[i] == 1 and ds.shape[i] != 1]
    return ds.sum(dim=dims, keepdim=True) if dims else ds


def attn_lowp(q, k, v, do, bias=None, causal: bool = False, softmax_scale: float | None = None):
    """Low-precision eager attention (every op in q.dtype), forward and
    backward through autograd: the yardstick the reference's own tests use for
    "error at most 2x that of a PyTorch implementation" (tests/test_flash_attn.py:18-62)."""
    scale = softmax_scale or 1.0 / math.sqrt(q.shape[-1])
    q, k, v = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
    s = torch.einsum("bthd,bshd->bhts", q * scale, k)
    if bias is not None:
        s = s + bias.to(s.dtype)
    if causal:
        tq, tk = s.shape[-2:]
        keep = torch.arange(tq)[:, None] >= torch.arange(tk)[None, :]
        s = s.masked_fill(~keep, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhts,bshd->bthd", p, v)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
    return o.detach(), dq, dk, dv
