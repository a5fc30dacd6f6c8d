"""Generate the golden vectors under tests/golden/ by running the REFERENCE.

The reference's Triton kernels run on the CPU under Triton's interpreter, so
this script needs no GPU — but it needs the reference checkout, which exists
only in the build container:

    TRITON_INTERPRET=1 python -O tests/golden/make_golden.py /path/to/reference

(the checkout's path is the one argument, or the RGD_REFERENCE environment variable).

``-O`` is required because the reference's host wrappers ``assert x.is_cuda``.
The env var must be set before Triton is imported (this script checks).  Each
case stores its inputs and the reference's outputs in one ``.npz``; the tests
only ever read the ``.npz`` files.  bf16 is not generated: the interpreter is
not bit-faithful for bf16.
"""
import os
import sys
from pathlib import Path

if os.environ.get("TRITON_INTERPRET") != "1":
    sys.exit("run with TRITON_INTERPRET=1 (and python -O)")
if __debug__:
    sys.exit("run with python -O (the reference asserts .is_cuda)")

if len(sys.argv) < 2 and not os.environ.get("RGD_REFERENCE"):
    sys.exit("give the path of the reference checkout as the argument (or in RGD_REFERENCE)")
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["RGD_REFERENCE"])
sys.path.insert(0, str(REF))
OUT = Path(__file__).resolve().parent

import numpy as np  # noqa: E402
import torch  # noqa: E402

from rgd_triton.triton.flash_attn.flash_attn_triton_cached import flash_attn_func  # noqa: E402
from rgd_triton.triton.normalization.fused_l2normalize_cached import triton_fused_norm_func_fn  # noqa: E402
from rgd_triton.triton.normalization.fused_rmsnorm_cached import triton_fused_rms_func_fn  # noqa: E402
from rgd_triton.triton.normalization.head_layernorm_cached import triton_fused_ln_func_fn  # noqa: E402
from rgd_triton.triton.normalization.l2normalize_cached import triton_norm_func_fn  # noqa: E402
from rgd_triton.triton.normalization.rmsnorm_cached import triton_rms_func_fn  # noqa: E402
from rgd_triton.triton.rope.fused_ln_rope_cached import triton_fused_ln_rope_fn  # noqa: E402
from rgd_triton.triton.rope.head_rope_cached import triton_rope_fn  # noqa: E402


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def randn(g, *shape, dtype=torch.float32, scale=1.0):
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(OUT / f"{name}.npz", **out)
    print(f"wrote {name}.npz ({(OUT / f'{name}.npz').stat().st_size} bytes)", flush=True)


def rotary_table(P, R, dtype):
    """[2, P, R]: sin, cos; each angle repeated for its channel pair."""
    inv = 1.0 / (10000.0 ** (torch.arange(0, R, 2, dtype=torch.float32) / R))
    ang = (torch.arange(P, dtype=torch.float32)[:, None] * inv[None, :]).repeat_interleave(2, dim=-1)
    return torch.stack([ang.sin(), ang.cos()]).to(dtype)


def tag(dtype):
    return {torch.float32: "f32", torch.float16: "f16"}[dtype]


def grads(outs, ins, gs):
    return torch.autograd.grad(outs, ins, gs)


def case_rms(dtype):
    g = gen(1)
    x = randn(g, 2, 9, 40, dtype=dtype).requires_grad_(True)
    w = (1 + 0.02 * torch.randn(40, generator=g)).to(dtype).requires_grad_(True)
    wb = (1 + 0.02 * torch.randn(2, 1, 40, generator=g)).to(dtype).requires_grad_(True)
    dy = randn(g, 2, 9, 40, dtype=dtype)
    y = triton_rms_func_fn(x, w, 1e-6)
    dx, dw = grads(y, (x, w), dy)
    yb = triton_rms_func_fn(x, wb, 1e-6)
    dxb, dwb = grads(yb, (x, wb), dy)
    save(f"rms_{tag(dtype)}", x=x, w=w, wb=wb, dy=dy, y=y, dx=dx, dw=dw, yb=yb, dxb=dxb, dwb=dwb, eps=1e-6)


def case_rms2(dtype):
    g = gen(2)
    a = randn(g, 2, 9, 40, dtype=dtype).requires_grad_(True)
    b = randn(g, 2, 5, 24, dtype=dtype).requires_grad_(True)
    w1 = (1 + 0.02 * torch.randn(40, generator=g)).to(dtype).requires_grad_(True)
    w2 = (1 + 0.02 * torch.randn(24, generator=g)).to(dtype).requires_grad_(True)
    g1, g2 = randn(g, 2, 9, 40, dtype=dtype), randn(g, 2, 5, 24, dtype=dtype)
    ya, yb = triton_fused_rms_func_fn(a, b, w1, w2, 1e-6)
    da, db, dw1, dw2 = grads((ya, yb), (a, b, w1, w2), (g1, g2))
    save(f"rms2_{tag(dtype)}", a=a, b=b, w1=w1, w2=w2, g1=g1, g2=g2, ya=ya, yb=yb, da=da, db=db, dw1=dw1, dw2=dw2,
         eps=1e-6)


def case_l2(dtype):
    g = gen(3)
    x = randn(g, 2, 9, 40, dtype=dtype)
    x[0, 0] = 0.0                       # exercises the eps gate
    x[1, 3] *= 1e-4 if dtype == torch.float32 else 1e-2
    x.requires_grad_(True)
    dy = randn(g, 2, 9, 40, dtype=dtype)
    y = triton_norm_func_fn(x, 1e-6)
    (dx,) = grads(y, (x,), dy)
    a = randn(g, 2, 9, 40, dtype=dtype).requires_grad_(True)
    b = randn(g, 2, 5, 24, dtype=dtype).requires_grad_(True)
    g1, g2 = randn(g, 2, 9, 40, dtype=dtype), randn(g, 2, 5, 24, dtype=dtype)
    ya, yb = triton_fused_norm_func_fn(a, b, 1e-6)
    da, db = grads((ya, yb), (a, b), (g1, g2))
    save(f"l2_{tag(dtype)}", x=x, dy=dy, y=y, dx=dx, a=a, b=b, g1=g1, g2=g2, ya=ya, yb=yb, da=da, db=db, eps=1e-6)


def case_heads(dtype):
    """Head LayerNorm, RoPE and LN->RoPE on the same q/k, both layouts."""
    g = gen(4)
    B, H, NQ, NK, D, R, P = 2, 3, 9, 5, 64, 32, 16
    pos = rotary_table(P, R, dtype)
    arrays = dict(pos=pos, cut_q=6, cut_k=5, eps=1e-5)
    for hs in (False, True):
        sfx = "hs" if hs else "ns"
        shape_q = (B, H, NQ, D) if hs else (B, NQ, H, D)
        shape_k = (B, H, NK, D) if hs else (B, NK, H, D)
        q = randn(g, *shape_q, dtype=dtype).requires_grad_(True)
        k = randn(g, *shape_k, dtype=dtype).requires_grad_(True)
        gq, gk = randn(g, *shape_q, dtype=dtype), randn(g, *shape_k, dtype=dtype)
        lq, lk = triton_fused_ln_func_fn(q, k, hs, 1e-5)
        dlq, dlk = grads((lq, lk), (q, k), (gq, gk))
        rq, rk = triton_rope_fn(q, k, pos, seq_cutoff=(6, 5), heads_second=hs)
        drq, drk = grads((rq, rk), (q, k), (gq, gk))
        fq, fk = triton_fused_ln_rope_fn(q, k, pos, seq_cutoff=(6, 5), heads_second=hs, norm_eps=1e-5)
        dfq, dfk = grads((fq, fk), (q, k), (gq, gk))
        for n, v in dict(q=q, k=k, gq=gq, gk=gk, lq=lq, lk=lk, dlq=dlq, dlk=dlk, rq=rq, rk=rk, drq=drq, drk=drk,
                         fq=fq, fk=fk, dfq=dfq, dfk=dfk).items():
            arrays[f"{n}_{sfx}"] = v
    save(f"heads_{tag(dtype)}", **arrays)


def case_attn():
    """fp16 attention, odd lengths, every bias kind, causal."""
    g = gen(5)
    dtype = torch.float16
    B, TQ, TK, H, D = 1, 80, 112, 2, 64
    q = randn(g, B, TQ, H, D, dtype=dtype).requires_grad_(True)
    k = randn(g, B, TK, H, D, dtype=dtype).requires_grad_(True)
    v = randn(g, B, TK, H, D, dtype=dtype).requires_grad_(True)
    do = randn(g, B, TQ, H, D, dtype=dtype)
    bm = randn(g, 1, H, TQ, TK, dtype=dtype)
    bv = randn(g, B, 1, 1, TK, dtype=dtype)
    arrays = dict(q=q, k=k, v=v, do=do, bias_matrix=bm, bias_vector=bv)
    for name, bias, causal in (("none", None, False), ("matrix", bm, False), ("vector", bv, False),
                               ("causal", None, True)):
        o, lse = flash_attn_func(q, k, v, bias, causal, None, True)
        dq, dk, dv = grads(o, (q, k, v), do)
        arrays.update({f"o_{name}": o, f"lse_{name}": lse, f"dq_{name}": dq, f"dk_{name}": dk, f"dv_{name}": dv})
    save("attn_f16", **arrays)


def case_config1():
    """FusedRMSNorm at the size of the first benchmark configuration:
    x [4, 256, 1024] fp32, seed 0.  Inputs are regenerated from the seed by the
    test; stored are the full dweight and every 16th row of y and dx."""
    g = gen(0)
    x = torch.randn(4, 256, 1024, generator=g).requires_grad_(True)
    w = (1 + 0.02 * torch.randn(1024, generator=g)).requires_grad_(True)
    dy = torch.randn(4, 256, 1024, generator=g)
    y = triton_rms_func_fn(x, w, 1e-6)
    dx, dw = grads(y, (x, w), dy)
    save("config1_rms_f32", y_rows=y[:, ::16], dx_rows=dx[:, ::16], dw=dw, row_step=16, eps=1e-6,
         x_probe=x[0, 0, :8], dy_probe=dy[3, 255, -8:])


if __name__ == "__main__":
    which = set(sys.argv[2:]) or {"rms", "rms2", "l2", "heads", "attn", "config1"}
    for dt in (torch.float32, torch.float16):
        if "rms" in which:
            case_rms(dt)
        if "rms2" in which:
            case_rms2(dt)
        if "l2" in which:
            case_l2(dt)
        if "heads" in which:
            case_heads(dt)
    if "attn" in which:
        case_attn()
    if "config1" in which:
        case_config1()
