"""Shared helpers for the parity tests."""
import math

import numpy as np
import torch

from oracle import oracle as O

DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def randn(g, *shape, dtype=torch.float32, scale=1.0):
    """Seeded N(0,1) generated on the CPU in fp32, then cast: CPU oracle and GPU
    kernel see identical bits."""
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def rotary_table(P, R, dtype):
    """[2, P, R]: sin, cos of t * 10000^(-2i/R), each angle repeated for its pair."""
    inv = 1.0 / (10000.0 ** (torch.arange(0, R, 2, dtype=torch.float32) / R))
    ang = (torch.arange(P, dtype=torch.float32)[:, None] * inv[None, :]).repeat_interleave(2, dim=-1)[:, :R]
    return torch.stack([ang.sin(), ang.cos()]).to(dtype)


def assert_parity(got: torch.Tensor, want: torch.Tensor, what: str, atol_rel: float = 2e-6):
    """Norm / RoPE parity bar: 16-bit outputs within 1 unit in the last place of
    the oracle, fp32 within 1e-5 relative.  Elements whose absolute error is
    below `atol_rel` x (largest magnitude of the tensor) also pass: they are
    cancellation results whose own ulp is far below fp32 rounding of the inputs."""
    got = got.detach().cpu()
    want = want.detach().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert got.dtype == want.dtype, f"{what}: dtype {got.dtype} vs {want.dtype}"
    if got.numel() == 0:
        return
    gf, wf = got.float(), want.float()
    assert torch.isfinite(gf).all(), f"{what}: non-finite output"
    scale = max(wf.abs().max().item(), 1e-30)
    err = (gf - wf).abs()
    small = err <= atol_rel * scale
    if got.dtype == torch.float32:
        ok = small | (err <= 1e-5 * wf.abs())
    else:
        ok = small | (O.ulp_distance(got, want) <= 1)
    if not ok.all():
        idx = (~ok).nonzero()[0].tolist()
        raise AssertionError(
            f"{what}: {int((~ok).sum())}/{ok.numel()} elements out of tolerance; first at {idx}: "
            f"got {gf[tuple(idx)].item()!r} want {wf[tuple(idx)].item()!r} (tensor scale {scale:.3g})")


def attn_error(got: torch.Tensor, exact: torch.Tensor) -> float:
    return (got.detach().cpu().float() - exact.detach().cpu().float()).abs().max().item()


def assert_attn(got, exact_f32, lowp, what, factor=2.0, floor=1e-4):
    """Attention parity bar: max-abs error against the exact fp32 evaluation at
    most `factor` x the error of the low-precision eager implementation on the
    same inputs (the yardstick of the reference's own tests)."""
    e_got = attn_error(got, exact_f32)
    e_low = attn_error(lowp, exact_f32)
    assert math.isfinite(e_got), f"{what}: non-finite"
    assert e_got <= factor * e_low + floor, f"{what}: error {e_got:.3e} > {factor} x eager {e_low:.3e}"
    return e_got, e_low


def T(a):
    return torch.from_numpy(np.asarray(a))


import contextlib


@contextlib.contextmanager
def attention_backward(mode):
    """Run the body with the attention backward in "two_kernel" (every output bit-reproducible)
    or "single_pass" (head_dim 64: dQ is summed with reductions whose order is not fixed) mode."""
    from rgd_triton_b200 import functional as F_
    prev = F_.set_attention_backward(mode)
    try:
        yield
    finally:
        F_.set_attention_backward(prev)
