"""Side by side with the reference's own Triton kernels on the same GPU.

Runs only where the unmodified reference is importable from ``baseline/_ref``
(an offline ``pip install --target`` of the reference project; not part of this
repository) and Triton can compile for the device; skipped otherwise.  The
reference entries are called with ``kernel_cache=None``: every call goes through
Triton's normal launcher.

Rules checked (the bars this library is built to):
* attention: max-abs error of out / dq / dk / dv against the exact fp32
  evaluation at most 2x the reference kernel's error on the same inputs;
* stand-alone RoPE on 16-bit tensors: bit-identical to the reference kernel;
* FusedLNRoPE, head LayerNorm, RMS and L2 norms: 16-bit results within one unit
  in the last place of the reference kernel's (elements that are cancellation
  results near zero are compared on the tensor's scale, see ``assert_parity``);
* RMSNorm dweight: at least as close to the fp32 value as the reference's (the
  reference sums batches in the weight dtype, this library in fp32).
"""
import sys
from pathlib import Path

import pytest
import torch

from oracle import oracle as O
from rgd_triton_b200 import functional as F_
from tests._util import assert_parity, attn_error, gen, randn, rotary_table

pytestmark = pytest.mark.gpu

REF_ROOT = Path(__file__).resolve().parent.parent / "baseline" / "_ref"


@pytest.fixture(scope="module")
def ref():
    if not (REF_ROOT / "rgd_triton").is_dir():
        pytest.skip("reference project is not installed under baseline/_ref")
    sys.path.insert(0, str(REF_ROOT))
    try:
        import triton  # noqa: F401
        from rgd_triton.triton.flash_attn.flash_attn_triton_cached import flash_attn_func
        from rgd_triton.triton.normalization.fused_l2normalize_cached import triton_fused_norm_func_fn
        from rgd_triton.triton.normalization.fused_rmsnorm_cached import triton_fused_rms_func_fn
        from rgd_triton.triton.normalization.head_layernorm_cached import triton_fused_ln_func_fn
        from rgd_triton.triton.normalization.rmsnorm_cached import triton_rms_func_fn
        from rgd_triton.triton.rope.fused_ln_rope_cached import triton_fused_ln_rope_fn
        from rgd_triton.triton.rope.head_rope_cached import triton_rope_fn
    except Exception as e:  # no Triton, or an incompatible one
        pytest.skip(f"reference kernels cannot be imported here: {e!r}")
    finally:
        sys.path.remove(str(REF_ROOT))

    class R:
        attn = staticmethod(flash_attn_func)
        l2_2 = staticmethod(triton_fused_norm_func_fn)
        rms2 = staticmethod(triton_fused_rms_func_fn)
        headln = staticmethod(triton_fused_ln_func_fn)
        rms = staticmethod(triton_rms_func_fn)
        lnrope = staticmethod(triton_fused_ln_rope_fn)
        rope = staticmethod(triton_rope_fn)
    yield R
    # give the import names back, so that nothing that runs later in this process picks the
    # reference up by accident
    for name in [n for n in sys.modules if n == "rgd_triton" or n.startswith("rgd_triton.")]:
        del sys.modules[name]


def _fwd_bwd(fn, inputs, grads):
    dev = [t.detach().cuda().requires_grad_(True) for t in inputs]
    outs = fn(*dev)
    outs = outs if isinstance(outs, tuple) else (outs,)
    gs = torch.autograd.grad(outs, dev, [g.cuda() for g in grads])
    torch.cuda.synchronize()
    return [o.detach().cpu() for o in outs], [g.cpu() for g in gs]


@pytest.mark.parametrize("d,dt,with_bias", [(128, torch.bfloat16, False), (64, torch.float16, True),
                                            (64, torch.bfloat16, False), (32, torch.float16, True)])
def test_attention_error_at_most_twice_the_reference_kernels(ref, d, dt, with_bias):
    g = gen(100 + d)
    B, Tn, H = 1, 1024, 4
    q, k, v, do = (randn(g, B, Tn, H, d, dtype=dt) for _ in range(4))
    bias = randn(g, B, H, Tn, Tn, dtype=dt) if with_bias else None
    fb = None if bias is None else bias.float()
    eo, _ = O.attn_fwd(q.float(), k.float(), v.float(), fb)
    exact = [eo.float(), *[t.float() for t in O.attn_bwd(q.float(), k.float(), v.float(), do.float(), fb)]]
    errs = {}
    for name, fn in (("reference", ref.attn), ("here", F_.flash_attn_func)):
        bd = None if bias is None else bias.cuda()
        (o,), grads = _fwd_bwd(lambda a, b, c: fn(a, b, c, bd), [q, k, v], [do])
        errs[name] = [attn_error(t, e) for t, e in zip([o, *grads], exact)]
    for what, e_here, e_ref in zip(("out", "dq", "dk", "dv"), errs["here"], errs["reference"]):
        assert e_here <= 2.0 * e_ref + 1e-6, f"{what}: error {e_here:.3e} vs reference kernel {e_ref:.3e}"


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_rope_is_bit_identical_to_the_reference_kernel(ref, dt):
    g = gen(7)
    q, k = randn(g, 2, 1100, 6, 128, dtype=dt), randn(g, 2, 900, 6, 128, dtype=dt)
    pos = rotary_table(1101, 64, dt).cuda()
    a_q, a_k = ref.rope(q.cuda(), k.cuda(), pos, (1000, 800), False)
    b_q, b_k = F_.triton_rope_fn(q.cuda(), k.cuda(), pos, (1000, 800), False)
    assert torch.equal(a_q, b_q) and torch.equal(a_k, b_k)


def test_fused_ln_rope_within_one_ulp_of_the_reference_kernel(ref):
    g = gen(8)
    q, k = randn(g, 2, 1024, 8, 128, dtype=torch.bfloat16), randn(g, 2, 777, 8, 128, dtype=torch.bfloat16)
    gq, gk = randn(g, *q.shape, dtype=torch.bfloat16), randn(g, *k.shape, dtype=torch.bfloat16)
    pos = rotary_table(1025, 64, torch.bfloat16).cuda()
    call = lambda fn: _fwd_bwd(lambda a, b: fn(a, b, pos, (1024, 700), False, 1e-5), [q, k], [gq, gk])
    (ra, rb), (rga, rgb) = call(ref.lnrope)
    (ha, hb), (hga, hgb) = call(F_.triton_fused_ln_rope_fn)
    for got, want, what in ((ha, ra, "q"), (hb, rb, "k"), (hga, rga, "dq"), (hgb, rgb, "dk")):
        assert_parity(got, want, f"lnrope {what}", atol_rel=1e-5)


def test_head_layernorm_within_one_ulp_of_the_reference_kernel(ref):
    g = gen(9)
    q, k = randn(g, 2, 600, 8, 128, dtype=torch.bfloat16), randn(g, 2, 333, 8, 128, dtype=torch.bfloat16)
    gq, gk = randn(g, *q.shape, dtype=torch.bfloat16), randn(g, *k.shape, dtype=torch.bfloat16)
    call = lambda fn: _fwd_bwd(lambda a, b: fn(a, b, False, 1e-6), [q, k], [gq, gk])
    (ra, rb), (rga, rgb) = call(ref.headln)
    (ha, hb), (hga, hgb) = call(F_.triton_fused_ln_func_fn)
    for got, want, what in ((ha, ra, "q"), (hb, rb, "k"), (hga, rga, "dq"), (hgb, rgb, "dk")):
        assert_parity(got, want, f"headln {what}", atol_rel=1e-5)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_rms_and_l2_norms_against_the_reference_kernels(ref, dt):
    g = gen(10)
    B, n1, n2, C = 2, 300, 513, 1024 if dt == torch.float32 else 3072
    a, b = randn(g, B, n1, C, dtype=dt), randn(g, B, n2, C, dtype=dt)
    ga, gb = randn(g, B, n1, C, dtype=dt), randn(g, B, n2, C, dtype=dt)
    w1 = (1 + 0.02 * torch.randn(C, generator=g)).to(dt)
    w2 = (1 + 0.02 * torch.randn(C, generator=g)).to(dt)
    call = lambda fn: _fwd_bwd(lambda *t: fn(*t, 1e-6), [a, b, w1, w2], [ga, gb])
    (ry1, ry2), (rd1, rd2, rdw1, rdw2) = call(ref.rms2)
    (hy1, hy2), (hd1, hd2, hdw1, hdw2) = call(F_.triton_fused_rms_func_fn)
    for got, want, what in ((hy1, ry1, "y1"), (hy2, ry2, "y2"), (hd1, rd1, "dx1"), (hd2, rd2, "dx2")):
        assert_parity(got, want, f"rms2 {what}", atol_rel=1e-5)
    # dweight: compare both with the fp32 value
    for x, dy, w, h_dw, r_dw, what in ((a, ga, w1, hdw1, rdw1, "dw1"), (b, gb, w2, hdw2, rdw2, "dw2")):
        exact = O.rmsnorm_bwd(x.float(), w.float(), dy.float(), 1e-6)[1]
        e_here, e_ref = attn_error(h_dw, exact), attn_error(r_dw, exact)
        assert e_here <= e_ref + 1e-5 * exact.abs().max().item(), f"{what}: {e_here:.3e} vs reference {e_ref:.3e}"
    call = lambda fn: _fwd_bwd(lambda *t: fn(*t, 1e-6), [a, b], [ga, gb])
    (ry1, ry2), (rd1, rd2) = call(ref.l2_2)
    (hy1, hy2), (hd1, hd2) = call(F_.triton_fused_norm_func_fn)
    for got, want, what in ((hy1, ry1, "y1"), (hy2, ry2, "y2"), (hd1, rd1, "dx1"), (hd2, rd2, "dx2")):
        assert_parity(got, want, f"l2 {what}", atol_rel=1e-5)
