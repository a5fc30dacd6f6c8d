"""GPU parity of FlashAttention forward / backward.

Bar (from the reference's own tests, tests/test_flash_attn.py:175-178,
:307-309): the max-abs error against the exact fp32 evaluation must be at most
2x the error a low-precision eager implementation makes on the same inputs.
Shapes follow the reference's grid (d in {32, 64}, odd and unequal lengths)
and add d in {40, 96, 128}, every bias kind incl. broadcast and fp32 bias,
causal, non-contiguous inputs and the benchmark configurations' sizes."""
import math

import pytest
import torch

from oracle import oracle as O
from rgd_triton_b200 import functional as F_, ops
from tests._util import DTYPES, T, assert_attn, attention_backward, attn_error, gen, randn

pytestmark = pytest.mark.gpu

@pytest.fixture(autouse=True)
def _no_device_wait_timed_out():
    """Every bounded device-side wait of the tensor-memory kernels must have
    completed normally."""
    yield
    from rgd_triton_b200 import _lib
    assert _lib.load().rgd_device_status() == 0, "a bounded device-side wait expired (RGD_E_TIMEOUT)"


LENS = [(113, 203), (128, 217), (108, 256), (256, 512), (1, 1), (3, 1023), (1023, 1024), (64, 64)]


def run_attn(q, k, v, do, bias=None, causal=False, scale=None):
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    bd = bias.cuda() if bias is not None else None
    o, lse = F_.flash_attn_func(qd, kd, vd, bd, causal, scale, return_lse=True)
    dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), do.cuda())
    torch.cuda.synchronize()
    return o.detach().cpu(), lse.cpu(), dq.cpu(), dk.cpu(), dv.cpu()


# Additive slack on top of "2x the low-precision eager error": half a unit in the last place of
# a bf16 value of magnitude ~0.1, so the eager error is what decides, not the slack.
GRAD_FLOOR = 5e-4


def check(q, k, v, do, bias=None, causal=False, what="", scale=None):
    o, lse, dq, dk, dv = run_attn(q, k, v, do, bias, causal, scale)
    fb = None if bias is None else bias.float()
    eo, elsed = O.attn_fwd(q.float(), k.float(), v.float(), fb, causal, scale)
    edq, edk, edv = O.attn_bwd(q.float(), k.float(), v.float(), do.float(), fb, causal, scale)
    lo, ldq, ldk, ldv = O.attn_lowp(q, k, v, do, bias, causal, scale)
    tq = q.shape[1]
    torch.testing.assert_close(lse[:, :, :tq], elsed, rtol=1e-3, atol=2e-3, msg=lambda m: f"{what} lse: {m}")
    assert_attn(o, eo, lo, f"{what} o")
    # the reference's own tests allow 2x (out) and up to 5x (gradients); 2x is asked of all four here
    assert_attn(dq, edq, ldq, f"{what} dq", factor=2.0, floor=GRAD_FLOOR)
    assert_attn(dk, edk, ldk, f"{what} dk", factor=2.0, floor=GRAD_FLOOR)
    assert_attn(dv, edv, ldv, f"{what} dv", factor=2.0, floor=GRAD_FLOOR)


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("d", [32, 64, 128, 40, 96])
@pytest.mark.parametrize("causal", [False, True])
def test_no_bias(dt, d, causal):
    dtype = DTYPES[dt]
    g = gen(d)
    for tq, tk in LENS:
        q, k, v = randn(g, 2, tq, 3, d, dtype=dtype), randn(g, 2, tk, 3, d, dtype=dtype), randn(g, 2, tk, 3, d, dtype=dtype)
        do = randn(g, 2, tq, 3, d, dtype=dtype)
        check(q, k, v, do, None, causal, f"d={d} ({tq},{tk}) causal={causal}")


BIAS_KINDS = ["vector", "matrix", "matrix_bcast_b", "matrix_bcast_h", "vector_bcast", "matrix_f32"]


def make_bias(g, kind, B, H, tq, tk, dtype):
    shape = {"vector": (B, H, 1, tk), "matrix": (B, H, tq, tk), "matrix_bcast_b": (1, H, tq, tk),
             "matrix_bcast_h": (B, 1, tq, tk), "vector_bcast": (1, 1, 1, tk), "matrix_f32": (B, H, tq, tk)}[kind]
    return randn(g, *shape, dtype=torch.float32 if kind == "matrix_f32" else dtype)


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("d", [64, 128, 32, 40, 96])
@pytest.mark.parametrize("kind", BIAS_KINDS)
def test_bias(dt, d, kind):
    """Every bias kind on the tensor-memory kernels (d = 64, 128) and on the general
    kernels (d = 32, 40, 96; the reference's own grid is bias kind x d in {32, 64},
    tests/test_flash_attn.py:70-73)."""
    dtype = DTYPES[dt]
    g = gen(d + len(kind))
    B, H = 2, 3
    for tq, tk in [(113, 203), (128, 217), (256, 512), (3, 1023)]:
        q, k, v = randn(g, B, tq, H, d, dtype=dtype), randn(g, B, tk, H, d, dtype=dtype), randn(g, B, tk, H, d, dtype=dtype)
        do = randn(g, B, tq, H, d, dtype=dtype)
        bias = make_bias(g, kind, B, H, tq, tk, dtype)
        check(q, k, v, do, bias, False, f"{kind} d={d} ({tq},{tk})")


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("d", [64, 128, 32, 96])
@pytest.mark.parametrize("kind", ["vector", "matrix", "matrix_bcast_b", "matrix_f32"])
def test_causal_with_bias(dt, d, kind):
    """The causal mask together with a bias, on both kernel families."""
    dtype = DTYPES[dt]
    g = gen(3 * d + len(kind))
    B, H = 2, 2
    for tq, tk in [(113, 203), (256, 256), (200, 136), (384, 640)]:
        q, k, v = randn(g, B, tq, H, d, dtype=dtype), randn(g, B, tk, H, d, dtype=dtype), randn(g, B, tk, H, d, dtype=dtype)
        do = randn(g, B, tq, H, d, dtype=dtype)
        bias = make_bias(g, kind, B, H, tq, tk, dtype)
        check(q, k, v, do, bias, True, f"causal {kind} d={d} ({tq},{tk})")


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("kind", [None, "vector", "matrix"])
@pytest.mark.parametrize("shape", [(384, 384, True), (256, 300, False), (200, 330, True)])
def test_scores_growing_along_the_keys(d, kind, shape):
    """Scores that grow by about 7 nats per 128 keys: the softmax's reference maximum is raised in
    every key block, the last one included - the block that crosses the causal diagonal or the
    end of the keys, which has code of its own in the forward."""
    tq, tk, causal = shape
    g = gen(5 * d + tq + (0 if kind is None else len(kind)))
    B, H = 1, 2
    u = torch.ones(d)
    ramp = 7.0 / (128 * d ** 0.5) * torch.arange(tk, dtype=torch.float32)
    q = (0.3 * randn(g, B, tq, H, d) + u).to(torch.bfloat16)
    k = (0.3 * randn(g, B, tk, H, d) + ramp[None, :, None, None] * u).to(torch.bfloat16)
    v, do = randn(g, B, tk, H, d, dtype=torch.bfloat16), randn(g, B, tq, H, d, dtype=torch.bfloat16)
    bias = None if kind is None else make_bias(g, kind, B, H, tq, tk, torch.bfloat16)
    check(q, k, v, do, bias, causal, f"growing scores d={d} {kind} ({tq},{tk}) causal={causal}")


def _uses_tmem_fwd(q, k, v):
    import ctypes as C
    from rgd_triton_b200 import _lib
    hv = lambda t: C.byref(F_._attn_heads(t))
    o = torch.empty_like(q)
    return _lib.load().rgd_attn_fwd_uses_tmem(hv(q), hv(k), hv(v), hv(o), q.shape[0], q.shape[2], q.shape[1],
                                              k.shape[1], q.shape[3], 1.0, _lib.dtype_code(q.dtype))


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("kind", [None, "matrix", "vector"])
def test_misaligned_views_take_the_general_kernels(d, kind):
    """q, k, v as channel slices [3 : 3 + d] of wider tensors: rows are not 16-byte
    addressable, so the call must leave the tensor-memory kernels and still be right."""
    g = gen(70 + d)
    B, H, tq, tk = 2, 2, 150, 217
    wide = [randn(g, B, n, H, d + 8, dtype=torch.bfloat16) for n in (tq, tk, tk)]
    q, k, v = (w[..., 3:3 + d] for w in wide)
    do = randn(g, B, tq, H, d, dtype=torch.bfloat16)
    bias = None if kind is None else make_bias(g, kind, B, H, tq, tk, torch.bfloat16)
    qd, kd, vd = (w.cuda()[..., 3:3 + d] for w in wide)
    assert _uses_tmem_fwd(qd, kd, vd) == 0
    assert _uses_tmem_fwd(qd.contiguous(), kd.contiguous(), vd.contiguous()) == 1
    qd, kd, vd = (t.requires_grad_(True) for t in (qd, kd, vd))
    o = F_.flash_attn_func(qd, kd, vd, None if bias is None else bias.cuda())
    dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), do.cuda())
    fb = None if bias is None else bias.float()
    eo, _ = O.attn_fwd(q.float(), k.float(), v.float(), fb)
    edq, edk, edv = O.attn_bwd(q.float(), k.float(), v.float(), do.float(), fb)
    lo, ldq, ldk, ldv = O.attn_lowp(q, k, v, do, bias)
    assert_attn(o, eo, lo, "o")
    assert_attn(dq, edq, ldq, "dq", floor=GRAD_FLOOR)
    assert_attn(dk, edk, ldk, "dk", floor=GRAD_FLOOR)
    assert_attn(dv, edv, ldv, "dv", floor=GRAD_FLOOR)


@pytest.mark.parametrize("d", [64, 128])
def test_batch_expanded_keys_and_values(d):
    """k and v expanded over the batch (stride 0): no tensor map describes that, the call
    runs on the general kernels instead of failing."""
    g = gen(90 + d)
    B, H, tq, tk = 3, 2, 140, 200
    q, do = randn(g, B, tq, H, d, dtype=torch.float16), randn(g, B, tq, H, d, dtype=torch.float16)
    k1, v1 = randn(g, 1, tk, H, d, dtype=torch.float16), randn(g, 1, tk, H, d, dtype=torch.float16)
    k, v = k1.expand(B, -1, -1, -1), v1.expand(B, -1, -1, -1)
    qd = q.cuda().requires_grad_(True)
    kd, vd = k1.cuda().expand(B, -1, -1, -1), v1.cuda().expand(B, -1, -1, -1)
    assert _uses_tmem_fwd(qd, kd, vd) == 0
    o = F_.flash_attn_func(qd, kd, vd)
    (dq,) = torch.autograd.grad(o, (qd,), do.cuda())
    eo, _ = O.attn_fwd(q.float(), k.float(), v.float())
    edq, _, _ = O.attn_bwd(q.float(), k.float(), v.float(), do.float())
    lo, ldq, _, _ = O.attn_lowp(q, k, v, do)
    assert_attn(o, eo, lo, "o")
    assert_attn(dq, edq, ldq, "dq", floor=GRAD_FLOOR)


@pytest.mark.parametrize("d,with_bias", [(96, False), (32, True), (40, False)])
def test_odd_head_dims_large_problems_are_padded_onto_the_tensor_memory_kernels(d, with_bias):
    """Head dims other than 64 / 128 run on the general kernels when the problem is small and are
    zero-padded to 64 / 128 when it is large; both must agree with the oracle (same scale
    1/sqrt(d), padded channels cut off again) and with each other."""
    g = gen(200 + d)
    B, Tn, H = 1, 2048, 4                             # B * H * Tq * Tk = 2^24: the padded path
    q, k, v, do = (randn(g, B, Tn, H, d, dtype=torch.bfloat16) for _ in range(4))
    bias = randn(g, B, H, Tn, Tn, dtype=torch.bfloat16) if with_bias else None
    assert F_._pad_head_dim_pays(q.cuda(), k.cuda())
    check(q, k, v, do, bias, False, f"padded d={d}")
    o, lse, dq, dk, dv = run_attn(q, k, v, do, bias)
    assert o.shape == q.shape and dq.shape == q.shape and dk.shape == k.shape and o.is_contiguous()
    # the same rows through the general kernels (a slice small enough not to be padded)
    qs, dos = q[:, :512].contiguous(), do[:, :512].contiguous()
    bs = None if bias is None else bias[:, :, :512].contiguous()
    assert not F_._pad_head_dim_pays(qs.cuda(), k.cuda())
    o2, lse2, _, _, _ = run_attn(qs, k, v, dos, bs)
    torch.testing.assert_close(o[:, :512].float(), o2.float(), rtol=2e-2, atol=2e-3)
    torch.testing.assert_close(lse[:, :, :512], lse2[:, :, :512], rtol=1e-3, atol=2e-3)


@pytest.mark.parametrize("d", [64, 32])
def test_negative_softmax_scale(d):
    """The reference accepts any scale; a negative one must not reach the forward fast
    path that takes the block maximum before scaling."""
    g = gen(5 + d)
    q, k, v, do = (randn(g, 2, 160, 2, d, dtype=torch.bfloat16) for _ in range(4))
    check(q, k, v, do, None, False, f"negative scale d={d}", scale=-0.2)


def test_block_mask_bias_like_config4():
    """-1e4 on random 64x64 blocks (diagonal kept), the bias of the fourth
    benchmark configuration at a size the oracle handles quickly."""
    g = gen(44)
    B, H, Tn, d = 1, 2, 512, 64
    q, k, v, do = (randn(g, B, Tn, H, d, dtype=torch.float16) for _ in range(4))
    bias = randn(g, B, H, Tn, Tn)
    blk = (torch.rand(B, H, Tn // 64, Tn // 64, generator=g) < 0.1)
    blk &= ~torch.eye(Tn // 64, dtype=torch.bool)
    bias = (bias - 1e4 * blk.repeat_interleave(64, 2).repeat_interleave(64, 3)).to(torch.float16)
    check(q, k, v, do, bias, False, "block mask")
    check(q, k, v, do, bias[:1].clone(), False, "block mask broadcast")


def test_bias_shape_error_is_runtime_error():
    q = torch.zeros(1, 8, 2, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError):
        F_.flash_attn_func(q, q, q, torch.zeros(1, 2, 4, 8, device="cuda", dtype=torch.float16))
    with pytest.raises(AssertionError):
        F_.flash_attn_func(q, q, q, torch.zeros(1, 2, 8, 8, device="cuda", dtype=torch.float64))
    # a bias that requires grad is not refused (the reference does, flash_attn_triton_cached.py:1107):
    # its gradient is produced, see test_bias_gradient
    b = torch.zeros(1, 2, 8, 8, device="cuda", dtype=torch.float16, requires_grad=True)
    o = F_.flash_attn_func(q.clone().requires_grad_(True), q, q, b)
    o.sum().backward()
    assert b.grad is not None and b.grad.shape == b.shape


def test_golden_vectors(golden):
    """Against outputs of the reference's own kernel (fp16)."""
    g = golden("attn_f16")
    q, k, v, do = T(g["q"]), T(g["k"]), T(g["v"]), T(g["do"])
    for kind in ("none", "matrix", "vector", "causal"):
        bias = {"none": None, "causal": None, "matrix": T(g["bias_matrix"]), "vector": T(g["bias_vector"])}[kind]
        o, lse, dq, dk, dv = run_attn(q, k, v, do, bias, kind == "causal")
        tq = q.shape[1]
        torch.testing.assert_close(lse[:, :, :tq], T(g[f"lse_{kind}"])[:, :, :tq], rtol=1e-4, atol=1e-4)
        for got, name in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
            want = T(g[f"{name}_{kind}"])
            err = attn_error(got, want)
            assert err <= 4e-3 * max(want.float().abs().max().item(), 1.0), f"{name}_{kind}: {err}"


def test_noncontiguous_inputs_and_grad():
    """(B,h,T,d) tensors passed as transposed views, and a non-contiguous dO
    (tests/test_flash_attn.py:463-513)."""
    g = gen(8)
    B, H, Tn, d = 2, 3, 200, 64
    qh, kh, vh = (randn(g, B, H, Tn, d, dtype=torch.bfloat16) for _ in range(3))
    q, k, v = qh.transpose(1, 2), kh.transpose(1, 2), vh.transpose(1, 2)
    do = randn(g, B, Tn, d, H, dtype=torch.bfloat16).transpose(2, 3)       # channel stride != 1
    qd, kd, vd = (t.cuda().transpose(1, 2).requires_grad_(True) for t in (qh, kh, vh))
    o = F_.flash_attn_func(qd, kd, vd)
    dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), do.cuda())
    eo, _ = O.attn_fwd(q.float(), k.float(), v.float())
    edq, edk, edv = O.attn_bwd(q.float(), k.float(), v.float(), do.float())
    lo, ldq, ldk, ldv = O.attn_lowp(q, k, v, do)
    assert_attn(o, eo, lo, "o")
    assert_attn(dq, edq, ldq, "dq", floor=GRAD_FLOOR)
    assert_attn(dk, edk, ldk, "dk", floor=GRAD_FLOOR)
    assert_attn(dv, edv, ldv, "dv", floor=GRAD_FLOOR)


def test_backward_overflow_small_seqlens():
    """Scaled inputs at tiny lengths (tests/test_flash_attn.py:399-451)."""
    g = gen(9)
    for tq, tk in [(15, 15), (31, 17), (64, 129)]:
        q, k, v = (randn(g, 2, n, 4, 64, dtype=torch.float16, scale=5.0) for n in (tq, tk, tk))
        do = randn(g, 2, tq, 4, 64, dtype=torch.float16)
        o, lse, dq, dk, dv = run_attn(q, k, v, do)
        for t in (o, dq, dk, dv):
            assert torch.isfinite(t.float()).all()
        edq, edk, edv = O.attn_bwd(q.float(), k.float(), v.float(), do.float())
        _, ldq, ldk, ldv = O.attn_lowp(q, k, v, do)
        assert_attn(dq, edq, ldq, "dq", factor=5.0, floor=2e-2)
        assert_attn(dk, edk, ldk, "dk", factor=5.0, floor=2e-2)
        assert_attn(dv, edv, ldv, "dv", factor=5.0, floor=2e-2)


@pytest.mark.parametrize("mode", ["two_kernel", "single_pass"])
def test_repeat_runs_are_bit_identical(mode):
    """tests/test_flash_attn.py:341-388: outputs and dK/dV bit-equal across repeated launches, dQ
    within 2 * max |(dq + 0.3 - 0.3) - dq| (the reference adds into dq with atomics).  The
    two-kernel backward has no atomics anywhere, so there dQ is bit-equal as well; the single-pass
    backward (head_dim 64) holds exactly the reference's contract."""
    g = gen(10)
    q, k, v = (randn(g, 6, n, 5, 64, dtype=torch.bfloat16).cuda() for n in (239, 127, 127))
    do = randn(g, 6, 239, 5, 64, dtype=torch.bfloat16).cuda()
    m = ops.FlashAttention()
    first = None
    with attention_backward(mode):
        for _ in range(10):
            qi, ki, vi = (t.clone().requires_grad_(True) for t in (q, k, v))
            o = m(qi, ki, vi)
            cur = [o, *torch.autograd.grad(o, (qi, ki, vi), do)]
            if first is None:
                first = [t.clone() for t in cur]
                dq_atol = 2 * ((first[1] + 0.3 - 0.3) - first[1]).abs().max().item()
            else:
                for i in (0, 2, 3):
                    assert torch.equal(first[i], cur[i])
                if mode == "two_kernel":
                    assert torch.equal(first[1], cur[1])
                else:
                    assert (first[1].float() - cur[1].float()).abs().max().item() <= dq_atol
    assert m.cache.fwd is not None and m.cache.bwd is not None


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("bias_kind", [None, "vector", "matrix"])
@pytest.mark.parametrize("causal", [False, True])
def test_single_pass_backward_against_two_kernel(dt, bias_kind, causal):
    """head_dim 64: the single-pass backward returns bit-identical dK and dV and a dQ within one
    rounding step of the two-kernel form (same arithmetic per tile; only the order of the fp32 sums
    into dQ differs), on sizes with ragged ends and several key and query blocks."""
    dtype = DTYPES[dt]
    g = gen(64 + int(causal) + len(bias_kind or ""))
    B, H, tq, tk = 2, 3, 1100, 904
    q, do = randn(g, B, tq, H, 64, dtype=dtype), randn(g, B, tq, H, 64, dtype=dtype)
    k, v = randn(g, B, tk, H, 64, dtype=dtype), randn(g, B, tk, H, 64, dtype=dtype)
    bias = None
    if bias_kind == "vector":
        bias = randn(g, B, H, 1, tk, dtype=dtype)
    elif bias_kind == "matrix":
        bias = randn(g, 1, H, tq, tk, dtype=dtype)
    with attention_backward("two_kernel"):
        a = run_attn(q, k, v, do, bias, causal)
    with attention_backward("single_pass"):
        b = run_attn(q, k, v, do, bias, causal)
    assert torch.equal(a[3], b[3]) and torch.equal(a[4], b[4])
    ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    assert (a[2].float() - b[2].float()).abs().max().item() <= 2 * ulp * a[2].float().abs().max().item()


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_long_sequences_steady_state_pipeline(d, causal):
    """Many key / query blocks per CTA, so the software pipelines of the tensor-memory kernels
    (tile rings, double-buffered score columns, several MMA-issuing threads) run in steady
    state: parity against the oracle, and bit-equal results over repeated launches (a race
    between the issuing threads would show up as run-to-run differences)."""
    g = gen(21 + d + int(causal))
    q, k, v, do = (randn(g, 1, 1664, 2, d, dtype=torch.bfloat16) for _ in range(4))
    check(q, k, v, do, None, causal, f"long d={d} causal={causal}")
    first = None
    with attention_backward("two_kernel"):
        for _ in range(4):
            cur = run_attn(q, k, v, do, None, causal)
            if first is None:
                first = cur
            else:
                assert all(torch.equal(a, b) for a, b in zip(first, cur))
    # the default backward (single-pass at head_dim 64): everything but dQ stays bit-equal
    for _ in range(3):
        cur = run_attn(q, k, v, do, None, causal)
        assert all(torch.equal(first[i], cur[i]) for i in (0, 1, 3, 4))


def _check_sampled_heads(cfg, q, k, v, do, bias_dev, o, grads, pairs):
    """Exact fp32 oracle on a few (batch, head) pairs of a full-size problem; the bias slice
    of each pair is brought back from the device, so oracle and kernel see the same bits."""
    dq, dk, dv = grads
    for b, h in pairs:
        sq, sk, sv, sdo = (t[b:b + 1, :, h:h + 1] for t in (q, k, v, do))
        sb = None
        if bias_dev is not None:
            bb = b if bias_dev.shape[0] > 1 else 0
            hh = h if bias_dev.shape[1] > 1 else 0
            sb = bias_dev[bb:bb + 1, hh:hh + 1].cpu()
        fb = None if sb is None else sb.float()
        eo, _ = O.attn_fwd(sq.float(), sk.float(), sv.float(), fb)
        edq, edk, edv = O.attn_bwd(sq.float(), sk.float(), sv.float(), sdo.float(), fb)
        lo, ldq, ldk, ldv = O.attn_lowp(sq, sk, sv, sdo, sb)
        sl = lambda t: t.detach().cpu()[b:b + 1, :, h:h + 1]
        assert_attn(sl(o), eo, lo, f"{cfg} o[{b},{h}]")
        assert_attn(sl(dq), edq, ldq, f"{cfg} dq[{b},{h}]", floor=GRAD_FLOOR)
        assert_attn(sl(dk), edk, ldk, f"{cfg} dk[{b},{h}]", floor=GRAD_FLOOR)
        assert_attn(sl(dv), edv, ldv, f"{cfg} dv[{b},{h}]", floor=GRAD_FLOOR)


def _block_mask_bias(Bb, H, Tn, dtype, seed):
    """N(0,1) plus -1e4 on 64x64 blocks chosen Bernoulli(0.1), diagonal blocks kept: the bias
    of the fourth benchmark configuration, generated on the device (1.6 GB at full size)."""
    gd = torch.Generator(device="cuda").manual_seed(seed)
    bias = torch.randn(Bb, H, Tn, Tn, device="cuda", generator=gd, dtype=torch.float32).to(dtype)
    nb = Tn // 64
    blk = (torch.rand(Bb, H, nb, nb, device="cuda", generator=gd) < 0.1) & ~torch.eye(nb, dtype=torch.bool, device="cuda")
    bias.view(Bb, H, nb, 64, nb, 64).masked_fill_(blk[:, :, :, None, :, None], -1e4)
    return bias


@pytest.mark.parametrize("cfg", ["config3", "config4_full_bias", "config4_broadcast_bias", "config5_attention"])
def test_benchmark_configurations_full_size(cfg):
    """Third, fourth and fifth benchmark configurations' attention at full (per-GPU) size.
    The exact oracle is evaluated for sampled (batch, head) pairs, and linearity in dO is
    checked on the whole tensors."""
    g = gen(0)
    pairs = None
    if cfg == "config3":
        B, Tn, H, d, dtype = 4, 4096, 16, 128, torch.bfloat16
        bias = None
    elif cfg.startswith("config4"):
        B, Tn, H, d, dtype = 2, 4096, 24, 64, torch.float16
        bias = _block_mask_bias(2 if cfg == "config4_full_bias" else 1, H, Tn, dtype, 4)
    else:
        # MMDiT joint attention, one GPU's share of the batch: 4096 image tokens then 512 text
        # tokens, keys of padded text positions masked by -1e4 in a dense (B, h, T, T) bias
        B, Tn, H, d, dtype = 2, 4608, 24, 128, torch.bfloat16
        text_len = [64, 389]                         # the shortest allowed length and a typical one
        bias = torch.zeros(B, H, Tn, Tn, device="cuda", dtype=dtype)
        for b, L in enumerate(text_len):
            bias[b, :, :, 4096 + L:] = -1e4
        pairs = ((0, 0), (1, H - 1), (0, 11))
    pairs = pairs or ((0, 0), (B - 1, H - 1))
    q, k, v, do = (randn(g, B, Tn, H, d, dtype=dtype) for _ in range(4))
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = F_.flash_attn_func(qd, kd, vd, bias)
    dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), do.cuda(), retain_graph=True)
    _check_sampled_heads(cfg, q, k, v, do, bias, o, (dq, dk, dv), pairs)
    if cfg == "config5_attention":
        # masked keys get no gradient and contribute nothing
        for b, L in enumerate(text_len):
            assert torch.count_nonzero(dk[b, 4096 + L:]) == 0 and torch.count_nonzero(dv[b, 4096 + L:]) == 0
    # linearity of the backward in dO: scaling dO by a power of two scales every
    # gradient by it — exactly in bf16; in fp16 up to subnormal rounding of dS
    dq2, dk2, dv2 = torch.autograd.grad(o, (qd, kd, vd), 2 * do.cuda())
    for a, b2 in ((dq, dq2), (dk, dk2), (dv, dv2)):
        if dtype == torch.bfloat16:
            assert torch.equal((2 * a.float()).to(a.dtype), b2)
        else:
            torch.testing.assert_close(2 * a.float(), b2.float(), rtol=2e-3, atol=2e-4)


def test_bounded_wait_gives_up_and_reports():
    """A device-side wait that nothing ever satisfies ends after its time limit, the kernel
    returns normally, and the status word reports the time-out exactly once."""
    from rgd_triton_b200 import _lib
    lib = _lib.load()
    assert lib.rgd_device_status() == 0
    assert lib.rgd_selftest_bounded_wait(0, None) == _lib.RGD_E_INVALID          # limit outside 1 us .. 100 ms
    assert lib.rgd_selftest_bounded_wait(1_000_000, torch.cuda.current_stream().cuda_stream) == 0   # 1 ms
    torch.cuda.synchronize()
    assert lib.rgd_device_status() == _lib.RGD_E_TIMEOUT
    assert lib.rgd_device_status() == 0
    # the context is intact: an attention call right after works and leaves the status clear
    g = gen(12)
    q, k, v, do = (randn(g, 1, 256, 2, 64, dtype=torch.bfloat16) for _ in range(4))
    check(q, k, v, do, None, False, "after time-out")


# ----------------------------------------------------------------------------- bias gradient
BIAS_GRAD_SHAPES = {
    "vector": lambda B, H, tq, tk: (B, H, 1, tk),
    "vector-shared": lambda B, H, tq, tk: (1, 1, 1, tk),
    "vector-per-head": lambda B, H, tq, tk: (1, H, 1, tk),
    "matrix": lambda B, H, tq, tk: (B, H, tq, tk),
    "matrix-batch-shared": lambda B, H, tq, tk: (1, H, tq, tk),
    "matrix-shared": lambda B, H, tq, tk: (1, 1, tq, tk),
}


def _lowp_bias_grad(q, k, v, do, bias, causal):
    """Bias gradient of the low-precision eager attention (every op in q.dtype)."""
    scale = 1.0 / math.sqrt(q.shape[-1])
    b = bias.detach().clone().requires_grad_(True)
    s = torch.einsum("bthd,bshd->bhts", q * scale, k) + b
    if causal:
        tq, tk = s.shape[-2:]
        keep = torch.arange(tq)[:, None] >= torch.arange(tk)[None, :]
        s = s.masked_fill(~keep, float("-inf"))
    o = torch.einsum("bhts,bshd->bthd", torch.softmax(s, dim=-1), v)
    return torch.autograd.grad(o, b, do)[0]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("kind", sorted(BIAS_GRAD_SHAPES))
@pytest.mark.parametrize("d,tq,tk", [(64, 300, 328), (128, 257, 384), (128, 200, 333), (32, 130, 77), (64, 128, 128)])
def test_bias_gradient(d, tq, tk, kind, causal, dt):
    """The gradient of the additive bias (which the reference refuses,
    flash_attn_triton_cached.py:1107): d bias = P (dP - delta) summed over the broadcast
    dimensions, against the exact fp32 evaluation with the low-precision eager error as the
    yardstick.  Sizes cover the kernels that stage a matrix bias by TMA (key count a multiple
    of 8), the general kernels (odd key count, head_dim 32) and both vector-bias kernels."""
    dtype = DTYPES[dt]
    g = gen(7 * d + tq + len(kind) + int(causal))
    B, H = 2, 3
    q, do = randn(g, B, tq, H, d, dtype=dtype), randn(g, B, tq, H, d, dtype=dtype)
    k, v = randn(g, B, tk, H, d, dtype=dtype), randn(g, B, tk, H, d, dtype=dtype)
    bias = randn(g, *BIAS_GRAD_SHAPES[kind](B, H, tq, tk), dtype=dtype)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    bd = bias.cuda().requires_grad_(True)
    o = F_.flash_attn_func(qd, kd, vd, bd, causal)
    dq, dk, dv, db = torch.autograd.grad(o, (qd, kd, vd, bd), do.cuda())
    torch.cuda.synchronize()
    assert db.shape == bias.shape and db.dtype == bias.dtype
    exact = O.attn_bwd_dbias(q.float(), k.float(), v.float(), do.float(), bias.float(), causal)
    lowp = _lowp_bias_grad(q, k, v, do, bias, causal)
    # sums over up to B * H * tq terms: the floor scales with the magnitude of the result
    floor = GRAD_FLOOR * max(1.0, exact.abs().max().item())
    assert_attn(db.cpu(), exact, lowp, f"dbias {kind} d={d} causal={causal}", factor=2.0, floor=floor)
    # dq, dk, dv of the same call hold the usual bar (a call that also wants the bias gradient may
    # take other kernels than one that does not)
    fb = bias.float()
    exact3 = O.attn_bwd(q.float(), k.float(), v.float(), do.float(), fb, causal)
    lowp3 = O.attn_lowp(q, k, v, do, bias, causal)[1:]
    for got, e, l, name in zip((dq, dk, dv), exact3, lowp3, ("dq", "dk", "dv")):
        assert_attn(got.cpu(), e, l, f"{name} with dbias {kind} d={d}", factor=2.0, floor=GRAD_FLOOR)


def test_bias_gradient_fp32_bias_and_module():
    """fp32 bias (its gradient comes back in fp32) through the module API."""
    g = gen(77)
    q, k, v, do = (randn(g, 1, 256, 2, 64, dtype=torch.bfloat16) for _ in range(4))
    bias = randn(g, 1, 2, 256, 256, dtype=torch.float32)
    m = ops.FlashAttention()
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    bd = bias.cuda().requires_grad_(True)
    for _ in range(2):      # second call: launch cache hit
        o = m(qd, kd, vd, bd)
        db, = torch.autograd.grad(o, (bd,), do.cuda())
    assert db.dtype == torch.float32
    exact = O.attn_bwd_dbias(q.float(), k.float(), v.float(), do.float(), bias, False)
    lowp = _lowp_bias_grad(q, k, v, do, bias.to(torch.bfloat16), False)
    assert_attn(db.cpu(), exact, lowp.float(), "dbias fp32", factor=2.0, floor=GRAD_FLOOR)


# ----------------------------------------------------------------------------- masked bias tiles
def _tile_layout(slices, tq, tk):
    """Offsets (16-bit words) of the tile-list buffer, as include/rgd_b200.h's builder lays it out."""
    nqb, nq2, nkb = (tq + 127) // 128, (tq + 255) // 256, (tk + 127) // 128
    off, w = {}, 0
    for name, n in (("qcnt", nqb), ("qlist", nqb * nkb), ("q2cnt", nq2), ("q2list", nq2 * nkb), ("kcnt", nkb),
                    ("klist", nkb * nqb)):
        off[name] = w
        w += slices * n
    return off, nqb, nq2, nkb


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("form", ["full", "batch-shared", "head-shared"])
@pytest.mark.parametrize("mask", ["blocks", "key-padding", "dead-row"])
def test_masked_bias_tiles_are_skipped_with_identical_results(d, form, mask):
    """Block-sparse skip (the reference has only the dense form,
    flash_attn_triton_cached.py:151-175): a bias reused through a module's cache gets tile lists
    from its second forward on, the kernels visit only listed tiles, and o, dq, dk, dv are
    bit-identical to the dense evaluation.  The lists themselves are checked against the mask."""
    dt = torch.bfloat16 if d == 128 else torch.float16
    g = gen(31 * d + len(form) + len(mask))
    B, H, tq, tk = 2, 3, 1100, 1160
    q, do = randn(g, B, tq, H, d, dtype=dt), randn(g, B, tq, H, d, dtype=dt)
    k, v = randn(g, B, tk, H, d, dtype=dt), randn(g, B, tk, H, d, dtype=dt)
    Bb, Hb = (1 if form == "batch-shared" else B), (1 if form == "head-shared" else H)
    bias = torch.randn(Bb, Hb, tq, tk, generator=g)
    nqb, nkb = (tq + 127) // 128, (tk + 127) // 128
    if mask == "blocks":
        blk = torch.rand(Bb, Hb, nqb, nkb, generator=g) < 0.4
        blk[..., torch.arange(nqb), torch.arange(nqb)] = False          # every row keeps its diagonal tile
        big = blk.repeat_interleave(128, 2).repeat_interleave(128, 3)[:, :, :tq, :tk]
    elif mask == "key-padding":
        big = torch.zeros(Bb, Hb, tq, tk, dtype=torch.bool)
        big[..., tk - 300:] = True                                       # 300 padded keys: two whole tiles and a part
    else:
        big = torch.zeros(Bb, Hb, tq, tk, dtype=torch.bool)
        big[..., 128:] = True                                            # only the first key tile is alive ...
        big[0, 0, 700, :] = True                                         # ... and one row has no unmasked key at all
    bias = (bias - 1e4 * big).to(dt)

    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    bd, dod = bias.cuda(), do.cuda()

    def run(module):
        o = module(qd, kd, vd, bd)
        return [o.detach(), *torch.autograd.grad(o, (qd, kd, vd), dod)]

    prev = F_.set_skip_masked_tiles(False)
    prev_mode = F_.set_attention_backward("two_kernel")     # the list-following backward is the two-kernel form
    try:
        dense = run(ops.FlashAttention())
    finally:
        F_.set_skip_masked_tiles(prev)
        F_.set_attention_backward(prev_mode)
    # the dense evaluation itself against the oracle (so that "identical" cannot mean "equally wrong")
    fb = bias.float()
    eo, _ = O.attn_fwd(q.float(), k.float(), v.float(), fb)
    exact = [eo, *O.attn_bwd(q.float(), k.float(), v.float(), do.float(), fb)]
    lowp = O.attn_lowp(q, k, v, do, bias)
    for got_, e_, l_, name in zip(dense, exact, lowp, ("o", "dq", "dk", "dv")):
        assert_attn(got_.cpu(), e_, l_, f"dense {name} ({mask}, {form}, d={d})", factor=2.0,
                    floor=1e-4 if name == "o" else GRAD_FLOOR)
    m = ops.FlashAttention()
    with attention_backward("two_kernel"):
        for call in range(3):
            got = run(m)
            for a, b_, name in zip(got, dense, ("o", "dq", "dk", "dv")):
                assert torch.equal(a, b_), f"call {call}: {name} differs from the dense evaluation"
    torch.cuda.synchronize()
    ent = m.cache._tiles
    assert ent[0]() is bd and torch.is_tensor(ent[2]), "the bias was not scanned on its second use"

    # the lists against the mask: a tile is listed iff it has an element > -9984 (bf16's -1e4), except
    # that a query block holding a row without any element >= -4992 lists every tile
    words = ent[2].cpu().view(torch.int16).to(torch.int32) & 0xFFFF
    off, nqb, nq2, nkb = _tile_layout(Bb * Hb, tq, tk)
    bf = bias.float()
    for s_ in range(Bb * Hb):
        sl = bf[s_ // Hb, s_ % Hb]
        live = torch.zeros(nqb, nkb, dtype=torch.bool)
        for i in range(nqb):
            rows = sl[128 * i:128 * i + 128]
            for j in range(nkb):
                live[i, j] = bool((rows[:, 128 * j:128 * j + 128] > -9984.0).any())
            if bool((rows.max(dim=1).values < -4992.0).any()):
                live[i, :] = True
        for i in range(nqb):
            n = int(words[off["qcnt"] + s_ * nqb + i])
            lst = words[off["qlist"] + (s_ * nqb + i) * nkb:][:n].tolist()
            assert lst == torch.nonzero(live[i]).flatten().tolist(), f"slice {s_} query block {i}"
        for j in range(nkb):
            n = int(words[off["kcnt"] + s_ * nkb + j])
            lst = words[off["klist"] + (s_ * nkb + j) * nqb:][:n].tolist()
            assert lst == torch.nonzero(live[:, j]).flatten().tolist(), f"slice {s_} key block {j}"
        for i2 in range(nq2):
            n = int(words[off["q2cnt"] + s_ * nq2 + i2])
            lst = words[off["q2list"] + (s_ * nq2 + i2) * nkb:][:n].tolist()
            both = live[2 * i2] | live[min(2 * i2 + 1, nqb - 1)]
            assert lst == torch.nonzero(both).flatten().tolist(), f"slice {s_} 256-query block {i2}"
    if mask != "dead-row":
        assert int(words[off["qcnt"]:off["qcnt"] + Bb * Hb * nqb].sum()) < Bb * Hb * nqb * nkb, "nothing was skipped"


def test_masked_bias_tiles_follow_the_tensor():
    """A bias modified in place, or another tensor of the same shape, is not served stale lists."""
    g = gen(5)
    B, H, T_, d = 1, 2, 1024, 64
    q, k, v, do = (randn(g, B, T_, H, d, dtype=torch.float16) for _ in range(4))
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    bias = torch.zeros(B, H, T_, T_)
    bias[..., 512:] = -1e4
    bd = bias.half().cuda()
    m = ops.FlashAttention()
    for _ in range(3):
        m(qd, kd, vd, bd)
    assert torch.is_tensor(m.cache._tiles[2])
    bd[..., 512:] = 0.0                                   # unmask in place: the version counter moves
    o = m(qd, kd, vd, bd)
    eo, _ = O.attn_fwd(q.float(), k.float(), v.float(), bd.float().cpu())
    lo = O.attn_lowp(q, k, v, do, bd.cpu())[0]
    assert_attn(o.detach().cpu(), eo, lo, "after in-place unmasking")
    other = torch.zeros_like(bd)
    o2 = m(qd, kd, vd, other)
    eo2, _ = O.attn_fwd(q.float(), k.float(), v.float(), None)
    assert_attn(o2.detach().cpu(), eo2, O.attn_lowp(q, k, v, do, None)[0], "another bias tensor")
