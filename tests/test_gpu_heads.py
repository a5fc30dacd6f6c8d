"""GPU parity of the head operators (FusedHeadLayerNorm, RoPE, FusedLNRoPE)
against the CPU oracle and the reference's golden vectors, on the reference's
own test grid (tests/test_head_layernorm.py:71, tests/test_head_rope.py:228-239,
tests/test_fused_ln_rope.py) plus misaligned and benchmark-sized cases."""
import pytest
import torch

from oracle import oracle as O
from rgd_triton_b200 import functional as F_, ops
from tests._util import DTYPES, T, assert_parity, gen, randn, rotary_table

pytestmark = pytest.mark.gpu

D_R = [(32, 32), (64, 32), (64, 64), (128, 32), (128, 64), (128, 96), (128, 128), (40, 20), (36, 36)]
LENS = [(14, 14), (97, 97), (31, 11), (113, 203), (128, 217), (200, 200)]


def _shape(B, H, N, D, hs):
    return (B, H, N, D) if hs else (B, N, H, D)


def _run(fn, q, k, gq, gk):
    qd, kd = q.cuda().requires_grad_(True), k.cuda().requires_grad_(True)
    qo, ko = fn(qd, kd)
    dq, dk = torch.autograd.grad((qo, ko), (qd, kd), (gq.cuda(), gk.cuda()))
    torch.cuda.synchronize()
    return qo.detach().cpu(), ko.detach().cpu(), dq.cpu(), dk.cpu()


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("hs", [True, False])
@pytest.mark.parametrize("d", [32, 64, 96, 128, 256, 36, 50])
def test_head_layernorm(dt, hs, d):
    dtype = DTYPES[dt]
    g = gen(d)
    for nq, nk in LENS[:4]:
        q, k = randn(g, *_shape(3, 5, nq, d, hs), dtype=dtype), randn(g, *_shape(3, 5, nk, d, hs), dtype=dtype)
        gq, gk = randn(g, *q.shape, dtype=dtype), randn(g, *k.shape, dtype=dtype)
        qo, ko, dq, dk = _run(lambda a, b: F_.triton_fused_ln_func_fn(a, b, hs, 1e-5), q, k, gq, gk)
        assert_parity(qo, O.headln_fwd(q, 1e-5), "q")
        assert_parity(ko, O.headln_fwd(k, 1e-5), "k")
        assert_parity(dq, O.headln_bwd(q, gq, 1e-5), "dq", atol_rel=1e-5)
        assert_parity(dk, O.headln_bwd(k, gk, 1e-5), "dk", atol_rel=1e-5)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("hs", [True, False])
@pytest.mark.parametrize("d,R", D_R)
def test_rope(dt, hs, d, R):
    dtype = DTYPES[dt]
    g = gen(d * 7 + R)
    for (nq, nk), frac in zip(LENS, (0, 0.5, 0.75, 1.0, 0.5, 1.0)):
        pos = rotary_table(max(nq, nk) + 1, R, dtype)
        cq, ck = int(frac * nq), int(frac * nk)
        q, k = randn(g, *_shape(2, 3, nq, d, hs), dtype=dtype), randn(g, *_shape(2, 3, nk, d, hs), dtype=dtype)
        gq, gk = randn(g, *q.shape, dtype=dtype), randn(g, *k.shape, dtype=dtype)
        qo, ko, dq, dk = _run(lambda a, b: F_.triton_rope_fn(a, b, pos.cuda(), (cq, ck), hs), q, k, gq, gk)
        assert_parity(qo, O.rope(q, pos, cq, hs), "q")
        assert_parity(ko, O.rope(k, pos, ck, hs), "k")
        assert_parity(dq, O.rope(gq, pos, cq, hs, transposed=True), "dq")
        assert_parity(dk, O.rope(gk, pos, ck, hs, transposed=True), "dk")


@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_rope_fp32_table_promotes(dt):
    """A 16-bit tensor with an fp32 table computes in fp32 (promoted type)."""
    dtype = DTYPES[dt]
    g = gen(3)
    pos = rotary_table(70, 64, torch.float32)
    q, k = randn(g, 2, 64, 3, 128, dtype=dtype), randn(g, 2, 50, 3, 128, dtype=dtype)
    qo, ko, dq, dk = _run(lambda a, b: F_.triton_rope_fn(a, b, pos.cuda(), None, False), q, k, q, k)
    assert_parity(qo, O.rope(q, pos, None, False), "q")
    assert_parity(ko, O.rope(k, pos, None, False), "k")
    assert_parity(dq, O.rope(q, pos, None, False, transposed=True), "dq")


def test_rope_default_out_of_place_and_in_place_flag():
    g = gen(4)
    pos = rotary_table(40, 32, torch.float32).cuda()
    q, k = randn(g, 2, 3, 33, 64).cuda(), randn(g, 2, 3, 20, 64).cuda()
    q0, k0 = q.clone(), k.clone()
    m = ops.RoPE()
    qo, ko = m(q, k, pos, seq_cutoff=20)
    assert torch.equal(q, q0) and torch.equal(k, k0), "module path must not overwrite its inputs"
    qi, ki = F_.triton_rope_fn(q, k, pos, 20, True, in_place=True)
    assert qi.data_ptr() == q.data_ptr() and torch.equal(qi, qo) and torch.equal(ki, ko)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("hs", [True, False])
@pytest.mark.parametrize("d,R", D_R)
def test_fused_ln_rope(dt, hs, d, R):
    dtype = DTYPES[dt]
    g = gen(d * 13 + R)
    for (nq, nk), frac in zip(LENS, (1.0, 0.5, 0.75, 0, 0.5, 1.0)):
        pos = rotary_table(max(nq, nk) + 1, R, dtype)
        cq, ck = int(frac * nq), int(frac * nk)
        q, k = randn(g, *_shape(2, 3, nq, d, hs), dtype=dtype), randn(g, *_shape(2, 3, nk, d, hs), dtype=dtype)
        gq, gk = randn(g, *q.shape, dtype=dtype), randn(g, *k.shape, dtype=dtype)
        qo, ko, dq, dk = _run(lambda a, b: F_.triton_fused_ln_rope_fn(a, b, pos.cuda(), (cq, ck), hs, 1e-5),
                              q, k, gq, gk)
        assert_parity(qo, O.lnrope_fwd(q, pos, cq, hs, 1e-5), "q")
        assert_parity(ko, O.lnrope_fwd(k, pos, ck, hs, 1e-5), "k")
        assert_parity(dq, O.lnrope_bwd(q, gq, pos, cq, hs, 1e-5), "dq", atol_rel=1e-5)
        assert_parity(dk, O.lnrope_bwd(k, gk, pos, ck, hs, 1e-5), "dk", atol_rel=1e-5)


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("hs", [False, True])
def test_golden_vectors(golden, dt, hs):
    g = golden(f"heads_{dt}")
    s = "hs" if hs else "ns"
    pos, eps, cuts = T(g["pos"]), float(g["eps"]), (int(g["cut_q"]), int(g["cut_k"]))
    q, k, gq, gk = (T(g[f"{n}_{s}"]) for n in ("q", "k", "gq", "gk"))
    for name, fn, tol in (("l", lambda a, b: F_.triton_fused_ln_func_fn(a, b, hs, eps), 1e-5),
                          # the interpreter rounds after every operation, the GPU kernels (the reference's
                          # and ours) fuse rot*sin into the sum: up to 1 ulp of the larger product apart
                          ("r", lambda a, b: F_.triton_rope_fn(a, b, pos.cuda(), cuts, hs), 2e-6 if dt == "f32" else 1e-3),
                          ("f", lambda a, b: F_.triton_fused_ln_rope_fn(a, b, pos.cuda(), cuts, hs, eps), 1e-5)):
        qo, ko, dq, dk = _run(fn, q, k, gq, gk)
        assert_parity(qo, T(g[f"{name}q_{s}"]), f"golden {name}q", atol_rel=tol if name == "r" else 2e-6)
        assert_parity(ko, T(g[f"{name}k_{s}"]), f"golden {name}k", atol_rel=tol if name == "r" else 2e-6)
        assert_parity(dq, T(g[f"d{name}q_{s}"]), f"golden d{name}q", atol_rel=tol)
        assert_parity(dk, T(g[f"d{name}k_{s}"]), f"golden d{name}k", atol_rel=tol)


def test_misaligned_views_take_the_scalar_path():
    """Views whose rows are not 16-byte addressable (odd offsets / strides)."""
    g = gen(9)
    base_q, base_k = randn(g, 2, 19, 3, 67, dtype=torch.bfloat16), randn(g, 2, 11, 3, 67, dtype=torch.bfloat16)
    q, k = base_q[..., 3:67], base_k[..., 3:67]          # d = 64, row starts misaligned
    pos = rotary_table(32, 32, torch.bfloat16)
    qd, kd = base_q.cuda()[..., 3:67], base_k.cuda()[..., 3:67]
    qo, ko = F_.triton_fused_ln_rope_fn(qd, kd, pos.cuda(), (10, 5), False, 1e-5)
    assert_parity(qo.cpu(), O.lnrope_fwd(q, pos, 10, False, 1e-5), "q misaligned")
    assert_parity(ko.cpu(), O.lnrope_fwd(k, pos, 5, False, 1e-5), "k misaligned")
    ro, _ = F_.triton_rope_fn(qd, kd, pos.cuda(), (10, 5), False)
    assert_parity(ro.cpu(), O.rope(q, pos, 10, False), "rope misaligned")


def test_repeat_runs_are_bit_identical():
    g = gen(12)
    q, k = randn(g, 60, 97, 4, 64, dtype=torch.bfloat16).cuda(), randn(g, 60, 50, 4, 64, dtype=torch.bfloat16).cuda()
    pos = rotary_table(128, 32, torch.bfloat16).cuda()
    gq, gk = torch.randn_like(q), torch.randn_like(k)
    first = None
    for _ in range(20):
        qi, ki = q.clone().requires_grad_(True), k.clone().requires_grad_(True)
        qo, ko = F_.triton_fused_ln_rope_fn(qi, ki, pos, (60, 50), False, 1e-5)
        cur = [qo, ko, *torch.autograd.grad((qo, ko), (qi, ki), (gq, gk))]
        if first is None:
            first = [t.clone() for t in cur]
        else:
            assert all(torch.equal(a, b) for a, b in zip(first, cur))


def test_errors():
    q = torch.zeros(1, 4, 2, 64, device="cuda")
    pos = torch.zeros(2, 4, 32, device="cuda")     # P must exceed the sequence length
    with pytest.raises(AssertionError):
        F_.triton_rope_fn(q, q, pos, None, False)
    with pytest.raises(AssertionError):
        F_.triton_fused_ln_rope_fn(torch.zeros(1, 4, 2, 256, device="cuda"), torch.zeros(1, 4, 2, 256, device="cuda"),
                                   torch.zeros(2, 8, 32, device="cuda"), None, False)
    with pytest.raises(AssertionError):
        F_.triton_fused_ln_func_fn(q, torch.zeros(1, 4, 3, 64, device="cuda"), False)
    pg = torch.zeros(2, 8, 32, device="cuda", requires_grad=True)
    qq = q.clone().requires_grad_(True)
    qo, ko = F_.triton_rope_fn(qq, qq, pg, None, False)
    with pytest.raises(AssertionError):
        (qo.sum() + ko.sum()).backward()


def test_config2_slice_full_size():
    """Second benchmark configuration at full size (q, k [8,4096,16,128] bf16,
    R=64, cutoffs 4096): the operator is row-wise, so the oracle is evaluated
    on a sampled set of tokens of every batch."""
    g = gen(0)
    B, N, H, D = 8, 4096, 16, 128
    q, k = randn(g, B, N, H, D, dtype=torch.bfloat16), randn(g, B, N, H, D, dtype=torch.bfloat16)
    gq = randn(g, B, N, H, D, dtype=torch.bfloat16)
    pos = rotary_table(N + 1, 64, torch.bfloat16)
    qd, kd = q.cuda().requires_grad_(True), k.cuda().requires_grad_(True)
    qo, ko = ops.FusedLNRoPE()(qd, kd, pos.cuda(), seq_cutoff=(4096, 4096), heads_second=False, eps=1e-5)
    dq, dk = torch.autograd.grad((qo, ko), (qd, kd), (gq.cuda(), gq.cuda()))
    tok = torch.tensor([0, 1, 63, 64, 1000, 2047, 2048, 4095])
    # oracle on the sampled tokens: build a table whose rows are those tokens' rows
    sub_pos = pos[:, tok]
    for got, x, name in ((qo, q, "q"), (ko, k, "k")):
        want = torch.stack([O.lnrope_fwd(x[:, t:t + 1], sub_pos[:, i:i + 1].repeat(1, 2, 1), 1, False, 1e-5)
                            for i, t in enumerate(tok.tolist())], dim=1).squeeze(2)
        assert_parity(got.detach().cpu()[:, tok], want, f"config2 {name}")
    want = torch.stack([O.lnrope_bwd(q[:, t:t + 1], gq[:, t:t + 1], sub_pos[:, i:i + 1].repeat(1, 2, 1), 1, False, 1e-5)
                        for i, t in enumerate(tok.tolist())], dim=1).squeeze(2)
    assert_parity(dq.cpu()[:, tok], want, "config2 dq", atol_rel=1e-5)
    # size-independent property: the rotation preserves the norm of every channel pair
    y = qo.detach().float()
    ln = torch.nn.functional.layer_norm(qd.detach().float(), (D,), eps=1e-5)
    pn = lambda t: (t[..., :64].reshape(B, N, H, 32, 2) ** 2).sum(-1)
    torch.testing.assert_close(pn(y), pn(ln), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(y[..., 64:], ln[..., 64:].to(torch.bfloat16).float(), rtol=1.6e-2, atol=1e-2)
