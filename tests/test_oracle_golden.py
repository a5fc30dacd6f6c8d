"""Pin the CPU oracle against outputs of the reference itself.

tests/golden/*.npz were produced by running the reference's Triton kernels
under Triton's interpreter (tests/golden/make_golden.py).  Every oracle
function must reproduce them: fp32 to ~1e-6 relative (the two differ only in
summation order), fp16 to one unit in the last place.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O


def T(a):
    return torch.from_numpy(np.asarray(a))


def close(got, want, dtype, what, atol_scale=1.0):
    got, want = got.detach(), T(want)
    assert got.shape == want.shape, what
    if dtype == "f32":
        torch.testing.assert_close(got, want, rtol=2e-5, atol=2e-6 * atol_scale, msg=lambda m: f"{what}: {m}")
    else:
        ulp = O.ulp_distance(got, want)
        # one 16-bit ulp, plus absolute slack near zero where an ulp is tiny
        bad = (ulp > 1) & ((got.float() - want.float()).abs() > 1e-4 * atol_scale)
        assert not bad.any(), f"{what}: {int(bad.sum())} elements off by more than 1 ulp (max {int(ulp.max())})"


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_rmsnorm(golden, dt):
    g = golden(f"rms_{dt}")
    x, w, wb, dy, eps = T(g["x"]), T(g["w"]), T(g["wb"]), T(g["dy"]), float(g["eps"])
    close(O.rmsnorm_fwd(x, w, eps), g["y"], dt, "y")
    dx, dw = O.rmsnorm_bwd(x, w, dy, eps)
    close(dx, g["dx"], dt, "dx")
    close(dw, g["dw"], dt, "dw", atol_scale=30)
    close(O.rmsnorm_fwd(x, wb, eps), g["yb"], dt, "y per-batch weight")
    dxb, dwb = O.rmsnorm_bwd(x, wb, dy, eps)
    close(dxb, g["dxb"], dt, "dx per-batch weight")
    close(dwb, g["dwb"], dt, "dw per-batch weight", atol_scale=30)


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_rmsnorm2(golden, dt):
    g = golden(f"rms2_{dt}")
    eps = float(g["eps"])
    for x, w, gy, y, dx, dw in (("a", "w1", "g1", "ya", "da", "dw1"), ("b", "w2", "g2", "yb", "db", "dw2")):
        close(O.rmsnorm_fwd(T(g[x]), T(g[w]), eps), g[y], dt, y)
        odx, odw = O.rmsnorm_bwd(T(g[x]), T(g[w]), T(g[gy]), eps)
        close(odx, g[dx], dt, dx)
        close(odw, g[dw], dt, dw, atol_scale=30)


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_l2norm(golden, dt):
    g = golden(f"l2_{dt}")
    eps = float(g["eps"])
    close(O.l2norm_fwd(T(g["x"]), eps), g["y"], dt, "y")
    # the all-zero row has scale 1/eps = 1e6: compare dx relative to that scale
    dx = O.l2norm_bwd(T(g["x"]), T(g["dy"]), eps)
    want = T(g["dx"])
    if dt == "f32":
        torch.testing.assert_close(dx, want, rtol=1e-4, atol=1e-5)
    else:
        finite = torch.isfinite(want.float()) & torch.isfinite(dx.float())
        assert (torch.isfinite(want.float()) == torch.isfinite(dx.float())).all()
        torch.testing.assert_close(dx[finite].float(), want[finite].float(), rtol=2e-3, atol=1e-3)
    for x, gy, y, d in (("a", "g1", "ya", "da"), ("b", "g2", "yb", "db")):
        close(O.l2norm_fwd(T(g[x]), eps), g[y], dt, y)
        close(O.l2norm_bwd(T(g[x]), T(g[gy]), eps), g[d], dt, d)


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("hs", [False, True])
def test_head_ops(golden, dt, hs):
    g = golden(f"heads_{dt}")
    s = "hs" if hs else "ns"
    pos, eps = T(g["pos"]), float(g["eps"])
    cuts = {"q": int(g["cut_q"]), "k": int(g["cut_k"])}
    for t in ("q", "k"):
        x, gy = T(g[f"{t}_{s}"]), T(g[f"g{t}_{s}"])
        close(O.headln_fwd(x, eps), g[f"l{t}_{s}"], dt, f"headln {t}")
        close(O.headln_bwd(x, gy, eps), g[f"dl{t}_{s}"], dt, f"headln d{t}")
        # the golden vectors come from Triton's interpreter: one rounding per operation
        close(O.rope(x, pos, cuts[t], hs, mode="interpreted"), g[f"r{t}_{s}"], dt, f"rope {t}")
        close(O.rope(gy, pos, cuts[t], hs, transposed=True, mode="interpreted"), g[f"dr{t}_{s}"], dt, f"rope d{t}")
        close(O.lnrope_fwd(x, pos, cuts[t], hs, eps), g[f"f{t}_{s}"], dt, f"lnrope {t}")
        close(O.lnrope_bwd(x, gy, pos, cuts[t], hs, eps), g[f"df{t}_{s}"], dt, f"lnrope d{t}")


@pytest.mark.parametrize("kind", ["none", "matrix", "vector", "causal"])
def test_attention(golden, kind):
    """The reference kernel rounds P and dS to fp16 inside; the oracle is the
    exact fp32 evaluation, so the two agree to fp16 accumulation error."""
    g = golden("attn_f16")
    q, k, v, do = T(g["q"]), T(g["k"]), T(g["v"]), T(g["do"])
    bias = {"none": None, "causal": None, "matrix": T(g["bias_matrix"]), "vector": T(g["bias_vector"])}[kind]
    causal = kind == "causal"
    o, lse = O.attn_fwd(q, k, v, bias, causal)
    dq, dk, dv = O.attn_bwd(q, k, v, do, bias, causal)
    tq = q.shape[1]
    torch.testing.assert_close(lse, T(g[f"lse_{kind}"])[:, :, :tq], rtol=1e-3, atol=2e-3)
    for got, name in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        want = T(g[f"{name}_{kind}"])
        err = (got.float() - want.float()).abs().max().item()
        scale = want.float().abs().max().item()
        assert err <= 4e-3 * max(scale, 1.0), f"{name}_{kind}: max abs err {err} (scale {scale})"


def test_config1_rmsnorm(golden):
    """First benchmark configuration at full size: x [4,256,1024] fp32, seed 0."""
    g = golden("config1_rms_f32")
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(4, 256, 1024, generator=gen)
    w = 1 + 0.02 * torch.randn(1024, generator=gen)
    dy = torch.randn(4, 256, 1024, generator=gen)
    np.testing.assert_array_equal(x[0, 0, :8].numpy(), g["x_probe"])       # same inputs as the generator saw
    np.testing.assert_array_equal(dy[3, 255, -8:].numpy(), g["dy_probe"])
    step, eps = int(g["row_step"]), float(g["eps"])
    y = O.rmsnorm_fwd(x, w, eps)
    dx, dw = O.rmsnorm_bwd(x, w, dy, eps)
    torch.testing.assert_close(y[:, ::step], T(g["y_rows"]), rtol=1e-5, atol=2e-6)
    torch.testing.assert_close(dx[:, ::step], T(g["dx_rows"]), rtol=1e-5, atol=2e-6)
    # dweight sums 1024 rows of O(1) terms: compare relative to its own scale (~30)
    want = T(g["dw"])
    assert (dw - want).abs().max().item() <= 1e-5 * want.abs().max().item() + 1e-4


def test_ulp_distance():
    a = torch.tensor([1.0, -1.0, 0.0, 1.0], dtype=torch.bfloat16)
    b = torch.tensor([1.0078125, -1.0078125, -0.0, 1.0], dtype=torch.bfloat16)
    assert O.ulp_distance(a, b).tolist() == [1, 1, 0, 0]
