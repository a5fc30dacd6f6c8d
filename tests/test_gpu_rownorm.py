"""GPU parity of the row norms (L2Normalize, FusedL2Normalize2, FusedRMSNorm,
FusedRMSNorm2) against the CPU oracle and the reference's golden vectors.
Shapes follow the reference's own test grid (tests/test_rms.py:127-130,
tests/test_fused_rms.py:218-256): odd channel counts, unequal lengths and
widths, plus the benchmark configurations' sizes."""
import pytest
import torch

from oracle import oracle as O
from rgd_triton_b200 import functional as F_, ops
from tests._util import DTYPES, T, assert_parity, gen, randn

pytestmark = pytest.mark.gpu

DIMS = [32, 63, 97, 122, 257, 384, 510, 740, 1023, 1024, 2048, 3072, 4096]
SEQS = [14, 97, 200]


def _run(fn, inputs, grads):
    """Run fn on CUDA copies of `inputs` (all requiring grad), return outputs and input grads on CPU."""
    dev = [t.detach().cuda().requires_grad_(True) for t in inputs]
    outs = fn(*dev)
    outs = outs if isinstance(outs, tuple) else (outs,)
    gs = torch.autograd.grad(outs, dev, [g.cuda() for g in grads])
    torch.cuda.synchronize()
    return [o.detach().cpu() for o in outs], [g.cpu() for g in gs]


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("C", DIMS)
def test_rmsnorm_shared_weight(dt, C):
    dtype = DTYPES[dt]
    g = gen(C)
    for N in SEQS:
        x, dy = randn(g, 3, N, C, dtype=dtype), randn(g, 3, N, C, dtype=dtype)
        w = (1 + 0.02 * torch.randn(C, generator=g)).to(dtype)
        (y,), (dx, dw) = _run(lambda a, b: F_.triton_rms_func_fn(a, b, 1e-6), [x, w], [dy])
        assert_parity(y, O.rmsnorm_fwd(x, w, 1e-6), f"y N={N}")
        odx, odw = O.rmsnorm_bwd(x, w, dy, 1e-6)
        assert_parity(dx, odx, f"dx N={N}", atol_rel=1e-5)
        assert_parity(dw, odw, f"dw N={N}", atol_rel=1e-5)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("wdt", ["f32", "bf16"])
def test_rmsnorm_per_batch_and_mixed_weight_dtype(dt, wdt):
    dtype, wdtype = DTYPES[dt], DTYPES[wdt]
    g = gen(7)
    x, dy = randn(g, 4, 50, 264, dtype=dtype), randn(g, 4, 50, 264, dtype=dtype)
    for wshape in ((264,), (1, 1, 264), (4, 1, 264)):
        w = (1 + 0.02 * torch.randn(*wshape, generator=g)).to(wdtype)
        (y,), (dx, dw) = _run(lambda a, b: F_.triton_rms_func_fn(a, b, 1e-6), [x, w], [dy])
        assert dw.shape == w.shape and dw.dtype == w.dtype
        assert_parity(y, O.rmsnorm_fwd(x, w, 1e-6), f"y {wshape}")
        odx, odw = O.rmsnorm_bwd(x, w, dy, 1e-6)
        assert_parity(dx, odx, f"dx {wshape}", atol_rel=1e-5)
        assert_parity(dw, odw, f"dw {wshape}", atol_rel=1e-5)


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("per_batch", [False, True])
def test_weight_views_that_are_not_16_byte_addressable(dt, per_batch):
    """Rows of 3072 (16-bit) / 1024 (fp32) channels normally run on the kernel that reads the
    weight with 16-byte loads.  A weight that starts one element into a larger buffer, or
    per-batch weights whose batch stride is odd, must take the other kernel and still match."""
    dtype = DTYPES[dt]
    C = 3072 if dt == "bf16" else 1024
    g = gen(C + int(per_batch))
    B, N = 2, 70
    x, dy = randn(g, B, N, C, dtype=dtype), randn(g, B, N, C, dtype=dtype)
    if per_batch:
        wbuf = (1 + 0.02 * torch.randn(B, 1, C + 3, generator=g)).to(dtype)        # batch stride C + 3
        w = wbuf[:, :, 1:C + 1]
    else:
        wbuf = (1 + 0.02 * torch.randn(C + 8, generator=g)).to(dtype)
        w = wbuf[1:C + 1]
    xd = x.cuda().requires_grad_(True)
    wd = (wbuf.cuda()[:, :, 1:C + 1] if per_batch else wbuf.cuda()[1:C + 1]).requires_grad_(True)
    assert wd.data_ptr() % 16 != 0
    y = F_.triton_rms_func_fn(xd, wd, 1e-6)
    dx, dw = torch.autograd.grad(y, (xd, wd), dy.cuda())
    assert_parity(y.detach().cpu(), O.rmsnorm_fwd(x, w, 1e-6), "y")
    odx, odw = O.rmsnorm_bwd(x, w, dy, 1e-6)
    assert_parity(dx.cpu(), odx, "dx", atol_rel=1e-5)
    assert_parity(dw.cpu(), odw.reshape(dw.shape), "dw", atol_rel=2e-5)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("n1,n2,c1,c2", [(97, 97, 128, 128), (1023, 1024, 257, 514), (108, 256, 740, 370),
                                          (512, 4096, 3072, 3072), (14, 31, 63, 32)])
def test_rmsnorm2(dt, n1, n2, c1, c2):
    dtype = DTYPES[dt]
    g = gen(n1 + c2)
    B = 2
    a, b = randn(g, B, n1, c1, dtype=dtype), randn(g, B, n2, c2, dtype=dtype)
    w1 = (1 + 0.02 * torch.randn(c1, generator=g)).to(dtype)
    w2 = (1 + 0.02 * torch.randn(c2, generator=g)).to(dtype)
    g1, g2 = randn(g, B, n1, c1, dtype=dtype), randn(g, B, n2, c2, dtype=dtype)
    (ya, yb), (da, db, dw1, dw2) = _run(lambda *t: F_.triton_fused_rms_func_fn(*t, 1e-6), [a, b, w1, w2], [g1, g2])
    assert_parity(ya, O.rmsnorm_fwd(a, w1, 1e-6), "y1")
    assert_parity(yb, O.rmsnorm_fwd(b, w2, 1e-6), "y2")
    oda, odw1 = O.rmsnorm_bwd(a, w1, g1, 1e-6)
    odb, odw2 = O.rmsnorm_bwd(b, w2, g2, 1e-6)
    assert_parity(da, oda, "dx1", atol_rel=1e-5)
    assert_parity(db, odb, "dx2", atol_rel=1e-5)
    assert_parity(dw1, odw1, "dw1", atol_rel=2e-5)
    assert_parity(dw2, odw2, "dw2", atol_rel=2e-5)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("C", DIMS)
def test_l2norm(dt, C):
    dtype = DTYPES[dt]
    g = gen(1000 + C)
    for N in SEQS:
        x, dy = randn(g, 3, N, C, dtype=dtype), randn(g, 3, N, C, dtype=dtype)
        (y,), (dx,) = _run(lambda a: F_.triton_norm_func_fn(a, 1e-6), [x], [dy])
        assert_parity(y, O.l2norm_fwd(x, 1e-6), f"y N={N}")
        assert_parity(dx, O.l2norm_bwd(x, dy, 1e-6), f"dx N={N}", atol_rel=1e-5)


def test_l2norm_eps_gate():
    """Rows shorter than eps are scaled by 1/eps, not by 1/length (l2normalize_cached.py:76-77)."""
    x = torch.zeros(1, 4, 64)
    x[0, 1] = 1e-9
    x[0, 2] = 1.0
    x[0, 3, 0] = 3e-7
    (y,), _ = _run(lambda a: F_.triton_norm_func_fn(a, 1e-6), [x], [torch.ones_like(x)])
    assert_parity(y, O.l2norm_fwd(x, 1e-6), "gated rows")
    assert torch.all(y[0, 0] == 0) and abs(y[0, 1, 0].item() - 1e-3) < 1e-9


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("n1,n2,c1,c2", [(97, 97, 128, 128), (23, 138, 97, 194), (512, 4096, 3072, 3072)])
def test_l2norm2(dt, n1, n2, c1, c2):
    dtype = DTYPES[dt]
    g = gen(n2 + c1)
    a, b = randn(g, 2, n1, c1, dtype=dtype), randn(g, 2, n2, c2, dtype=dtype)
    g1, g2 = randn(g, 2, n1, c1, dtype=dtype), randn(g, 2, n2, c2, dtype=dtype)
    (ya, yb), (da, db) = _run(lambda *t: F_.triton_fused_norm_func_fn(*t, 1e-6), [a, b], [g1, g2])
    assert_parity(ya, O.l2norm_fwd(a, 1e-6), "y1")
    assert_parity(yb, O.l2norm_fwd(b, 1e-6), "y2")
    assert_parity(da, O.l2norm_bwd(a, g1, 1e-6), "dx1", atol_rel=1e-5)
    assert_parity(db, O.l2norm_bwd(b, g2, 1e-6), "dx2", atol_rel=1e-5)


@pytest.mark.parametrize("dt,C", [("bf16", 2048), ("f16", 3072), ("bf16", 4096), ("f32", 1024), ("f32", 1536)])
def test_exact_row_lengths_strided_views_and_weight_kinds(dt, C):
    """Rows of exactly 128 * {2, 3, 4} 16-byte vectors take the lean kernel: strided row and
    batch views (a slice of a wider, longer tensor), rows that do not fill the last CTA
    iteration, per-batch and fp32 weights, and L2 with a zero row."""
    dtype = DTYPES[dt]
    g = gen(C + 3)
    host = randn(g, 3, 2 * 37, 2 * C, dtype=dtype)
    view = lambda t: t[:, 1::2, C // 2:C // 2 + C]      # row stride 4C, batch stride 148C, 16-byte aligned offset
    x = view(host)
    dy = randn(g, *x.shape, dtype=dtype)
    for wshape, wdt in (((C,), dtype), ((3, 1, C), torch.float32)):
        w = (1 + 0.02 * torch.randn(*wshape, generator=g)).to(wdt)
        xin = view(host.cuda()).detach().requires_grad_(True)
        assert xin.stride() == x.stride()
        wd = w.cuda().requires_grad_(True)
        y = F_.triton_rms_func_fn(xin, wd, 1e-6)
        dx, dw = torch.autograd.grad(y, (xin, wd), dy.cuda())
        assert_parity(y.cpu(), O.rmsnorm_fwd(x, w, 1e-6), f"y {wshape}")
        odx, odw = O.rmsnorm_bwd(x, w, dy, 1e-6)
        assert_parity(dx.cpu(), odx, f"dx {wshape}", atol_rel=1e-5)
        assert_parity(dw.cpu(), odw, f"dw {wshape}", atol_rel=1e-5)
    xz = x.clone()
    xz[1, 5] = 0                                        # forward only: its gradient is dy / eps, beyond fp16
    (y,), _ = _run(lambda a: F_.triton_norm_func_fn(a, 1e-6), [xz], [dy])
    assert_parity(y, O.l2norm_fwd(xz, 1e-6), "l2 y")
    (_,), (dxl,) = _run(lambda a: F_.triton_norm_func_fn(a, 1e-6), [x.contiguous()], [dy])
    assert_parity(dxl, O.l2norm_bwd(x, dy, 1e-6), "l2 dx", atol_rel=1e-5)


def test_strided_and_noncontiguous_inputs():
    """Row / batch strides are honoured as passed; a non-unit channel stride
    falls back to .contiguous() like the reference (rmsnorm_cached.py:578)."""
    g = gen(5)
    base = randn(g, 2, 40, 2 * 96)
    base_t = randn(g, 2, 96, 20)
    w = 1 + 0.02 * torch.randn(96, generator=g)
    views = (lambda t: t[:, ::2, :96],        # strided rows, channel stride 1
             lambda t: t.transpose(1, 2))     # channel stride != 1
    for view, host in zip(views, (base, base_t)):
        inp = view(host)
        dy = randn(g, *inp.shape)
        dev = view(host.cuda())
        assert dev.stride() == inp.stride()
        xin = dev.detach().requires_grad_(True)
        y = F_.triton_rms_func_fn(xin, w.cuda(), 1e-6)
        (dx,) = torch.autograd.grad(y, xin, dy.cuda())
        assert_parity(y.cpu(), O.rmsnorm_fwd(inp, w, 1e-6), "y strided")
        assert_parity(dx.cpu(), O.rmsnorm_bwd(inp, w, dy, 1e-6)[0], "dx strided", atol_rel=1e-5)
        y2 = F_.triton_norm_func_fn(dev)
        assert_parity(y2.cpu(), O.l2norm_fwd(inp), "l2 strided")


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_golden_vectors(golden, dt):
    """The CUDA kernels against outputs of the reference's own kernels."""
    dtype = DTYPES[dt]
    g = golden(f"rms_{dt}")
    x, w, wb, dy = T(g["x"]), T(g["w"]), T(g["wb"]), T(g["dy"])
    (y,), (dx, dw) = _run(lambda a, b: F_.triton_rms_func_fn(a, b, 1e-6), [x, w], [dy])
    assert_parity(y, T(g["y"]), "golden y")
    assert_parity(dx, T(g["dx"]), "golden dx", atol_rel=1e-5)
    assert_parity(dw, T(g["dw"]), "golden dw", atol_rel=3e-3 if dt == "f16" else 1e-5)
    (yb,), (dxb, dwb) = _run(lambda a, b: F_.triton_rms_func_fn(a, b, 1e-6), [x, wb], [dy])
    assert_parity(yb, T(g["yb"]), "golden y per-batch")
    assert_parity(dwb, T(g["dwb"]), "golden dw per-batch", atol_rel=1e-5)
    g2 = golden(f"rms2_{dt}")
    (ya, yb2), (da, db, dw1, dw2) = _run(lambda *t: F_.triton_fused_rms_func_fn(*t, 1e-6),
                                         [T(g2["a"]), T(g2["b"]), T(g2["w1"]), T(g2["w2"])], [T(g2["g1"]), T(g2["g2"])])
    assert_parity(ya, T(g2["ya"]), "golden rms2 y1")
    assert_parity(yb2, T(g2["yb"]), "golden rms2 y2")
    assert_parity(da, T(g2["da"]), "golden rms2 dx1", atol_rel=1e-5)
    assert_parity(db, T(g2["db"]), "golden rms2 dx2", atol_rel=1e-5)
    gl = golden(f"l2_{dt}")
    (ya, yb3), (da, db) = _run(lambda *t: F_.triton_fused_norm_func_fn(*t, 1e-6), [T(gl["a"]), T(gl["b"])],
                               [T(gl["g1"]), T(gl["g2"])])
    assert_parity(ya, T(gl["ya"]), "golden l2 y1")
    assert_parity(yb3, T(gl["yb"]), "golden l2 y2")
    assert_parity(da, T(gl["da"]), "golden l2 dx1", atol_rel=1e-5)
    assert_parity(db, T(gl["db"]), "golden l2 dx2", atol_rel=1e-5)
    assert dtype == y.dtype


def test_config1_full_size_against_reference_output(golden):
    """First benchmark configuration: x [4,256,1024] fp32, seed 0; y, dx, dweight
    against the reference kernel's own output."""
    g = golden("config1_rms_f32")
    gn = torch.Generator().manual_seed(0)
    x = torch.randn(4, 256, 1024, generator=gn)
    w = 1 + 0.02 * torch.randn(1024, generator=gn)
    dy = torch.randn(4, 256, 1024, generator=gn)
    m = ops.FusedRMSNorm(1024, eps=1e-6).cuda()
    with torch.no_grad():
        m.weight.copy_(w)
    xin = x.cuda().requires_grad_(True)
    y = m(xin)
    y.backward(dy.cuda())
    step = int(g["row_step"])
    torch.testing.assert_close(y.detach().cpu()[:, ::step], T(g["y_rows"]), rtol=1e-5, atol=2e-6)
    torch.testing.assert_close(xin.grad.cpu()[:, ::step], T(g["dx_rows"]), rtol=1e-5, atol=2e-6)
    want = T(g["dw"])
    assert (m.weight.grad.cpu() - want).abs().max().item() <= 1e-5 * want.abs().max().item() + 1e-4
    assert m.cache.fwd is not None and m.cache.bwd is not None


def test_repeat_runs_are_bit_identical():
    """The reference's race-condition tests (tests/test_fused_rms.py: batch 60,
    repeated launches, torch.equal): here including dweight, which is reduced
    in a fixed order."""
    g = gen(11)
    a, b = randn(g, 60, 97, 384, dtype=torch.bfloat16).cuda(), randn(g, 60, 31, 740, dtype=torch.bfloat16).cuda()
    w1, w2 = torch.ones(384, device="cuda", requires_grad=True), torch.ones(740, device="cuda", requires_grad=True)
    g1, g2 = torch.randn_like(a), torch.randn_like(b)
    first = None
    for _ in range(20):
        ai, bi = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
        ya, yb = F_.triton_fused_rms_func_fn(ai, bi, w1, w2, 1e-6)
        grads = torch.autograd.grad((ya, yb), (ai, bi, w1, w2), (g1, g2))
        cur = [ya, yb, *grads]
        if first is None:
            first = [t.clone() for t in cur]
        else:
            for x, y in zip(first, cur):
                assert torch.equal(x, y)


def test_empty_and_single_row():
    x = torch.zeros(2, 0, 64, device="cuda", requires_grad=True)
    y = F_.triton_norm_func_fn(x)
    assert y.shape == (2, 0, 64)
    w = torch.ones(64, device="cuda", requires_grad=True)
    y = F_.triton_rms_func_fn(x, w)
    (dw,) = torch.autograd.grad(y.sum() + 0 * w.sum(), w, allow_unused=True)
    x1 = torch.randn(1, 1, 64)
    assert_parity(F_.triton_rms_func_fn(x1.cuda(), w.detach()).cpu(), O.rmsnorm_fwd(x1, torch.ones(64)), "1 row")


def test_module_reuse_across_shapes_and_dtypes():
    """One module, changing shapes and dtypes: the launch cache re-validates
    instead of replaying a stale configuration."""
    m = ops.L2Normalize()
    for shape, dt in (((2, 10, 64), torch.float32), ((3, 7, 97), torch.bfloat16), ((2, 10, 64), torch.float16)):
        x = torch.randn(*shape).to(dt)
        assert_parity(m(x.cuda()).cpu(), O.l2norm_fwd(x), f"{shape} {dt}")
