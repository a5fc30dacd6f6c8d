"""rgd_rmsnorm_bwd_static: the RMSNorm backward for callers that cannot
allocate device memory (a plugin inside an application that owns all device
memory, or a loop section that must avoid an allocation's synchronisation).
Its dweight partial rows live in a fixed device array inside the library, so
the call takes no workspace and allocates nothing.

Checked here, through the C ABI: two calls in a row give the same dx and
dweight as the existing rgd_rmsnorm_bwd with a caller-allocated workspace, and
a size beyond the array's capacity is refused with RGD_E_WORKSPACE.  The file
name sorts last so that a run that stops at the first failure has already run
every other test.
"""
import ctypes as C

import pytest
import torch

from rgd_triton_b200 import _lib

pytestmark = pytest.mark.gpu


def _args(xs, ws, dys, dxs, dws):
    n = len(xs)
    return dict(
        n=n,
        xa=(_lib.Rows * n)(*[_lib.rows(t) for t in xs]),
        wp=(C.c_void_p * n)(*[t.data_ptr() for t in ws]),
        wsb=(C.c_int64 * n)(*[0] * n),
        da=(_lib.Rows * n)(*[_lib.rows(t) for t in dys]),
        oa=(_lib.Rows * n)(*[_lib.rows(t) for t in dxs]),
        dwp=(C.c_void_p * n)(*[t.data_ptr() for t in dws]),
        per=(C.c_int * n)(*[0] * n),
        N=(C.c_int64 * n)(*[t.shape[1] for t in xs]),
        Cc=(C.c_int64 * n)(*[t.shape[2] for t in xs]),
        B=xs[0].shape[0],
    )


def _run_existing(lib, xs, ws, dys, eps):
    dxs = [torch.empty_like(t) for t in xs]
    dws = [torch.empty_like(t) for t in ws]
    a = _args(xs, ws, dys, dxs, dws)
    nbytes = lib.rgd_rmsnorm_bwd_workspace_bytes(a["n"], a["N"], a["Cc"], a["B"])
    work = torch.empty(int(nbytes), dtype=torch.uint8, device=xs[0].device)
    rc = lib.rgd_rmsnorm_bwd(a["n"], a["xa"], a["wp"], a["wsb"], a["da"], a["oa"], a["dwp"], a["per"], a["N"], a["Cc"],
                             a["B"], eps, _lib.dtype_code(xs[0].dtype), _lib.dtype_code(ws[0].dtype),
                             work.data_ptr(), work.numel(), _lib.stream_ptr())
    assert rc == 0, _lib.status_string(rc)
    return dxs, dws


def _run_static(lib, xs, ws, dys, eps):
    dxs = [torch.empty_like(t) for t in xs]
    dws = [torch.empty_like(t) for t in ws]
    a = _args(xs, ws, dys, dxs, dws)
    rc = lib.rgd_rmsnorm_bwd_static(a["n"], a["xa"], a["wp"], a["wsb"], a["da"], a["oa"], a["dwp"], a["per"], a["N"],
                                    a["Cc"], a["B"], eps, _lib.dtype_code(xs[0].dtype), _lib.dtype_code(ws[0].dtype),
                                    _lib.stream_ptr())
    return rc, dxs, dws


def test_static_scratch_backward_matches_workspace_backward_twice():
    lib = _lib.load()
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(21)
    eps = 1e-6
    cases = [
        # first call: two streams of different length and width, bf16 data, fp32 weights
        ([(3, 200, 768), (3, 77, 384)], torch.bfloat16, torch.float32),
        # second call, right after: one stream, fp32, odd width (scalar path), larger partial count
        ([(2, 1023, 257)], torch.float32, torch.float32),
    ]
    for shapes, dt, wdt in cases:
        xs = [torch.randn(*s, generator=g).to(dt).cuda() for s in shapes]
        dys = [torch.randn(*s, generator=g).to(dt).cuda() for s in shapes]
        ws = [(1 + 0.02 * torch.randn(s[2], generator=g)).to(wdt).cuda() for s in shapes]
        want_dx, want_dw = _run_existing(lib, xs, ws, dys, eps)
        rc, got_dx, got_dw = _run_static(lib, xs, ws, dys, eps)
        assert rc == 0, _lib.status_string(rc)
        torch.cuda.synchronize()
        for a, b in zip(got_dx + got_dw, want_dx + want_dw):
            # same kernels, same CTA partition, same reduction order: bit-equal
            # (tolerance of the other RMSNorm tests would be 1 ulp / 1e-5 relative)
            assert torch.equal(a, b)


def test_static_scratch_refuses_sizes_beyond_its_capacity():
    lib = _lib.load()
    torch.cuda.set_device(0)
    n = 1
    N = (C.c_int64 * n)(16)
    Cc = (C.c_int64 * n)(16384)          # partial rows of 16384 fp32 channels exceed 16 MiB
    need = lib.rgd_rmsnorm_bwd_workspace_bytes(n, N, Cc, 2)
    assert need > (16 << 20)
    x = torch.zeros(2, 16, 16384, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(16384, device="cuda")
    rc, _, _ = _run_static(lib, [x], [w], [x], 1e-6)
    assert rc == _lib.RGD_E_WORKSPACE
    assert "workspace" in _lib.status_string(rc)
