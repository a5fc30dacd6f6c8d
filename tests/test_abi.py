"""The C-ABI library builds, loads, and exports exactly what include/rgd_b200.h
declares.  No compute calls: these run without a GPU."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "rgd_b200.h"


@pytest.fixture(scope="module")
def lib():
    from rgd_triton_b200 import build
    path = build.build()
    return ctypes.CDLL(str(path))


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(rgd_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operator_set():
    names = declared_functions()
    for op in ("l2norm_fwd", "l2norm_bwd", "rmsnorm_fwd", "rmsnorm_bwd", "headln_fwd", "headln_bwd", "rope",
               "lnrope_fwd", "lnrope_bwd", "attn_fwd", "attn_bwd"):
        assert f"rgd_{op}" in names


def test_library_exports_every_declared_symbol(lib):
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_python_binding_covers_the_header():
    from rgd_triton_b200 import _lib
    declared = set(declared_functions())
    bound = set(_lib.SIGNATURES)
    assert declared == bound, f"header-only: {declared - bound}; binding-only: {bound - declared}"
    _lib.load()


def test_status_strings_and_version(lib):
    lib.rgd_status_string.restype = ctypes.c_char_p
    assert lib.rgd_status_string(0) == b"ok"
    assert b"bias" in lib.rgd_status_string(-8)
    assert b"unknown" in lib.rgd_status_string(-999)
    assert lib.rgd_abi_version() >= 3
    lib.rgd_attn_lse_rows.restype = ctypes.c_int64
    lib.rgd_attn_lse_rows.argtypes = [ctypes.c_int64]
    assert [lib.rgd_attn_lse_rows(n) for n in (0, 1, 64, 65, 4096)] == [0, 64, 64, 128, 4096]


def test_argument_errors_need_no_gpu(lib):
    """Validation runs before any CUDA call, so bad arguments are reported even
    on a machine without a device."""
    from rgd_triton_b200 import _lib
    L = _lib.load()
    n = (ctypes.c_int64 * 1)(4)
    c = (ctypes.c_int64 * 1)(8)
    rows = (_lib.Rows * 1)(_lib.Rows(None, 0, 0))
    assert L.rgd_l2norm_fwd(3, rows, rows, n, c, 1, 1e-6, 0, None) == _lib.RGD_E_INVALID
    assert L.rgd_l2norm_fwd(1, rows, rows, n, c, 1, 1e-6, 7, None) == _lib.RGD_E_DTYPE
    assert L.rgd_l2norm_fwd(1, rows, rows, n, c, 1, 1e-6, 0, None) == _lib.RGD_E_NULL
    h = _lib.Heads(None, 0, 0, 0)
    hp = ctypes.byref(h)
    assert L.rgd_headln_fwd(hp, hp, hp, hp, 1, 1, 4, 4, 512, 1e-6, 0, None) == _lib.RGD_E_SIZE
    b = _lib.Bias(None, 0, 0, 0, 5, 0, None)
    assert L.rgd_attn_fwd(hp, hp, hp, ctypes.byref(b), hp, None, 1, 1, 4, 4, 64, 1.0, 0, 2, None, None) \
        == _lib.RGD_E_BIAS_SHAPE
    assert L.rgd_attn_fwd(hp, hp, hp, None, hp, None, 1, 1, 4, 4, 256, 1.0, 0, 2, None, None) == _lib.RGD_E_SIZE
    assert L.rgd_attn_fwd(hp, hp, hp, None, hp, None, 1, 1, 4, 4, 64, 1.0, 0, 0, None, None) == _lib.RGD_E_DTYPE
    with pytest.raises(AssertionError):
        _lib.check(_lib.RGD_E_SIZE, "x")
    with pytest.raises(RuntimeError):
        _lib.check(_lib.RGD_E_BIAS_SHAPE, "x")


def test_bias_gradient_and_tile_list_arguments_need_no_gpu(lib):
    """rgd_attn_bwd_dbias and the tile-list entry points validate before any CUDA call."""
    from rgd_triton_b200 import _lib
    L = _lib.load()
    h = _lib.Heads(None, 0, 0, 0)
    hp = ctypes.byref(h)
    mat = _lib.Bias(None, 0, 0, 8, _lib.RGD_BIAS_MATRIX, _lib.RGD_F16, None)
    vec = _lib.Bias(None, 0, 0, 0, _lib.RGD_BIAS_VECTOR, _lib.RGD_F16, None)
    # the gradient's kind must be the bias's kind
    rc = L.rgd_attn_bwd_dbias(hp, hp, hp, ctypes.byref(mat), hp, None, hp, hp, hp, hp, ctypes.byref(vec),
                              0, 1, 8, 8, 64, 1.0, 0, _lib.RGD_F16, None, 0, None, None)
    assert rc == _lib.RGD_E_BIAS_SHAPE
    # a vector-bias gradient is dense fp32 [B, H, Tk]
    rc = L.rgd_attn_bwd_dbias(hp, hp, hp, ctypes.byref(vec), hp, None, hp, hp, hp, hp, ctypes.byref(vec),
                              0, 1, 8, 8, 64, 1.0, 0, _lib.RGD_F16, None, 0, None, None)
    assert rc == _lib.RGD_E_DTYPE
    # tile lists: size formula, and refusals
    def layout_bytes(B, H, tq, tk):
        nqb, nq2, nkb = (tq + 127) // 128, (tq + 255) // 256, (tk + 127) // 128
        words = B * H * (nqb + nqb * nkb + nq2 + nq2 * nkb + nkb + nkb * nqb)
        words = (words + 7) // 8 * 8
        return words * 2 + (B * H * nqb * nkb + 15) // 16 * 16
    for dims in ((2, 3, 1100, 1160), (1, 1, 1, 1), (4, 16, 4096, 4096), (2, 24, 4608, 4608)):
        assert L.rgd_attn_bias_tiles_bytes(*dims) == layout_bytes(*dims)
    assert L.rgd_attn_bias_tiles_bytes(0, 3, 5, 5) == 0
    buf = ctypes.create_string_buffer(64)
    assert L.rgd_attn_bias_tiles_build(ctypes.byref(vec), 1, 1, 8, 8, -9984.0, buf, 64, None) == _lib.RGD_E_BIAS_SHAPE
    assert L.rgd_attn_bias_tiles_build(ctypes.byref(mat), 1, 1, 8, 8, 1.0, buf, 64, None) == _lib.RGD_E_INVALID
    f32 = _lib.Bias(None, 0, 0, 8, _lib.RGD_BIAS_MATRIX, _lib.RGD_F32, None)
    assert L.rgd_attn_bias_tiles_build(ctypes.byref(f32), 1, 1, 8, 8, -9984.0, buf, 64, None) == _lib.RGD_E_DTYPE
    big = _lib.Bias(None, 0, 0, 4096, _lib.RGD_BIAS_MATRIX, _lib.RGD_F16, None)
    assert L.rgd_attn_bias_tiles_build(ctypes.byref(big), 1, 1, 4096, 4096, -9984.0, buf, 64, None) == _lib.RGD_E_WORKSPACE
    assert L.rgd_attn_bias_tiles_build(ctypes.byref(mat), 1, 1, 4096, 4096, -9984.0, buf, 64, None) == _lib.RGD_E_STRIDE
