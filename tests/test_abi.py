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
