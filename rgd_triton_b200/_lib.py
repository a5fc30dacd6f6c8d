"""ctypes binding of librgd_b200.so (the C ABI declared in include/rgd_b200.h).

The library is the only compute path of this package: there is no CPU or
PyTorch fallback.  If the shared object is missing, or the current device is
not a compute-capability-10 GPU, the operators raise instead of silently
computing something else.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "librgd_b200.so"

RGD_F32, RGD_F16, RGD_BF16 = 0, 1, 2
RGD_BIAS_NONE, RGD_BIAS_VECTOR, RGD_BIAS_MATRIX = 0, 1, 2

RGD_E_INVALID, RGD_E_DTYPE, RGD_E_SIZE, RGD_E_STRIDE = -1, -2, -3, -4
RGD_E_NULL, RGD_E_WORKSPACE, RGD_E_DEVICE, RGD_E_BIAS_SHAPE = -5, -6, -7, -8
RGD_E_TIMEOUT = 2001

DTYPE_CODE = {torch.float32: RGD_F32, torch.float16: RGD_F16, torch.bfloat16: RGD_BF16}


class Rows(C.Structure):
    """rgd_rows: [B, N, C] view, channel stride 1."""
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_n", C.c_int64)]


class Heads(C.Structure):
    """rgd_heads: (batch, head, token, channel) view of a 4-D tensor."""
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_n", C.c_int64)]


class Bias(C.Structure):
    """rgd_bias: additive attention bias, logically (B, H, Tq, Tk)."""
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_q", C.c_int64),
                ("kind", C.c_int), ("dtype", C.c_int), ("tiles", C.c_void_p)]


_i64, _i32, _f32, _vp = C.c_int64, C.c_int, C.c_float, C.c_void_p
_pRows, _pHeads, _pBias = C.POINTER(Rows), C.POINTER(Heads), C.POINTER(Bias)
_pi64, _pi32, _pvp = C.POINTER(C.c_int64), C.POINTER(C.c_int), C.POINTER(C.c_void_p)

# name -> (restype, argtypes); must list every function of include/rgd_b200.h.
SIGNATURES = {
    "rgd_device_supported": (_i32, [_i32]),
    "rgd_status_string": (C.c_char_p, [_i32]),
    "rgd_abi_version": (_i32, []),
    "rgd_launch_count": (_i64, []),
    "rgd_device_status": (_i32, []),
    "rgd_selftest_bounded_wait": (_i32, [_i64, _vp]),
    "rgd_cache_create": (_vp, []),
    "rgd_cache_destroy": (None, [_vp]),
    "rgd_cache_stats": (_i32, [_vp, _pi64, _pi64, _pi64]),
    "rgd_l2norm_fwd": (_i32, [_i32, _pRows, _pRows, _pi64, _pi64, _i64, _f32, _i32, _vp]),
    "rgd_l2norm_bwd": (_i32, [_i32, _pRows, _pRows, _pRows, _pi64, _pi64, _i64, _f32, _i32, _vp]),
    "rgd_rmsnorm_fwd": (_i32, [_i32, _pRows, _pvp, _pi64, _pRows, _pi64, _pi64, _i64, _f32, _i32, _i32, _vp]),
    "rgd_rmsnorm_bwd_workspace_bytes": (_i64, [_i32, _pi64, _pi64, _i64]),
    "rgd_rmsnorm_bwd": (_i32, [_i32, _pRows, _pvp, _pi64, _pRows, _pRows, _pvp, _pi32, _pi64, _pi64, _i64, _f32,
                               _i32, _i32, _vp, _i64, _vp]),
    "rgd_rmsnorm_bwd_static": (_i32, [_i32, _pRows, _pvp, _pi64, _pRows, _pRows, _pvp, _pi32, _pi64, _pi64, _i64, _f32,
                                      _i32, _i32, _vp]),
    "rgd_headln_fwd": (_i32, [_pHeads, _pHeads, _pHeads, _pHeads, _i64, _i64, _i64, _i64, _i64, _f32, _i32, _vp]),
    "rgd_headln_bwd": (_i32, [_pHeads] * 6 + [_i64, _i64, _i64, _i64, _i64, _f32, _i32, _vp]),
    "rgd_rope": (_i32, [_pHeads, _pHeads, _vp, _i64, _i64, _pHeads, _pHeads] + [_i64] * 9 + [_i32, _i32, _i32, _vp]),
    "rgd_lnrope_fwd": (_i32, [_pHeads, _pHeads, _vp, _i64, _i64, _pHeads, _pHeads] + [_i64] * 9
                       + [_f32, _i32, _i32, _vp]),
    "rgd_lnrope_bwd": (_i32, [_pHeads, _pHeads, _pHeads, _pHeads, _vp, _i64, _i64, _pHeads, _pHeads] + [_i64] * 9
                       + [_f32, _i32, _i32, _vp]),
    "rgd_attn_lse_rows": (_i64, [_i64]),
    "rgd_attn_fwd": (_i32, [_pHeads, _pHeads, _pHeads, _pBias, _pHeads, _vp] + [_i64] * 5
                     + [_f32, _i32, _i32, _vp, _vp]),
    "rgd_attn_bwd_workspace_bytes": (_i64, [_i64] * 5 + [_i32]),
    "rgd_attn_bwd_single_pass_workspace_bytes": (_i64, [_i64] * 5 + [_i32]),
    "rgd_attn_bwd": (_i32, [_pHeads, _pHeads, _pHeads, _pBias, _pHeads, _vp, _pHeads, _pHeads, _pHeads, _pHeads]
                     + [_i64] * 5 + [_f32, _i32, _i32, _vp, _i64, _vp, _vp]),
    "rgd_attn_bwd_dbias": (_i32, [_pHeads, _pHeads, _pHeads, _pBias, _pHeads, _vp, _pHeads, _pHeads, _pHeads, _pHeads, _pBias]
                           + [_i64] * 5 + [_f32, _i32, _i32, _vp, _i64, _vp, _vp]),
    "rgd_attn_bias_tiles_bytes": (_i64, [_i64] * 4),
    "rgd_attn_bias_tiles_build": (_i32, [_pBias, _i64, _i64, _i64, _i64, _f32, _vp, _i64, _vp]),
    "rgd_attn_fwd_uses_tmem": (_i32, [_pHeads] * 4 + [_i64] * 5 + [_f32, _i32]),
    "rgd_attn_bwd_uses_tmem": (_i32, [_pHeads] * 8 + [_i64] * 5 + [_i32]),
}

_lib = None


def load() -> C.CDLL:
    """dlopen the library once and attach the prototypes.  Raises if absent."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("RGD_B200_LIB", LIB_PATH))
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m rgd_triton_b200.build` "
            "(nvcc, sm_100a).  This package has no CPU or PyTorch fallback."
        )
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_string(code: int) -> str:
    return load().rgd_status_string(int(code)).decode()


_ASSERT_CODES = {RGD_E_INVALID, RGD_E_DTYPE, RGD_E_SIZE, RGD_E_STRIDE, RGD_E_NULL, RGD_E_WORKSPACE}


def check(code: int, what: str) -> None:
    """Turn a status code into the exception type the reference would raise."""
    if code == 0:
        return
    msg = f"{what}: {status_string(code)} (status {code})"
    if code in _ASSERT_CODES:
        raise AssertionError(msg)
    raise RuntimeError(msg)


_checked_devices: set[int] = set()


def require_device(t: torch.Tensor) -> None:
    """Operators run only on sm_100 CUDA tensors; anything else is an error."""
    if not t.is_cuda:
        raise AssertionError("rgd_triton_b200 operators need CUDA tensors (there is no CPU path)")
    idx = t.device.index if t.device.index is not None else torch.cuda.current_device()
    if idx in _checked_devices:
        return
    ok = load().rgd_device_supported(idx)
    if ok != 1:
        raise RuntimeError(f"cuda:{idx} is not a compute-capability-10 (B200) device; "
                           "rgd_triton_b200 ships sm_100a kernels only")
    _checked_devices.add(idx)


# The raw accessors skip the Stream / device-index objects torch.cuda.current_stream() builds (several
# microseconds per call, as much as a small operator's whole launch); the public path is the fallback.
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def stream_ptr() -> int:
    """The current CUDA stream of the current device as an integer handle."""
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return _RAW_STREAM(_RAW_DEVICE())
    return torch.cuda.current_stream().cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def device_guard(t: torch.Tensor):
    """Context that makes t's device current for the launch; free of charge
    when it already is (the common case), which matters for the small operators
    whose host path is as long as their kernel."""
    if t.device.index == (_RAW_DEVICE() if _RAW_DEVICE is not None else torch.cuda.current_device()):
        return _NO_GUARD
    return torch.cuda.device(t.device)


def dtype_code(dt: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dt]
    except KeyError:
        raise AssertionError("Only support fp16, bf16, and fp32") from None


def rows(t: torch.Tensor) -> Rows:
    return Rows(t.data_ptr(), t.stride(0), t.stride(1))


def heads(t: torch.Tensor, heads_second: bool) -> Heads:
    if heads_second:   # [B, H, N, d]
        return Heads(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
    return Heads(t.data_ptr(), t.stride(0), t.stride(2), t.stride(1))   # [B, N, H, d]
