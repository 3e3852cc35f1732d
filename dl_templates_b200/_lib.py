"""ctypes binding of the C ABI declared in ``include/swa2d.h``.

The shared library is the only implementation: if it is missing or does not
load, importing this module raises -- there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libswa2d.so")

SWA_F32, SWA_F16, SWA_BF16 = 0, 1, 2
NOALLOC_MAX_ROWS = 1 << 21          # SWA_NOALLOC_MAX_ROWS of include/swa2d.h
IMPL_AUTO, IMPL_SIMT, IMPL_TC = 0, 1, 2
_IMPL_BY_NAME = {"auto": IMPL_AUTO, "simt": IMPL_SIMT, "tc": IMPL_TC}
_DTYPES = {torch.float32: SWA_F32, torch.float16: SWA_F16, torch.bfloat16: SWA_BF16}


class Tensor4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride", C.c_int64 * 4)]


class Geom(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("B", C.c_int32), ("H", C.c_int32), ("b_size", C.c_int32),
                ("t_height", C.c_int32), ("t_width", C.c_int32), ("row_size", C.c_int32), ("col_size", C.c_int32),
                ("d_qk", C.c_int32), ("d_v", C.c_int32), ("sm_scale", C.c_float), ("impl", C.c_int32)]


class Rope(C.Structure):
    _fields_ = [("idx", C.c_void_p), ("row_cs", C.c_void_p), ("col_cs", C.c_void_p),
                ("n_rdim", C.c_int32), ("max_h", C.c_int32), ("max_w", C.c_int32)]


EXPORTS = ("swa_fwd", "swa_bwd_delta", "swa_bwd_dq", "swa_bwd_dkdv", "swa_fwd_rot", "swa_bwd_dq_rot", "swa_bwd_dkdv_rot",
           "swa_bwd_noalloc", "rope2d_apply",
           "rope2d_apply_to", "swa_select_impl", "swa_describe_plan", "swa_refresh_env", "swa_launch_count", "swa_last_error", "swa_version")


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python dl_templates_b200/build.py` "
            "(nvcc, sm_100a). This package has no fallback implementation.")
    lib = C.CDLL(LIB_PATH)
    P = C.POINTER
    lib.swa_fwd.argtypes = [P(Geom), P(Rope), P(Tensor4), P(Tensor4), P(Tensor4), P(Tensor4), C.c_void_p, C.c_void_p,
                            C.c_void_p]
    lib.swa_bwd_delta.argtypes = [P(Geom), P(Tensor4), P(Tensor4), C.c_void_p, C.c_void_p]
    lib.swa_bwd_dq.argtypes = [P(Geom), P(Rope), P(Tensor4), P(Tensor4), P(Tensor4), P(Tensor4), C.c_void_p,
                               C.c_void_p, P(Tensor4), C.c_void_p, C.c_void_p]
    lib.swa_bwd_dkdv.argtypes = [P(Geom), P(Rope), P(Tensor4), P(Tensor4), P(Tensor4), P(Tensor4), C.c_void_p,
                                 C.c_void_p, P(Tensor4), P(Tensor4), C.c_void_p, C.c_void_p]
    lib.swa_fwd_rot.argtypes = [P(Geom), P(Rope), P(Tensor4), P(Tensor4), P(Tensor4), P(Tensor4), C.c_void_p, P(Tensor4),
                                P(Tensor4), C.c_void_p, C.c_void_p]
    lib.swa_bwd_dq_rot.argtypes = lib.swa_bwd_dq.argtypes
    lib.swa_bwd_dkdv_rot.argtypes = lib.swa_bwd_dkdv.argtypes
    lib.swa_bwd_noalloc.argtypes = [P(Geom), P(Rope), P(Tensor4), P(Tensor4), P(Tensor4), P(Tensor4), P(Tensor4),
                                    C.c_void_p, P(Tensor4), P(Tensor4), P(Tensor4), C.c_void_p, C.c_void_p]
    lib.rope2d_apply.argtypes = [C.c_int32, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, P(C.c_int64), P(Rope),
                                 C.c_int32, C.c_void_p]
    lib.rope2d_apply_to.argtypes = [C.c_int32, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, P(C.c_int64),
                                    P(C.c_int64), P(Rope), C.c_int32, C.c_void_p]
    lib.swa_select_impl.argtypes = [P(Geom), P(Rope), C.c_int32]
    lib.swa_describe_plan.argtypes = [P(Geom), P(Rope), C.c_int32, P(C.c_int32)]
    for name in ("swa_fwd", "swa_bwd_delta", "swa_bwd_dq", "swa_bwd_dkdv", "swa_fwd_rot", "swa_bwd_dq_rot",
                 "swa_bwd_dkdv_rot", "swa_bwd_noalloc", "rope2d_apply",
                 "rope2d_apply_to", "swa_select_impl", "swa_describe_plan", "swa_version"):
        getattr(lib, name).restype = C.c_int
    lib.swa_refresh_env.restype = None
    lib.swa_launch_count.restype = C.c_int64
    lib.swa_last_error.restype = C.c_char_p
    return lib


lib = _load()


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}; supported: float32, float16, bfloat16") from None


def impl_code(name) -> int:
    if isinstance(name, int):
        return name
    return _IMPL_BY_NAME[os.environ.get("SWA_FORCE_IMPL", name)]


def tensor4(t: torch.Tensor) -> Tensor4:
    assert t.dim() == 4
    r = Tensor4()
    r.ptr = t.data_ptr()
    for i in range(4):
        r.stride[i] = t.stride(i)
    return r


def make_geom(dtype, B, H, b_size, t_height, t_width, row_size, col_size, d_qk, d_v, sm_scale, impl="auto") -> Geom:
    return Geom(dtype_code(dtype), B, H, b_size, t_height, t_width, row_size, col_size, d_qk, d_v, float(sm_scale),
                impl_code(impl))


def make_rope(idx, row_cs, col_cs):
    """ctypes view of (idx, row table, col table); ``None`` index -> NULL (no RoPE)."""
    if idx is None:
        return None
    assert idx.dtype == torch.int32 and idx.is_contiguous()
    assert row_cs.dtype == torch.float32 and col_cs.dtype == torch.float32
    assert row_cs.is_contiguous() and col_cs.is_contiguous()
    assert row_cs.dim() == 3 and row_cs.shape[2] == 2 and row_cs.shape[1] == col_cs.shape[1]
    return Rope(idx.data_ptr(), row_cs.data_ptr(), col_cs.data_ptr(), row_cs.shape[1], row_cs.shape[0],
                col_cs.shape[0])


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed ({code}): {lib.swa_last_error().decode()}")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def launch_count() -> int:
    return int(lib.swa_launch_count())
