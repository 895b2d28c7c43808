"""ctypes binding of the C ABI declared in ``include/lloom_b200.h``.

There is no fallback: if the shared library is missing the import of any compute entry point
raises, and every non-zero status from the library becomes a ``LloomError``.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "liblloom_b200.so")

OK, ERR_DTYPE, ERR_SHAPE, ERR_ALIGN, ERR_NULL, ERR_WORKSPACE, ERR_LAUNCH, ERR_TIMEOUT, ERR_DEVICE, ERR_STATIC_LIMIT = range(10)

# Every symbol include/lloom_b200.h declares: (name, restype, argtypes)
_i64, _vp, _int = C.c_int64, C.c_void_p, C.c_int
SYMBOLS = [
    ("lloom_b200_version", _int, []),
    ("lloom_b200_error_string", C.c_char_p, [_int]),
    ("lloom_b200_last_cuda_error", _int, []),
    ("lloom_b200_device_status", _int, [C.POINTER(_int)]),
    ("lloom_b200_set_launch_overlap", _int, [_int]),
    ("lloom_b200_set_wait_limit_ns", _int, [C.c_uint64]),
    ("lloom_b200_weight_image_bytes", _i64, [_int, _i64, _i64]),
    ("lloom_b200_weight_image_build", _int, [_int, _vp, _i64, _i64, _vp, _i64, _vp]),
    ("lloom_b200_workspace_bytes_with_image", _i64, [_int, _i64, _i64, _i64]),
    ("lloom_b200_qmatmul_fwd_image", _int, [_int, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    ("lloom_b200_qmatmul_fwd_group", _int, [_int, _int, C.POINTER(_vp), _vp, C.POINTER(_vp), C.POINTER(_i64),
                                            C.POINTER(_i64), C.POINTER(_int), _i64, _i64, _vp, _i64, _vp]),
    ("lloom_b200_indexed_moe_forward", _int, [_int, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _vp, _i64, _vp]),
    ("lloom_b200_qmatmul_fwd_gather_sync", _int, [_int, _vp, _vp, _i64, _i64, _i64, _i64, _i64, C.POINTER(_vp), _int, _int,
                                                  C.POINTER(_vp), _vp, _vp, _i64, _vp]),
    ("lloom_b200_qmatmul_fwd_after_gather", _int, [_int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _int, _vp, _i64, _vp]),
    ("lloom_b200_peer_wait", _int, [_int, _vp, _vp]),
    ("lloom_b200_block_elems", _i64, [_int]),
    ("lloom_b200_block_bytes", _i64, [_int]),
    ("lloom_b200_act_dtype", _int, [_int]),
    ("lloom_b200_act_row_bytes", _i64, [_int, _i64]),
    ("lloom_b200_workspace_bytes", _i64, [_int, _i64, _i64, _i64]),
    ("lloom_b200_quantize_act", _int, [_int, _vp, _i64, _i64, _vp, _vp]),
    ("lloom_b200_gemv", _int, [_int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    ("lloom_b200_gemm", _int, [_int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    ("lloom_b200_qmatmul_fwd", _int, [_int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    ("lloom_b200_qmatmul_fwd_static", _int, [_int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    ("lloom_b200_qmatmul_fwd_store", _int, [_int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp, _i64, _vp]),
    ("lloom_b200_qmatmul_fwd_gather", _int, [_int, _vp, _vp, _i64, _i64, _i64, _i64, _i64, C.POINTER(_vp), _int, _vp, _i64, _vp]),
    ("lloom_b200_peer_barrier", _int, [_int, _int, C.POINTER(_vp), _vp]),
    ("lloom_b200_peer_alloc", _int, [_i64, C.POINTER(_vp)]),
    ("lloom_b200_peer_free", _int, [_vp]),
    ("lloom_b200_peer_export", _int, [_vp, C.c_char_p]),
    ("lloom_b200_peer_open", _int, [C.c_char_p, C.POINTER(_vp)]),
    ("lloom_b200_peer_close", _int, [_vp]),
    ("lloom_b200_dequantize", _int, [_int, _vp, _i64, _vp, _int, _vp]),
    ("lloom_b200_get_rows", _int, [_int, _vp, _i64, _i64, _vp, _i64, _vp, _vp]),
    # include/lloom_b200_host.h: C view of the C++ host layer
    ("lloom_b200_host_last_error", C.c_char_p, []),
    ("lloom_b200_host_quantize_rows", _int, [_int, _vp, _vp, _i64, _i64, _int]),
    ("lloom_b200_host_quantize_rows_imatrix", _int, [_int, _vp, _vp, _vp, _i64, _i64, _int]),
    ("lloom_b200_host_qtensor_quantize_imatrix", _int, [_int, _vp, _vp, _vp, _i64, _i64, _int, _int, C.POINTER(_vp)]),
    ("lloom_b200_host_qtensor_quantize", _int, [_int, _vp, _vp, _i64, _i64, _int, _int, C.POINTER(_vp)]),
    ("lloom_b200_host_qtensor_from_data", _int, [_int, _vp, _vp, _i64, _int, _i64, _i64, C.POINTER(_vp)]),
    ("lloom_b200_host_qtensor_free", None, [_vp]),
    ("lloom_b200_host_qtensor_nbytes", _i64, [_vp]),
    ("lloom_b200_host_qtensor_device_ptr", _vp, [_vp]),
    ("lloom_b200_host_qtensor_data", _int, [_vp, _vp, _i64]),
    ("lloom_b200_host_qmatmul_forward", _int, [_vp, _vp, _i64, _vp]),
    ("lloom_b200_host_qtensor_dequantize", _int, [_vp, _vp, _int]),
    ("lloom_b200_host_qtensor_embedding", _int, [_vp, _vp, _i64, _vp]),
]


class LloomError(RuntimeError):
    """A non-zero status from the library (the shim maps these to ``Error::Cuda`` on the Rust side)."""

    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        super().__init__(f"{where}: status {status} ({detail})")


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m lloom_b200.build` "
                "(there is no CPU or PyTorch fallback for this library)")
        L = C.CDLL(LIB_PATH)
        for name, res, args in SYMBOLS:
            fn = getattr(L, name)  # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int, where: str) -> None:
    if status != OK:
        L = lib()
        detail = L.lloom_b200_error_string(status).decode()
        if status == ERR_LAUNCH:
            detail += f", cudaError {L.lloom_b200_last_cuda_error()}"
        raise LloomError(status, where, detail)
