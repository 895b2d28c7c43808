"""ctypes front end of the CPU oracle (``liblloom_oracle.so``).

TEST INFRASTRUCTURE ONLY.  Importable from ``tests/``, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``; the product
package never imports it.

The oracle restates lloom-tensor's CPU ``QMatMul`` path
(lloom-tensor/src/quantized/k_quants.rs, utils.rs, avx.rs); parity is pinned by
the reference's own golden values in ``tests/test_oracle_golden.py``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

Q8_0, Q4_K, Q6_K, Q8_K = 8, 12, 14, 15
Q4_0, Q5_0, Q5_K = 2, 6, 13
ORDER_UNOPT, ORDER_AVX2_EMU, ORDER_AVX2 = 0, 1, 2

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblloom_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (gcc only)."""
    src = os.path.join(_HERE, "lloom_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        i64, f32p, vp = C.c_int64, C.POINTER(C.c_float), C.c_void_p
        L.lo_has_avx2.restype = C.c_int
        L.lo_block_elems.restype = i64
        L.lo_block_elems.argtypes = [C.c_int]
        L.lo_block_bytes.restype = i64
        L.lo_block_bytes.argtypes = [C.c_int]
        L.lo_f32_to_f16.restype = C.c_uint16
        L.lo_f32_to_f16.argtypes = [C.c_float]
        L.lo_f16_to_f32.restype = C.c_float
        L.lo_f16_to_f32.argtypes = [C.c_uint16]
        L.lo_quantize_rows.restype = C.c_int
        L.lo_quantize_rows.argtypes = [C.c_int, vp, vp, i64, i64, C.c_int]
        L.lo_quantize_row_imatrix.restype = C.c_int
        L.lo_quantize_row_imatrix.argtypes = [C.c_int, vp, vp, i64, vp]
        L.lo_dequantize_row.restype = C.c_int
        L.lo_dequantize_row.argtypes = [C.c_int, vp, vp, i64]
        L.lo_vec_dot.restype = C.c_float
        L.lo_vec_dot.argtypes = [C.c_int, i64, vp, vp, C.c_int]
        L.lo_vec_dot_absum.restype = C.c_float
        L.lo_vec_dot_absum.argtypes = [C.c_int, i64, vp, vp]
        L.lo_matmul.restype = C.c_int
        L.lo_matmul.argtypes = [C.c_int, i64, i64, i64, vp, vp, vp, i64, C.c_int, C.c_int]
        L.lo_matmul_absum.restype = C.c_int
        L.lo_matmul_absum.argtypes = [C.c_int, i64, i64, i64, vp, vp, vp, C.c_int]
        L.lo_quantize_act.restype = C.c_int
        L.lo_quantize_act.argtypes = [C.c_int, vp, vp, i64, i64]
        L.lo_set_cluster_size.restype = None
        L.lo_set_cluster_size.argtypes = [C.c_int]
        _lib = L
    return _lib


def block_elems(dtype: int) -> int:
    return int(lib().lo_block_elems(dtype))


def block_bytes(dtype: int) -> int:
    return int(lib().lo_block_bytes(dtype))


def row_bytes(dtype: int, k: int) -> int:
    return k // block_elems(dtype) * block_bytes(dtype)


def act_dtype(w_dtype: int) -> int:
    """VecDotType of a weight type (k_quants.rs:717, 1507, 2082)."""
    return Q8_0 if w_dtype in (Q8_0, Q4_0, Q5_0) else Q8_K


def best_order() -> int:
    """The order the reference's x86 build runs (AVX2 arm); emulated when the host has no AVX2."""
    return ORDER_AVX2 if lib().lo_has_avx2() else ORDER_AVX2_EMU


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def quantize(dtype: int, x, nthreads: int = 1) -> np.ndarray:
    """``T::from_float`` over each row of ``x`` ([rows, k] or [k]); returns uint8 [rows, row_bytes]."""
    x = _f32(x)
    if x.ndim == 1:
        x = x[None, :]
    rows, k = x.shape
    out = np.zeros((rows, row_bytes(dtype, k)), dtype=np.uint8)
    rc = lib().lo_quantize_rows(dtype, _ptr(x), _ptr(out), rows, k, nthreads)
    if rc != 0:
        raise ValueError(f"oracle quantize failed rc={rc} dtype={dtype} k={k}")
    return out


def quantize_imatrix(dtype: int, x, imatrix) -> np.ndarray:
    """``T::from_float_imatrix`` over each row of ``x`` with one importance weight per column (``QTensor::quantize_imatrix``)."""
    x = _f32(x)
    if x.ndim == 1:
        x = x[None, :]
    imatrix = _f32(imatrix)
    rows, k = x.shape
    assert imatrix.shape == (k,)
    out = np.zeros((rows, row_bytes(dtype, k)), dtype=np.uint8)
    for r in range(rows):
        rc = lib().lo_quantize_row_imatrix(dtype, _ptr(x[r]), _ptr(out[r]), k, _ptr(imatrix))
        if rc != 0:
            raise ValueError(f"oracle quantize_imatrix failed rc={rc} dtype={dtype} k={k}")
    return out


def dequantize(dtype: int, blocks: np.ndarray, k: int) -> np.ndarray:
    """``T::to_float`` over each row of packed blocks; returns f32 [rows, k]."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, row_bytes(dtype, k))
    out = np.empty((blocks.shape[0], k), dtype=np.float32)
    for r in range(blocks.shape[0]):
        rc = lib().lo_dequantize_row(dtype, _ptr(blocks[r]), _ptr(out[r]), k)
        if rc != 0:
            raise ValueError(f"oracle dequantize failed rc={rc}")
    return out


def quantize_act(w_dtype: int, x) -> np.ndarray:
    """The activation quantizer ``matmul`` applies to its LHS (Q8_0 or Q8_K by weight type)."""
    x = _f32(x)
    if x.ndim == 1:
        x = x[None, :]
    m, k = x.shape
    out = np.zeros((m, row_bytes(act_dtype(w_dtype), k)), dtype=np.uint8)
    rc = lib().lo_quantize_act(w_dtype, _ptr(x), _ptr(out), m, k)
    if rc != 0:
        raise ValueError(f"oracle quantize_act failed rc={rc}")
    return out


def vec_dot(w_dtype: int, k: int, w_row: np.ndarray, act_row: np.ndarray, order: int) -> float:
    w_row = np.ascontiguousarray(w_row, dtype=np.uint8)
    act_row = np.ascontiguousarray(act_row, dtype=np.uint8)
    return float(np.float32(lib().lo_vec_dot(w_dtype, k, _ptr(w_row), _ptr(act_row), order)))


def matmul(w_dtype: int, lhs, w_blocks: np.ndarray, n: int, order: int | None = None, nthreads: int = 1,
           dst_len: int | None = None) -> np.ndarray:
    """``k_quants::matmul((m,k,n), lhs, W, dst)``; returns f32 [m, n]."""
    lhs = _f32(lhs)
    if lhs.ndim == 1:
        lhs = lhs[None, :]
    m, k = lhs.shape
    w_blocks = np.ascontiguousarray(w_blocks, dtype=np.uint8)
    assert w_blocks.size == n * row_bytes(w_dtype, k), (w_blocks.size, n, k)
    if order is None:
        order = best_order()
    dst = np.full(m * n if dst_len is None else max(dst_len, 1), np.nan, dtype=np.float32)
    rc = lib().lo_matmul(w_dtype, m, k, n, _ptr(lhs), _ptr(w_blocks), _ptr(dst),
                         m * n if dst_len is None else dst_len, nthreads, order)
    if rc == -1:
        raise ValueError(f"quantized matmul destination is too short for {m}x{n}")
    if rc != 0:
        raise ValueError(f"oracle matmul failed rc={rc}")
    return dst[: m * n].reshape(m, n) if dst_len is None else dst


def set_cluster_size(cluster_size: int) -> None:
    """Cluster size of the thread pool's two-level tree (utils::BarrierPool; 0 = flat, the reference's choice off macOS)."""
    lib().lo_set_cluster_size(int(cluster_size))


def matmul_absum(w_dtype: int, lhs, w_blocks: np.ndarray, n: int, nthreads: int = 1) -> np.ndarray:
    """Per output element, the sum of magnitudes of its per-block f32 terms."""
    lhs = _f32(lhs)
    if lhs.ndim == 1:
        lhs = lhs[None, :]
    m, k = lhs.shape
    w_blocks = np.ascontiguousarray(w_blocks, dtype=np.uint8)
    dst = np.empty(m * n, dtype=np.float32)
    rc = lib().lo_matmul_absum(w_dtype, m, k, n, _ptr(lhs), _ptr(w_blocks), _ptr(dst), nthreads)
    if rc != 0:
        raise ValueError(f"oracle matmul_absum failed rc={rc}")
    return dst.reshape(m, n)
