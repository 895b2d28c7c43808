"""Seeded synthetic weights and activations in the shapes and distributions of the benchmark configurations.

No checkpoint exists where this library is measured, so the benchmark and the full-size parity tests draw
their matrices here: ``numpy.random.default_rng(seed).standard_normal(...) * sigma`` in float32, quantized with
the host layer's CPU weight quantizer (the reference's ``T::from_float``, what ``QTensor::quantize`` runs before
the upload, lloom-tensor/src/quantized/mod.rs:919-938).  Large matrices are drawn in chunks of 4096 rows, each
chunk from its own generator ``default_rng([seed, chunk])``, so that chunks can be produced by several threads
and any row shard of a matrix sees the same values as the whole.
"""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

CHUNK_ROWS = 4096


def host_threads() -> int:
    try:
        import psutil

        return psutil.cpu_count(logical=False) or os.cpu_count() or 1
    except Exception:
        return os.cpu_count() or 1


def weight_chunk_f32(seed: int, chunk: int, k: int, sigma: float = 0.02) -> np.ndarray:
    """Rows [chunk * 4096, (chunk + 1) * 4096) of the f32 matrix of ``seed``."""
    rng = np.random.default_rng([seed, chunk])
    return rng.standard_normal((CHUNK_ROWS, k)).astype(np.float32) * np.float32(sigma)


def weight_rows_f32(seed: int, lo: int, hi: int, k: int, sigma: float = 0.02) -> np.ndarray:
    parts = []
    c0 = lo
    while c0 < hi:
        c1 = min(hi, (c0 // CHUNK_ROWS + 1) * CHUNK_ROWS)
        blk = weight_chunk_f32(seed, c0 // CHUNK_ROWS, k, sigma)
        parts.append(blk[c0 % CHUNK_ROWS: c0 % CHUNK_ROWS + (c1 - c0)])
        c0 = c1
    return np.concatenate(parts) if len(parts) > 1 else np.ascontiguousarray(parts[0])


def quantized_rows(seed: int, lo: int, hi: int, k: int, dtype: int, sigma: float = 0.02, threads: int = 0) -> np.ndarray:
    """Packed blocks (uint8 ``[hi - lo, row_bytes]``) of rows [lo, hi) of the matrix of ``seed``."""
    from .quantized import quantize_weights_host

    threads = threads or host_threads()
    spans = []
    c0 = lo
    while c0 < hi:
        c1 = min(hi, (c0 // CHUNK_ROWS + 1) * CHUNK_ROWS)
        spans.append((c0, c1))
        c0 = c1

    def one(span):
        a, b = span
        blk = weight_chunk_f32(seed, a // CHUNK_ROWS, k, sigma)
        return quantize_weights_host(blk[a % CHUNK_ROWS: a % CHUNK_ROWS + (b - a)], dtype, nthreads=1)

    if len(spans) == 1:
        a, b = spans[0]
        blk = weight_chunk_f32(seed, a // CHUNK_ROWS, k, sigma)
        return quantize_weights_host(blk[a % CHUNK_ROWS: a % CHUNK_ROWS + (b - a)], dtype, nthreads=threads)
    with ThreadPoolExecutor(max_workers=threads) as pool:
        parts = list(pool.map(one, spans))
    return np.concatenate(parts)


def quantized_matrix(seed: int, n: int, k: int, dtype: int, sigma: float = 0.02, threads: int = 0) -> np.ndarray:
    return quantized_rows(seed, 0, n, k, dtype, sigma, threads)


def activations(seed: int, m: int, k: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)
