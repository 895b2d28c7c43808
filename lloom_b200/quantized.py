"""Host-side mirror of lloom-tensor's quantized API for the CUDA slot.

Names and semantics follow ``lloom-tensor/src/quantized/mod.rs`` (``GgmlDType`` :404-716, ``QTensor``
:94-101/908-1666, ``QMatMul`` :1698-1752/2022-2069) and the backend slot ``QCudaStorage``
(``lloom-tensor/src/quantized/cuda.rs`` :586-1024).  Everything that computes goes through the C ABI in
``include/lloom_b200.h``; PyTorch only provides device memory and the current stream.
"""
from __future__ import annotations

import enum
from typing import Sequence

import numpy as np
import torch

from . import _lib
from ._lib import LloomError, check


class GgmlDType(enum.IntEnum):
    """GGUF type ids of the formats this backend implements (mod.rs:505-568)."""

    Q4_0 = 2
    Q5_0 = 6
    Q8_0 = 8
    Q4K = 12
    Q5K = 13
    Q6K = 14
    Q8K = 15  # activation-only (mod.rs:448-451)

    def block_size(self) -> int:
        """Elements per block (mod.rs:699-715)."""
        return int(_lib.lib().lloom_b200_block_elems(int(self)))

    def type_size(self) -> int:
        """Bytes per block (mod.rs:663-697)."""
        return int(_lib.lib().lloom_b200_block_bytes(int(self)))

    @classmethod
    def from_u32(cls, u: int) -> "GgmlDType":
        try:
            return cls(u)
        except ValueError:
            raise LloomError(_lib.ERR_DTYPE, "GgmlDType.from_u32", f"unsupported dtype id {u}") from None


_WEIGHT_TYPES = (GgmlDType.Q4_0, GgmlDType.Q5_0, GgmlDType.Q8_0, GgmlDType.Q4K, GgmlDType.Q5K, GgmlDType.Q6K)
# The reference pads device weight buffers by 512 elements' worth of blocks (cuda.rs MATRIX_ROW_PADDING).
MATRIX_ROW_PADDING = 512


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class _Workspace:
    """Grow-only scratch per (device, stream), the role of fast_mmvq.rs:44-81 / fast_mmq.rs:135-174.

    Launches on different streams never share a buffer.  A buffer that has been outgrown is kept alive for the
    life of the process instead of being freed: a CUDA graph captured earlier may still hold its address."""

    _bufs: dict[tuple[int, int], torch.Tensor] = {}
    _retired: list[torch.Tensor] = []

    @classmethod
    def get(cls, device: torch.device, nbytes: int) -> torch.Tensor:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        key = (idx, torch.cuda.current_stream(device).cuda_stream)
        buf = cls._bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            if buf is not None:
                cls._retired.append(buf)
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            cls._bufs[key] = buf
        return buf


class QCudaStorage:
    """Device owner of packed GGUF blocks: the ``QStorage::Cuda`` slot (cuda.rs:586-1024)."""

    def __init__(self, data: torch.Tensor, nbytes: int, dtype: GgmlDType):
        self._data = data  # uint8, padded
        self._len = nbytes
        self._dtype = dtype
        self._image = None  # optional prebuilt f16 operand image for the prefill GEMM (build_prefill_image)

    # cuda.rs:1005-1024 load_quantized: one H2D copy of the raw block bytes, no repack, zero padding.
    @classmethod
    def load_quantized(cls, device, data, dtype: GgmlDType) -> "QCudaStorage":
        dtype = GgmlDType(dtype)
        if dtype not in _WEIGHT_TYPES:
            raise LloomError(_lib.ERR_DTYPE, "load_quantized", f"{dtype!r} is not a weight type of this backend")
        device = torch.device(device)
        if isinstance(data, torch.Tensor):
            host = data.detach().to("cpu").contiguous().view(torch.uint8).reshape(-1)
        else:
            host = torch.from_numpy(np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8)
                                                         if isinstance(data, (bytes, bytearray, memoryview))
                                                         else np.asarray(data, dtype=np.uint8)).reshape(-1))
        nbytes = host.numel()
        if nbytes % dtype.type_size() != 0:
            raise LloomError(_lib.ERR_SHAPE, "load_quantized", f"{nbytes} bytes is not a whole number of blocks")
        pad = MATRIX_ROW_PADDING * dtype.type_size() // dtype.block_size()
        buf = torch.zeros(nbytes + pad, dtype=torch.uint8, device=device)
        buf[:nbytes].copy_(host, non_blocking=host.is_pinned())  # pinned staging buffer: one asynchronous copy
        return cls(buf, nbytes, dtype)

    # cuda.rs:624-637 zeros
    @classmethod
    def zeros(cls, device, el_count: int, dtype: GgmlDType) -> "QCudaStorage":
        dtype = GgmlDType(dtype)
        nbytes = -(-el_count // dtype.block_size()) * dtype.type_size()
        padded = -(-(el_count + MATRIX_ROW_PADDING) // dtype.block_size()) * dtype.type_size()
        return cls(torch.zeros(padded, dtype=torch.uint8, device=torch.device(device)), nbytes, dtype)

    def dtype(self) -> GgmlDType:
        return self._dtype

    def device(self) -> torch.device:
        return self._data.device

    def storage_size_in_bytes(self) -> int:
        return self._len

    def device_ptr(self) -> int:
        return self._data.data_ptr()

    # cuda.rs:894-900 data(): the exact packed bytes.
    def data(self) -> bytes:
        return self._data[: self._len].cpu().numpy().tobytes()

    def build_prefill_image(self, self_shape: Sequence[int]) -> bool:
        """Builds, once, the f16 operand image the tensor-core GEMM reads (``lloom_b200_weight_image_build``) and keeps
        it beside the packed blocks: later forwards with more than 8 rows skip the per-call expansion.  Costs about
        4x the packed bytes of device memory.  Returns False (and keeps nothing) when no GEMM exists for the shape."""
        n, k = int(self_shape[0]), int(self_shape[1])
        L = _lib.lib()
        nbytes = int(L.lloom_b200_weight_image_bytes(int(self._dtype), n, k))
        if nbytes <= 0:
            return False
        dev = self.device()
        img = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
        off = (-img.data_ptr()) % 1024
        with torch.cuda.device(dev):
            check(L.lloom_b200_weight_image_build(int(self._dtype), self._data.data_ptr(), n, k, img.data_ptr() + off, nbytes,
                                                  _stream_ptr(dev)), "weight_image_build")
        self._image = (img, off)
        return True

    def drop_prefill_image(self) -> None:
        self._image = None

    # cuda.rs:647-718 dequantize / dequantize_f16
    def dequantize(self, elem_count: int) -> torch.Tensor:
        return self._dequantize(elem_count, False)

    def dequantize_f16(self, elem_count: int) -> torch.Tensor:
        return self._dequantize(elem_count, True)

    def _dequantize(self, elem_count: int, f16: bool) -> torch.Tensor:
        dev = self.device()
        out = torch.empty(elem_count, dtype=torch.float16 if f16 else torch.float32, device=dev)
        with torch.cuda.device(dev):
            check(_lib.lib().lloom_b200_dequantize(int(self._dtype), self._data.data_ptr(), elem_count,
                                                   out.data_ptr(), int(f16), _stream_ptr(dev)), "dequantize")
        return out

    # cuda.rs:828-860 embedding -> get_rows (cuda.rs:225-316)
    def embedding(self, rows: int, hidden: int, ids: torch.Tensor) -> torch.Tensor:
        if not ids.is_contiguous():
            raise LloomError(_lib.ERR_SHAPE, "embedding", "quantized embedding requires contiguous ids")
        if hidden % self._dtype.block_size() != 0:
            raise LloomError(_lib.ERR_SHAPE, "embedding",
                             f"quantized embedding hidden size {hidden} is not divisible by block size "
                             f"{self._dtype.block_size()}")
        expected = rows * hidden * self._dtype.type_size() // self._dtype.block_size()
        if self._len != expected:
            raise LloomError(_lib.ERR_SHAPE, "embedding", f"quantized tensor has {self._len} bytes, expected {expected}")
        dev = self.device()
        ids32 = ids.to(device=dev, dtype=torch.int64).to(torch.int32).contiguous()  # u32 bit pattern
        out = torch.empty(ids.numel(), hidden, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            check(_lib.lib().lloom_b200_get_rows(int(self._dtype), self._data.data_ptr(), rows, hidden,
                                                 ids32.data_ptr(), ids.numel(), out.data_ptr(), _stream_ptr(dev)),
                  "get_rows")
        return out

    # cuda.rs:862-894 fwd: weight [n,k]; x [..., k] contiguous f32 (f16/bf16 widen first); out [..., n].
    def fwd(self, self_shape: Sequence[int], x: torch.Tensor, out: torch.Tensor | None = None,
            out_col_offset: int = 0, store: int = 0) -> torch.Tensor:
        """``store``: block on the GEMV's store (the reference's MvStore, mod.rs:1668-1696): 0 plain, 1 ``silu(W.x)``,
        2 ``out <- out * (W.x)`` (needs ``out``); served for at most 8 rows, like the reference's matvec store."""
        if len(self_shape) != 2:
            raise LloomError(_lib.ERR_SHAPE, "fwd", f"weight shape {tuple(self_shape)} is not [n, k]")
        n, k = int(self_shape[0]), int(self_shape[1])
        if x.dim() < 2:
            raise LloomError(_lib.ERR_SHAPE, "fwd", f"input tensor has only one dimension {tuple(x.shape)}")
        if not x.is_contiguous():
            raise LloomError(_lib.ERR_SHAPE, "fwd", f"input tensor is not contiguous {tuple(x.shape)}")
        if x.shape[-1] != k:
            raise LloomError(_lib.ERR_SHAPE, "fwd", f"input tensor {tuple(x.shape)} incompatible with {(n, k)}")
        dev = self.device()
        if x.device != dev:
            raise LloomError(_lib.ERR_DEVICE, "fwd", f"input on {x.device}, weights on {dev}")
        in_dtype = x.dtype
        if in_dtype in (torch.float16, torch.bfloat16):
            x = x.float()  # the CPU f16 arm widens to f32 and quantizes the same way (k_quants.rs:2802-2835)
        elif in_dtype != torch.float32:
            raise LloomError(_lib.ERR_DTYPE, "fwd", "Expected f32/f16")
        m = x.numel() // k
        L = _lib.lib()
        with torch.cuda.device(dev):
            if out is None:
                y = torch.empty(*x.shape[:-1], n, dtype=torch.float32, device=dev)
                ldy, yptr = n, y.data_ptr()
            else:  # caller-provided [m, ld] buffer: write columns [off, off+n) (row-sharded weights)
                y = out
                ldy, yptr = out.stride(-2) if out.dim() >= 2 else out.numel(), out.data_ptr() + 4 * out_col_offset
            image = self._image if m > 8 else None
            ws_bytes = int((L.lloom_b200_workspace_bytes_with_image if image else L.lloom_b200_workspace_bytes)(
                int(self._dtype), m, n, k))
            if ws_bytes <= 0:
                raise LloomError(_lib.ERR_SHAPE, "fwd", f"unsupported shape m={m} n={n} k={k} for {self._dtype!r}")
            ws = _Workspace.get(dev, ws_bytes)
            if image is not None and not store:
                check(L.lloom_b200_qmatmul_fwd_image(int(self._dtype), self._data.data_ptr(),
                                                     image[0].data_ptr() + image[1], x.data_ptr(), yptr, m, n, k, ldy,
                                                     ws.data_ptr(), ws.numel(), _stream_ptr(dev)), "qmatmul_fwd_image")
            elif store:
                if store == 2 and out is None:
                    raise LloomError(_lib.ERR_NULL, "fwd", "the multiply-into store needs the destination buffer")
                check(L.lloom_b200_qmatmul_fwd_store(int(self._dtype), self._data.data_ptr(), x.data_ptr(), yptr, m, n, k,
                                                     ldy, int(store), ws.data_ptr(), ws.numel(), _stream_ptr(dev)),
                      "qmatmul_fwd_store")
            else:
                check(L.lloom_b200_qmatmul_fwd(int(self._dtype), self._data.data_ptr(), x.data_ptr(), yptr, m, n, k, ldy,
                                               ws.data_ptr(), ws.numel(), _stream_ptr(dev)), "qmatmul_fwd")
        if out is None and in_dtype != torch.float32:
            y = y.to(in_dtype)
        return y


class QTensor:
    """(storage, shape) pair, shape ``[n, k]`` with k a whole number of blocks (mod.rs:94-101, 894-906)."""

    def __init__(self, storage: QCudaStorage, shape: Sequence[int]):
        shape = tuple(int(s) for s in shape)
        dtype = storage.dtype()
        if len(shape) == 0 or shape[-1] % dtype.block_size() != 0:
            raise LloomError(_lib.ERR_SHAPE, "QTensor.new",
                             f"quantized tensor must have their last dim divisible by block size "
                             f"{tuple(shape)} {dtype.block_size()}")
        elems = int(np.prod(shape))
        if elems // dtype.block_size() * dtype.type_size() != storage.storage_size_in_bytes():
            raise LloomError(_lib.ERR_SHAPE, "QTensor.new", "storage size does not match shape")
        self.storage = storage
        self.shape = shape

    @classmethod
    def from_data(cls, data, dtype: GgmlDType, shape: Sequence[int], device="cuda") -> "QTensor":
        """``QStorage::from_data`` + ``load_quantized`` (mod.rs:136-223): raw GGUF block bytes to the device."""
        return cls(QCudaStorage.load_quantized(device, data, GgmlDType(dtype)), shape)

    @classmethod
    def quantize(cls, src, dtype: GgmlDType, device="cuda", nthreads: int = 0) -> "QTensor":
        """``QTensor::quantize`` (mod.rs:919-938): f32 ``[.., k]`` -> packed blocks on the device.  As in the
        reference's CUDA slot (cuda.rs:720-741) the weight quantizer runs on the CPU (the library's host
        layer), then the blocks are uploaded."""
        return cls.from_data(quantize_weights_host(src, dtype, nthreads), dtype,
                             tuple(src.shape), device)

    @classmethod
    def quantize_imatrix(cls, src, imatrix_weights, dtype: GgmlDType, device="cuda", nthreads: int = 0) -> "QTensor":
        """``QTensor::quantize_imatrix`` / ``quantize_imatrix_onto`` (mod.rs:940-1020): importance-weighted CPU
        quantization (one weight per column of ``src``), then upload.  Q4K, Q5K and Q6K, like the reference."""
        imatrix_weights = np.ascontiguousarray(imatrix_weights, dtype=np.float32)
        if imatrix_weights.ndim != 1 or imatrix_weights.shape[0] != src.shape[-1]:
            raise LloomError(_lib.ERR_SHAPE, "quantize_imatrix",
                             f"imatrix weights must have the same length {imatrix_weights.shape} as the last dim of src "
                             f"{src.shape[-1]}")
        return cls.from_data(quantize_weights_host(src, dtype, nthreads, imatrix=imatrix_weights), dtype,
                             tuple(src.shape), device)

    def dtype(self) -> GgmlDType:
        return self.storage.dtype()

    def device(self) -> torch.device:
        return self.storage.device()

    def rank(self) -> int:
        return len(self.shape)

    def storage_size_in_bytes(self) -> int:
        return self.storage.storage_size_in_bytes()

    def device_ptr(self) -> int:
        return self.storage.device_ptr()

    def data(self) -> bytes:
        return self.storage.data()

    def dequantize(self) -> torch.Tensor:
        return self.storage.dequantize(int(np.prod(self.shape))).reshape(self.shape)

    def dequantize_f16(self) -> torch.Tensor:
        return self.storage.dequantize_f16(int(np.prod(self.shape))).reshape(self.shape)

    def embedding(self, ids: torch.Tensor) -> torch.Tensor:
        """Rows of the dequantized table for ``ids`` (mod.rs:1101-1144): output ``ids.shape + [hidden]``."""
        if len(self.shape) != 2:
            raise LloomError(_lib.ERR_SHAPE, "embedding", "quantized embedding requires a rank-2 table")
        rows, hidden = self.shape
        return self.storage.embedding(rows, hidden, ids.contiguous()).reshape(*ids.shape, hidden)

    def fwd(self, x: torch.Tensor) -> torch.Tensor:
        """``CustomOp1::cuda_fwd`` (mod.rs:2009-2019)."""
        return self.storage.fwd(self.shape, x)

    def indexed_moe_forward(self, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """Routed matmul over stacked experts (mod.rs:1539-1650, cuda.rs:505-622): weight ``[n_experts, n, k]``,
        ``x [batch, 1 or topk, k]`` f32, ``ids [batch, topk]`` on the device -> ``[batch, topk, n]`` with
        ``out[b, t] = W[ids[b, t]] @ x[b, 0 or t]``.  Shape errors follow the reference's CPU arm."""
        if len(self.shape) != 3:
            raise LloomError(_lib.ERR_SHAPE, "indexed_moe_forward", f"weight shape {self.shape} is not [experts, n, k]")
        n_experts, n, k = self.shape
        if x.dim() != 3 or ids.dim() != 2:
            raise LloomError(_lib.ERR_SHAPE, "indexed_moe_forward", "x is [batch, in_dim1, k], ids [batch, topk]")
        batch, in_dim1, k_in = x.shape
        batch_ids, topk = ids.shape
        if k_in != k or batch != batch_ids or (in_dim1 != 1 and in_dim1 != topk):
            raise LloomError(_lib.ERR_SHAPE, "indexed_moe_forward",
                             f"x {tuple(x.shape)} / ids {tuple(ids.shape)} do not fit weight {self.shape}")
        dev = self.device()
        if x.device != dev or ids.device != dev:
            raise LloomError(_lib.ERR_DEVICE, "indexed_moe_forward", "x and ids must be on the weight's device")
        x = x.float().contiguous()
        ids32 = ids.to(torch.int64).to(torch.int32).contiguous()  # u32 bit pattern
        out = torch.empty(batch, topk, n, dtype=torch.float32, device=dev)
        L = _lib.lib()
        with torch.cuda.device(dev):
            ws_bytes = int(L.lloom_b200_workspace_bytes(int(self.dtype()), 1, n, k))
            ws = _Workspace.get(dev, ws_bytes)
            check(L.lloom_b200_indexed_moe_forward(int(self.dtype()), self.device_ptr(), n_experts, n, k, x.data_ptr(), batch,
                                                   in_dim1, ids32.data_ptr(), topk, out.data_ptr(), ws.data_ptr(), ws.numel(),
                                                   _stream_ptr(dev)), "indexed_moe_forward")
        return out


class QMatMul:
    """``QMatMul::QTensor`` arm (mod.rs:1698-1752): ``forward(xs) = xs @ W^T`` over packed weights."""

    def __init__(self, qtensor: QTensor):
        self.qtensor = qtensor

    @classmethod
    def from_qtensor(cls, qtensor: QTensor) -> "QMatMul":
        return cls(qtensor)

    from_arc = from_qtensor

    def forward(self, xs: torch.Tensor) -> torch.Tensor:
        return self.qtensor.fwd(xs)

    __call__ = forward

    MV_STORE_MAX_ROWS = 8

    def mv_store_serves(self, xs: torch.Tensor) -> bool:
        """Whether the store blocks serve this input (mod.rs ``mv_store_serves``): f32, contiguous, at most 8 rows."""
        k = self.qtensor.shape[1]
        return (xs.dtype == torch.float32 and xs.is_contiguous() and xs.dim() >= 2 and xs.shape[-1] == k
                and xs.numel() // k <= self.MV_STORE_MAX_ROWS)

    def forward_silu(self, xs: torch.Tensor):
        """``silu(W.x)`` with the SiLU on the GEMV's store, one launch (mod.rs:2105-2122).  ``None`` where the
        store block does not serve: the caller composes."""
        if not self.mv_store_serves(xs):
            return None
        return self.qtensor.storage.fwd(self.qtensor.shape, xs, store=1)

    def forward_mul_into(self, xs: torch.Tensor, gate: torch.Tensor):
        """``gate <- gate * (W.x)`` in ``gate``'s own buffer (mod.rs:2124-2155): the SwiGLU's up projection landing as
        ``silu(g) * u``.  ``gate`` is overwritten.  ``None`` where the store block does not serve."""
        n, k = self.qtensor.shape
        rows = xs.numel() // k if xs.dim() >= 2 else 0
        if (not self.mv_store_serves(xs) or gate.dtype != torch.float32 or not gate.is_contiguous()
                or gate.device != xs.device or gate.numel() != rows * n):
            return None
        self.qtensor.storage.fwd(self.qtensor.shape, xs, out=gate.view(rows, n), store=2)
        return gate


def forward_group(mats: Sequence["QMatMul"], xs: torch.Tensor, stores: Sequence[int] | None = None,
                  outs: Sequence[torch.Tensor] | None = None) -> list[torch.Tensor]:
    """Decode forward of several ``QMatMul`` that share the input ``xs`` (gate|up, q|k|v) through
    ``lloom_b200_qmatmul_fwd_group``: one activation read and, for a single row, one launch for all of them.
    All weights must have the same dtype, k and device; at most 8 rows.  ``stores[g]``: block on matrix g's store
    (0 plain, 1 SiLU, 2 multiply into ``outs[g]``).  Each result equals that matrix's own ``forward`` bit for bit."""
    import ctypes as C

    if not 1 <= len(mats) <= 8:
        raise LloomError(_lib.ERR_SHAPE, "forward_group", "1 to 8 matrices")
    st0 = mats[0].qtensor.storage
    dt, dev = st0.dtype(), st0.device()
    k = mats[0].qtensor.shape[1]
    if any(mm.qtensor.storage.dtype() != dt or mm.qtensor.shape[1] != k or mm.qtensor.device() != dev for mm in mats):
        raise LloomError(_lib.ERR_SHAPE, "forward_group", "matrices of a group share dtype, k and device")
    if xs.dtype != torch.float32 or not xs.is_contiguous() or xs.dim() < 2 or xs.shape[-1] != k or xs.device != dev:
        raise LloomError(_lib.ERR_SHAPE, "forward_group", f"input {tuple(xs.shape)} {xs.dtype}")
    m = xs.numel() // k
    ns = [mm.qtensor.shape[0] for mm in mats]
    if outs is None:
        outs = [torch.empty(*xs.shape[:-1], n, dtype=torch.float32, device=dev) for n in ns]
    G = len(mats)
    L = _lib.lib()
    with torch.cuda.device(dev):
        ws_bytes = int(L.lloom_b200_workspace_bytes(int(dt), m, max(ns), k))
        ws = _Workspace.get(dev, ws_bytes)
        w_arr = (C.c_void_p * G)(*[mm.qtensor.device_ptr() for mm in mats])
        y_arr = (C.c_void_p * G)(*[o.data_ptr() for o in outs])
        n_arr = (C.c_int64 * G)(*ns)
        ld_arr = (C.c_int64 * G)(*[o.stride(-2) if o.dim() >= 2 else o.numel() for o in outs])
        st_arr = (C.c_int * G)(*([int(s) for s in stores] if stores is not None else [0] * G))
        check(L.lloom_b200_qmatmul_fwd_group(int(dt), G, w_arr, xs.data_ptr(), y_arr, n_arr, ld_arr, st_arr, m, k,
                                             ws.data_ptr(), ws.numel(), _stream_ptr(dev)), "qmatmul_fwd_group")
    return list(outs)


def quantize_weights_host(src, dtype: GgmlDType, nthreads: int = 0, imatrix=None) -> np.ndarray:
    """CPU ``T::from_float`` (``from_float_imatrix`` when ``imatrix`` is given) over the rows of ``src`` through the
    library's host layer; uint8 [rows, row_bytes]."""
    import os

    dtype = GgmlDType(dtype)
    if isinstance(src, torch.Tensor):
        src = src.detach().to("cpu", torch.float32).numpy()
    src = np.ascontiguousarray(src, dtype=np.float32)
    k = src.shape[-1]
    if dtype not in _WEIGHT_TYPES or k % dtype.block_size() != 0:
        raise LloomError(_lib.ERR_SHAPE, "quantize", f"cannot quantize shape {src.shape} to {dtype!r}")
    rows = src.size // k
    out = np.zeros((rows, k // dtype.block_size() * dtype.type_size()), dtype=np.uint8)
    L = _lib.lib()
    if imatrix is not None:
        imatrix = np.ascontiguousarray(imatrix, dtype=np.float32)
        rc = L.lloom_b200_host_quantize_rows_imatrix(int(dtype), src.ctypes.data, imatrix.ctypes.data, out.ctypes.data, rows,
                                                     k, nthreads or (os.cpu_count() or 1))
    else:
        rc = L.lloom_b200_host_quantize_rows(int(dtype), src.ctypes.data, out.ctypes.data, rows, k,
                                             nthreads or (os.cpu_count() or 1))
    if rc != 0:
        raise LloomError(rc, "quantize", L.lloom_b200_host_last_error().decode())
    return out


# ---- thin functional access to the individual kernels (used by the parity tests and the bench) ----

def quantize_act(w_dtype: GgmlDType, x: torch.Tensor) -> torch.Tensor:
    """Activation quantizer alone: f32 [m,k] -> canonical Q8_0 / Q8_K blocks, uint8 [m, row_bytes]."""
    L = _lib.lib()
    x = x.contiguous()
    m, k = x.shape
    rb = int(L.lloom_b200_act_row_bytes(int(w_dtype), k))
    if rb <= 0:
        raise LloomError(_lib.ERR_SHAPE, "quantize_act", f"k={k} is not a whole number of blocks")
    out = torch.empty(m, rb, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(L.lloom_b200_quantize_act(int(w_dtype), x.data_ptr(), m, k, out.data_ptr(), _stream_ptr(x.device)),
              "quantize_act")
    return out


def gemv(w: QTensor, act_blocks: torch.Tensor, m: int) -> torch.Tensor:
    n, k = w.shape
    y = torch.empty(m, n, dtype=torch.float32, device=w.device())
    with torch.cuda.device(w.device()):
        check(_lib.lib().lloom_b200_gemv(int(w.dtype()), w.device_ptr(), act_blocks.data_ptr(), y.data_ptr(), m, n, k,
                                         n, _stream_ptr(w.device())), "gemv")
    return y


def gemm(w: QTensor, act_blocks: torch.Tensor, m: int) -> torch.Tensor:
    n, k = w.shape
    L = _lib.lib()
    y = torch.empty(m, n, dtype=torch.float32, device=w.device())
    ws_bytes = max(int(L.lloom_b200_workspace_bytes(int(w.dtype()), m, n, k)), 256)
    ws = _Workspace.get(w.device(), ws_bytes)
    with torch.cuda.device(w.device()):
        check(L.lloom_b200_gemm(int(w.dtype()), w.device_ptr(), act_blocks.data_ptr(), y.data_ptr(), m, n, k, n,
                                ws.data_ptr(), ws.numel(), _stream_ptr(w.device())), "gemm")
    return y


def device_status() -> int:
    v = _lib.C.c_int(0)
    check(_lib.lib().lloom_b200_device_status(_lib.C.byref(v)), "device_status")
    return v.value


def set_wait_limit_ns(ns: int) -> None:
    """Time limit of the kernels' bounded waits on the current device (0: the default, 2 s)."""
    check(_lib.lib().lloom_b200_set_wait_limit_ns(int(ns)), "set_wait_limit_ns")
