"""Row-sharded QMatMul across the GPUs of one node.

Output element ``y[r, c]`` depends only on weight row ``c`` (k_quants::matmul,
lloom-tensor/src/quantized/k_quants.rs:2455-2641), and the canonical block stream is row-major
``[n][k/block]``, so rank g of G owns the contiguous rows ``[g*ceil(n/G), ...)``, holds only those
bytes, runs the ordinary forward on its slice, and the ranks exchange their ``[m, n_local]`` f32
slices with one all-gather (NCCL over NVLink through ``torch.distributed``; ``gloo`` in the CPU
tests).  Per-row arithmetic does not depend on the shard, so the gathered result equals the
unsharded one bit for bit.  The reference has no distributed layer for this path; its only
collective code is the tensor-parallel example candle-examples/examples/llama_multiprocess/model.rs:31-98.

Decode batches (m <= 8) can skip the collective: with ``enable_fused_gather`` the GEMV stores every output
value into the output buffer of each GPU of the node (peer memory mapped through CUDA IPC), followed by one
small cross-GPU barrier kernel -- same bits, no NCCL launch on the critical path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardPlan:
    """Contiguous row ranges: every rank gets ``rows_per`` rows except possibly the last ones."""

    n: int
    world: int

    @property
    def rows_per(self) -> int:
        return -(-self.n // self.world)

    def range_of(self, rank: int) -> tuple[int, int]:
        lo = min(self.n, rank * self.rows_per)
        return lo, min(self.n, lo + self.rows_per)

    def rows_of(self, rank: int) -> int:
        lo, hi = self.range_of(rank)
        return hi - lo

    def byte_range(self, rank: int, row_bytes: int) -> tuple[int, int]:
        lo, hi = self.range_of(rank)
        return lo * row_bytes, hi * row_bytes


def gather_rows(y_local: torch.Tensor, plan: ShardPlan, group=None) -> torch.Tensor:
    """All-gather of ``[m, rows_of(rank)]`` slices into ``[m, n]``.  Slices are padded to ``rows_per`` columns
    for the collective (equal message sizes) and trimmed afterwards."""
    m = y_local.shape[0]
    rank = dist.get_rank(group)
    per = plan.rows_per
    if y_local.shape[1] != plan.rows_of(rank):
        raise ValueError(f"rank {rank}: local slice has {y_local.shape[1]} columns, plan says {plan.rows_of(rank)}")
    if y_local.shape[1] != per:
        padded = y_local.new_zeros(m, per)
        padded[:, : y_local.shape[1]] = y_local
        y_local = padded
    gathered = y_local.new_empty(plan.world, m, per)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(gathered, y_local.contiguous(), group=group)
    else:  # gloo (CPU tests): list form
        dist.all_gather(list(gathered.unbind(0)), y_local.contiguous(), group=group)
    if m == 1:
        out = gathered.reshape(1, plan.world * per)  # already in row order: no copy
    else:
        out = gathered.permute(1, 0, 2).reshape(m, plan.world * per)
    return out[:, : plan.n]


class _DeviceBytes:
    """Zero-copy view of raw device memory for ``torch.as_tensor``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerBuffer:
    """One zeroed device buffer per rank, each mapped into every process of the group (CUDA IPC): ``ptrs[g]`` is
    rank g's buffer as seen from this process.  Set-up only; collective over the group."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        import ctypes as C

        from . import _lib

        L = _lib.lib()
        self._L, self.nbytes, self.device, self.rank = L, int(nbytes), device, dist.get_rank(group)
        world = dist.get_world_size(group)
        with torch.cuda.device(device):
            own = C.c_void_p()
            _lib.check(L.lloom_b200_peer_alloc(self.nbytes, C.byref(own)), "peer_alloc")
            handle = C.create_string_buffer(64)
            _lib.check(L.lloom_b200_peer_export(own, handle), "peer_export")
            handles = [None] * world
            dist.all_gather_object(handles, handle.raw, group=group)
            self.ptrs = []
            for g in range(world):
                if g == self.rank:
                    self.ptrs.append(own.value)
                else:
                    p = C.c_void_p()
                    _lib.check(L.lloom_b200_peer_open(handles[g], C.byref(p)), "peer_open")
                    self.ptrs.append(p.value)
            self.array = (C.c_void_p * world)(*self.ptrs)  # host array of device pointers for the C ABI
        dist.barrier(group=group)

    def own_tensor(self) -> torch.Tensor:
        return torch.as_tensor(_DeviceBytes(self.ptrs[self.rank], self.nbytes), device=self.device)

    def close(self, group=None) -> None:
        """Collective: every rank unmaps its peers, then frees its own buffer."""
        if not self.ptrs:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for g, p in enumerate(self.ptrs):
                if g != self.rank:
                    self._L.lloom_b200_peer_close(p)
            dist.barrier(group=group)
            self._L.lloom_b200_peer_free(self.ptrs[self.rank])
        self.ptrs = []


class ShardedQMatMul:
    """``QMatMul`` whose weight rows are split over the ranks of a process group."""

    def __init__(self, local_forward: Callable[[torch.Tensor], torch.Tensor], plan: ShardPlan, group=None, local=None):
        self._fwd = local_forward
        self.plan = plan
        self.group = group
        self._local = local  # the shard's QMatMul (None on a rank without rows)
        self._fused = None

    @classmethod
    def from_data(cls, data, dtype, shape: Sequence[int], device, group=None) -> "ShardedQMatMul":
        """Every rank passes the full packed matrix (bytes / uint8 array); each keeps only its own rows on its GPU."""
        import numpy as np

        from .quantized import GgmlDType, QMatMul, QTensor

        dtype = GgmlDType(dtype)
        n, k = int(shape[0]), int(shape[1])
        plan = ShardPlan(n, dist.get_world_size(group))
        row_bytes = k // dtype.block_size() * dtype.type_size()
        raw = np.frombuffer(data, dtype=np.uint8) if isinstance(data, (bytes, bytearray, memoryview)) else np.asarray(data, dtype=np.uint8).reshape(-1)
        lo, hi = plan.byte_range(dist.get_rank(group), row_bytes)
        rows = plan.rows_of(dist.get_rank(group))
        if rows == 0:
            return cls(lambda x: x.new_empty(x.shape[0], 0, dtype=torch.float32), plan, group)
        mm = QMatMul.from_qtensor(QTensor.from_data(np.ascontiguousarray(raw[lo:hi]), dtype, (rows, k), device))
        return cls(lambda x: mm.forward(x.reshape(-1, k)), plan, group, local=mm)

    def enable_fused_gather(self, max_m: int = 8, sync: str = "fused") -> bool:
        """Collective.  Prepares the peer-store path for batches of up to ``max_m`` (<= 8) rows: two output buffers
        per rank (alternated call by call, so a buffer is rewritten only two forwards later) and one flag array,
        all mapped into every process.  ``sync``: "fused" -- the GEMV's last CTA publishes the completion flags and
        the consumer waits (``lloom_b200_qmatmul_fwd_gather_sync``); "barrier" -- a separate barrier kernel after
        the GEMV (``lloom_b200_peer_barrier``).  Returns False, changing nothing, when some rank holds no rows or
        the group has more than eight ranks."""
        world = self.plan.world
        if world > 8 or any(self.plan.rows_of(r) == 0 for r in range(world)) or self._local is None:
            return False
        if sync not in ("fused", "barrier"):
            raise ValueError(sync)
        max_m = max(1, min(8, int(max_m)))
        dev = self._local.qtensor.device()
        outs = [PeerBuffer(4 * max_m * self.plan.n, dev, self.group) for _ in range(2)]
        flags = PeerBuffer(256, dev, self.group)
        self._fused = {"max_m": max_m, "outs": outs, "flags": flags, "turn": 0, "sync": sync,
                       "stream": torch.cuda.current_stream(dev).cuda_stream,
                       "views": [o.own_tensor().view(torch.float32) for o in outs]}
        return True

    def close(self) -> None:
        if self._fused is not None:
            for b in self._fused["outs"] + [self._fused["flags"]]:
                b.close(self.group)
            self._fused = None

    def own_flags_ptr(self) -> int:
        """Device address of this rank's flag array of the fused gather (what a consumer's prologue waits on)."""
        f = self._fused
        return f["flags"].ptrs[dist.get_rank(self.group)]

    def _forward_fused(self, x2: torch.Tensor, after: "Optional[ShardedQMatMul]", wait: bool) -> torch.Tensor:
        from . import _lib
        from .quantized import _Workspace, _stream_ptr

        f, L = self._fused, _lib.lib()
        st = self._local.qtensor.storage
        rows, k = self._local.qtensor.shape
        m, n = x2.shape[0], self.plan.n
        rank = dist.get_rank(self.group)
        lo, _ = self.plan.range_of(rank)
        out, view = f["outs"][f["turn"]], f["views"][f["turn"]]
        f["turn"] ^= 1
        dev = st.device()
        stream = _stream_ptr(dev)
        if stream != f["stream"]:
            raise RuntimeError("the fused gather must run on the stream it was enabled on: the two output buffers and "
                               "the flag array are ordered by that stream alone")
        with torch.cuda.device(dev):
            ws_bytes = int(L.lloom_b200_workspace_bytes(int(st.dtype()), m, rows, k))
            ws = _Workspace.get(dev, ws_bytes)
            if f["sync"] == "barrier":
                _lib.check(L.lloom_b200_qmatmul_fwd_gather(int(st.dtype()), st.device_ptr(), x2.data_ptr(), m, rows, k, n,
                                                           lo, out.array, self.plan.world, ws.data_ptr(), ws.numel(), stream),
                           "qmatmul_fwd_gather")
                _lib.check(L.lloom_b200_peer_barrier(rank, self.plan.world, f["flags"].array, stream), "peer_barrier")
            else:
                wait_flags = after.own_flags_ptr() if after is not None else None
                _lib.check(L.lloom_b200_qmatmul_fwd_gather_sync(int(st.dtype()), st.device_ptr(), x2.data_ptr(), m, rows, k,
                                                                n, lo, out.array, self.plan.world, rank, f["flags"].array,
                                                                wait_flags, ws.data_ptr(), ws.numel(), stream),
                           "qmatmul_fwd_gather_sync")
                if wait:
                    _lib.check(L.lloom_b200_peer_wait(self.plan.world, self.own_flags_ptr(), stream), "peer_wait")
        return view[: m * n].view(m, n)

    def forward(self, xs: torch.Tensor, after: "Optional[ShardedQMatMul]" = None, wait: bool = True) -> torch.Tensor:
        """``xs @ W^T`` with the rows of ``W`` split over the ranks; every rank gets the full ``[.., n]`` result.

        With the fused gather enabled (and at most ``max_m`` contiguous f32 rows) the result is a *view* into this
        rank's peer-mapped output buffer: it stays valid until the second-next fused forward of this object, and
        every consumer of it must be ordered on the stream the gather was enabled on (each rank's next gather on
        that stream is what tells the peers that the buffer may be rewritten).  Clone it to keep it longer.

        ``wait=False`` (fused sync only) leaves out the wait kernel: the returned rows may then only be read by a
        forward that is told so -- ``other.forward(y, after=this)`` or ``forward_after_gather`` -- whose own
        prologue waits for all ranks' rows.  ``after``: the ShardedQMatMul whose un-waited output ``xs`` is
        (batches of up to two rows)."""
        lead = xs.shape[:-1]
        x2 = xs.reshape(-1, xs.shape[-1])
        if (self._fused is not None and x2.shape[0] <= self._fused["max_m"] and x2.dtype == torch.float32
                and x2.is_contiguous()):
            return self._forward_fused(x2, after, wait).reshape(*lead, self.plan.n)
        if after is not None or not wait:
            raise RuntimeError("after= / wait=False need the fused gather")
        y_local = self._fwd(x2)
        return gather_rows(y_local, self.plan, self.group).reshape(*lead, self.plan.n)

    __call__ = forward


def forward_after_gather(mm, xs: torch.Tensor, producer: ShardedQMatMul, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A replicated ``QMatMul`` forward (at most two rows) whose input is the un-waited output of ``producer``'s fused
    gather: the GEMV waits for the gather's completion flags in its own prologue (``lloom_b200_qmatmul_fwd_after_gather``)."""
    from . import _lib
    from .quantized import _Workspace, _stream_ptr

    L = _lib.lib()
    st = mm.qtensor.storage
    n, k = mm.qtensor.shape
    x2 = xs.reshape(-1, k)
    m = x2.shape[0]
    dev = st.device()
    y = out if out is not None else torch.empty(m, n, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        ws_bytes = int(L.lloom_b200_workspace_bytes(int(st.dtype()), m, n, k))
        ws = _Workspace.get(dev, ws_bytes)
        _lib.check(L.lloom_b200_qmatmul_fwd_after_gather(int(st.dtype()), st.device_ptr(), x2.data_ptr(), y.data_ptr(), m, n, k,
                                                         y.stride(0), producer.own_flags_ptr(), producer.plan.world,
                                                         ws.data_ptr(), ws.numel(), _stream_ptr(dev)), "qmatmul_fwd_after_gather")
    return y
