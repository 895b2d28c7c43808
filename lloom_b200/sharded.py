"""Row-sharded QMatMul across the GPUs of one node.

Output element ``y[r, c]`` depends only on weight row ``c`` (k_quants::matmul,
lloom-tensor/src/quantized/k_quants.rs:2455-2641), and the canonical block stream is row-major
``[n][k/block]``, so rank g of G owns the contiguous rows ``[g*ceil(n/G), ...)``, holds only those
bytes, runs the ordinary forward on its slice, and the ranks exchange their ``[m, n_local]`` f32
slices with one all-gather (NCCL over NVLink through ``torch.distributed``; ``gloo`` in the CPU
tests).  Per-row arithmetic does not depend on the shard, so the gathered result equals the
unsharded one bit for bit.  The reference has no distributed layer for this path; its only
collective code is the tensor-parallel example candle-examples/examples/llama_multiprocess/model.rs:31-98.
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


class ShardedQMatMul:
    """``QMatMul`` whose weight rows are split over the ranks of a process group."""

    def __init__(self, local_forward: Callable[[torch.Tensor], torch.Tensor], plan: ShardPlan, group=None):
        self._fwd = local_forward
        self.plan = plan
        self.group = group

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
        return cls(lambda x: mm.forward(x.reshape(-1, k)), plan, group)

    def forward(self, xs: torch.Tensor) -> torch.Tensor:
        lead = xs.shape[:-1]
        y_local = self._fwd(xs.reshape(-1, xs.shape[-1]))
        return gather_rows(y_local, self.plan, self.group).reshape(*lead, self.plan.n)

    __call__ = forward
