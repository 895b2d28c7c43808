"""Multi-rank host logic of the row-sharded forward, on CPU with the gloo backend (world_size 2 and 3).
The per-rank matmul is stood in for by the CPU oracle (no GPU here); what is tested is the shard plan,
the padded all-gather and its ordering: the gathered result must equal the unsharded one bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, dt, n, k, m, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lloom_b200.sharded import ShardedQMatMul, ShardPlan
        from oracle import oracle as O

        rng = np.random.default_rng(123)
        w = rng.standard_normal((n, k)).astype(np.float32) * np.float32(0.02)
        x = rng.standard_normal((m, k)).astype(np.float32)
        wq = O.quantize(dt, w)
        plan = ShardPlan(n, world)
        lo, hi = plan.range_of(rank)

        def local(xt):
            if hi == lo:
                return torch.empty(xt.shape[0], 0, dtype=torch.float32)
            return torch.from_numpy(O.matmul(dt, xt.numpy(), np.ascontiguousarray(wq[lo:hi]), hi - lo,
                                             order=O.ORDER_AVX2_EMU))

        y = ShardedQMatMul(local, plan).forward(torch.from_numpy(x).reshape(1, m, k))
        assert tuple(y.shape) == (1, m, n)
        full = O.matmul(dt, x, wq, n, order=O.ORDER_AVX2_EMU)
        assert y.reshape(m, n).numpy().tobytes() == full.tobytes(), f"rank {rank}: gathered != unsharded"
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,dt,n,k,m", [(2, 12, 64, 256, 1), (2, 14, 37, 256, 3), (3, 8, 10, 256, 2), (2, 12, 1, 256, 1)])
def test_sharded_forward_gloo(tmp_path, world, dt, n, k, m):
    from oracle import oracle as O

    O.build()
    port = _free_port()
    mp.spawn(_worker, args=(world, port, dt, n, k, m, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_plan_ranges():
    from lloom_b200.sharded import ShardPlan

    p = ShardPlan(128256, 8)  # the lm_head: 16032 rows per GPU
    assert p.rows_per == 16032 and [p.rows_of(r) for r in range(8)] == [16032] * 8
    assert p.byte_range(3, 3360) == (3 * 16032 * 3360, 4 * 16032 * 3360)
    p = ShardPlan(10, 4)
    assert [p.range_of(r) for r in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    p = ShardPlan(2, 4)
    assert [p.rows_of(r) for r in range(4)] == [1, 1, 0, 0]
