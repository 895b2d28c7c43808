"""Row-sharded forward on real GPUs (needs at least two): each rank loads only its rows, the logits are
all-gathered with NCCL, and every rank ends up with exactly the unsharded result."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import lloom_b200 as lb
        from lloom_b200.quantized import quantize_weights_host
        from lloom_b200.sharded import ShardedQMatMul

        for dt, n, k, m in ((14, 4008, 4096, 1), (12, 1792, 4096, 8), (8, 1030, 2048, 2), (12, 640, 1024, 40)):
            rng = np.random.default_rng(dt + n)
            w = rng.standard_normal((n, k)).astype(np.float32) * np.float32(0.02)
            x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dev)
            wq = quantize_weights_host(w, dt)
            sharded = ShardedQMatMul.from_data(wq, dt, (n, k), dev)
            y = sharded.forward(x)
            full = lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq, dt, (n, k), dev)).forward(x)
            torch.cuda.synchronize()
            assert tuple(y.shape) == (m, n)
            if m <= 8:  # same kernel on both sides: identical bits
                assert y.cpu().numpy().tobytes() == full.cpu().numpy().tobytes(), (rank, dt, n, k, m)
            else:       # a shard changes the GEMM's tile boundaries, not the per-element arithmetic
                assert y.cpu().numpy().tobytes() == full.cpu().numpy().tobytes(), (rank, dt, n, k, m)
            if m <= 8:
                # gather fused into the GEMV: peer stores + barrier kernel, no collective call; several forwards
                # in a row (the two output buffers alternate), each on a fresh activation
                assert sharded.enable_fused_gather(8)
                for it in range(5):
                    xi = x + float(it)
                    yi = sharded.forward(xi).clone()
                    fi = lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq, dt, (n, k), dev)).forward(xi)
                    torch.cuda.synchronize()
                    assert yi.cpu().numpy().tobytes() == fi.cpu().numpy().tobytes(), (rank, dt, n, k, m, it, "fused")
                from lloom_b200.quantized import device_status
                assert device_status() == 0
                sharded.close()
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_sharded_forward_nccl(tmp_path, cuda_lib):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = 2
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
