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
                # gather fused into the GEMV: peer stores, no collective call; several forwards in a row (the two
                # output buffers alternate), each on a fresh activation.  Both completion protocols: flags published
                # by the GEMV's last CTA + a wait kernel, and the separate barrier kernel.
                from lloom_b200.quantized import device_status
                ref_mm = lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq, dt, (n, k), dev))
                for sync in ("fused", "barrier"):
                    assert sharded.enable_fused_gather(8, sync=sync)
                    for it in range(5):
                        xi = x + float(it)
                        yi = sharded.forward(xi).clone()
                        fi = ref_mm.forward(xi)
                        torch.cuda.synchronize()
                        assert yi.cpu().numpy().tobytes() == fi.cpu().numpy().tobytes(), (rank, dt, n, k, m, it, sync)
                    assert device_status() == 0
                    sharded.close()
        # a chain without wait kernels: sharded up-projection -> replicated square matrix -> sharded down-projection,
        # each consumer waiting for its producer's completion flags in its own prologue (one row)
        from lloom_b200.sharded import forward_after_gather
        rng = np.random.default_rng(99)
        k0, n1 = 1024, 2048
        w_up = quantize_weights_host(rng.standard_normal((n1, k0)).astype(np.float32) * np.float32(0.02), 12)
        w_mid = quantize_weights_host(rng.standard_normal((n1, n1)).astype(np.float32) * np.float32(0.02), 12)
        w_down = quantize_weights_host(rng.standard_normal((k0, n1)).astype(np.float32) * np.float32(0.02), 12)
        up = ShardedQMatMul.from_data(w_up, 12, (n1, k0), dev)
        down = ShardedQMatMul.from_data(w_down, 12, (k0, n1), dev)
        mid = lb.QMatMul.from_qtensor(lb.QTensor.from_data(w_mid, 12, (n1, n1), dev))
        full_up = lb.QMatMul.from_qtensor(lb.QTensor.from_data(w_up, 12, (n1, k0), dev))
        full_down = lb.QMatMul.from_qtensor(lb.QTensor.from_data(w_down, 12, (k0, n1), dev))
        assert up.enable_fused_gather(1) and down.enable_fused_gather(1)
        x0 = torch.from_numpy(rng.standard_normal((1, k0)).astype(np.float32)).to(dev)
        for it in range(4):
            xi = x0 + float(it)
            h = up.forward(xi, wait=False)
            h2 = forward_after_gather(mid, h, up)
            y = down.forward(h, after=up, wait=True)
            torch.cuda.synchronize()
            want_h = full_up.forward(xi)
            assert torch.equal(h, want_h), (rank, it, "up")
            assert torch.equal(h2, mid.forward(want_h)), (rank, it, "mid")
            assert torch.equal(y, full_down.forward(want_h)), (rank, it, "down")
        from lloom_b200.quantized import device_status
        assert device_status() == 0
        up.close()
        down.close()
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


def test_fused_gather_entry_one_gpu(cuda_lib, oracle):
    """The gather entry on one GPU: with two output buffers standing in for two GPUs' buffers the GEMV writes
    identical rows into both at the shard's column offset and leaves the other columns alone; the barrier kernel
    with a group of one returns at once.  Covers both GEMV kernels (dp4a and tensor-core)."""
    import ctypes as C

    import lloom_b200 as lb
    from lloom_b200 import _lib
    from lloom_b200.quantized import device_status, quantize_weights_host

    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    for dt, n, k, m in ((12, 520, 1024, 1), (12, 520, 1024, 5), (14, 300, 512, 1), (8, 257, 256, 8)):
        rng = np.random.default_rng(dt * 1000 + n + m)
        w = rng.standard_normal((n, k)).astype(np.float32) * np.float32(0.02)
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dev)
        wq = quantize_weights_host(w, dt)
        qt = lb.QTensor.from_data(wq, dt, (n, k), dev)
        full = lb.QMatMul.from_qtensor(qt).forward(x)
        ldy, col0 = n + 40, 24
        bufs = [torch.full((m, ldy), -7.0, dtype=torch.float32, device=dev) for _ in range(2)]
        ptrs = (C.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
        ws_bytes = int(L.lloom_b200_workspace_bytes(dt, m, n, k))
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        rc = L.lloom_b200_qmatmul_fwd_gather(dt, qt.device_ptr(), x.data_ptr(), m, n, k, ldy, col0, ptrs, 2,
                                             ws.data_ptr(), ws.numel(), stream)
        assert rc == 0, rc
        flags = torch.zeros(16, dtype=torch.int32, device=dev)
        fptr = (C.c_void_p * 1)(flags.data_ptr())
        assert L.lloom_b200_peer_barrier(0, 1, fptr, stream) == 0
        torch.cuda.synchronize()
        assert device_status() == 0
        assert int(flags[0].item()) == 1 and int(flags[8].item()) == 1  # slot of rank 0 and the call counter
        # the same gather with the completion flags published by the GEMV itself (a group of one GPU: its own slot),
        # then the wait kernel, then a forward that waits for those flags in its prologue
        if True:
            flags2 = torch.zeros(16, dtype=torch.int32, device=dev)
            f2 = (C.c_void_p * 1)(flags2.data_ptr())
            one = (C.c_void_p * 1)(bufs[0].data_ptr())
            bufs[0].fill_(-7.0)
            for call in (1, 2):
                assert L.lloom_b200_qmatmul_fwd_gather_sync(dt, qt.device_ptr(), x.data_ptr(), m, n, k, ldy, col0, one, 1, 0,
                                                            f2, None, ws.data_ptr(), ws.numel(), stream) == 0
                assert L.lloom_b200_peer_wait(1, flags2.data_ptr(), stream) == 0
                torch.cuda.synchronize()
                assert device_status() == 0
                assert int(flags2[0].item()) == call and int(flags2[8].item()) == call and int(flags2[9].item()) == 0
            assert bufs[0].cpu().numpy()[:, col0:col0 + n].tobytes() == full.cpu().numpy().tobytes(), (dt, n, k, m, "sync")
        if m <= 2:
            y2 = torch.empty(m, n, dtype=torch.float32, device=dev)
            assert L.lloom_b200_qmatmul_fwd_after_gather(dt, qt.device_ptr(), x.data_ptr(), y2.data_ptr(), m, n, k, n,
                                                         flags2.data_ptr(), 1, ws.data_ptr(), ws.numel(), stream) == 0
            torch.cuda.synchronize()
            assert device_status() == 0
            assert torch.equal(y2, full)
        for b in bufs:
            got = b.cpu().numpy()
            assert got[:, col0:col0 + n].tobytes() == full.cpu().numpy().tobytes(), (dt, n, k, m)
            assert (got[:, :col0] == -7.0).all() and (got[:, col0 + n:] == -7.0).all()
    # argument checks
    assert L.lloom_b200_qmatmul_fwd_gather(12, qt.device_ptr(), x.data_ptr(), 9, n, k, ldy, col0, ptrs, 2,
                                           ws.data_ptr(), ws.numel(), stream) == _lib.ERR_SHAPE
    assert L.lloom_b200_peer_barrier(1, 1, fptr, stream) == _lib.ERR_SHAPE
