"""The C++ host layer (QTensor / QMatMul / QCudaStorage in lloom_b200/csrc/host) driven through its C view:
the object path a compiled host program uses, checked against the oracle."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _err(L):
    return L.lloom_b200_host_last_error().decode()


@pytest.mark.parametrize("dt,n,k,m", [(12, 130, 1024, 3), (14, 77, 512, 8), (8, 64, 256, 1), (12, 96, 512, 40)])
def test_host_qtensor_roundtrip_and_forward(cuda_lib, oracle, dt, n, k, m):
    L = cuda_lib
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(dt + n)
    w = rng.standard_normal((n, k)).astype(np.float32) * np.float32(0.02)
    x = rng.standard_normal((m, k)).astype(np.float32)
    wq = oracle.quantize(dt, w)
    h = C.c_void_p()
    stream = torch.cuda.current_stream(dev).cuda_stream
    # QTensor::quantize: host quantizer + upload
    assert L.lloom_b200_host_qtensor_quantize(0, stream, w.ctypes.data, n, k, dt, 4, C.byref(h)) == 0, _err(L)
    try:
        assert L.lloom_b200_host_qtensor_nbytes(h) == wq.size
        back = np.zeros(wq.size, np.uint8)
        assert L.lloom_b200_host_qtensor_data(h, back.ctypes.data, back.size) == 0, _err(L)
        np.testing.assert_array_equal(back, wq.reshape(-1))  # data() returns the exact packed bytes
        xt = torch.from_numpy(x).to(dev)
        y = torch.empty(m, n, dtype=torch.float32, device=dev)
        assert L.lloom_b200_host_qmatmul_forward(h, xt.data_ptr(), m, y.data_ptr()) == 0, _err(L)
        deq = torch.empty(n, k, dtype=torch.float32, device=dev)
        assert L.lloom_b200_host_qtensor_dequantize(h, deq.data_ptr(), 0) == 0, _err(L)
        ids = torch.tensor([n - 1, 0, 5], dtype=torch.int32, device=dev)
        emb = torch.empty(3, k, dtype=torch.float32, device=dev)
        assert L.lloom_b200_host_qtensor_embedding(h, ids.data_ptr(), 3, emb.data_ptr()) == 0, _err(L)
        torch.cuda.synchronize()
        ref = oracle.matmul(dt, x, wq, n)
        absum = oracle.matmul_absum(dt, x, wq, n)
        err = np.abs(y.cpu().numpy().astype(np.float64) - ref)
        assert (err / np.maximum(absum, 1e-30)).max() <= 1e-5
        dref = oracle.dequantize(dt, wq, k)
        assert deq.cpu().numpy().tobytes() == dref.tobytes()
        assert emb.cpu().numpy().tobytes() == dref[[n - 1, 0, 5]].tobytes()
    finally:
        L.lloom_b200_host_qtensor_free(h)
    # from_data refuses a short payload and a last dim that is not a whole number of blocks
    h2 = C.c_void_p()
    assert L.lloom_b200_host_qtensor_from_data(0, stream, wq.ctypes.data, wq.size - 1, dt, n, k, C.byref(h2)) != 0
    assert "payload length" in _err(L)
    assert L.lloom_b200_host_qtensor_from_data(0, stream, wq.ctypes.data, wq.size, dt, n * 2, k // 2 + 1, C.byref(h2)) != 0
