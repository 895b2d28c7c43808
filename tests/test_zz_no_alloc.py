"""The allocation-free decode entry point, lloom_b200_qmatmul_fwd_static.

Some callers cannot hand the library a workspace: a plugin that only receives input and output
buffers, or a thread that is not allowed to touch the device allocator.  For them the library keeps
a fixed 256 KiB scratch array of its own.  This test calls that entry point through the C ABI twice
in a row (the second call finds the first call's leftovers in the shared array) and checks both
results against the regular workspace-taking entry point, which runs the same kernels: equal bits.

Collected last on purpose: a failure here cannot hide any other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_static_scratch_forward_matches_workspace_forward(cuda_lib):
    from lloom_b200 import _lib
    from lloom_b200.quantized import quantize_weights_host

    assert torch.cuda.is_available()
    L = cuda_lib
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    rng = np.random.default_rng(42)
    # two calls in a row with different shapes and formats: the second must not see the first one's bytes
    cases = [(12, 384, 4096, 8), (14, 200, 2048, 3), (8, 96, 2048, 1), (12, 64, 1024, 8)]
    for dt, n, k, m in cases:
        w = rng.standard_normal((n, k)).astype(np.float32) * np.float32(0.02)
        wq = torch.from_numpy(quantize_weights_host(w, dt).reshape(-1)).to(dev)
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dev)
        ws_bytes = int(L.lloom_b200_workspace_bytes(dt, m, n, k))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        y_ref = torch.zeros(m, n, dtype=torch.float32, device=dev)
        assert L.lloom_b200_qmatmul_fwd(dt, wq.data_ptr(), x.data_ptr(), y_ref.data_ptr(), m, n, k, n,
                                        ws.data_ptr(), ws_bytes, stream) == _lib.OK
        for call in range(2):
            y = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
            rc = L.lloom_b200_qmatmul_fwd_static(dt, wq.data_ptr(), x.data_ptr(), y.data_ptr(), m, n, k, n, stream)
            assert rc == _lib.OK, L.lloom_b200_error_string(rc)
            torch.cuda.synchronize()
            assert y.cpu().numpy().tobytes() == y_ref.cpu().numpy().tobytes(), (dt, n, k, m, call)
    # beyond the built-in scratch: refused with its own status, nothing launched
    big_k = 32768
    assert 8 * int(L.lloom_b200_act_row_bytes(12, big_k)) > 256 * 1024
    dummy = torch.zeros(64, dtype=torch.uint8, device=dev)
    xbig = torch.zeros(8, big_k, dtype=torch.float32, device=dev)
    ybig = torch.zeros(8, 4, dtype=torch.float32, device=dev)
    assert L.lloom_b200_qmatmul_fwd_static(12, dummy.data_ptr(), xbig.data_ptr(), ybig.data_ptr(), 8, 4, big_k, 4,
                                           stream) == _lib.ERR_STATIC_LIMIT
    x9 = torch.zeros(9, 256, dtype=torch.float32, device=dev)
    y9 = torch.zeros(9, 4, dtype=torch.float32, device=dev)
    assert L.lloom_b200_qmatmul_fwd_static(12, dummy.data_ptr(), x9.data_ptr(), y9.data_ptr(), 9, 4, 256, 4,
                                           stream) == _lib.ERR_STATIC_LIMIT
    assert b"built-in scratch" in L.lloom_b200_error_string(_lib.ERR_STATIC_LIMIT)
    torch.cuda.synchronize()
