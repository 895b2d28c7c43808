"""CPU-only checks of the C ABI: the library loads, exports every declared symbol, and validates
arguments before touching a device.  No kernel is launched here."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for header in sorted(os.listdir(inc)):
        if header.endswith(".h"):
            text = open(os.path.join(inc, header)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(lloom_b200_\w+)\s*\(", text))
    return sorted(names)


def test_header_and_binding_agree(cuda_lib):
    from lloom_b200 import _lib

    bound = sorted(name for name, _, _ in _lib.SYMBOLS)
    assert bound == declared_symbols()
    for name in bound:
        assert hasattr(cuda_lib, name), f"library does not export {name}"


def test_version_and_format_tables(cuda_lib):
    assert cuda_lib.lloom_b200_version() == 100
    sizes = {8: (32, 34), 12: (256, 144), 14: (256, 210), 15: (256, 292), 2: (32, 18), 6: (32, 22), 13: (256, 176)}  # mod.rs:663-715
    for dt, (elems, nbytes) in sizes.items():
        assert cuda_lib.lloom_b200_block_elems(dt) == elems
        assert cuda_lib.lloom_b200_block_bytes(dt) == nbytes
    assert cuda_lib.lloom_b200_block_elems(3) == 0  # Q4_1: not implemented, no fallback
    assert cuda_lib.lloom_b200_act_dtype(2) == 8 and cuda_lib.lloom_b200_act_dtype(6) == 8 and cuda_lib.lloom_b200_act_dtype(13) == 15
    assert cuda_lib.lloom_b200_act_dtype(8) == 8 and cuda_lib.lloom_b200_act_dtype(12) == 15
    assert cuda_lib.lloom_b200_act_dtype(14) == 15 and cuda_lib.lloom_b200_act_dtype(0) == 0
    assert cuda_lib.lloom_b200_act_row_bytes(12, 4096) == 16 * 292
    assert cuda_lib.lloom_b200_act_row_bytes(8, 2048) == 64 * 34
    assert cuda_lib.lloom_b200_act_row_bytes(12, 100) == 0
    assert cuda_lib.lloom_b200_workspace_bytes(12, 1, 14336, 4096) >= 16 * 292
    assert cuda_lib.lloom_b200_workspace_bytes(12, 1, 14336, 4100) == 0
    assert b"unsupported" in cuda_lib.lloom_b200_error_string(1)


def test_argument_validation_happens_before_any_launch(cuda_lib):
    from lloom_b200 import _lib

    L = cuda_lib
    buf = (C.c_uint8 * 4096)()
    p = C.addressof(buf)
    p16 = (p + 15) & ~15
    # unsupported dtypes are refused by name, never routed elsewhere (mod.rs:206-221)
    assert L.lloom_b200_gemv(3, p16, p16, p16, 1, 4, 256, 4, None) == _lib.ERR_DTYPE
    assert L.lloom_b200_qmatmul_fwd(10, p16, p16, p16, 1, 4, 256, 4, p16, 4096, None) == _lib.ERR_DTYPE
    assert L.lloom_b200_dequantize(3, p16, 256, p16, 0, None) == _lib.ERR_DTYPE
    # shapes
    assert L.lloom_b200_gemv(12, p16, p16, p16, 1, 4, 100, 4, None) == _lib.ERR_SHAPE
    assert L.lloom_b200_gemv(12, p16, p16, p16, 9, 4, 256, 4, None) == _lib.ERR_SHAPE  # GEMV is m <= 8
    assert L.lloom_b200_gemv(12, p16, p16, p16, 1, 4, 256, 3, None) == _lib.ERR_SHAPE  # ldy < n
    assert L.lloom_b200_gemv(12, p16, p16, p16, 0, 4, 256, 4, None) == _lib.ERR_SHAPE
    assert L.lloom_b200_dequantize(12, p16, 100, p16, 0, None) == _lib.ERR_SHAPE
    # null and alignment
    assert L.lloom_b200_gemv(12, None, p16, p16, 1, 4, 256, 4, None) == _lib.ERR_NULL
    assert L.lloom_b200_gemv(12, p16 + 2, p16, p16, 1, 4, 256, 4, None) == _lib.ERR_ALIGN
    assert L.lloom_b200_quantize_act(12, p16 + 4, 1, 256, p16, None) == _lib.ERR_ALIGN
    # workspace
    assert L.lloom_b200_qmatmul_fwd(12, p16, p16, p16, 1, 4, 256, 4, None, 0, None) == _lib.ERR_WORKSPACE
    assert L.lloom_b200_qmatmul_fwd(12, p16, p16, p16, 1, 4, 256, 4, p16, 16, None) == _lib.ERR_WORKSPACE
    assert L.lloom_b200_device_status(None) == _lib.ERR_NULL


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from lloom_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_host_mirror_metadata(cuda_lib):
    from lloom_b200 import GgmlDType, LloomError

    assert GgmlDType.Q4K.block_size() == 256 and GgmlDType.Q4K.type_size() == 144
    assert GgmlDType.from_u32(14) is GgmlDType.Q6K
    with pytest.raises(LloomError):
        GgmlDType.from_u32(3)


def test_abi_is_reentrant_from_host_threads(cuda_lib):
    """The entry points that need no device (tables, planning, argument checks) called from eight host threads at
    once: same answers as single-threaded (QTensor is shared across threads in the reference, mod.rs:1700)."""
    import threading

    from lloom_b200 import _lib

    L = cuda_lib
    want = [(dt, m, int(L.lloom_b200_workspace_bytes(dt, m, 4096, 4096)), int(L.lloom_b200_weight_image_bytes(dt, 4096, 4096)))
            for dt in (2, 6, 8, 12, 13, 14) for m in (1, 8, 64, 512)]
    buf = (C.c_uint8 * 4096)()
    p16 = (C.addressof(buf) + 15) & ~15
    bad = []

    def worker():
        for _ in range(200):
            for dt, m, ws, img in want:
                if int(L.lloom_b200_workspace_bytes(dt, m, 4096, 4096)) != ws or int(L.lloom_b200_weight_image_bytes(dt, 4096, 4096)) != img:
                    bad.append((dt, m))
            if L.lloom_b200_gemv(3, p16, p16, p16, 1, 4, 256, 4, None) != _lib.ERR_DTYPE:
                bad.append("dtype")
            if L.lloom_b200_qmatmul_fwd(12, p16, p16, p16, 1, 4, 256, 4, None, 0, None) != _lib.ERR_WORKSPACE:
                bad.append("workspace")

    threads = [threading.Thread(target=worker) for _ in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not bad, bad[:5]


@pytest.mark.parametrize("dt", [8, 12, 14, 2, 6, 13])
def test_host_weight_quantizer_matches_oracle(cuda_lib, oracle, dt):
    """The host layer's CPU weight quantizer (what QCudaStorage::quantize runs before the upload) is
    byte-identical with the oracle's restatement of T::from_float, including all-zero blocks."""
    import numpy as np

    from lloom_b200.quantized import quantize_weights_host

    rng = np.random.default_rng(dt)
    w = rng.standard_normal((37, 1024)).astype(np.float32) * np.float32(0.02)
    w[3] = 0.0
    w[5, :256] = 0.0
    w[7] = np.float32(1.5)
    np.testing.assert_array_equal(quantize_weights_host(w, dt, nthreads=3), oracle.quantize(dt, w))
    i = np.arange(4096, dtype=np.float32)
    cosv = (np.float32(0.1) + np.float32(2.0) * np.cos(i)).astype(np.float32)[None, :]
    np.testing.assert_array_equal(quantize_weights_host(cosv, dt), oracle.quantize(dt, cosv))


@pytest.mark.parametrize("dt", [12, 13, 14])
def test_imatrix_quantizer(cuda_lib, oracle, dt):
    """from_float_imatrix (k_quants.rs:1682, 1959, 2246): the host layer's blocks equal the oracle's byte for byte, and
    the reference's own property holds (imatrix_quantize_q4k/q5k/q6k, quantized_tests.rs:571-690): with importance
    weights accumulated from activations the mean absolute dequantization error does not exceed the plain quantizer's."""
    import numpy as np

    from lloom_b200.quantized import LloomError, quantize_weights_host

    rng = np.random.default_rng(dt)
    values, rows, ncall = np.zeros(768, np.float64), 0, 0
    for _ in range(10):
        res = rng.standard_normal((256, 512)).astype(np.float32) @ rng.standard_normal((512, 768)).astype(np.float32)
        values += (res.astype(np.float64) ** 2).sum(0)
        rows += res.shape[0]
        ncall += 1
    imatrix = (values / rows * ncall).astype(np.float32)
    xs = rng.standard_normal((96, 768)).astype(np.float32)
    xs[5] = 0.0
    xs[7, :256] = 0.0
    q_imat = quantize_weights_host(xs, dt, nthreads=3, imatrix=imatrix)
    np.testing.assert_array_equal(q_imat, oracle.quantize_imatrix(dt, xs, imatrix))
    q_plain = quantize_weights_host(xs, dt)
    err_plain = np.abs(oracle.dequantize(dt, q_plain, 768) - xs).mean()
    err_imat = np.abs(oracle.dequantize(dt, q_imat, 768) - xs).mean()
    assert err_imat < err_plain, (err_imat, err_plain)
    with pytest.raises(LloomError):  # Q8_0 has no from_float_imatrix in the reference either
        quantize_weights_host(xs, 8, imatrix=imatrix)
