"""Pins the CPU oracle to the golden values of the reference's own tests.

Sources (paths inside the reference project):
  lloom-tensor/tests/quantized_tests.rs   :490-568 helpers, :862-1048 quantize ramps,
                                          :1106-1222 ggml matmul error test, :1769-1921 GEMM == GEMV rows
  lloom-tensor/src/quantized/ggml_file_tests.rs :11-14, :140-265 literal block images and sizes
The three seeded-RNG pins (quantized_matmul_q4k/q6k/q8k, :1441-1542) need Rust's StdRng and are not reproducible here.
"""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = json.load(open(os.path.join(HERE, "golden", "reference_pins.json")))

GGML_TEST_SIZE = 32 * 128


def test_vector2(bound, size):
    # get_test_vector2 (quantized_tests.rs:490-503)
    v = np.arange(size, dtype=np.float32)
    return ((v - np.float32(size / 2)) * np.float32(bound) / np.float32(size / 2)).astype(np.float32)


test_vector2.__test__ = False


def round3(v):
    # round_vector (:505-511): f32 (1000*x).round()/1000, half away from zero
    v = np.asarray(v, dtype=np.float32) * np.float32(1000.0)
    r = np.where(v >= 0, np.floor(v + np.float32(0.5)), np.ceil(v - np.float32(0.5))).astype(np.float32)
    return (r / np.float32(1000.0)).astype(np.float32)


def ggml_like(offset):
    # create_ggml_like_vector (:525-531)
    i = np.arange(GGML_TEST_SIZE, dtype=np.float32)
    return (np.float32(0.1) + np.float32(2.0) * np.cos(i + np.float32(offset))).astype(np.float32)


DT = {"Q8_0": 8, "Q4K": 12, "Q6K": 14, "Q8K": 15, "Q4_0": 2, "Q5_0": 6, "Q5K": 13}


def test_block_sizes(oracle):
    for name, (elems, size) in GOLD["block_sizes"].items():
        assert oracle.block_elems(DT[name]) == elems
        assert oracle.block_bytes(DT[name]) == size


def test_literal_block_images(oracle):
    """Field order of every block struct, from the literal byte images the reference asserts."""
    h1, hmin = bytes([0x00, 0x3C]), bytes([0x00, 0x38])  # f16 1.0, 0.5
    q8 = np.frombuffer(h1 + bytes([0xFD] * 32), dtype=np.uint8)
    np.testing.assert_array_equal(oracle.dequantize(8, q8, 32)[0], np.full(32, -3.0, np.float32))
    # Q4K: d=1, dmin=.5, scales all 0x23 -> (sc,m)=(35,35) for j<4 and (3,2) for j>=4; qs 0x98 -> low 8, high 9
    q4 = np.frombuffer(h1 + hmin + bytes([0x23] * 12) + bytes([0x98] * 128), dtype=np.uint8)
    got = oracle.dequantize(12, q4, 256)[0]
    exp = np.empty(256, np.float32)
    for j in range(8):
        sc, m = (35, 35) if j < 4 else (3, 2)
        q = 8 if j % 2 == 0 else 9
        exp[32 * j:32 * j + 32] = np.float32(sc) * np.float32(q) - np.float32(0.5) * np.float32(m)
    np.testing.assert_array_equal(got, exp)
    # Q6K: ql 0x9a, qh 0x5a, scales -5, d=1
    q6 = np.frombuffer(bytes([0x9A] * 128) + bytes([0x5A] * 64) + bytes([0xFB] * 16) + h1, dtype=np.uint8)
    got = oracle.dequantize(14, q6, 256)[0]
    exp = np.empty(256, np.float32)
    for h in range(2):
        for gq, (nib, hb) in enumerate([(0xA, 0x5A & 3), (0xA, (0x5A >> 2) & 3), (0x9, (0x5A >> 4) & 3), (0x9, 0x5A >> 6)]):
            exp[128 * h + 32 * gq:128 * h + 32 * gq + 32] = np.float32(-5.0) * np.float32((nib | (hb << 4)) - 32)
    np.testing.assert_array_equal(got, exp)


def test_q4_0_q5_0_ramp_pins(oracle):
    """quantize_q4_0 / quantize_q5_0 (quantized_tests.rs:361-393, 428-459): the ramp 0..127 through quantize and
    dequantize, all 128 values (Q4_0 exactly, Q5_0 to three decimals as the reference rounds them)."""
    src = np.arange(128, dtype=np.float32)
    d4 = oracle.dequantize(2, oracle.quantize(2, src), 128)[0]
    np.testing.assert_array_equal(d4, np.array(GOLD["ramp_0_127"]["Q4_0"], np.float32))
    assert np.signbit(d4[0]) and np.signbit(d4[1])  # the reference's -0.0
    d5 = oracle.dequantize(6, oracle.quantize(6, src), 128)[0]
    np.testing.assert_array_equal(round3(d5), np.array(GOLD["ramp_0_127"]["Q5_0"], np.float32))


@pytest.mark.parametrize("name", ["Q4K", "Q5K", "Q6K", "Q8K"])
def test_quantize_ramp_pins(oracle, name):
    """quantize_q4k / _q5k / _q6k / _q8k (quantized_tests.rs:862-1048)."""
    g = GOLD["quantize_ramp"][name]
    dt = DT[name]
    src = test_vector2(0.5, 1024)
    idx = [0, 128, 256, 512, 800, 1023]
    np.testing.assert_array_equal(src[idx], np.array(GOLD["quantize_ramp"]["src_points"], np.float32))
    dst = oracle.dequantize(dt, oracle.quantize(dt, src), 1024)[0]
    assert np.abs(dst - src).max() < g["max_err_small"]
    np.testing.assert_array_equal(round3(dst)[idx], np.array(g["points"], np.float32))
    big = test_vector2(128.0, 1024)
    dbig = oracle.dequantize(dt, oracle.quantize(dt, big), 1024)[0]
    assert np.abs(dbig - big).max() < g["max_err_big"]


@pytest.mark.parametrize("name", ["Q8_0", "Q4K", "Q6K", "Q8K", "Q4_0", "Q5_0", "Q5K"])
def test_ggml_quantization_error(oracle, name):
    """ggml_quantization_error_test (:545-568): RMSE/len on 0.1 + 2cos(i) stays under 0.002."""
    src = ggml_like(0.0)
    dst = oracle.dequantize(DT[name], oracle.quantize(DT[name], src), GGML_TEST_SIZE)[0]
    diff = (src - dst).astype(np.float32)
    rmse = np.sqrt(np.sum(diff * diff, dtype=np.float32)) / np.float32(GGML_TEST_SIZE)
    assert rmse <= GOLD["max_quantization_total_error"]


@pytest.mark.parametrize("name", ["Q8_0", "Q4K", "Q6K", "Q4_0", "Q5_0", "Q5K"])
def test_ggml_matmul_error(oracle, name):
    """ggml_matmul_error_test (:1157-1222) on the cosine vectors and on the ramp."""
    dt = DT[name]
    ramp = (np.arange(GGML_TEST_SIZE, dtype=np.float32) / np.float32(GGML_TEST_SIZE)).astype(np.float32)
    for a, b, err_m in [(ggml_like(0.0), ggml_like(1.0), 1.0), (ramp, ramp, 2.0)]:
        n = len(a)
        wq = oracle.quantize(dt, a)
        aq = oracle.quantize_act(dt, b)
        opt = oracle.vec_dot(dt, n, wq, aq, oracle.ORDER_AVX2_EMU)
        unopt = oracle.vec_dot(dt, n, wq, aq, oracle.ORDER_UNOPT)
        assert abs(opt - unopt) / n <= 1e-6
        mm = float(oracle.matmul(dt, b, wq, 1, order=oracle.ORDER_AVX2_EMU)[0, 0])
        assert abs(mm - opt) / n <= 1e-6
        assert mm == opt  # same function underneath
        ref = float(np.sum(a * b, dtype=np.float32))  # vec_dot_reference: f32 products, f32 left fold
        ref = float(np.float32(np.add.reduce((a * b).astype(np.float32), dtype=np.float32)))
        for r in (opt, unopt):
            err = abs(r - ref) / n
            assert np.isfinite(err) and err <= GOLD["max_dot_product_error"]
            assert err - 1e-5 <= GOLD["ggml_matmul_error"][name] * err_m, (name, err)
        if oracle.lib().lo_has_avx2():
            assert oracle.vec_dot(dt, n, wq, aq, oracle.ORDER_AVX2) == opt


@pytest.mark.parametrize("name", ["Q8_0", "Q4K", "Q6K", "Q4_0", "Q5_0", "Q5K"])
def test_prompt_gemm_is_bit_identical_to_decode_rows(oracle, name):
    """cpu_prompt_gemm_is_bit_identical_to_decode_rows (:1769-1903): integer-pattern inputs."""
    dt = DT[name]
    for m in (2, 17, 33):
        for n in (1, 2, 3, 4, 7, 65):
            for k in (256, 768):
                i = np.arange(m * k, dtype=np.int64)
                lhs = (((i * 17 % 211).astype(np.float32) - np.float32(103.0)) / np.float32(73.0)).reshape(m, k)
                i = np.arange(n * k, dtype=np.int64)
                w = (((i * 31 % 173).astype(np.float32) - np.float32(87.0)) / np.float32(61.0)).reshape(n, k)
                wq = oracle.quantize(dt, w)
                expected = np.stack([oracle.matmul(dt, lhs[r], wq, n, nthreads=1)[0] for r in range(m)])
                dense_w = oracle.dequantize(dt, wq, k).astype(np.float64)
                aq = oracle.quantize_act(dt, lhs)
                dense_a = oracle.dequantize(oracle.act_dtype(dt), aq, k).astype(np.float64)
                scalar = dense_a @ dense_w.T
                for threads in (1, 3):
                    got = oracle.matmul(dt, lhs, wq, n, nthreads=threads)
                    assert got.tobytes() == expected.tobytes(), (name, m, n, k)
                    err = np.abs(got.astype(np.float64) - scalar) / np.maximum(np.abs(scalar), 1.0)
                    assert err.max() <= GOLD["max_dot_product_error"]


def test_matmul_destination_too_short(oracle):
    """cpu_prompt_gemm_checks_destination_before_unsafe_stores (:1905-1921), on a quantized type."""
    m, k, n = 17, 256, 7
    lhs = np.ones((m, k), np.float32)
    wq = oracle.quantize(8, np.ones((n, k), np.float32))
    for length in (0, 1, m * n - 1):
        with pytest.raises(ValueError, match="destination is too short"):
            oracle.matmul(8, lhs, wq, n, dst_len=length)
    dst = oracle.matmul(8, lhs, wq, n, dst_len=m * n + 1)
    np.testing.assert_allclose(dst[: m * n], np.float32(k), rtol=1e-3)  # f16 scale rounding of 1/127
    assert np.isnan(dst[m * n])  # extra space is not written


def test_f16_conversions_match_ieee(oracle):
    L = oracle.lib()
    halves = np.arange(65536, dtype=np.uint16)
    as_f32 = halves.view(np.float16).astype(np.float32)
    mine = np.array([L.lo_f16_to_f32(int(h)) for h in halves[::7]], dtype=np.float32)
    np.testing.assert_array_equal(mine.view(np.uint32)[~np.isnan(mine)], as_f32[::7].view(np.uint32)[~np.isnan(mine)])
    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 5, 4000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5, np.inf, -np.inf], np.float32),
        (halves[::11].view(np.float16).astype(np.float32) * np.float32(1.0004883)),  # near rounding boundaries
    ]).astype(np.float32)
    vals = vals[~np.isnan(vals)]
    with np.errstate(over="ignore"):
        expect = vals.astype(np.float16).view(np.uint16)
    got = np.array([L.lo_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    np.testing.assert_array_equal(got, expect)


def test_avx2_arm_equals_lane_emulation(oracle):
    if not oracle.lib().lo_has_avx2():
        pytest.skip("host has no AVX2+FMA")
    rng = np.random.default_rng(7)
    for dt in (8, 12, 14):
        for k in (256, 2048, 4096):
            w = rng.standard_normal((5, k)).astype(np.float32) * np.float32(0.02)
            x = rng.standard_normal((3, k)).astype(np.float32)
            wq = oracle.quantize(dt, w)
            a = oracle.matmul(dt, x, wq, 5, order=oracle.ORDER_AVX2)
            b = oracle.matmul(dt, x, wq, 5, order=oracle.ORDER_AVX2_EMU)
            assert a.tobytes() == b.tobytes()


def test_special_blocks(oracle):
    """All-zero blocks and blocks with a tie for the largest magnitude (first occurrence wins)."""
    z = np.zeros(256, np.float32)
    for dt in (8, 12, 14, 15, 2, 6, 13):
        q = oracle.quantize(dt, z)
        np.testing.assert_array_equal(oracle.dequantize(dt, q, 256)[0], z)
    q6 = oracle.quantize(14, z)[0]
    assert q6[208] == 0x00 and q6[209] == 0x80  # d = f16(-0.0): 1 / (-128 / 0)
    x = np.zeros(256, np.float32)
    x[10], x[200] = 2.0, -2.0  # tie: +2 comes first, so iscale = -127/2 and d < 0
    q = oracle.quantize(15, x)[0]
    d = q[:4].view(np.float32)[0]
    assert d == np.float32(1.0) / (np.float32(-127.0) / np.float32(2.0))
    assert q[4 + 10].view(np.int8) == -127 and q[4 + 200].view(np.int8) == 127
    x[10], x[200] = -2.0, 2.0
    q = oracle.quantize(15, x)[0]
    assert q[:4].view(np.float32)[0] > 0 and q[4 + 10].view(np.int8) == -127


def test_gguf_package_layout_crosscheck(oracle):
    """Third-party layout check: python `gguf` dequantizes the oracle's bytes to the same values."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants

    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 512)).astype(np.float32)
    for dt, qt in ((8, gguf.GGMLQuantizationType.Q8_0), (12, gguf.GGMLQuantizationType.Q4_K),
                   (14, gguf.GGMLQuantizationType.Q6_K), (2, gguf.GGMLQuantizationType.Q4_0),
                   (6, gguf.GGMLQuantizationType.Q5_0), (13, gguf.GGMLQuantizationType.Q5_K)):
        q = oracle.quantize(dt, x)
        theirs = quants.dequantize(q, qt).astype(np.float32)
        mine = oracle.dequantize(dt, q, 512)
        np.testing.assert_allclose(theirs, mine, rtol=2e-6, atol=1e-7)


def test_committed_fixtures_match_oracle(oracle):
    """tests/golden/qmatmul_small.npz was written by make_golden.py from this oracle; it must not drift."""
    z = np.load(os.path.join(HERE, "golden", "qmatmul_small.npz"))
    for key in [k[:-2] for k in z.files if k.endswith("_w")]:
        dt, n, k, m = [int(v) for v in z[key + "_meta"]]
        wq = oracle.quantize(dt, z[key + "_w"])
        np.testing.assert_array_equal(wq, z[key + "_wq"])
        np.testing.assert_array_equal(oracle.quantize_act(dt, z[key + "_x"]), z[key + "_aq"])
        y = oracle.matmul(dt, z[key + "_x"], wq, n, order=oracle.ORDER_AVX2_EMU)
        assert y.tobytes() == z[key + "_y"].tobytes()


def test_barrier_pool_tree_shapes_give_the_same_result():
    """The oracle's thread pool restates utils::BarrierPool (utils.rs:10-307): flat (the reference's tree off macOS) and
    two-level trees of several cluster sizes, growing and shrinking thread counts, many generations -- the matmul's
    output does not depend on any of it."""
    from oracle import oracle as O

    rng = np.random.default_rng(11)
    n, k, m = 203, 512, 3
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    wq = O.quantize(12, w, nthreads=1)
    want = O.matmul(12, x, wq, n, nthreads=1).tobytes()
    try:
        for cluster in (0, 2, 3, 6, 64):
            O.set_cluster_size(cluster)
            for nthreads in (2, 7, 16, 5, 1, 12):
                for _ in range(20):
                    assert O.matmul(12, x, wq, n, nthreads=nthreads).tobytes() == want, (cluster, nthreads)
            assert O.quantize(12, w, nthreads=9).tobytes() == wq.tobytes()
    finally:
        O.set_cluster_size(0)
