"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle and the committed
golden fixtures.

Tolerances (stated here, used everywhere below):
  * quantized activation blocks: bit-exact (byte equality).
  * dequantize / get_rows: bit-exact.
  * f32 matmul outputs: |got - ref| <= 1e-6 * A, where A is the sum of the magnitudes of the f32
    summands the reference's AVX2 arm adds for that element (eight lane terms per block, plus the four
    min-lane terms of Q4_K) -- the scale any re-ordered f32 summation, the reference's own included, is
    bounded by (measured: 2-5e-7 for the GEMVs, below 1e-7 for the tensor-core GEMMs; the reference's own
    scalar and AVX2 arms differ by up to 8e-8 * A) -- and plain relative error |got - ref| <= 1e-5 * |ref|
    (the figure the specification names) for every element that is not a cancellation (|ref| >= A / 32;
    with N(0, 0.02) weights most Q4_K outputs do cancel below that: the min term eats the main term).
    Integer block sums are exact on both sides; only the f32 summation order differs from the AVX2 arm.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
HERE = os.path.dirname(os.path.abspath(__file__))

REL_TOL = 1e-5   # plain relative error, outputs that are not cancellations
A_TOL = 1e-6     # |err| / A, every output
DT_NAMES = {8: "Q8_0", 12: "Q4K", 14: "Q6K", 2: "Q4_0", 6: "Q5_0", 13: "Q5K"}
ALL_DT = [8, 12, 14, 2, 6, 13]


@pytest.fixture(scope="module")
def dev(cuda_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def assert_matmul_close(got, ref, absum, what=""):
    got, ref, absum = np.asarray(got, np.float64), np.asarray(ref, np.float64), np.asarray(absum, np.float64)
    assert got.shape == ref.shape
    err = np.abs(got - ref)
    scaled = err / np.maximum(absum, 1e-30)
    assert scaled.max() <= A_TOL, f"{what}: max |err|/A = {scaled.max():.3e}"
    solid = np.abs(ref) >= absum / 32
    if solid.any():
        rel = err[solid] / np.abs(ref[solid])
        assert rel.max() <= REL_TOL, f"{what}: max relative error {rel.max():.3e}"


def make_case(oracle, dt, n, k, m, seed, sigma_w=0.02):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((n, k)).astype(np.float32) * np.float32(sigma_w)
    x = rng.standard_normal((m, k)).astype(np.float32)
    wq = oracle.quantize(dt, w, nthreads=8)
    return w, x, wq


def run_fwd(dev, dt, wq, n, k, x):
    import lloom_b200 as lb

    qt = lb.QTensor.from_data(wq.tobytes(), dt, (n, k), dev)
    y = lb.QMatMul.from_qtensor(qt).forward(torch.from_numpy(x).to(dev))
    torch.cuda.synchronize()
    return y.cpu().numpy()


def test_golden_fixtures(dev):
    """Committed vectors: activation blocks byte-equal, outputs within tolerance, through the C ABI."""
    import lloom_b200 as lb
    from lloom_b200 import quantized as Q

    z = np.load(os.path.join(HERE, "golden", "qmatmul_small.npz"))
    for key in [k[:-2] for k in z.files if k.endswith("_w")]:
        dt, n, k, m = [int(v) for v in z[key + "_meta"]]
        xt = torch.from_numpy(z[key + "_x"]).to(dev)
        aq = Q.quantize_act(lb.GgmlDType(dt), xt)
        np.testing.assert_array_equal(aq.cpu().numpy(), z[key + "_aq"], err_msg=key)
        got = run_fwd(dev, dt, z[key + "_wq"], n, k, z[key + "_x"])
        assert_matmul_close(got, z[key + "_y"], z[key + "_absum"], key)
    assert Q.device_status() == 0


@pytest.mark.parametrize("dt", ALL_DT)
def test_activation_quantizer_bit_exact(dev, oracle, dt):
    """Seeded normals plus adversarial rows: ties, zeros, denormals, huge values, infinities, NaN."""
    import lloom_b200 as lb
    from lloom_b200 import quantized as Q

    rng = np.random.default_rng(100 + dt)
    k = 2048
    rows = [rng.standard_normal(k).astype(np.float32) for _ in range(6)]
    rows.append(np.zeros(k, np.float32))
    t = np.zeros(k, np.float32); t[5], t[300], t[301], t[700] = 3.0, -3.0, 3.0, -3.0  # magnitude ties
    rows.append(t)
    t = np.zeros(k, np.float32); t[::2] = -1.5; t[1::2] = 1.5  # every element ties; first is negative
    rows.append(t)
    rows.append((rng.standard_normal(k) * 1e-41).astype(np.float32))  # denormals
    rows.append((rng.standard_normal(k) * 1e37).astype(np.float32))   # near overflow
    h = (rng.integers(-254, 255, k) / 2.0).astype(np.float32)          # exact .5 rounding cases
    h[0] = 127.0
    rows.append(h)
    s = rng.standard_normal(k).astype(np.float32); s[3] = np.inf; s[900] = -np.inf
    rows.append(s)
    s = rng.standard_normal(k).astype(np.float32); s[17] = np.nan
    rows.append(s)
    x = np.stack(rows)
    with np.errstate(all="ignore"):
        ref = oracle.quantize_act(dt, x)
    got = Q.quantize_act(lb.GgmlDType(dt), torch.from_numpy(x).to(dev)).cpu().numpy()
    np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("dt", ALL_DT)
def test_gemv_exhaustive_small_shapes(dev, oracle, dt):
    """k in {256,512,768}, n in {1..9,65}, m in 1..8: ragged tiles, partial warps, unaligned rows."""
    for k in (256, 512, 768):
        for n in (1, 2, 3, 4, 5, 6, 7, 8, 9, 65):
            for m in (1, 2, 3, 4, 5, 6, 7, 8):
                _, x, wq = make_case(oracle, dt, n, k, m, seed=1000 * k + 10 * n + m)
                ref = oracle.matmul(dt, x, wq, n)
                absum = oracle.matmul_absum(dt, x, wq, n)
                got = run_fwd(dev, dt, wq, n, k, x)
                assert_matmul_close(got, ref, absum, f"{DT_NAMES[dt]} n={n} k={k} m={m}")


@pytest.mark.parametrize("dt,n,k", [(8, 8192, 2048), (12, 1792, 4096), (14, 2004, 4096), (12, 512, 14336),
                                    (13, 1792, 4096), (2, 2048, 4096), (6, 2048, 4096), (13, 300, 14336), (2, 300, 14336),
                                    (6, 257, 11008)])
@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_gemv_config_shapes(dev, oracle, dt, n, k, m):
    """Row counts and K of the decode configurations (full C1; one 8-GPU shard of C2/C3; the down projection)."""
    _, x, wq = make_case(oracle, dt, n, k, m, seed=dt * 7 + m)
    ref = oracle.matmul(dt, x, wq, n, nthreads=8)
    absum = oracle.matmul_absum(dt, x, wq, n, nthreads=8)
    got = run_fwd(dev, dt, wq, n, k, x)
    assert_matmul_close(got, ref, absum, f"{DT_NAMES[dt]} n={n} k={k} m={m}")


def test_reference_integer_pattern_inputs(dev, oracle):
    """Inputs of cpu_prompt_gemm_is_bit_identical_to_decode_rows (quantized_tests.rs:1816-1823): each row
    of a batch equals the same row run alone, bit for bit, and matches the oracle within tolerance."""
    for dt in ALL_DT:
        for m in (2, 8, 17, 33):
            for n in (1, 3, 7, 65):
                for k in (256, 768):
                    i = np.arange(m * k, dtype=np.int64)
                    lhs = (((i * 17 % 211).astype(np.float32) - np.float32(103.0)) / np.float32(73.0)).reshape(m, k)
                    i = np.arange(n * k, dtype=np.int64)
                    w = (((i * 31 % 173).astype(np.float32) - np.float32(87.0)) / np.float32(61.0)).reshape(n, k)
                    wq = oracle.quantize(dt, w)
                    got = run_fwd(dev, dt, wq, n, k, lhs)
                    ref = oracle.matmul(dt, lhs, wq, n)
                    assert_matmul_close(got, ref, oracle.matmul_absum(dt, lhs, wq, n), f"{DT_NAMES[dt]} m={m} n={n} k={k}")
                    if m <= 8:  # rows of a batch do not depend on the batch (qmm_batch, :239-275): bit for bit
                        # within one kernel, within tolerance across kernels (Q4_K batches of 2+ rows run on
                        # the tensor-core GEMV, single rows on the dp4a GEMV)
                        alone = np.concatenate([run_fwd(dev, dt, wq, n, k, lhs[r:r + 1]) for r in range(m)])
                        if dt == 12 and m >= 2:
                            assert_matmul_close(alone, ref, oracle.matmul_absum(dt, lhs, wq, n), "rows alone")
                        else:
                            assert alone.tobytes() == got.tobytes()


def test_run_to_run_bit_stable_and_shard_invariant(dev, oracle):
    """Same launch twice gives identical bits; a row shard computed alone equals the same rows of the
    full product (what N-sharding across GPUs relies on)."""
    import lloom_b200 as lb

    for dt, n, k in ((12, 1792, 4096), (14, 1336, 4096), (8, 1024, 2048)):
        for m in (1, 8):
            _, x, wq = make_case(oracle, dt, n, k, m, seed=5)
            a = run_fwd(dev, dt, wq, n, k, x)
            b = run_fwd(dev, dt, wq, n, k, x)
            assert a.tobytes() == b.tobytes()
            g = 8
            rows = n // g
            full = torch.empty(m, n, dtype=torch.float32, device=dev)
            xt = torch.from_numpy(x).to(dev)
            for r in range(g):
                shard = lb.QCudaStorage.load_quantized(dev, wq[r * rows:(r + 1) * rows].tobytes(), lb.GgmlDType(dt))
                shard.fwd((rows, k), xt, out=full, out_col_offset=r * rows)
            torch.cuda.synchronize()
            assert full.cpu().numpy().tobytes() == a.tobytes()


def test_full_size_properties_q4k(dev, oracle):
    """C2 at full size [14336, 4096]: linearity in the weights' row order and agreement with the oracle on
    a row sample (the oracle on all 14336 x 8 outputs would take minutes)."""
    n, k = 14336, 4096
    rng = np.random.default_rng(2)
    w = rng.standard_normal((n, k)).astype(np.float32) * np.float32(0.02)
    wq = oracle.quantize(12, w, nthreads=8)
    x = np.random.default_rng(3).standard_normal((8, k)).astype(np.float32)
    got = run_fwd(dev, 12, wq, n, k, x)
    perm = rng.permutation(n)
    got_perm = run_fwd(dev, 12, np.ascontiguousarray(wq[perm]), n, k, x)
    assert got_perm.tobytes() == np.ascontiguousarray(got[:, perm]).tobytes()  # rows are independent
    sample = np.sort(rng.choice(n, 1024, replace=False))
    ref = oracle.matmul(12, x, np.ascontiguousarray(wq[sample]), len(sample), nthreads=8)
    absum = oracle.matmul_absum(12, x, np.ascontiguousarray(wq[sample]), len(sample), nthreads=8)
    assert_matmul_close(got[:, sample], ref, absum, "C2 sample")
    # a row's result does not depend on its batch: bit for bit within one kernel (batches of 2..8 rows run on the
    # tensor-core GEMV, single rows on the dp4a GEMV), within the tolerance across the two
    assert run_fwd(dev, 12, wq, n, k, x[:4]).tobytes() == got[:4].tobytes()
    assert run_fwd(dev, 12, wq, n, k, x[:2]).tobytes() == got[:2].tobytes()
    one = run_fwd(dev, 12, wq, n, k, x[:1])
    assert_matmul_close(one[:, sample], ref[:1], absum[:1], "C2 sample, 1 row")


@pytest.mark.parametrize("n,k,m", [(128, 256, 128), (130, 512, 70), (256, 1024, 96), (384, 2048, 9), (1000, 4096, 200),
                                   (64, 768, 129)])
def test_gemm_q4k_tensor_core_path(dev, oracle, n, k, m):
    """Prefill GEMM (m > 8, Q4_K) on the tcgen05 kernel: ragged tiles in both directions, 1..16 superblocks."""
    _, x, wq = make_case(oracle, 12, n, k, m, seed=n + k + m)
    ref = oracle.matmul(12, x, wq, n, nthreads=8)
    absum = oracle.matmul_absum(12, x, wq, n, nthreads=8)
    got = run_fwd(dev, 12, wq, n, k, x)
    assert_matmul_close(got, ref, absum, f"Q4K gemm n={n} k={k} m={m}")
    assert run_fwd(dev, 12, wq, n, k, x).tobytes() == got.tobytes()  # run-to-run bit-stable


def test_gemm_q4k_prefill_config(dev, oracle):
    """C4 shape [14336, 4096] at M = 512: oracle parity on a sample of rows and columns (the CPU needs minutes for
    all of it), agreement with the decode GEMV on the same tokens, and every output finite."""
    from lloom_b200 import quantized as Q

    n, k, m = 14336, 4096, 512
    w = np.random.default_rng(6).standard_normal((n, k)).astype(np.float32) * np.float32(0.02)
    wq = oracle.quantize(12, w, nthreads=8)
    x = np.random.default_rng(7).standard_normal((m, k)).astype(np.float32)
    got = run_fwd(dev, 12, wq, n, k, x)
    assert np.isfinite(got).all()
    rng = np.random.default_rng(1)
    rows = np.sort(rng.choice(m, 24, replace=False))
    cols = np.sort(rng.choice(n, 1536, replace=False))
    wsub = np.ascontiguousarray(wq[cols])
    ref = oracle.matmul(12, x[rows], wsub, len(cols), nthreads=8)
    absum = oracle.matmul_absum(12, x[rows], wsub, len(cols), nthreads=8)
    assert_matmul_close(got[np.ix_(rows, cols)], ref, absum, "C4 sample")
    gemv = run_fwd(dev, 12, wq, n, k, x[:8])  # the same first eight tokens through the decode kernel
    absum8 = oracle.matmul_absum(12, x[:8], np.ascontiguousarray(wq[:4096]), 4096, nthreads=8)
    err = np.abs(gemv[:, :4096].astype(np.float64) - got[:8, :4096]) / np.maximum(absum8, 1e-30)
    assert err.max() <= 2 * A_TOL
    assert Q.device_status() == 0


@pytest.mark.parametrize("dt", ALL_DT)
def test_dequantize_and_embedding_bit_exact(dev, oracle, dt):
    """T::to_float parity (f32 and f16) and the embedding gather (run_quantized_embedding, :304-315)."""
    import lloom_b200 as lb

    i = np.arange(8 * 256, dtype=np.float32)
    table = (np.sin(i * np.float32(0.003)) * np.float32(0.5) + np.cos(i * np.float32(0.007)) * np.float32(0.25)).astype(np.float32).reshape(8, 256)
    wq = oracle.quantize(dt, table)
    qt = lb.QTensor.from_data(wq.tobytes(), dt, (8, 256), dev)
    ref = oracle.dequantize(dt, wq, 256)
    deq = qt.dequantize().cpu().numpy()
    assert deq.tobytes() == ref.tobytes()
    f16 = qt.dequantize_f16().cpu().numpy()
    assert f16.tobytes() == ref.astype(np.float16).tobytes()
    ids = torch.tensor([[3, 1], [3, 7]], dtype=torch.int64, device=dev)
    emb = qt.embedding(ids).cpu().numpy()
    assert emb.shape == (2, 2, 256)
    assert emb.tobytes() == ref[[3, 1, 3, 7]].reshape(2, 2, 256).tobytes()
    assert qt.data() == wq.tobytes()  # packed byte identity (ggml_file_tests.rs:78-82)
    # larger random table
    rng = np.random.default_rng(9)
    w = rng.standard_normal((300, 1024)).astype(np.float32)
    wq = oracle.quantize(dt, w, nthreads=8)
    qt = lb.QTensor.from_data(wq.tobytes(), dt, (300, 1024), dev)
    assert qt.dequantize().cpu().numpy().tobytes() == oracle.dequantize(dt, wq, 1024).tobytes()


def test_fwd_shape_rules_and_errors(dev, oracle):
    """QTensor::cuda_fwd layout rules (mod.rs:1906-1925): rank >= 2, contiguous, last dim == k; batch dims kept."""
    import lloom_b200 as lb

    _, x, wq = make_case(oracle, 12, 16, 256, 6, seed=1)
    qt = lb.QTensor.from_data(wq.tobytes(), 12, (16, 256), dev)
    mm = lb.QMatMul.from_qtensor(qt)
    xt = torch.from_numpy(x).to(dev)
    y3 = mm.forward(xt.reshape(2, 3, 256))
    assert tuple(y3.shape) == (2, 3, 16)
    assert y3.reshape(6, 16).cpu().numpy().tobytes() == mm.forward(xt).cpu().numpy().tobytes()
    with pytest.raises(lb.LloomError, match="only one dimension"):
        mm.forward(xt[0])
    with pytest.raises(lb.LloomError, match="incompatible"):
        mm.forward(torch.zeros(2, 512, device=dev))
    with pytest.raises(lb.LloomError, match="not contiguous"):
        mm.forward(torch.zeros(256, 2, device=dev).t())
    with pytest.raises(lb.LloomError):
        lb.QTensor.from_data(wq.tobytes(), 12, (16, 250), dev)
    # f16 input widens to f32, output returns in f16 (the CPU f16 arm, k_quants.rs:2802-2835)
    yh = mm.forward(xt.half())
    assert yh.dtype == torch.float16
    ref = mm.forward(xt.half().float()).half()
    assert yh.cpu().numpy().tobytes() == ref.cpu().numpy().tobytes()


@pytest.mark.parametrize("dt,n,k", [(12, 520, 1024), (14, 300, 512), (8, 257, 256), (13, 300, 512), (2, 257, 256), (6, 130, 512)])
def test_store_blocks_silu_and_mul_into(dev, oracle, dt, n, k):
    """forward_silu / forward_mul_into (mod.rs:2105-2155): the product is the plain forward's, bit for bit; SiLU is
    v / (1 + exp(-v)) in f32 (exp within a few ulp of the host's); the multiply-into is one exact f32 product."""
    import torch

    import lloom_b200 as lb

    for m in (1, 2, 5, 8):
        _, x, wq = make_case(oracle, dt, n, k, m, seed=dt + m)
        mm = lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq.tobytes(), dt, (n, k), dev))
        xt = torch.from_numpy(x).to(dev)
        plain = mm.forward(xt)
        got = mm.forward_silu(xt)
        assert got is not None and tuple(got.shape) == (m, n)
        p64 = plain.double()
        want = (p64 / (1.0 + torch.exp(-p64))).float()
        torch.testing.assert_close(got, want, rtol=3e-6, atol=1e-9)
        gate0 = torch.from_numpy(np.random.default_rng(m).standard_normal((m, n)).astype(np.float32)).to(dev)
        gate = gate0.clone()
        assert mm.forward_mul_into(xt, gate) is gate
        assert gate.cpu().numpy().tobytes() == (gate0 * plain).cpu().numpy().tobytes()
    # more than eight rows: the store blocks do not serve, the caller composes
    xt = torch.zeros(9, k, device=dev)
    assert mm.forward_silu(xt) is None and mm.forward_mul_into(xt, torch.zeros(9, n, device=dev)) is None


@pytest.mark.parametrize("n,m", [(40, 8), (130, 5), (97, 2), (64, 1)])
def test_q4k_long_rows(dev, oracle, n, m):
    """K = 14336 (an FFN down projection): the tensor-core GEMV cuts the rows into several stages' worth of
    superblocks and carries each warp's partial sums across the pieces (a single row stays on the dp4a kernel)."""
    k = 14336
    _, x, wq = make_case(oracle, 12, n, k, m, seed=n + m)
    ref = oracle.matmul(12, x, wq, n, nthreads=8)
    absum = oracle.matmul_absum(12, x, wq, n, nthreads=8)
    got = run_fwd(dev, 12, wq, n, k, x)
    assert_matmul_close(got, ref, absum, f"Q4K long rows n={n} m={m}")
    assert run_fwd(dev, 12, wq, n, k, x).tobytes() == got.tobytes()  # run-to-run bit-stable
    half = n // 2  # a row shard gives the same bits for its rows
    assert run_fwd(dev, 12, np.ascontiguousarray(wq[half:]), n - half, k, x).tobytes() == np.ascontiguousarray(got[:, half:]).tobytes()


@pytest.mark.parametrize("n,k", [(130, 11008), (257, 16384), (64, 5120), (100, 12288), (96, 20480), (48, 8192)])
def test_q4k_single_row_long_k(dev, oracle, n, k):
    """One activation row, K beyond 4096: the dp4a kernel cuts the rows into pieces of 16 superblocks (the last one
    shorter where K is no multiple of 4096).  Oracle parity, the same bits from run to run, for a row shard, and
    from a grouped launch."""
    _, x, wq = make_case(oracle, 12, n, k, 1, seed=n + k)
    ref = oracle.matmul(12, x, wq, n, nthreads=8)
    absum = oracle.matmul_absum(12, x, wq, n, nthreads=8)
    got = run_fwd(dev, 12, wq, n, k, x)
    assert_matmul_close(got, ref, absum, f"Q4K single row n={n} k={k}")
    assert run_fwd(dev, 12, wq, n, k, x).tobytes() == got.tobytes()
    half = n // 2
    assert run_fwd(dev, 12, np.ascontiguousarray(wq[half:]), n - half, k, x).tobytes() == np.ascontiguousarray(got[:, half:]).tobytes()
    import lloom_b200 as lb
    from lloom_b200 import quantized as Q
    mats = [lb.QMatMul.from_qtensor(lb.QTensor.from_data(w.tobytes(), 12, (w.shape[0], k), dev))
            for w in (wq, np.ascontiguousarray(wq[half:]))]
    outs = Q.forward_group(mats, torch.from_numpy(x).to(dev))
    assert outs[0].cpu().numpy().tobytes() == got.tobytes()
    assert outs[1].cpu().numpy().tobytes() == np.ascontiguousarray(got[:, half:]).tobytes()


def test_gemm_q4k_prefill_config_m2048(dev, oracle):
    """C4 at M = 2048 (the size the prefill throughput is quoted on): oracle parity on a sample of rows and
    columns, every output finite, and the prebuilt weight image gives the same bits as the per-call expansion."""
    import lloom_b200 as lb
    from lloom_b200 import quantized as Q
    from lloom_b200 import synthetic as S

    n, k, m = 14336, 4096, 2048
    wq = S.quantized_matrix(6, n, k, 12)
    x = S.activations(7, m, k)
    qt = lb.QTensor.from_data(wq, 12, (n, k), dev)
    xt = torch.from_numpy(x).to(dev)
    got_t = lb.QMatMul.from_qtensor(qt).forward(xt)
    got = got_t.cpu().numpy()
    assert np.isfinite(got).all()
    rng = np.random.default_rng(11)
    rows = np.sort(rng.choice(m, 16, replace=False))
    cols = np.sort(rng.choice(n, 2048, replace=False))
    wsub = np.ascontiguousarray(wq[cols])
    ref = oracle.matmul(12, x[rows], wsub, len(cols), nthreads=8)
    absum = oracle.matmul_absum(12, x[rows], wsub, len(cols), nthreads=8)
    assert_matmul_close(got[np.ix_(rows, cols)], ref, absum, "C4 M=2048 sample")
    assert qt.storage.build_prefill_image(qt.shape)
    again = lb.QMatMul.from_qtensor(qt).forward(xt)
    assert torch.equal(again, got_t)
    assert Q.device_status() == 0


def test_lm_head_q6k_full_size_and_shard(dev, oracle):
    """C3 at full size, Q6_K [128256, 4096], M = 1: oracle parity on a row sample, and the 16032-row shard of one of
    eight GPUs computed alone equals the same rows of the full product bit for bit."""
    import lloom_b200 as lb
    from lloom_b200 import quantized as Q
    from lloom_b200 import synthetic as S

    n, k = 128256, 4096
    wq = S.quantized_matrix(4, n, k, 14)
    x = S.activations(5, 1, k)
    xt = torch.from_numpy(x).to(dev)
    full = lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq, 14, (n, k), dev)).forward(xt)
    got = full.cpu().numpy()
    rng = np.random.default_rng(3)
    sample = np.sort(rng.choice(n, 4096, replace=False))
    wsub = np.ascontiguousarray(wq[sample])
    ref = oracle.matmul(14, x, wsub, len(sample), nthreads=8)
    absum = oracle.matmul_absum(14, x, wsub, len(sample), nthreads=8)
    assert_matmul_close(got[:, sample], ref, absum, "C3 sample")
    rows = n // 8
    for g in (0, 5, 7):
        shard = lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq[g * rows:(g + 1) * rows], 14, (rows, k), dev)).forward(xt)
        assert torch.equal(shard, full[:, g * rows:(g + 1) * rows]), g
    assert Q.device_status() == 0


@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("m", [1, 8])
def test_decode_stack_shapes_q4k(dev, oracle, n, k, m):
    """The Q4_K shapes of the decode matmul stack (q/o, k/v, gate/up, down) at M = 1 and 8 against the oracle (row sample
    for the large ones)."""
    from lloom_b200 import synthetic as S

    wq = S.quantized_matrix(1000 + n % 7, n, k, 12)
    x = S.activations(9001, m, k)
    got = run_fwd(dev, 12, wq, n, k, x)
    sample = np.sort(np.random.default_rng(n + k).choice(n, min(n, 1024), replace=False))
    wsub = np.ascontiguousarray(wq[sample])
    ref = oracle.matmul(12, x, wsub, len(sample), nthreads=8)
    absum = oracle.matmul_absum(12, x, wsub, len(sample), nthreads=8)
    assert_matmul_close(got[:, sample], ref, absum, f"stack shape n={n} k={k} m={m}")


@pytest.mark.parametrize("dt,n,k,m", [(8, 128, 128, 128), (8, 130, 256, 9), (8, 300, 1024, 64), (8, 8192, 2048, 512),
                                      (8, 77, 2048, 200), (14, 128, 256, 128), (14, 130, 512, 9), (14, 300, 1024, 64),
                                      (14, 2004, 4096, 512), (14, 77, 2048, 200), (8, 64, 192, 40),
                                      (14, 2004, 4096, 100), (14, 300, 4096, 700), (14, 1100, 2048, 129),
                                      (13, 128, 256, 128), (13, 300, 1024, 64), (13, 2004, 4096, 200), (2, 130, 256, 9),
                                      (2, 300, 1024, 64), (2, 1030, 2048, 200), (6, 130, 256, 9), (6, 300, 1024, 64),
                                      (6, 1030, 2048, 200), (2, 64, 192, 40)])
def test_gemm_q8_0_q6k_tensor_core_path(dev, oracle, dt, n, k, m):
    """Prefill GEMM (m > 8) on the tcgen05 kernels for the formats beside Q4_K -- Q8_0, Q4_0, Q5_0 (one frame), Q6_K,
    Q5_K (Q4_K's frame): ragged tiles in both directions, one to many drain groups, several CTAs at once; Q6_K with
    128-row (m <= 128) and 256-row activation tiles; (the 32-element-block formats with k not a multiple of 128 run as
    slabs of the GEMV)."""
    from lloom_b200 import quantized as Q

    _, x, wq = make_case(oracle, dt, n, k, m, seed=dt + n + k + m)
    ref = oracle.matmul(dt, x, wq, n, nthreads=8)
    absum = oracle.matmul_absum(dt, x, wq, n, nthreads=8)
    got = run_fwd(dev, dt, wq, n, k, x)
    assert_matmul_close(got, ref, absum, f"{DT_NAMES[dt]} gemm n={n} k={k} m={m}")
    assert run_fwd(dev, dt, wq, n, k, x).tobytes() == got.tobytes()  # run-to-run bit-stable
    assert Q.device_status() == 0


@pytest.mark.parametrize("dt,n,k,m", [(12, 520, 2048, 70), (12, 300, 1024, 300), (13, 200, 512, 9), (14, 300, 1024, 40),
                                      (14, 200, 2048, 300), (8, 300, 1024, 70), (8, 200, 1152, 300), (2, 200, 640, 40),
                                      (6, 130, 384, 9)])
def test_prefill_forward_equals_quantizer_plus_gemm(dev, oracle, dt, n, k, m):
    """The forward entry of the prefill quantizes the activations in the pass that builds the GEMM's operand images;
    the result equals the explicit route -- lloom_b200_quantize_act, then lloom_b200_gemm on the canonical blocks --
    bit for bit (Q8_K activations for the K-quants; Q8_0 activations, with k ending in the middle of a 256-element
    span, for the 32-element formats)."""
    import lloom_b200 as lb
    from lloom_b200 import quantized as Q

    _, x, wq = make_case(oracle, dt, n, k, m, seed=dt + n + m)
    x[m // 2] = 0.0  # an all-zero activation row: d = 0, codes and sums 0
    qt = lb.QTensor.from_data(wq.tobytes(), dt, (n, k), dev)
    xt = torch.from_numpy(x).to(dev)
    fwd = lb.QMatMul.from_qtensor(qt).forward(xt)
    two_step = Q.gemm(qt, Q.quantize_act(lb.GgmlDType(dt), xt), m)
    assert torch.equal(fwd, two_step)
    assert Q.device_status() == 0


@pytest.mark.parametrize("dt", [8, 12, 14, 13, 2, 6])
def test_prefill_image_same_bits(dev, oracle, dt):
    """A forward with the prebuilt weight image equals the per-call expansion bit for bit (m > 8), and decode batches
    ignore the image."""
    import lloom_b200 as lb

    n, k = 520, 2048
    _, x, wq = make_case(oracle, dt, n, k, 70, seed=dt)
    qt = lb.QTensor.from_data(wq.tobytes(), dt, (n, k), dev)
    mm = lb.QMatMul.from_qtensor(qt)
    xt = torch.from_numpy(x).to(dev)
    plain, plain8 = mm.forward(xt), mm.forward(xt[:8])
    assert qt.storage.build_prefill_image(qt.shape)
    assert torch.equal(mm.forward(xt), plain) and torch.equal(mm.forward(xt[:8]), plain8)


@pytest.mark.parametrize("dt,k", [(12, 4096), (14, 1024), (8, 2048), (13, 2048), (2, 1024), (6, 2048)])
@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_grouped_forward_same_bits(dev, oracle, dt, k, m):
    """lloom_b200_qmatmul_fwd_group (gate|up, q|k|v behind one activation read): each matrix's rows equal its own
    forward bit for bit, with and without launch overlap, plain and with the store blocks."""
    import lloom_b200 as lb
    from lloom_b200 import _lib
    from lloom_b200 import quantized as Q

    ns = (1030, 257, 520)
    mats = []
    for i, n in enumerate(ns):
        _, _, wq = make_case(oracle, dt, n, k, 1, seed=dt + 10 * i)
        mats.append(lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq.tobytes(), dt, (n, k), dev)))
    xt = torch.from_numpy(np.random.default_rng(m).standard_normal((m, k)).astype(np.float32)).to(dev)
    want = [mm.forward(xt) for mm in mats]
    for overlap in (0, 1):
        prev = _lib.lib().lloom_b200_set_launch_overlap(overlap)
        try:
            got = Q.forward_group(mats, xt)
            for g, w in zip(got, want):
                assert torch.equal(g, w)
            got2 = Q.forward_group(mats[:2], xt)
            assert torch.equal(got2[0], want[0]) and torch.equal(got2[1], want[1])
            # SwiGLU through the group: silu on the first, multiply-into on a copy of it afterwards
            gate = Q.forward_group(mats[:1], xt, stores=[1])[0]
            assert torch.equal(gate, mats[0].forward_silu(xt))
        finally:
            _lib.lib().lloom_b200_set_launch_overlap(prev)
    assert Q.device_status() == 0


def test_bounded_wait_runs_out_and_context_survives(dev, oracle):
    """A device-side wait that nothing satisfies: the peer wait on a flag array whose second slot is never published.
    With the limit lowered to 50 ms the kernel returns by itself, the status word reads LLOOM_ERR_TIMEOUT once and
    then 0 again, and a forward launched afterwards is still correct.  Nothing faults and nothing hangs."""
    import ctypes as C
    import time

    from lloom_b200 import _lib
    from lloom_b200 import quantized as Q

    L = _lib.lib()
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert Q.device_status() == 0
    Q.set_wait_limit_ns(50_000_000)
    try:
        flags = torch.zeros(16, dtype=torch.int32, device=dev)
        flags[8] = 1   # this GPU's own call counter: one gather published ...
        flags[0] = 1   # ... its own slot has arrived, slot 1 (a peer that does not exist) never will
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        assert L.lloom_b200_peer_wait(2, flags.data_ptr(), stream) == _lib.OK
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert 0.03 < waited < 1.5, waited
        assert Q.device_status() == _lib.ERR_TIMEOUT
        assert Q.device_status() == 0  # read-and-clear
        # the barrier kernel's wait, same way: rank 0 of 2 on two local flag arrays, slot 1 never published
        fl = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(2)]
        ptrs = (C.c_void_p * 2)(fl[0].data_ptr(), fl[1].data_ptr())
        assert L.lloom_b200_peer_barrier(0, 2, ptrs, stream) == _lib.OK
        torch.cuda.synchronize()
        assert Q.device_status() == _lib.ERR_TIMEOUT
    finally:
        Q.set_wait_limit_ns(0)
    # the context is intact: an ordinary forward still matches the oracle
    _, x, wq = make_case(oracle, 12, 300, 1024, 3, seed=77)
    got = run_fwd(dev, 12, wq, 300, 1024, x)
    assert_matmul_close(got, oracle.matmul(12, x, wq, 300), oracle.matmul_absum(12, x, wq, 300), "after time-out")
    assert Q.device_status() == 0


def test_abi_from_several_host_threads(dev, oracle):
    """QTensor is shared across threads in the reference (Arc): forwards issued from several host threads, each on its
    own stream with its own workspace, all give the single-threaded bits."""
    import threading

    import lloom_b200 as lb

    cases = [(12, 777, 2048, 1), (14, 300, 1024, 4), (8, 515, 2048, 2), (12, 260, 1024, 40)]
    mats, xs, want = [], [], []
    for dt, n, k, m in cases:
        _, x, wq = make_case(oracle, dt, n, k, m, seed=dt + m)
        mats.append(lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq.tobytes(), dt, (n, k), dev)))
        xs.append(torch.from_numpy(x).to(dev))
        want.append(mats[-1].forward(xs[-1]).cpu())
    torch.cuda.synchronize()
    errors = []

    def worker(tid):
        try:
            st = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(st):
                for rep in range(20):
                    i = (tid + rep) % len(cases)
                    y = mats[i].forward(xs[i])
                    st.synchronize()
                    if not torch.equal(y.cpu(), want[i]):
                        errors.append((tid, rep, i))
        except Exception as e:  # noqa: BLE001
            errors.append((tid, repr(e)))

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:4]


def test_second_device_in_one_process(oracle):
    """Per-device launch configuration: a prefill GEMM and a decode GEMV on cuda:1 after the process has already run
    them on cuda:0 (the shared-memory opt-in of a kernel is per device)."""
    import lloom_b200 as lb

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _, x, wq = make_case(oracle, 12, 384, 1024, 40, seed=5)
    outs = []
    for d in (0, 1):
        dv = torch.device("cuda", d)
        mm = lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq.tobytes(), 12, (384, 1024), dv))
        xt = torch.from_numpy(x).to(dv)
        outs.append((mm.forward(xt).cpu(), mm.forward(xt[:1]).cpu()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("dt,n,k", [(12, 300, 1024), (14, 130, 512), (8, 257, 512), (13, 96, 2048), (12, 64, 14336)])
def test_indexed_moe_forward(dev, oracle, dt, n, k):
    """QTensor::indexed_moe_forward (mod.rs:1539-1650, cuda.rs:505-622): every (token, expert) product equals the plain
    forward of that expert's matrix on that row bit for bit, matches the oracle within tolerance, and stays close to
    the reference CPU arm's dequantize-and-dot (which does not quantize the activations)."""
    import lloom_b200 as lb
    from lloom_b200 import _lib
    from lloom_b200 import quantized as Q

    n_experts, batch, topk = 6, 3, 4
    rng = np.random.default_rng(dt + n)
    w = rng.standard_normal((n_experts, n, k)).astype(np.float32) * np.float32(0.02)
    wq = oracle.quantize(dt, w.reshape(n_experts * n, k), nthreads=8)
    rb = wq.shape[1]
    stacked = lb.QTensor.from_data(wq.tobytes(), dt, (n_experts, n, k), dev)
    experts = [lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq[e * n:(e + 1) * n].tobytes(), dt, (n, k), dev)) for e in range(n_experts)]
    ids_np = np.stack([rng.permutation(n_experts)[:topk] for _ in range(batch)]).astype(np.int64)
    ids = torch.from_numpy(ids_np).to(dev)
    for overlap in (0, 1):
        prev = _lib.lib().lloom_b200_set_launch_overlap(overlap)
        try:
            for in_dim1 in (1, topk):
                x_np = rng.standard_normal((batch, in_dim1, k)).astype(np.float32)
                x = torch.from_numpy(x_np).to(dev)
                got = stacked.indexed_moe_forward(x, ids)
                assert tuple(got.shape) == (batch, topk, n)
                got_np = got.cpu().numpy()
                dense = oracle.dequantize(dt, wq, k).reshape(n_experts, n, k).astype(np.float64)
                for b in range(batch):
                    for t in range(topk):
                        e = int(ids_np[b, t])
                        xi = 0 if in_dim1 == 1 else t
                        want = experts[e].forward(x[b, xi:xi + 1])
                        assert torch.equal(got[b, t:t + 1], want), (dt, b, t, in_dim1)
                        ref = oracle.matmul(dt, x_np[b, xi:xi + 1], wq[e * n:(e + 1) * n], n)
                        absum = oracle.matmul_absum(dt, x_np[b, xi:xi + 1], wq[e * n:(e + 1) * n], n)
                        assert_matmul_close(got_np[b, t:t + 1], ref, absum, f"moe {DT_NAMES[dt]} b={b} t={t}")
                        cpu_arm = dense[e] @ x_np[b, xi].astype(np.float64)
                        scale = np.abs(dense[e]) @ np.abs(x_np[b, xi].astype(np.float64))
                        assert (np.abs(got_np[b, t] - cpu_arm) <= 2e-2 * scale).all()
        finally:
            _lib.lib().lloom_b200_set_launch_overlap(prev)
    assert Q.device_status() == 0
    # an expert id past the stack is clamped and reported through the status word
    bad = ids.clone()
    bad[0, 0] = n_experts + 3
    stacked.indexed_moe_forward(torch.from_numpy(rng.standard_normal((batch, 1, k)).astype(np.float32)).to(dev), bad)
    torch.cuda.synchronize()
    assert Q.device_status() == _lib.ERR_SHAPE
    with pytest.raises(lb.LloomError):
        stacked.indexed_moe_forward(torch.zeros(batch, 2, k, device=dev), ids)
