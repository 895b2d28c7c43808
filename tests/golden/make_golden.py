"""Writes tests/golden/qmatmul_small.npz: small seeded cases of the hot path computed by the CPU oracle.

The reference itself (Rust) cannot be built in this environment, so these vectors come from the C
restatement in oracle/, which tests/test_oracle_golden.py pins to the reference's own literal test
values (reference_pins.json).  Each case stores the f32 weights and activations, the packed weight
blocks, the quantized activation blocks and the f32 outputs in the AVX2 arm's summation order.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

CASES = [  # (dtype, n, k, m, seed)
    (O.Q8_0, 9, 256, 1, 11), (O.Q8_0, 65, 768, 3, 12), (O.Q8_0, 33, 2048, 8, 13),
    (O.Q4_K, 9, 256, 1, 21), (O.Q4_K, 65, 768, 3, 22), (O.Q4_K, 33, 2048, 8, 23), (O.Q4_K, 130, 512, 70, 24),
    (O.Q6_K, 9, 256, 1, 31), (O.Q6_K, 65, 768, 3, 32), (O.Q6_K, 33, 2048, 8, 33), (O.Q6_K, 130, 512, 70, 34),
    (O.Q8_0, 130, 512, 70, 14),
    (O.Q4_0, 9, 256, 1, 41), (O.Q4_0, 33, 2048, 8, 42), (O.Q5_0, 9, 256, 1, 51), (O.Q5_0, 33, 2048, 8, 52),
    (O.Q5_K, 9, 256, 1, 61), (O.Q5_K, 65, 768, 3, 62), (O.Q5_K, 33, 2048, 8, 63),
]


def main():
    out = {}
    for dt, n, k, m, seed in CASES:
        rng = np.random.default_rng(seed)
        w = rng.standard_normal((n, k)).astype(np.float32) * np.float32(0.02)
        x = rng.standard_normal((m, k)).astype(np.float32)
        key = f"dt{dt}_n{n}_k{k}_m{m}"
        wq = O.quantize(dt, w)
        out[key + "_meta"] = np.array([dt, n, k, m], dtype=np.int64)
        out[key + "_w"] = w
        out[key + "_x"] = x
        out[key + "_wq"] = wq
        out[key + "_aq"] = O.quantize_act(dt, x)
        out[key + "_y"] = O.matmul(dt, x, wq, n, order=O.ORDER_AVX2_EMU)
        out[key + "_absum"] = O.matmul_absum(dt, x, wq, n)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qmatmul_small.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
