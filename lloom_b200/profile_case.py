"""Small, bounded cases of the hot path for profilers (``python -m lloom_b200.profile_case ...``).

A profiler that replays every captured launch many times needs a case that ends by itself in seconds and holds
little device memory: a handful of ``QMatMul::forward`` calls on seeded synthetic weights, rotating over a few
distinct copies of the matrix so that the weights of a launch are not already in L2.  The ncu summaries under
``profiles/`` name the exact command line used.

Examples:
    python -m lloom_b200.profile_case --dtype 12 --n 14336 --k 4096 --m 1 --copies 5 --calls 12
    python -m lloom_b200.profile_case --dtype 12 --n 14336 --k 4096 --m 2048 --copies 2 --calls 3 --image
    python -m lloom_b200.profile_case --dtype 12 --n 14336 --k 4096 --m 1 --copies 8 --calls 4 --group 4
"""
from __future__ import annotations

import argparse

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dtype", type=int, default=12, help="GGUF type id of the weights (2, 6, 8, 12, 13, 14)")
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--m", type=int, default=1, help="activation rows (<= 8: decode GEMV, else prefill GEMM)")
    ap.add_argument("--copies", type=int, default=5, help="distinct device copies of the matrix")
    ap.add_argument("--calls", type=int, default=12, help="forwards to issue, rotating over the copies")
    ap.add_argument("--group", type=int, default=1, help="matrices per grouped launch (1: one forward per matrix)")
    ap.add_argument("--image", action="store_true", help="prebuild the prefill weight image (m > 8)")
    ap.add_argument("--no-overlap", action="store_true", help="leave programmatic launch overlap off")
    args = ap.parse_args()

    import torch

    import lloom_b200 as lb
    from lloom_b200 import _lib
    from lloom_b200 import quantized as Q
    from lloom_b200 import synthetic as S

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    _lib.lib().lloom_b200_set_launch_overlap(0 if args.no_overlap else 1)
    wq = S.quantized_matrix(2, args.n, args.k, args.dtype)
    mats = [lb.QMatMul.from_qtensor(lb.QTensor.from_data(wq, args.dtype, (args.n, args.k), dev)) for _ in range(args.copies)]
    if args.image:
        for mm in mats:
            mm.qtensor.storage.build_prefill_image(mm.qtensor.shape)
    x = torch.from_numpy(S.activations(3, args.m, args.k)).to(dev)
    outs = [torch.empty(args.m, args.n, dtype=torch.float32, device=dev) for _ in range(args.copies)]
    torch.cuda.synchronize()
    for c in range(args.calls):
        i = (c * args.group) % args.copies
        if args.group > 1:
            idx = [(i + j) % args.copies for j in range(args.group)]
            Q.forward_group([mats[j] for j in idx], x, outs=[outs[j] for j in idx])
        else:
            mats[i].qtensor.storage.fwd((args.n, args.k), x, out=outs[i])
    torch.cuda.synchronize()
    status = Q.device_status()
    print(f"profile_case ok: {args.calls} calls, device status {status}, checksum {float(np.float64(outs[0].double().sum().item())):.6e}")
    if status != 0:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
