"""Times the Linear kernels (include/linear_sm100.h) on one B200 against the library GEMM the
reference uses for the same layers (cuBLAS in TF32 tensor-op math, here through torch.addmm /
torch.matmul with TF32 allowed), for the Linear shapes of GPT-2 124M at B=8, T=1024.

    python gpt.c_b200/bench_linear.py [--steps 30] [--cold] [--shape M,N,K] [--only fwd|dx|dw]

Prints one JSON line per shape: microseconds and algorithmic TFLOP/s (2*M*N*K per product) of
forward (with and without the fused bf16 planes), backward (dx + dW + db) and its two products
alone, next to the cuBLAS time of the same product.  Inputs stay resident; --cold writes a 512 MB
buffer between launches so that every launch starts with a cold L2 (default: warm, back to back).
--shape times one other shape instead (e.g. 8192,50257,768, the vocabulary projection; the planes
variant is skipped when N is not a multiple of 8); --only fwd|dx|dw launches nothing but that product
(for a profiler capture).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [  # name, M, N (out_features), K (in_features)
    ("qkv", 8192, 2304, 768),
    ("attn c_proj", 8192, 768, 768),
    ("mlp c_fc", 8192, 3072, 768),
    ("mlp c_proj", 8192, 768, 3072),
]


def main() -> None:
    import torch

    import __graft_entry__ as entry

    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--cold", action="store_true")
    ap.add_argument("--shape", default=None, metavar="M,N,K")
    ap.add_argument("--only", default=None, choices=["fwd", "dx", "dw"])
    args = ap.parse_args()

    pkg = entry.load_package()
    pkg.init()
    torch.backends.cuda.matmul.allow_tf32 = True
    flush = torch.empty(512 << 20, device="cuda", dtype=torch.uint8) if args.cold else None

    def timed(fn) -> float:
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        if flush is None:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                fn()
            b.record()
            torch.cuda.synchronize()
            total = a.elapsed_time(b)
        else:
            for _ in range(args.steps):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                total += a.elapsed_time(b)
        return total / args.steps * 1e3  # microseconds

    shapes = SHAPES
    if args.shape:
        m, n, k = (int(v) for v in args.shape.split(","))
        shapes = [("custom", m, n, k)]
    for name, M, N, K in shapes:
        x = torch.randn(M, K, device="cuda")
        w = torch.randn(N, K, device="cuda") * 0.05
        b = torch.randn(N, device="cuda")
        dy = torch.randn(M, N, device="cuda")
        dw = torch.zeros(N, K, device="cuda")
        db = torch.zeros(N, device="cuda")
        fl = 2.0 * M * N * K
        if args.only:
            one = {"fwd": lambda: pkg.linear_forward(x, w, b),
                   "dx": lambda: pkg.linear_backward(dy, x, w, None, None),
                   "dw": lambda: pkg.linear_backward(dy, x, w, dw, None, want_dx=False)}[args.only]
            t_us = timed(one)
            print(json.dumps({"layer": name, "M": M, "N": N, "K": K, "us": {args.only: round(t_us, 1)},
                              "tflops": {args.only: round(fl / t_us / 1e6, 1)}, "status": pkg.device_status()}), flush=True)
            continue
        planes = torch.empty(4 * M * N + 512, device="cuda", dtype=torch.uint8) if N % 8 == 0 else None

        def cublas_bwd():
            _ = dy @ w
            dw.addmm_(dy.t(), x)
            db.add_(dy.sum(0))

        us = {
            "fwd": timed(lambda: pkg.linear_forward(x, w, b)),
            "fwd_with_planes": timed(lambda: pkg.linear_forward(x, w, b, planes=planes)) if planes is not None else None,
            "fwd_cublas_tf32": timed(lambda: torch.addmm(b, x, w.t())),
            "bwd": timed(lambda: pkg.linear_backward(dy, x, w, dw, db)),
            "bwd_cublas_tf32": timed(cublas_bwd),
            "dx": timed(lambda: pkg.linear_backward(dy, x, w, None, None)),
            "dx_cublas_tf32": timed(lambda: dy @ w),
            "dw": timed(lambda: pkg.linear_backward(dy, x, w, dw, None, want_dx=False)),
            "dw_cublas_tf32": timed(lambda: dw.addmm_(dy.t(), x)),
        }
        status = pkg.device_status()
        if status != 0:
            raise SystemExit(f"kernel status word {status}")
        line = {"layer": name, "M": M, "N": N, "K": K, "l2": "cold" if args.cold else "warm",
                "us": {k: round(v, 1) for k, v in us.items() if v is not None},
                "tflops": {k: round((fl if k.startswith(("fwd", "dx", "dw")) else 2 * fl) / v / 1e6, 1)
                           for k, v in us.items() if v is not None}}
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
