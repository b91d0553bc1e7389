"""Per-kernel throughput on the shapes the reference's own benchmark sweeps, next to cuBLAS.

Mirrors python/bench/bench.py of apd10/RzLinear: (M, K, N) in {32, 128, 1024} x {1024, 10240}, forward,
hashed-weight gradient and input gradient, TFLOPS = 2*M*N*K / time, `torch.matmul` on a dense weight of
the same shape as the comparison line; once with tf32 tensor cores allowed and once in fp32.

    python -m rzlinear_b200.bench_shapes [--dtype fp32|tf32|bf16] [--reps 20]

Prints one JSON line per shape and precision.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from . import _lib

CONFIGS = [(32, 1024, 1024), (32, 10240, 10240), (128, 1024, 1024),
           (128, 10240, 10240), (1024, 1024, 1024), (1024, 10240, 10240)]
PRIME = 2038074743


def _time(fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def run(precision: str, reps: int, block_k: int = 32, block_n: int = 64, device="cuda:0"):
    dev = torch.device(device)
    dtype = torch.bfloat16 if precision == "bf16" else torch.float32
    prec = {"fp32": _lib.PREC_FP32, "tf32": _lib.PREC_TF32, "bf16": _lib.PREC_BF16}[precision]
    if precision == "bf16":
        block_k = max(block_k, 64)
    torch.backends.cuda.matmul.allow_tf32 = precision == "tf32"
    R = [PRIME] + [int(v) for v in np.random.RandomState(0).randint(1, 2**31 - 1, 7)]
    for (M, K, N) in CONFIGS:
        H = int(K * N * 0.0625)                     # the reference's default compress_ratio
        pb = _lib.make_problem(M, K, N, H, block_k, block_n, R, _lib.HASH_SINGLE, _lib.torch_io_dtype(dtype), prec)
        g = torch.Generator(device=dev).manual_seed(0)
        X = torch.randn((M, K), generator=g, device=dev).to(dtype)
        dY = torch.randn((M, N), generator=g, device=dev).to(dtype)
        h = (torch.rand(H, generator=g, device=dev) * 2 - 1) / K ** 0.5
        W = torch.randn((K, N), generator=g, device=dev).to(dtype)
        nbytes = _lib.shadow_bytes(pb)
        shadow = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
        if shadow is not None:
            _lib.shadow_refresh(pb, h, shadow)
        Y = torch.empty((M, N), dtype=dtype, device=dev)
        dX = torch.empty((M, K), dtype=dtype, device=dev)
        dH = torch.empty(H, dtype=torch.float32, device=dev)
        dW = torch.empty((K, N), dtype=dtype, device=dev)
        ms = {
            "forward": _time(lambda: _lib.forward(pb, X, h, shadow, None, Y), reps),
            "backward_weight": _time(lambda: _lib.backward_weight(pb, X, dY, dH), reps),
            "backward_input": _time(lambda: _lib.backward_input(pb, dY, h, shadow, dX), reps),
            "cublas_forward": _time(lambda: torch.matmul(X, W, out=Y), reps),
            "cublas_backward_weight": _time(lambda: torch.matmul(X.t(), dY, out=dW), reps),
            "cublas_backward_input": _time(lambda: torch.matmul(dY, W.t(), out=dX), reps),
        }
        tflops = {k: 2.0 * M * N * K * 1e-12 / (v * 1e-3) for k, v in ms.items()}
        print(json.dumps({"precision": precision, "M": M, "K": K, "N": N, "H": H, "block": [block_k, block_n],
                          "path": "tcgen05" if _lib.plan(pb, 0) == _lib.PATH_TCGEN05 else "fma",
                          "tflops": {k: round(v, 2) for k, v in tflops.items()}}), flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="all", choices=["all", "fp32", "tf32", "bf16"])
    ap.add_argument("--reps", type=int, default=20)
    a = ap.parse_args()
    for p in (["tf32", "fp32", "bf16"] if a.dtype == "all" else [a.dtype]):
        run(p, a.reps)
