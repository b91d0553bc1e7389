"""Per-kernel throughput on the shapes the reference's own benchmark sweeps, next to cuBLAS.

Mirrors python/bench/bench.py of apd10/RzLinear: (M, K, N) in {32, 128, 1024} x {1024, 10240}, forward,
hashed-weight gradient and input gradient, TFLOPS = 2*M*N*K / time, `torch.matmul` on a dense weight of
the same shape as the comparison line; once with tf32 tensor cores allowed and once in fp32.

    python -m rzlinear_b200.bench_shapes [--dtype fp32|tf32|bf16] [--reps 20]
    python -m rzlinear_b200.bench_shapes --baseline          # the single-layer and MLP baseline configurations
    python -m rzlinear_b200.bench_shapes --dtype bf16 --shape 128,10240,10240 [--hashed H --block BK,BN]

The hash tile defaults to the reference's 32 x 64 in every precision.

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


# Single-layer baseline configurations: (precision, M, K, N, H, BK, BN)
BASELINE = [("fp32", 1024, 1024, 1024, 65536, 32, 32),
            ("tf32", 16384, 4096, 4096, 1 << 20, 64, 64),
            ("bf16", 8192, 8192, 32768, 1 << 22, 128, 128)]


def _time_graph(fn, reps):
    """fn captured once in a CUDA graph, then replayed: the figure without per-launch host time."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()                      # first-use set-up happens outside the capture
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return _time(g.replay, reps)


def measure(precision: str, M: int, K: int, N: int, H: int, block_k: int, block_n: int, reps: int, device="cuda:0",
            graph: bool = False) -> dict:
    """forward / hashed-weight gradient / input gradient of one shape through the C ABI, and torch.matmul on a dense
    weight of the same shape (the reference's comparison line, python/bench/bench.py:40-42,78-79,120-121)."""
    dev = torch.device(device)
    dtype = torch.bfloat16 if precision == "bf16" else torch.float32
    prec = {"fp32": _lib.PREC_FP32, "tf32": _lib.PREC_TF32, "bf16": _lib.PREC_BF16}[precision]
    was_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = precision == "tf32"
    try:
        R = [PRIME] + [int(v) for v in np.random.RandomState(0).randint(1, 2**31 - 1, 7)]
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
        graphed = None
        if graph:   # launch-bound problems: the three products back to back as one CUDA graph, ours and cuBLAS
            def ours_all():
                _lib.forward(pb, X, h, shadow, None, Y)
                _lib.backward_weight(pb, X, dY, dH)
                _lib.backward_input(pb, dY, h, shadow, dX)

            def dense_all():
                torch.matmul(X, W, out=Y)
                torch.matmul(X.t(), dY, out=dW)
                torch.matmul(dY, W.t(), out=dX)

            g_ours, g_dense = _time_graph(ours_all, 5 * reps), _time_graph(dense_all, 5 * reps)
            graphed = {"fwd_bwd_tflops": round(6.0 * M * N * K * 1e-12 / (g_ours * 1e-3), 2),
                       "cublas_fwd_bwd_tflops": round(6.0 * M * N * K * 1e-12 / (g_dense * 1e-3), 2),
                       "pct_of_cublas": round(100.0 * g_dense / g_ours, 1),
                       "what": "forward + weight gradient + input gradient captured in one CUDA graph and replayed"}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = was_tf32
    tflops = {k: 2.0 * M * N * K * 1e-12 / (v * 1e-3) for k, v in ms.items()}
    ours = ms["forward"] + ms["backward_weight"] + ms["backward_input"]
    dense = ms["cublas_forward"] + ms["cublas_backward_weight"] + ms["cublas_backward_input"]
    return {"precision": precision, "M": M, "K": K, "N": N, "H": H, "block": [block_k, block_n],
            "path": "tcgen05" if _lib.plan(pb, 0) == _lib.PATH_TCGEN05 else "fma",
            "tflops": {k: round(v, 2) for k, v in tflops.items()},
            "fwd_bwd_tflops": round(6.0 * M * N * K * 1e-12 / (ours * 1e-3), 2),
            "pct_of_cublas": round(100.0 * dense / ours, 1), **({"cuda_graph": graphed} if graphed else {})}


def run(precision: str, reps: int, block_k: int = 32, block_n: int = 64, device="cuda:0", shapes=None, hashed=None):
    for (M, K, N) in (shapes or CONFIGS):
        H = hashed or int(K * N * 0.0625)           # default: the reference's default compress_ratio
        print(json.dumps(measure(precision, M, K, N, H, block_k, block_n, reps, device)), flush=True)


def measure_mlp(reps: int, batch: int = 65536, dims=(1024, 4096, 4096, 256), hashed: int = 1 << 18, device="cuda:0") -> dict:
    """Full training step (forward, MSE loss, backward) of the 3-layer ReLU MLP baseline configuration in bf16,
    next to the same MLP built from dense torch.nn.Linear layers (cuBLAS).  The input needs no gradient, so the
    step runs 3 forward, 3 weight-gradient and 2 input-gradient products."""
    from .RzLinear import RzLinear
    dev = torch.device(device)
    torch.manual_seed(4)
    rs = np.random.RandomState(4)
    ours = torch.nn.ModuleList([
        RzLinear(dims[i], dims[i + 1], hashed_weight=torch.nn.Parameter((torch.rand(hashed) * 2 - 1) / dims[i] ** 0.5),
                 hash_mode="single", random_numbers=[PRIME] + [int(v) for v in rs.randint(1, 2**31 - 1, 3)] + [0, 0, 0, 0],
                 block_size_k=64, block_size_n=64, relu=(i < 2)) for i in range(3)]).to(dev)
    dense = torch.nn.ModuleList([torch.nn.Linear(dims[i], dims[i + 1]) for i in range(3)]).to(dev).to(torch.bfloat16)
    x = torch.randn(batch, dims[0], device=dev).to(torch.bfloat16)
    target = torch.randn(batch, dims[-1], device=dev).to(torch.bfloat16)

    def step_ours():
        y = x
        for layer in ours:
            y = layer(y)
        torch.nn.functional.mse_loss(y.float(), target.float()).backward()

    def step_dense():
        y = x
        for i, layer in enumerate(dense):
            y = layer(y)
            if i < 2:
                y = torch.relu(y)
        torch.nn.functional.mse_loss(y.float(), target.float()).backward()

    flops = 2.0 * batch * (3 * sum(dims[i] * dims[i + 1] for i in range(3)) - dims[0] * dims[1])
    ms = {"rz_mlp_step": _time(step_ours, reps), "dense_mlp_step": _time(step_dense, reps)}
    return {"config": "mlp", "batch": batch, "dims": list(dims), "H": hashed, "ms": {k: round(v, 3) for k, v in ms.items()},
            "tflops": {k: round(flops * 1e-12 / (v * 1e-3), 1) for k, v in ms.items()},
            "pct_of_dense": round(100.0 * ms["dense_mlp_step"] / ms["rz_mlp_step"], 1)}


def run_mlp(reps: int, **kw):
    print(json.dumps(measure_mlp(reps, **kw)), flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="all", choices=["all", "fp32", "tf32", "bf16"])
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--baseline", action="store_true", help="run the baseline configurations instead of the sweep")
    ap.add_argument("--shape", default=None, help="M,K,N: one shape instead of the sweep")
    ap.add_argument("--hashed", type=int, default=None, help="length of the hashed array (default K*N/16)")
    ap.add_argument("--block", default=None, help="BK,BN hash tile (default 32,64)")
    a = ap.parse_args()
    if a.baseline:
        for (prec, M, K, N, H, bk, bn) in BASELINE:
            run(prec, a.reps, bk, bn, shapes=[(M, K, N)], hashed=H)
        run_mlp(a.reps)
    else:
        shapes = [tuple(int(v) for v in a.shape.split(","))] if a.shape else None
        bk, bn = (int(v) for v in a.block.split(",")) if a.block else (32, 64)
        for p in (["tf32", "fp32", "bf16"] if a.dtype == "all" else [a.dtype]):
            run(p, a.reps, bk, bn, shapes=shapes, hashed=a.hashed)
