"""Generate the golden fixtures in this directory from the reference implementation itself.

Run in a container that has the reference checkout (it is a Python/Triton package; its kernels
execute on the CPU under the Triton interpreter):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/RzLinear/python

The fixtures pin the CPU oracle (and, through it and directly, the CUDA kernels) to outputs of
the reference's own kernels:
  * random numbers produced by RzLinear._generate_random_numbers for a few seeds,
  * rz_linear_idx_tl (single-level hash, small prime) on a seeded hashed array,
  * rz_linear_forward_tl / rz_linear_backward_input_grad_tl / rz_linear_backward_weight_grad_tl
    (the two-level hash the reference's kernels execute) on seeded inputs, full and ragged shapes,
  * one RzLinear module forward+backward with bias and a 3-D input.
Everything is stored as float32/int64 in one compressed .npz per case.
"""
import argparse
import contextlib
import io
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout's python/ directory")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from rz_linear import RzLinear
    from rz_linear.impl.RzLinearIdx import rz_linear_idx_tl
    from rz_linear.impl.RzLinearForward import rz_linear_forward_tl
    from rz_linear.impl.RzLinearBackward import (rz_linear_backward_input_grad_tl,
                                                 rz_linear_backward_weight_grad_tl)

    def quiet_module(*a, **kw):
        with contextlib.redirect_stdout(io.StringIO()):
            return RzLinear(*a, **kw)

    # ---- random numbers -------------------------------------------------------------------
    seeds = [1024, 7, 0, 123456]
    rn = {}
    for s in seeds:
        rn[str(s)] = quiet_module(input_dim=64, output_dim=64, seed=s, compress_ratio=1.0
                                  )._random_numbers.numpy().astype(np.int64)
    np.savez_compressed(os.path.join(HERE, "random_numbers.npz"), **rn)

    # ---- single-level index kernel -------------------------------------------------------
    g = torch.Generator().manual_seed(11)
    for tag, (K, N, H, BK, BN, seed) in {
        "idx_a": (128, 256, 9001, 32, 64, 1024),
        "idx_b": (64, 128, 2500, 16, 128, 7),
    }.items():
        R = rn[str(seed)]
        h = torch.rand(H, generator=g, dtype=torch.float32)
        W = rz_linear_idx_tl(h, K, N, H, int(R[3]), int(R[2]), int(R[1]), int(R[0]), BK, BN)
        np.savez_compressed(os.path.join(HERE, tag + ".npz"), hashed=h.numpy(), W=W.numpy(), R=R,
                            dims=np.array([K, N, H, BK, BN], dtype=np.int64))

    # ---- the three kernels, two-level hash ----------------------------------------------
    cases = {
        #        M    K    N    H     BM  BK  BN  seed  init_factor
        "k_full":   (96, 128, 192, 8192, 32, 32, 64, 1024, 1.0),
        "k_ragged": (50, 80, 100, 4099, 32, 32, 64, 7, 0.5),
        "k_small_tiles": (40, 64, 96, 3000, 16, 16, 32, 123456, 2.0),
    }
    for tag, (M, K, N, H, BM, BK, BN, seed, alpha) in cases.items():
        R = [int(v) for v in rn[str(seed)]]
        g = torch.Generator().manual_seed(1000 + M)
        X = torch.randn(M, K, generator=g)
        dY = torch.randn(M, N, generator=g)
        h = (torch.rand(H, generator=g) - 0.5) * 0.25
        kw = dict(allow_tf32=False, allow_autotune=False, BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN,
                  BLOCK_SIZE_K=BK, GROUP_SIZE=1)
        Rargs = (R[7], R[6], R[5], R[4], R[3], R[2], R[1], R[0])
        Y = rz_linear_forward_tl(X, h, alpha, M, K, N, H, *Rargs, **kw)
        dX = rz_linear_backward_input_grad_tl(dY, h, alpha, M, K, N, H, *Rargs, **kw)
        dH = rz_linear_backward_weight_grad_tl(X, dY, alpha, M, K, N, H, *Rargs, **kw)
        np.savez_compressed(os.path.join(HERE, tag + ".npz"), X=X.numpy(), dY=dY.numpy(), hashed=h.numpy(),
                            Y=Y.numpy(), dX=dX.numpy(), dH=dH.numpy(), R=np.array(R, dtype=np.int64),
                            dims=np.array([M, K, N, H, BK, BN], dtype=np.int64),
                            alpha=np.array(alpha, dtype=np.float64))

    # ---- module forward + backward (default tiles 32 x 64, bias, 3-D input) ------------
    rz = quiet_module(input_dim=64, output_dim=128, seed=1024, compress_ratio=0.75, init_factor=0.125)
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        rz._hashed_weight.copy_((torch.rand(rz._hashed_weight.shape, generator=g) - 0.5))
        rz._bias.copy_(torch.randn(128, generator=g))
    x = torch.randn(3, 10, 64, generator=g, requires_grad=True)
    gy = torch.randn(3, 10, 128, generator=g)
    y = rz(x)
    y.backward(gy)
    np.savez_compressed(os.path.join(HERE, "module.npz"), x=x.detach().numpy(), gy=gy.numpy(),
                        hashed=rz._hashed_weight.detach().numpy(), bias=rz._bias.detach().numpy(),
                        y=y.detach().numpy(), dx=x.grad.numpy(), dh=rz._hashed_weight.grad.numpy(),
                        dbias=rz._bias.grad.numpy(), R=rz._random_numbers.numpy().astype(np.int64),
                        alpha=np.array(0.125))
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
