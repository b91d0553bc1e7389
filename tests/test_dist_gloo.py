"""World-size-2 check of the data-parallel step's host logic on CPU (gloo): sharding, the single
all-reduce, the SGD update.  The CUDA kernels are replaced by the CPU oracle here, which is what
the oracle is for; the shipped step never does that."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import rz_oracle as o
from rzlinear_b200.dist import RzDataParallelStep, shard_rows

M, K, N, H, BK, BN = 48, 64, 96, 3000, 16, 32
R = [2038074743, 12345, 6789, 1357, 0, 0, 0, 0]
LR = 0.05


class OracleKernels:
    def refresh(self, hashed):
        pass

    def forward(self, x, hashed, y):
        y.copy_(torch.from_numpy(o.forward(x.numpy(), hashed.numpy(), N, BK, BN, R, 0)).to(y.dtype))

    def backward_input(self, dy, hashed, dx):
        dx.copy_(torch.from_numpy(o.backward_input(dy.numpy(), hashed.numpy(), K, BK, BN, R, 0)).to(dx.dtype))

    def backward_weight(self, x, dy, dh):
        dh.copy_(torch.from_numpy(o.backward_weight(x.numpy(), dy.numpy(), H, BK, BN, R, 0)).to(dh.dtype))

    def sgd(self, hashed, dh, lr, velocity=None, momentum=0.0):
        if velocity is not None:
            velocity.mul_(momentum).add_(dh)
            dh = velocity
        hashed.sub_(lr * dh)


def _inputs():
    g = torch.Generator().manual_seed(0)
    return torch.randn(M, K, generator=g), torch.randn(M, N, generator=g), torch.rand(H, generator=g) - 0.5


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    X, dY, h = _inputs()
    lo, hi = shard_rows(M, rank, world)
    step = RzDataParallelStep(hi - lo, K, N, H, BK, BN, R, 0, torch.float32, LR, device="cpu", allow_tf32=False,
                              kernels=OracleKernels())
    step.load_weights(h)
    step.step(X[lo:hi].contiguous(), dY[lo:hi].contiguous())
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), h=step.hashed.numpy(), dH=step.dH.numpy(), Y=step.Y.numpy(),
             dX=step.dX.numpy(), lo=lo, hi=hi)
    dist.destroy_process_group()


def test_shard_rows_partition():
    for m, w in [(10, 4), (131072, 8), (7, 8), (48, 2)]:
        spans = [shard_rows(m, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == m
        assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))


def test_two_rank_step_equals_full_batch(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    X, dY, h = _inputs()
    dH_full = o.backward_weight(X.numpy(), dY.numpy(), H, BK, BN, R, 0)
    h_full = h.numpy().astype(np.float64) - LR * dH_full
    Y_full = o.forward(X.numpy(), h.numpy(), N, BK, BN, R, 0)
    dX_full = o.backward_input(dY.numpy(), h.numpy(), K, BK, BN, R, 0)
    outs = [np.load(tmp_path / f"r{r}.npz") for r in range(2)]
    assert np.array_equal(outs[0]["h"], outs[1]["h"])          # replicas stay identical
    assert np.array_equal(outs[0]["dH"], outs[1]["dH"])
    assert o.rel_l2(outs[0]["dH"], dH_full) < 1e-6
    assert o.rel_l2(outs[0]["h"], h_full) < 1e-6
    for r in range(2):
        lo, hi = int(outs[r]["lo"]), int(outs[r]["hi"])
        assert o.rel_l2(outs[r]["Y"], Y_full[lo:hi]) < 1e-6
        assert o.rel_l2(outs[r]["dX"], dX_full[lo:hi]) < 1e-6
