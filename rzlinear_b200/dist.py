"""Data-parallel training step of one RzLinear layer (batch rows sharded over ranks).

Each rank owns M_local rows of X and dY; the hashed array and the random numbers are replicated.
Forward and input gradient need no communication.  The only exchange is the sum of the
hashed-weight gradient over ranks (one all-reduce of H floats), launched right after the
weight-gradient kernel so that it overlaps the input-gradient kernel; every rank then applies the
same SGD update, so the replicas stay identical.

The reference has no distributed code; this follows its single-GPU step
(python/rz_linear/RzLinearFunction.py:14-60) per rank.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from . import _lib


class CudaKernels:
    """The C-ABI kernels (the only shipped implementation)."""

    def __init__(self, pb, device):
        self.pb = pb
        self.device = device
        nbytes = _lib.shadow_bytes(pb)
        self.shadow = torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None

    def refresh(self, hashed):
        if self.shadow is not None:
            _lib.shadow_refresh(self.pb, hashed, self.shadow)

    def forward(self, x, hashed, y):
        _lib.forward(self.pb, x, hashed, self.shadow, None, y)

    def backward_input(self, dy, hashed, dx):
        _lib.backward_input(self.pb, dy, hashed, self.shadow, dx)

    def backward_weight(self, x, dy, dh):
        _lib.backward_weight(self.pb, x, dy, dh)

    def sgd(self, hashed, dh, lr):
        _lib.sgd_step(self.pb, hashed, dh, lr, self.shadow)


def shard_rows(M_global: int, rank: int, world: int):
    """Rows [lo, hi) of the global batch owned by `rank` (contiguous blocks, remainder to the first ranks)."""
    base, rem = divmod(M_global, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class RzDataParallelStep:
    def __init__(self, M_local: int, K: int, N: int, H: int, BK: int, BN: int, R: Sequence[int],
                 hash_mode: int = _lib.HASH_SINGLE, dtype: torch.dtype = torch.bfloat16, lr: float = 1e-3,
                 device="cuda", init_factor: float = 1.0, allow_tf32: bool = True,
                 process_group: Optional[dist.ProcessGroup] = None, kernels=None):
        self.M, self.K, self.N, self.H = M_local, K, N, H
        self.device = torch.device(device)
        self.dtype = dtype
        self.lr = float(lr)
        self.group = process_group
        self.world = dist.get_world_size(process_group) if (dist.is_available() and dist.is_initialized()) else 1
        prec = _lib.PREC_BF16 if dtype == torch.bfloat16 else (_lib.PREC_TF32 if allow_tf32 else _lib.PREC_FP32)
        self.pb = _lib.make_problem(M_local, K, N, H, BK, BN, R, hash_mode, _lib.torch_io_dtype(dtype), prec,
                                    init_factor)
        self.kernels = kernels if kernels is not None else CudaKernels(self.pb, self.device)
        self.hashed = torch.zeros(H, dtype=torch.float32, device=self.device)
        self.dH = torch.empty(H, dtype=torch.float32, device=self.device)
        self.Y = torch.empty((M_local, N), dtype=dtype, device=self.device)
        self.dX = torch.empty((M_local, K), dtype=dtype, device=self.device)
        self._x_dev = self._dy_dev = None

    def load_weights(self, hashed: torch.Tensor) -> None:
        self.hashed.copy_(hashed.to(self.hashed.dtype), non_blocking=True)
        self.kernels.refresh(self.hashed)

    def step(self, X: torch.Tensor, dY: torch.Tensor, marks=None) -> None:
        """One training step on device-resident shards; results in self.Y, self.dX, self.dH, self.hashed.

        `marks`, if given, is a callable(name) invoked between kernels (the benchmark records events)."""
        k = self.kernels
        mark = marks if marks is not None else (lambda name: None)
        mark("start")
        k.forward(X, self.hashed, self.Y)
        mark("forward")
        k.backward_weight(X, dY, self.dH)
        mark("backward_weight")
        work = None
        if self.world > 1:
            work = dist.all_reduce(self.dH, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        k.backward_input(dY, self.hashed, self.dX)
        mark("backward_input")
        if work is not None:
            work.wait()
        k.sgd(self.hashed, self.dH, self.lr)
        mark("sgd")

    def step_host(self, X_host: torch.Tensor, dY_host: torch.Tensor, hashed_out_host: torch.Tensor) -> None:
        """The same step fed from (pinned) host memory: copies the shards in, runs, copies the updated
        hashed array back to `hashed_out_host`.  Asynchronous on the current stream."""
        if self._x_dev is None:
            self._x_dev = torch.empty((self.M, self.K), dtype=self.dtype, device=self.device)
            self._dy_dev = torch.empty((self.M, self.N), dtype=self.dtype, device=self.device)
        self._x_dev.copy_(X_host, non_blocking=True)
        self._dy_dev.copy_(dY_host, non_blocking=True)
        self.step(self._x_dev, self._dy_dev)
        hashed_out_host.copy_(self.hashed, non_blocking=True)
