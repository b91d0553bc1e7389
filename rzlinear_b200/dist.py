"""Data-parallel training step of one RzLinear layer (batch rows sharded over ranks).

Each rank owns M_local rows of X and dY; the hashed array and the random numbers are replicated.
Forward and input gradient need no communication.  The only exchange is the sum of the
hashed-weight gradient over ranks (one all-reduce of H floats), launched right after the
weight-gradient kernel so that it overlaps the input-gradient kernel; every rank then applies the
same SGD update, so the replicas stay identical.  The input-gradient kernel is persistent (one CTA
per SM), so with more than one rank it is launched on all SMs but `comm_sms`: the collective's
CTAs get those and run beside it instead of behind it.  For that the collective must fit those SMs: create the
NCCL process group with at most `comm_sms` CTAs (environment `NCCL_MAX_CTAS`, or the process-group option
`config.max_ctas`); with NCCL's default CTA count part of the collective still waits for the input gradient to end.

The reference has no distributed code; this follows its single-GPU step
(python/rz_linear/RzLinearFunction.py:14-60) per rank.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from . import _lib


class CudaKernels:
    """The C-ABI kernels (the only shipped implementation).

    `comm_sms` > 0: the input-gradient kernel leaves that many SMs idle (for the all-reduce that runs
    beside it).  The scratch is sized for the largest of the problems this object launches."""

    def __init__(self, pb, device, comm_sms: int = 0):
        self.pb = pb
        self.pb_dx = _lib.with_fields(pb, sm_reserve=int(comm_sms)) if comm_sms > 0 else pb
        self.device = device
        self.shadow = None
        self.reserve(max(_lib.shadow_bytes(pb), _lib.shadow_bytes(self.pb_dx)))

    def reserve(self, nbytes: int, hashed=None) -> None:
        """Grow the scratch to at least `nbytes` (never shrinks); refills it from `hashed` when it was replaced."""
        have = 0 if self.shadow is None else self.shadow.numel()
        if nbytes <= have:
            return
        self.shadow = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        if hashed is not None:
            self.refresh(hashed)

    def refresh(self, hashed):
        if self.shadow is not None:
            _lib.shadow_refresh(self.pb, hashed, self.shadow)

    def forward(self, x, hashed, y):
        _lib.forward(self.pb, x, hashed, self.shadow, None, y)

    def backward_input(self, dy, hashed, dx):
        _lib.backward_input(self.pb_dx, dy, hashed, self.shadow, dx)

    def backward_weight(self, x, dy, dh):
        _lib.backward_weight(self.pb, x, dy, dh)

    def sgd(self, hashed, dh, lr, velocity=None, momentum=0.0):
        if velocity is None:
            _lib.sgd_step(self.pb, hashed, dh, lr, self.shadow)
        else:
            _lib.sgd_momentum_step(self.pb, hashed, dh, velocity, lr, momentum, self.shadow)


def shard_rows(M_global: int, rank: int, world: int):
    """Rows [lo, hi) of the global batch owned by `rank` (contiguous blocks, remainder to the first ranks)."""
    base, rem = divmod(M_global, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class RzDataParallelStep:
    def __init__(self, M_local: int, K: int, N: int, H: int, BK: int, BN: int, R: Sequence[int],
                 hash_mode: int = _lib.HASH_SINGLE, dtype: torch.dtype = torch.bfloat16, lr: float = 1e-3,
                 device="cuda", init_factor: float = 1.0, allow_tf32: bool = True,
                 process_group: Optional[dist.ProcessGroup] = None, kernels=None, momentum: float = 0.0,
                 comm_sms: int = 8):
        self.M, self.K, self.N, self.H = M_local, K, N, H
        self.device = torch.device(device)
        self.dtype = dtype
        self.lr = float(lr)
        self.momentum = float(momentum)
        self.group = process_group
        self.world = dist.get_world_size(process_group) if (dist.is_available() and dist.is_initialized()) else 1
        prec = _lib.PREC_BF16 if dtype == torch.bfloat16 else (_lib.PREC_TF32 if allow_tf32 else _lib.PREC_FP32)
        self.pb = _lib.make_problem(M_local, K, N, H, BK, BN, R, hash_mode, _lib.torch_io_dtype(dtype), prec,
                                    init_factor)
        self.comm_sms = int(comm_sms) if self.world > 1 else 0
        self.kernels = kernels if kernels is not None else CudaKernels(self.pb, self.device, self.comm_sms)
        self.hashed = torch.zeros(H, dtype=torch.float32, device=self.device)
        self.dH = torch.empty(H, dtype=torch.float32, device=self.device)
        self.velocity = torch.zeros(H, dtype=torch.float32, device=self.device) if self.momentum != 0.0 else None
        self.Y = torch.empty((M_local, N), dtype=dtype, device=self.device)
        self.dX = torch.empty((M_local, K), dtype=dtype, device=self.device)
        self._pipe = None
        self._comm_stream = None

    def load_weights(self, hashed: torch.Tensor) -> None:
        self.hashed.copy_(hashed.to(self.hashed.dtype), non_blocking=True)
        self.kernels.refresh(self.hashed)

    def _update(self) -> None:
        if self.velocity is None:
            self.kernels.sgd(self.hashed, self.dH, self.lr)
        else:
            self.kernels.sgd(self.hashed, self.dH, self.lr, self.velocity, self.momentum)

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
        # The input gradient is queued BEFORE the collective, and the collective is issued from a side stream that
        # waits for the weight gradient only: when the weight gradient finishes, the persistent input-gradient CTAs
        # are placed first (on all SMs but `comm_sms`) and the collective's CTAs take the SMs left idle.  Issued
        # the other way round, the collective's CTAs land first, anywhere, and the input-gradient CTAs they displace
        # start only when it is over - with a static work split that delays the whole kernel by the collective's time.
        work = None
        on_gpu = self.device.type == "cuda"
        if self.world > 1 and on_gpu:
            dh_ready = torch.cuda.Event()
            dh_ready.record()
        elif self.world > 1:   # host-logic tests on CPU (gloo): no streams to order
            work = dist.all_reduce(self.dH, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        k.backward_input(dY, self.hashed, self.dX)
        if self.world > 1 and on_gpu:
            work = self._all_reduce_beside(dh_ready)
        mark("backward_input")
        if work is not None:
            work.wait()
        mark("comm_wait")   # what of the all-reduce was still running when the input gradient had finished
        self._update()
        mark("sgd")

    def _all_reduce_beside(self, dh_ready):
        """Start the all-reduce of dH on the communication stream, ordered after `dh_ready` only."""
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=self.device)
        self._comm_stream.wait_event(dh_ready)
        with torch.cuda.stream(self._comm_stream):
            return dist.all_reduce(self.dH, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    def _host_pipeline(self, chunk_rows: int):
        """Device staging buffers, the copy stream, per-chunk problems and events of step_host."""
        if getattr(self, "_pipe", None) is not None and self._pipe["chunk_rows"] == chunk_rows:
            return self._pipe
        spans = [(lo, min(self.M, lo + chunk_rows)) for lo in range(0, self.M, chunk_rows)]
        # What follows the last copy cannot overlap anything: the kernels of the last chunk, the update, the read-back.
        # So the last chunk is cut into halves of halves (down to 2048 rows): the copies stay large, the tail short.
        lo, hi = spans.pop()
        while hi - lo >= 2 * 2048:
            mid = lo + (hi - lo) // 2 // 128 * 128
            spans.append((lo, mid))
            lo = mid
        spans.append((lo, hi))
        base = self.pb
        problems = []
        for i, (lo, hi) in enumerate(spans):
            flags = base.flags | (_lib.FLAG_ACCUMULATE_DH if i > 0 else 0)
            # the all-reduce is issued before the last chunk's input gradient and runs beside it
            reserve = self.comm_sms if i == len(spans) - 1 else 0
            problems.append((_lib.with_fields(base, M=hi - lo, flags=flags),
                             _lib.with_fields(base, M=hi - lo, flags=flags, sm_reserve=reserve)))
        # the split-contraction workspace inside the scratch depends on the rows of a launch: a remainder chunk
        # can need more of it than the whole shard does
        self.kernels.reserve(max(_lib.shadow_bytes(pb) for pair in problems for pb in pair), self.hashed)
        self._pipe = {
            "chunk_rows": chunk_rows, "spans": spans, "problems": problems,
            "x": torch.empty((self.M, self.K), dtype=self.dtype, device=self.device),
            "dy": torch.empty((self.M, self.N), dtype=self.dtype, device=self.device),
            "stream": torch.cuda.Stream(device=self.device),
            "loaded": [torch.cuda.Event() for _ in spans],
            "consumed": [None for _ in spans],
        }
        return self._pipe

    def step_host(self, X_host: torch.Tensor, dY_host: torch.Tensor, hashed_out_host: torch.Tensor,
                  chunk_rows: int = 16384) -> None:
        """The same step fed from (pinned) host memory, asynchronous on the current stream.

        The shards are copied in row chunks on a side stream while the kernels work on the chunks that
        have already arrived (forward and input gradient are row-independent, the hashed-weight
        gradient accumulates over chunks); the updated hashed array is copied back to
        `hashed_out_host` at the end."""
        if not isinstance(self.kernels, CudaKernels):
            raise RuntimeError("step_host drives the CUDA kernels; use step() with injected kernels")
        pipe = self._host_pipeline(min(chunk_rows, self.M))   # (may replace the scratch by a larger one)
        main = torch.cuda.current_stream(self.device)
        side = pipe["stream"]
        shadow = self.kernels.shadow
        side.wait_stream(main)   # inputs pinned/filled by work queued on the main stream so far
        for i, (lo, hi) in enumerate(pipe["spans"]):
            if pipe["consumed"][i] is not None:
                side.wait_event(pipe["consumed"][i])   # the previous step has finished reading this chunk
            with torch.cuda.stream(side):
                pipe["x"][lo:hi].copy_(X_host[lo:hi], non_blocking=True)
                pipe["dy"][lo:hi].copy_(dY_host[lo:hi], non_blocking=True)
                pipe["loaded"][i].record(side)
        work = None
        last = len(pipe["spans"]) - 1
        for i, (lo, hi) in enumerate(pipe["spans"]):
            pb, pb_dx = pipe["problems"][i]
            x, dy = pipe["x"][lo:hi], pipe["dy"][lo:hi]
            main.wait_event(pipe["loaded"][i])
            _lib.forward(pb, x, self.hashed, shadow, None, self.Y[lo:hi])
            _lib.backward_weight(pb, x, dy, self.dH)
            if i == last and self.world > 1:
                dh_ready = torch.cuda.Event()
                dh_ready.record()
            _lib.backward_input(pb_dx, dy, self.hashed, shadow, self.dX[lo:hi])
            if i == last and self.world > 1:
                work = self._all_reduce_beside(dh_ready)
            ev = torch.cuda.Event()
            ev.record(main)
            pipe["consumed"][i] = ev
        if work is not None:
            work.wait()
        self._update()
        hashed_out_host.copy_(self.hashed, non_blocking=True)
