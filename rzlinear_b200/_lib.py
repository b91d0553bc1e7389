"""ctypes binding of librzlinear_b200.so (the C ABI declared in include/rzlinear_b200.h).

PyTorch is used for device memory and streams only; the library itself has no torch types in
its signatures.  There is no CPU fallback: a missing or unloadable library raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch  # also makes sure torch's libcudart.so.12 is the one the library binds to

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librzlinear_b200.so")

# enum values of include/rzlinear_b200.h
RZ_OK = 0
RZ_ERR_CUDA, RZ_ERR_PIPELINE, RZ_ERR_TOO_LARGE, RZ_ERR_SCRATCH = -7, -8, -10, -11
HASH_SINGLE, HASH_TWO_LEVEL = 0, 1
F32, BF16 = 0, 1
PREC_FP32, PREC_TF32, PREC_BF16 = 0, 1, 2
FLAG_ACCUMULATE_DH, FLAG_FORCE_SIMT, FLAG_RELU = 1, 2, 4
OP_FORWARD, OP_BACKWARD_INPUT, OP_BACKWARD_WEIGHT = 0, 1, 2
PATH_SIMT, PATH_TCGEN05 = 0, 1

EXPORTS = [
    "rz_version", "rz_status_string", "rz_last_cuda_error", "rz_hash_indices_host",
    "rz_hash_indices_device", "rz_plan", "rz_shadow_bytes", "rz_shadow_refresh",
    "rz_linear_forward", "rz_linear_backward_input", "rz_linear_backward_weight",
    "rz_linear_materialize", "rz_sgd_step", "rz_device_status", "rz_launch_count",
    "rz_selftest_bounded_wait", "rz_sgd_momentum_step", "rz_grad_prepare", "rz_linear_forward_noalloc",
    "rz_reload_env",
]


class RzProblem(ctypes.Structure):
    _fields_ = [
        ("M", ctypes.c_int64), ("K", ctypes.c_int64), ("N", ctypes.c_int64), ("H", ctypes.c_int64),
        ("BK", ctypes.c_int32), ("BN", ctypes.c_int32),
        ("hash_mode", ctypes.c_int32), ("io_dtype", ctypes.c_int32),
        ("precision", ctypes.c_int32), ("flags", ctypes.c_int32),
        ("R", ctypes.c_int64 * 8),
        ("alpha", ctypes.c_float), ("sm_reserve", ctypes.c_int32),
    ]


class RzLinearError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"rzlinear_b200: {message} (status {status})")
        self.status = status


_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load the library once; raise (never fall back) if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m rzlinear_b200.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback for the RzLinear kernels)")
        lib = ctypes.CDLL(LIB_PATH)
        vp, i64p = ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)
        pbp = ctypes.POINTER(RzProblem)
        lib.rz_version.restype = ctypes.c_int
        lib.rz_status_string.restype = ctypes.c_char_p
        lib.rz_status_string.argtypes = [ctypes.c_int]
        lib.rz_last_cuda_error.restype = ctypes.c_char_p
        lib.rz_hash_indices_host.argtypes = [pbp, i64p]
        lib.rz_hash_indices_device.argtypes = [pbp, vp, vp]
        lib.rz_plan.argtypes = [pbp, ctypes.c_int]
        lib.rz_shadow_bytes.restype = ctypes.c_size_t
        lib.rz_shadow_bytes.argtypes = [pbp]
        lib.rz_shadow_refresh.argtypes = [pbp, vp, vp, vp]
        lib.rz_linear_forward.argtypes = [pbp, vp, vp, vp, ctypes.c_size_t, vp, vp, vp]
        lib.rz_linear_backward_input.argtypes = [pbp, vp, vp, vp, ctypes.c_size_t, vp, vp]
        lib.rz_linear_backward_weight.argtypes = [pbp, vp, vp, vp, vp]
        lib.rz_linear_materialize.argtypes = [pbp, vp, vp, vp]
        lib.rz_grad_prepare.argtypes = [pbp, vp, vp, vp, vp, vp]
        lib.rz_grad_prepare.restype = ctypes.c_int
        lib.rz_sgd_step.argtypes = [pbp, vp, vp, ctypes.c_float, vp, vp]
        lib.rz_sgd_momentum_step.argtypes = [pbp, vp, vp, vp, ctypes.c_float, ctypes.c_float, vp, vp]
        lib.rz_selftest_bounded_wait.argtypes = [ctypes.c_int64, vp]
        lib.rz_linear_forward_noalloc.argtypes = [pbp, vp, vp, vp, vp, vp]
        lib.rz_reload_env.restype = None
        lib.rz_device_status.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        lib.rz_launch_count.restype = ctypes.c_uint64
        for name in ("rz_hash_indices_host", "rz_hash_indices_device", "rz_plan", "rz_shadow_refresh",
                     "rz_linear_forward", "rz_linear_backward_input", "rz_linear_backward_weight",
                     "rz_linear_materialize", "rz_sgd_step", "rz_device_status", "rz_sgd_momentum_step",
                     "rz_selftest_bounded_wait", "rz_linear_forward_noalloc"):
            getattr(lib, name).restype = ctypes.c_int
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status == RZ_OK:
        return
    lib = load()
    msg = lib.rz_status_string(status).decode()
    if status == RZ_ERR_CUDA:
        msg += ": " + lib.rz_last_cuda_error().decode()
    raise RzLinearError(status, msg)


def make_problem(M, K, N, H, BK, BN, R, hash_mode, io_dtype, precision, alpha=1.0, flags=0, sm_reserve=0) -> RzProblem:
    pb = RzProblem()
    pb.M, pb.K, pb.N, pb.H = int(M), int(K), int(N), int(H)
    pb.BK, pb.BN = int(BK), int(BN)
    pb.hash_mode, pb.io_dtype, pb.precision, pb.flags = int(hash_mode), int(io_dtype), int(precision), int(flags)
    R = [int(v) for v in R]
    if len(R) != 8:
        raise ValueError("random_numbers must have 8 entries (R[0] is the prime)")
    for i, v in enumerate(R):
        pb.R[i] = v
    pb.alpha = float(alpha)
    pb.sm_reserve = int(sm_reserve)
    return pb


def with_fields(pb: RzProblem, **fields) -> RzProblem:
    """A copy of `pb` with some fields replaced (M, flags, sm_reserve, ...)."""
    out = RzProblem()
    ctypes.memmove(ctypes.byref(out), ctypes.byref(pb), ctypes.sizeof(RzProblem))
    for name, value in fields.items():
        setattr(out, name, value)
    return out


def torch_io_dtype(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"rzlinear_b200 supports float32 and bfloat16 activations, got {dtype}")


class _on:
    """Makes `device` current around a call.  Cheaper than torch.cuda.device() in the common case where it
    already is (no device switch, no context-manager machinery): small problems are bound by host time."""
    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx = device.index

    def __enter__(self):
        self.prev = torch.cuda.current_device()
        if self.idx is not None and self.idx != self.prev:
            torch.cuda.set_device(self.idx)
        else:
            self.idx = None
        return self

    def __exit__(self, *exc):
        if self.idx is not None:
            torch.cuda.set_device(self.prev)
        return False


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("rzlinear_b200 kernels run on CUDA tensors only (there is no CPU path)")


def plan(pb: RzProblem, op: int) -> int:
    r = load().rz_plan(ctypes.byref(pb), op)
    if r < 0:
        check(r)
    return r


def shadow_bytes(pb: RzProblem) -> int:
    return int(load().rz_shadow_bytes(ctypes.byref(pb)))


def hash_indices_host(pb: RzProblem):
    import numpy as np
    nk = -(-pb.K // pb.BK)
    nn = -(-pb.N // pb.BN)
    out = np.empty((nk, nn), dtype=np.int64)
    check(load().rz_hash_indices_host(ctypes.byref(pb), out.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))))
    return out


def hash_indices_device(pb: RzProblem, device) -> torch.Tensor:
    nk = -(-pb.K // pb.BK)
    nn = -(-pb.N // pb.BN)
    out = torch.empty((nk, nn), dtype=torch.int64, device=device)
    with _on(out.device):
        check(load().rz_hash_indices_device(ctypes.byref(pb), _ptr(out), _stream(out.device)))
    return out


def shadow_refresh(pb: RzProblem, hashed: torch.Tensor, shadow: torch.Tensor) -> None:
    _require_cuda(hashed, shadow)
    with _on(hashed.device):
        check(load().rz_shadow_refresh(ctypes.byref(pb), _ptr(hashed), _ptr(shadow), _stream(hashed.device)))


def _nbytes(t) -> int:
    return 0 if t is None else t.numel() * t.element_size()


def forward(pb, x, hashed, shadow, bias, y) -> None:
    """Raises RzLinearError(RZ_ERR_SCRATCH) when `shadow` is smaller than shadow_bytes(pb)."""
    _require_cuda(x, hashed, shadow, bias, y)
    with _on(x.device):
        check(load().rz_linear_forward(ctypes.byref(pb), _ptr(x), _ptr(hashed), _ptr(shadow), _nbytes(shadow), _ptr(bias),
                                       _ptr(y), _stream(x.device)))


def backward_input(pb, dy, hashed, shadow, dx) -> None:
    _require_cuda(dy, hashed, shadow, dx)
    with _on(dy.device):
        check(load().rz_linear_backward_input(ctypes.byref(pb), _ptr(dy), _ptr(hashed), _ptr(shadow), _nbytes(shadow),
                                              _ptr(dx), _stream(dy.device)))


def backward_weight(pb, x, dy, dh) -> None:
    _require_cuda(x, dy, dh)
    with _on(x.device):
        check(load().rz_linear_backward_weight(ctypes.byref(pb), _ptr(x), _ptr(dy), _ptr(dh), _stream(x.device)))


def materialize(pb, hashed, w) -> None:
    _require_cuda(hashed, w)
    with _on(hashed.device):
        check(load().rz_linear_materialize(ctypes.byref(pb), _ptr(hashed), _ptr(w), _stream(hashed.device)))


def grad_prepare(pb, dy, y, dym, bias_grad) -> None:
    """dym = dy where y > 0 (y may be None: no mask), bias_grad = column sums of the (masked) gradient (may be None)."""
    _require_cuda(dy, y, dym, bias_grad)
    with _on(dy.device):
        check(load().rz_grad_prepare(ctypes.byref(pb), _ptr(dy), _ptr(y), _ptr(dym), _ptr(bias_grad), _stream(dy.device)))


def sgd_step(pb, hashed, dh, lr, shadow) -> None:
    _require_cuda(hashed, dh, shadow)
    with _on(hashed.device):
        check(load().rz_sgd_step(ctypes.byref(pb), _ptr(hashed), _ptr(dh), ctypes.c_float(lr), _ptr(shadow),
                                 _stream(hashed.device)))


def sgd_momentum_step(pb, hashed, dh, velocity, lr, momentum, shadow) -> None:
    _require_cuda(hashed, dh, velocity, shadow)
    fn = load().rz_sgd_momentum_step
    with _on(hashed.device):
        check(fn(ctypes.byref(pb), _ptr(hashed), _ptr(dh), _ptr(velocity), ctypes.c_float(lr), ctypes.c_float(momentum),
                 _ptr(shadow), _stream(hashed.device)))


def device_status():
    """(status, detail) of the device-side pipeline word; synchronises the device and clears the word."""
    st, detail = ctypes.c_int(0), ctypes.c_int(0)
    check(load().rz_device_status(ctypes.byref(st), ctypes.byref(detail)))
    return st.value, detail.value


def selftest_bounded_wait(limit_cycles: int, device="cuda") -> None:
    """Launch the bounded-wait self-test kernel; read the outcome with device_status()."""
    fn = load().rz_selftest_bounded_wait
    dev = torch.device(device)
    with _on(dev):
        check(fn(int(limit_cycles), _stream(dev)))


def launch_count() -> int:
    return int(load().rz_launch_count())


def reload_env() -> None:
    """Make the library read its RZ_TC_* bring-up knobs from the environment again."""
    load().rz_reload_env()


NOALLOC_SCRATCH_BYTES = 16 << 20


def forward_noalloc(pb, x, hashed, bias, y) -> None:
    """rz_linear_forward_noalloc: forward pass whose scratch is a fixed array inside the library.

    For hosts that cannot allocate device memory when they call (see include/rzlinear_b200.h for who
    that is and for the limits: shifted copies <= NOALLOC_SCRATCH_BYTES, one shared array per device, calls
    that overlap on the GPU race, first call per device before any stream capture)."""
    _require_cuda(x, hashed, bias, y)
    fn = load().rz_linear_forward_noalloc
    with _on(x.device):
        check(fn(ctypes.byref(pb), _ptr(x), _ptr(hashed), _ptr(bias), _ptr(y), _stream(x.device)))
