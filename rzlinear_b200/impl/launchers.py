"""Kernel launchers with the reference's names and argument order.

They replace python/rz_linear/impl/RzLinearForward.py:6-85 (rz_linear_forward_tl),
RzLinearBackward.py:7-20, 23-97, 374-449 (rz_linear_backward_tl, _weight_grad_tl, _input_grad_tl)
and RzLinearIdx.py:6-45 (rz_linear_idx_tl) of apd10/RzLinear: same positional arguments, outputs
allocated here, kernels launched asynchronously on the current stream through the C ABI.

Differences, all additive:
  * BLOCK_SIZE_K / BLOCK_SIZE_N are the hash tile (they define the virtual matrix, exactly as in
    the reference); BLOCK_SIZE_M, GROUP_SIZE and allow_autotune only steered Triton's scheduling
    and are accepted and ignored.
  * `hash_mode` selects the two-level hash the reference's forward/backward kernels execute
    (default, RzLinearForward.py:316) or the single-level hash of its index kernel and tests
    (RzLinearIdx.py:70-71).
  * bf16 activations run the bf16 tensor-core path; fp32 activations run tf32 tensor cores when
    allow_tf32 is set and fp32 FMA otherwise.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib

HASH_SINGLE = _lib.HASH_SINGLE
HASH_TWO_LEVEL = _lib.HASH_TWO_LEVEL


def _precision(dtype: torch.dtype, allow_tf32: bool) -> int:
    if dtype == torch.bfloat16:
        return _lib.PREC_BF16
    if dtype == torch.float32:
        return _lib.PREC_TF32 if allow_tf32 else _lib.PREC_FP32
    raise TypeError(f"RzLinear kernels take float32 or bfloat16 activations, got {dtype}")


def _hashed_f32(hashed_weight: torch.Tensor) -> torch.Tensor:
    h = hashed_weight.detach()
    if h.dim() != 1:
        h = h.reshape(-1)
    if h.dtype != torch.float32:
        h = h.float()
    return h.contiguous()


def make_problem(M, K, N, H, R, BLOCK_SIZE_K, BLOCK_SIZE_N, dtype, allow_tf32, init_factor, hash_mode, flags=0):
    if not H > BLOCK_SIZE_K * BLOCK_SIZE_N:
        # the reference's assert (RzLinearForward.py:28)
        raise AssertionError("H must be larger than BLOCK_SIZE_K * BLOCK_SIZE_N")
    return _lib.make_problem(M, K, N, H, BLOCK_SIZE_K, BLOCK_SIZE_N, R, hash_mode, _lib.torch_io_dtype(dtype),
                             _precision(dtype, allow_tf32), init_factor, flags)


def alloc_shadow(pb, hashed: torch.Tensor) -> Optional[torch.Tensor]:
    """Allocate and fill the shadow copies the tensor-core forward / input-gradient kernels read."""
    nbytes = _lib.shadow_bytes(pb)
    if nbytes == 0:
        return None
    shadow = torch.empty(nbytes, dtype=torch.uint8, device=hashed.device)
    _lib.shadow_refresh(pb, hashed, shadow)
    return shadow


_CACHE_ATTR = "_rz_shadow_cache"


def cached_shadow(pb, hashed_weight: torch.Tensor, hashed_f32: torch.Tensor) -> Optional[torch.Tensor]:
    """The shadow of `hashed_weight` for this problem, rebuilt only when the weights have changed.

    The cache lives on the tensor object itself (so it dies with it and can never be mistaken for another
    tensor that later reuses the address) as {(H, BK, BN, precision): entry}; an entry is valid while the
    tensor's autograd version counter and data pointer are the ones it was filled at.  In-place updates
    (optimisers, copy_, add_) bump the counter; writes through `.data` or from foreign code do not, exactly
    as for autograd's own saved-tensor check: call `drop_shadow_cache(hashed_weight)` after such a write.
    A forward on unchanged weights (evaluation, several layers sharing one hashed array, several
    micro-batches per optimiser step) therefore allocates nothing and launches no refresh.
    While a CUDA graph is being captured the refresh is always launched (it becomes a node of the graph): a replay
    runs none of this Python, so a graph that skipped the refresh would keep reading the shadow of the weights it
    was captured with."""
    _lib._require_cuda(hashed_f32)
    nbytes = _lib.shadow_bytes(pb)
    if nbytes == 0:
        return None
    cache = getattr(hashed_weight, _CACHE_ATTR, None)
    if cache is None:
        cache = {}
        try:
            setattr(hashed_weight, _CACHE_ATTR, cache)
        except AttributeError:      # a tensor subclass without a __dict__: no caching
            return alloc_shadow(pb, hashed_f32)
    key = (pb.H, pb.BK, pb.BN, pb.precision)
    try:
        version, ptr = hashed_weight._version, hashed_weight.data_ptr()
    except RuntimeError:            # inference tensors keep no version counter: nothing to key a cache on
        return alloc_shadow(pb, hashed_f32)
    stream = torch.cuda.current_stream(hashed_f32.device)
    if torch.cuda.is_current_stream_capturing():
        # a buffer from the graph's own memory pool, filled by a node of the graph; the eager cache is left alone
        shadow = torch.empty(nbytes, dtype=torch.uint8, device=hashed_f32.device)
        _lib.shadow_refresh(pb, hashed_f32, shadow)
        return shadow
    entry = cache.get(key)
    if entry is not None and entry["shadow"].numel() >= nbytes and entry["shadow"].device == hashed_f32.device:
        if entry["version"] == version and entry["ptr"] == ptr:
            if entry["stream"] != stream.cuda_stream:
                stream.wait_event(entry["filled"])    # the refresh ran on another stream
            return entry["shadow"]
        shadow = entry["shadow"]                      # same buffer, new contents
    else:
        shadow = torch.empty(nbytes, dtype=torch.uint8, device=hashed_f32.device)
    _lib.shadow_refresh(pb, hashed_f32, shadow)
    filled = torch.cuda.Event()
    filled.record(stream)
    cache[key] = {"version": version, "ptr": ptr, "shadow": shadow, "stream": stream.cuda_stream, "filled": filled}
    return shadow


def drop_shadow_cache(hashed_weight: torch.Tensor) -> None:
    """Forget the cached shadows of `hashed_weight` (after a write that autograd's version counter does not see)."""
    if getattr(hashed_weight, _CACHE_ATTR, None):
        getattr(hashed_weight, _CACHE_ATTR).clear()


def rz_linear_forward_tl(input: torch.Tensor, hashed_weight: torch.Tensor, init_factor: float,
                         M: int, K: int, N: int, H: int,
                         R7: int, R6: int, R5: int, R4: int,
                         R3: int, R2: int, R1: int, R0: int,
                         allow_tf32: bool = True, allow_autotune: bool = True,
                         BLOCK_SIZE_M: int = 64, BLOCK_SIZE_N: int = 64, BLOCK_SIZE_K: int = 32,
                         GROUP_SIZE: int = 4, *, hash_mode: int = HASH_TWO_LEVEL,
                         bias: Optional[torch.Tensor] = None, relu: bool = False,
                         shadow: Optional[torch.Tensor] = None) -> torch.Tensor:
    """output[M, N] = (input[M, K] @ W_virtual[K, N]) * init_factor (+ bias, ReLU when asked)."""
    x = input.contiguous()
    hashed = _hashed_f32(hashed_weight)
    flags = _lib.FLAG_RELU if relu else 0
    pb = make_problem(M, K, N, H, (R0, R1, R2, R3, R4, R5, R6, R7), BLOCK_SIZE_K, BLOCK_SIZE_N, x.dtype,
                      allow_tf32, init_factor, hash_mode, flags)
    if shadow is None:
        shadow = alloc_shadow(pb, hashed)
    out = torch.empty((M, N), device=x.device, dtype=x.dtype)
    b = None if bias is None else bias.detach().float().contiguous()
    _lib.forward(pb, x, hashed, shadow, b, out)
    return out


def rz_linear_backward_input_grad_tl(output_grad: torch.Tensor, hashed_weight: torch.Tensor, init_factor: float,
                                     M: int, K: int, N: int, H: int,
                                     R7: int, R6: int, R5: int, R4: int,
                                     R3: int, R2: int, R1: int, R0: int,
                                     allow_tf32: bool = True, allow_autotune: bool = True,
                                     BLOCK_SIZE_M: int = 64, BLOCK_SIZE_N: int = 64, BLOCK_SIZE_K: int = 32,
                                     GROUP_SIZE: int = 4, *, hash_mode: int = HASH_TWO_LEVEL,
                                     shadow: Optional[torch.Tensor] = None) -> torch.Tensor:
    """input_grad[M, K] = (output_grad[M, N] @ W_virtual^T) * init_factor."""
    dy = output_grad.contiguous()
    hashed = _hashed_f32(hashed_weight)
    pb = make_problem(M, K, N, H, (R0, R1, R2, R3, R4, R5, R6, R7), BLOCK_SIZE_K, BLOCK_SIZE_N, dy.dtype,
                      allow_tf32, init_factor, hash_mode)
    if shadow is None:
        shadow = alloc_shadow(pb, hashed)
    dx = torch.empty((M, K), device=dy.device, dtype=dy.dtype)
    _lib.backward_input(pb, dy, hashed, shadow, dx)
    return dx


def rz_linear_backward_weight_grad_tl(input: torch.Tensor, output_grad: torch.Tensor, init_factor: float,
                                      M: int, K: int, N: int, H: int,
                                      R7: int, R6: int, R5: int, R4: int,
                                      R3: int, R2: int, R1: int, R0: int,
                                      allow_tf32: bool = True, allow_autotune: bool = True,
                                      BLOCK_SIZE_M: int = 64, BLOCK_SIZE_N: int = 64, BLOCK_SIZE_K: int = 32,
                                      GROUP_SIZE: int = 8, *, hash_mode: int = HASH_TWO_LEVEL,
                                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """hashed_weight_grad[H] (fp32): every tile of input^T @ output_grad added into its slice."""
    x = input.contiguous()
    dy = output_grad.contiguous()
    if x.dtype != dy.dtype:
        raise TypeError("input and output_grad must have the same dtype")
    pb = make_problem(M, K, N, H, (R0, R1, R2, R3, R4, R5, R6, R7), BLOCK_SIZE_K, BLOCK_SIZE_N, x.dtype,
                      allow_tf32, init_factor, hash_mode)
    dh = out if out is not None else torch.empty((H,), device=x.device, dtype=torch.float32)
    _lib.backward_weight(pb, x, dy, dh)  # zeroes dh first
    return dh


def rz_linear_backward_tl(input: torch.Tensor, hashed_weight: torch.Tensor, output_grad: torch.Tensor,
                          init_factor: float, M: int, K: int, N: int, H: int,
                          R7: int, R6: int, R5: int, R4: int,
                          R3: int, R2: int, R1: int, R0: int,
                          allow_tf32: bool = True, allow_autotune: bool = False,
                          BLOCK_SIZE_M: int = 64, BLOCK_SIZE_N: int = 64, BLOCK_SIZE_K: int = 32,
                          GROUP_SIZE: int = 4, *, hash_mode: int = HASH_TWO_LEVEL,
                          shadow: Optional[torch.Tensor] = None,
                          need_input_grad: bool = True) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """(input_grad, hashed_weight_grad), the pair RzLinearBackward.py:7-20 returns."""
    kw = dict(allow_tf32=allow_tf32, allow_autotune=allow_autotune, BLOCK_SIZE_M=BLOCK_SIZE_M,
              BLOCK_SIZE_N=BLOCK_SIZE_N, BLOCK_SIZE_K=BLOCK_SIZE_K, GROUP_SIZE=GROUP_SIZE, hash_mode=hash_mode)
    input_grad = None
    if need_input_grad:
        input_grad = rz_linear_backward_input_grad_tl(output_grad, hashed_weight, init_factor, M, K, N, H,
                                                      R7, R6, R5, R4, R3, R2, R1, R0, shadow=shadow, **kw)
    weight_grad = rz_linear_backward_weight_grad_tl(input, output_grad, init_factor, M, K, N, H,
                                                    R7, R6, R5, R4, R3, R2, R1, R0, **kw)
    return input_grad, weight_grad


def rz_linear_idx_tl(hashed_weight: torch.Tensor, K: int, N: int, H: int,
                     R3: int, R2: int, R1: int, R0: int,
                     BLOCK_SIZE_K: int = 32, BLOCK_SIZE_N: int = 32, *, hash_mode: int = HASH_SINGLE,
                     R7: int = 0, R5: int = 0, R4: int = 0) -> torch.Tensor:
    """Dense K x N virtual weight rebuilt from the hashed array (RzLinearIdx.py:6-45)."""
    assert H > BLOCK_SIZE_K * BLOCK_SIZE_N
    hashed = _hashed_f32(hashed_weight)
    pb = _lib.make_problem(1, K, N, H, BLOCK_SIZE_K, BLOCK_SIZE_N, (R0, R1, R2, R3, R4, R5, 0, R7), hash_mode,
                           _lib.F32, _lib.PREC_FP32)
    w = torch.empty((K, N), device=hashed.device, dtype=torch.float32)
    _lib.materialize(pb, hashed, w)
    return w.to(hashed_weight.dtype)
