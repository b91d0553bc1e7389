"""autograd glue of the RzLinear layer (host code only).

Mirrors python/rz_linear/RzLinearFunction.py:7-60 of apd10/RzLinear: the same `controls` switches,
the same first six arguments of `RzLinearFunction.apply`, gradients for `input` and
`hashed_weight`.  Two optional trailing arguments are additive: `config` (hash tile, hash mode,
ReLU fusion) and `bias` (added in the forward kernel's epilogue instead of a separate pass,
python/rz_linear/RzLinear.py:93-94).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from .impl import launchers

controls = {}
controls['triton_allow_tf32'] = False      # fp32 activations: tf32 tensor cores instead of fp32 FMA
controls['triton_allow_autotune'] = False  # accepted for compatibility; scheduling is fixed


@dataclass(frozen=True)
class RzConfig:
    """What defines the virtual matrix besides the random numbers, plus epilogue fusion."""
    block_size_k: int = 32      # reference default tile: RzLinearForward.py:11 (BLOCK_SIZE_K=32)
    block_size_n: int = 64      #                          RzLinearForward.py:11 (BLOCK_SIZE_N=64)
    hash_mode: int = _lib.HASH_TWO_LEVEL
    relu: bool = False


DEFAULT_CONFIG = RzConfig()


def _unpack(random_numbers):
    assert random_numbers.numel() == 8
    return [int(v) for v in random_numbers.tolist()]


def _compute_view(t: torch.Tensor) -> torch.Tensor:
    """Contiguous activations in a dtype the kernels take.  float32 and bfloat16 pass through; anything else
    (float16, float64: the reference accepts whatever Triton does) is computed in float32 and cast back."""
    if t.dtype in (torch.float32, torch.bfloat16):
        return t.contiguous()
    if not t.is_floating_point():
        raise TypeError(f"RzLinear takes floating-point activations, got {t.dtype}")
    return t.float().contiguous()


class RzLinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input: torch.Tensor, hashed_weight: torch.Tensor, random_numbers: torch.Tensor,
                output_dim, chunk_size, init_factor, config: Optional[RzConfig] = None,
                bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        '''
            Args:
                input (Tensor): (M, input_dim)
                hashed_weight (Tensor): (H), the compressed weight
                random_numbers (Tensor): (8), R[0] the prime, on the CPU
                output_dim (int): N
                chunk_size (int): unused, as in the reference
                init_factor (float): scale applied to the product
                config (RzConfig): hash tile / hash mode / ReLU fusion (default: reference behaviour)
                bias (Tensor): (N), fused into the kernel epilogue when given

            Returns:
                output (Tensor): (M, output_dim)
        '''
        cfg = config if config is not None else DEFAULT_CONFIG
        R = _unpack(random_numbers)
        M, K, N, H = input.shape[0], input.shape[1], output_dim, hashed_weight.shape[0]
        allow_tf32 = controls['triton_allow_tf32']
        x = _compute_view(input)
        hashed = launchers._hashed_f32(hashed_weight)
        flags = _lib.FLAG_RELU if cfg.relu else 0
        pb = launchers.make_problem(M, K, N, H, R, cfg.block_size_k, cfg.block_size_n, x.dtype, allow_tf32,
                                    init_factor, cfg.hash_mode, flags)
        shadow = launchers.cached_shadow(pb, hashed_weight, hashed)   # refreshed only when the weights changed
        out = torch.empty((M, N), device=x.device, dtype=x.dtype)
        b = None if bias is None else bias.detach().float().contiguous()
        _lib.forward(pb, x, hashed, shadow, b, out)

        # (the saved output keeps the compute dtype: the backward masks with it)
        ctx.save_for_backward(input, hashed_weight, random_numbers, out if cfg.relu else None)
        ctx.shadow = shadow  # the backward reads the weights the forward saw
        ctx.output_dim = output_dim
        ctx.chunk_size = chunk_size
        ctx.init_factor = init_factor
        ctx.config = cfg
        ctx.allow_tf32 = allow_tf32
        ctx.has_bias = bias is not None
        return out if out.dtype == input.dtype else out.to(input.dtype)

    @staticmethod
    def backward(ctx, grad):
        input, hashed_weight, random_numbers, out = ctx.saved_tensors
        cfg = ctx.config
        R = _unpack(random_numbers)
        M, K, N, H = input.shape[0], input.shape[1], ctx.output_dim, hashed_weight.shape[0]
        x = _compute_view(input)
        grad = grad.contiguous() if grad.dtype == x.dtype else grad.to(x.dtype).contiguous()
        hashed = launchers._hashed_f32(hashed_weight)
        pb = launchers.make_problem(M, K, N, H, R, cfg.block_size_k, cfg.block_size_n, x.dtype, ctx.allow_tf32,
                                    ctx.init_factor, cfg.hash_mode)
        input_grad = weight_grad = bias_grad = None
        # one pass over the incoming gradient: ReLU mask from the saved output and the bias gradient (column sums)
        want_bias = ctx.has_bias and ctx.needs_input_grad[7]
        if cfg.relu or want_bias:
            masked = torch.empty_like(grad) if cfg.relu else None
            bias_grad = torch.empty((N,), device=x.device, dtype=torch.float32) if want_bias else None
            _lib.grad_prepare(pb, grad, out if cfg.relu else None, masked, bias_grad)
            if cfg.relu:
                grad = masked
        if ctx.needs_input_grad[0]:
            input_grad = torch.empty((M, K), device=x.device, dtype=x.dtype)
            _lib.backward_input(pb, grad, hashed, ctx.shadow, input_grad)
            if input_grad.dtype != input.dtype:
                input_grad = input_grad.to(input.dtype)
        if ctx.needs_input_grad[1]:
            dh = torch.empty((H,), device=x.device, dtype=torch.float32)
            _lib.backward_weight(pb, x, grad, dh)
            weight_grad = dh if hashed_weight.dtype == torch.float32 else dh.to(hashed_weight.dtype)
        ctx.shadow = None
        return input_grad, weight_grad, None, None, None, None, None, bias_grad
