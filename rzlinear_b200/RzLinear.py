"""The RzLinear layer: a linear layer over a virtual, ROBE-Z-hashed weight matrix.

Drop-in for python/rz_linear/RzLinear.py:7-97 of apd10/RzLinear: same constructor arguments,
attributes (`_hashed_weight`, `_bias`, `_random_numbers`, `_seed`, ...), class constants `P`, `R`
and forward semantics.  Keyword-only additions choose the hash tile, the hash form and the prime.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
from torch.nn.parameter import Parameter

from . import _lib
from .RzLinearFunction import RzLinearFunction, RzConfig


class RzLinear(torch.nn.Module):
    # the reference's working prime (RzLinear.py:8-10); the large prime 2038074743 can be passed as `prime`
    P = 45007
    R = 8
    LARGE_PRIME = 2038074743

    # P: default prime of the tile hash.  R: how many random numbers a layer carries (R[0] is the prime itself).

    def __init__(self, input_dim: int, output_dim: int, chunk_size: int = 1,
                 hashed_weight: Parameter = None, tiled=True, seed: int = 1024, bias: bool = True,
                 dtype: torch.dtype = torch.float32, compress_ratio: float = 0.0625,
                 init_factor: float = 1.0, *,
                 block_size_k: int = 32, block_size_n: int = 64, hash_mode: str = 'two_level',
                 prime: Optional[int] = None, random_numbers: Optional[Sequence[int]] = None,
                 relu: bool = False) -> None:
        '''
            Linear layer whose input_dim x output_dim weight is virtual: every block_size_k x block_size_n tile of it
            is a contiguous slice of one shared 1-D parameter, `hashed_weight`, at an offset given by a hash of the
            tile's coordinates (ROBE-Z).

            Positional arguments, same order and meaning as the reference's constructor:
                input_dim, output_dim (int): feature counts of the input and of the output (both below 10^5)
                chunk_size (int): kept for call compatibility; neither implementation uses it
                hashed_weight (Parameter): an existing compressed array to share with other layers; when given,
                    compress_ratio plays no part
                tiled (bool): kept for call compatibility, unused
                seed (int): seeds the draw of the layer's random numbers
                bias (bool): whether the layer owns a bias vector of output_dim entries
                dtype (torch.dtype): dtype of the parameters this layer creates
                compress_ratio (float): length of a newly created hashed_weight as a fraction of input_dim * output_dim
                init_factor (float): constant the product is multiplied by

            Keyword-only additions:
                block_size_k, block_size_n (int): the hash tile. It is part of what defines the virtual matrix; the
                    reference's kernels use 32 x 64 unless told otherwise
                hash_mode (str): 'two_level', the form the reference's kernels evaluate, or 'single',
                    ((pk*R3 + pn*R2 + R1) mod P) mod (H - BK*BN)
                prime (int): this layer's prime instead of RzLinear.P
                random_numbers (8 ints): use these instead of drawing from the seed; entry 0 is the prime
                relu (bool): fuse a ReLU into the forward kernel's epilogue
        '''

        super(RzLinear, self).__init__()

        assert (input_dim < 10**5 and output_dim < 10**5)
        if hash_mode not in ('two_level', 'single'):
            raise ValueError("hash_mode must be 'two_level' or 'single'")

        self._input_dim = input_dim
        self._output_dim = output_dim
        self._compress_ratio = compress_ratio
        self._chunk_size = chunk_size
        self._hashed_weight = hashed_weight
        self._bias = bias
        self._seed = seed
        self._init_factor = init_factor
        self._prime = int(prime) if prime is not None else RzLinear.P
        self._config = RzConfig(block_size_k=int(block_size_k), block_size_n=int(block_size_n),
                                hash_mode=_lib.HASH_TWO_LEVEL if hash_mode == 'two_level' else _lib.HASH_SINGLE,
                                relu=bool(relu))

        # random numbers are always on the CPU
        if random_numbers is not None:
            rn = [int(v) for v in random_numbers]
            assert len(rn) == RzLinear.R
            self._random_numbers = torch.tensor(rn, dtype=torch.int64)
            self._prime = rn[0]
        else:
            self._random_numbers = self._generate_random_numbers(seed)

        # weight
        if hashed_weight is None:
            self._hashed_weight = Parameter(
                torch.arange(int(input_dim * output_dim * compress_ratio)).type(dtype))
        else:
            self._hashed_weight = hashed_weight

        # bias term
        if bias:
            self._bias = Parameter(torch.zeros(self._output_dim, dtype=dtype))
        else:
            self._bias = None

    def __repr__(self):
        return 'RzLinear(mm={}x{} bias={} seed={} hashed_weight_size={}, init_factor={} hashed_weight_id={})'.format(
            self._input_dim, self._output_dim, (self._bias is not None), self._seed, self._hashed_weight.size(),
            self._init_factor, self._hashed_weight.data_ptr())

    def _generate_random_numbers(self, seed: int):
        # Same draw as the reference (RzLinear.py:68-74), including its reseeding of torch's global generator.
        torch.manual_seed(seed)
        P = self._prime
        x = torch.randint(0, P, (RzLinear.R - 1,)).type(torch.int32).requires_grad_(False)
        x = torch.cat([torch.tensor([P], dtype=torch.int32), x])
        return x.requires_grad_(False).cpu()

    def forward(self, x) -> torch.Tensor:
        '''
            x: (batch, ..., input_dim) -> (batch, ..., output_dim).  Leading dimensions are flattened for the kernel
            and restored afterwards; the bias (if any) and the optional ReLU are applied inside the kernel.
        '''
        assert (len(x.shape) >= 2)
        dim_gt_2 = x.dim() > 2
        if (dim_gt_2):
            shape = x.shape
            x = x.reshape(-1, shape[-1]).contiguous()
        x = RzLinearFunction.apply(
            x, self._hashed_weight, self._random_numbers, self._output_dim, self._chunk_size, self._init_factor,
            self._config, self._bias)
        if (dim_gt_2):
            x = x.view(*shape[:-1], x.shape[-1])
        return x
