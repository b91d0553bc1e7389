"""Host logic of the Python mirror of the reference's rz_linear package (no GPU needed)."""
import os

import numpy as np
import pytest
import torch

import rzlinear_b200
from rzlinear_b200 import RzLinear, RzLinearFunction, RzConfig, controls


def test_public_names_match_reference_package():
    assert {"RzLinear", "RzLinearFunction", "controls"} <= set(dir(rzlinear_b200))
    assert controls == {"triton_allow_tf32": False, "triton_allow_autotune": False}
    assert RzLinear.P == 45007 and RzLinear.R == 8
    from rzlinear_b200.impl.RzLinearForward import rz_linear_forward_tl  # noqa: F401
    from rzlinear_b200.impl.RzLinearBackward import (rz_linear_backward_tl, rz_linear_backward_input_grad_tl,  # noqa: F401
                                                     rz_linear_backward_weight_grad_tl)
    from rzlinear_b200.impl.RzLinearIdx import rz_linear_idx_tl  # noqa: F401


def test_constructor_defaults_and_attributes(golden_dir):
    rz = RzLinear(input_dim=1024, output_dim=512)
    assert rz._input_dim == 1024 and rz._output_dim == 512
    assert rz._compress_ratio == 0.0625 and rz._chunk_size == 1 and rz._seed == 1024 and rz._init_factor == 1.0
    H = int(1024 * 512 * 0.0625)
    assert rz._hashed_weight.shape == (H,) and rz._hashed_weight.dtype == torch.float32
    assert torch.equal(rz._hashed_weight.detach(), torch.arange(H).float())   # reference init: arange
    assert rz._bias.shape == (512,) and float(rz._bias.detach().abs().sum()) == 0.0
    assert not rz._random_numbers.is_cuda and rz._random_numbers.numel() == 8
    d = np.load(os.path.join(golden_dir, "random_numbers.npz"))
    for seed in d.files:
        got = RzLinear(64, 64, seed=int(seed), compress_ratio=1.0)._random_numbers
        assert got.dtype == torch.int32 and [int(v) for v in got] == [int(v) for v in d[seed]]
    assert set(dict(rz.named_parameters())) == {"_hashed_weight", "_bias"}
    assert "RzLinear(mm=1024x512 bias=True seed=1024" in repr(rz)
    assert rz._config == RzConfig(32, 64, 1, False)


def test_shared_hashed_weight_and_options():
    shared = torch.nn.Parameter(torch.randn(5000))
    a = RzLinear(64, 64, hashed_weight=shared, bias=False)
    b = RzLinear(64, 128, hashed_weight=shared, seed=3, hash_mode="single", prime=RzLinear.LARGE_PRIME,
                 block_size_k=64, block_size_n=64)
    assert a._hashed_weight is shared and b._hashed_weight is shared and a._bias is None
    assert int(b._random_numbers[0]) == RzLinear.LARGE_PRIME and b._config.hash_mode == 0
    c = RzLinear(64, 64, random_numbers=[RzLinear.LARGE_PRIME, 1, 2, 3, 4, 5, 6, 7])
    assert c._random_numbers.tolist() == [RzLinear.LARGE_PRIME, 1, 2, 3, 4, 5, 6, 7]
    with pytest.raises(AssertionError):
        RzLinear(10**5, 64)
    with pytest.raises(ValueError):
        RzLinear(64, 64, hash_mode="other")


def test_cpu_tensors_are_rejected_not_emulated():
    rz = RzLinear(64, 128, compress_ratio=0.5)
    with pytest.raises(RuntimeError, match="CUDA"):
        rz(torch.randn(4, 64))
    with pytest.raises(AssertionError):
        rz(torch.randn(64))
    small = RzLinear(64, 128)          # H = 512 <= 32*64: the reference's assert
    with pytest.raises(AssertionError):
        small(torch.randn(4, 64))
    with pytest.raises(TypeError):
        RzLinear(64, 128, compress_ratio=0.5)(torch.ones(4, 64, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="CUDA"):      # float16 is computed in float32, still only on the GPU
        RzLinear(64, 128, compress_ratio=0.5)(torch.randn(4, 64).half())


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from rzlinear_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()
