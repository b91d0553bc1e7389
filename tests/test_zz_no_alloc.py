"""rz_linear_forward_noalloc against the ordinary forward entry point.

The no-alloc variant serves hosts that cannot give the library scratch memory (their own pool owns
all of HBM, or they only pass pointers through a binding).  It must produce what rz_linear_forward
produces with a caller-allocated shadow.  Two calls in a row with different weights check that the
shared array's old contents do not leak into the second result.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
PRIME = 2038074743


def _case(rzlib, M, K, N, H, BK, BN, dtype, seed):
    rs = np.random.RandomState(seed)
    R = [PRIME] + [int(v) for v in rs.randint(1, 2**31 - 1, 7)]
    io, prec = (rzlib.BF16, rzlib.PREC_BF16) if dtype == torch.bfloat16 else (rzlib.F32, rzlib.PREC_TF32)
    pb = rzlib.make_problem(M, K, N, H, BK, BN, R, rzlib.HASH_SINGLE, io, prec, 0.5)
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(M, K, generator=g).to(dtype).to(DEV)
    h = ((torch.rand(H, generator=g) * 2 - 1) / K ** 0.5).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    return pb, X, h, bias


def _reference_forward(rzlib, pb, X, h, bias):
    nbytes = rzlib.shadow_bytes(pb)
    shadow = torch.empty(nbytes, dtype=torch.uint8, device=DEV) if nbytes else None
    if shadow is not None:
        rzlib.shadow_refresh(pb, h, shadow)
    Y = torch.empty((pb.M, pb.N), dtype=X.dtype, device=DEV)
    rzlib.forward(pb, X, h, shadow, bias, Y)
    return Y


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_forward_matches_forward_twice_in_a_row(rzlib, dtype):
    assert torch.cuda.is_available()
    # first call: a large hashed array fills most of the fixed scratch; second call: a smaller, different one
    cases = [_case(rzlib, 256, 512, 512, 1 << 20, 128, 128, dtype, 1),
             _case(rzlib, 384, 256, 768, 100003, 64, 128, dtype, 2)]
    for pb, X, h, bias in cases:
        assert rzlib.plan(pb, rzlib.OP_FORWARD) == rzlib.PATH_TCGEN05
        assert 0 < rzlib.shadow_bytes(pb) <= rzlib.NOALLOC_SCRATCH_BYTES
        want = _reference_forward(rzlib, pb, X, h, bias)
        got = torch.empty_like(want)
        rzlib.forward_noalloc(pb, X, h, bias, got)
        torch.cuda.synchronize()
        assert torch.equal(got, want)   # same kernels on the same shadow contents: bit-identical
        assert float(got.float().abs().sum()) > 0
    st, detail = rzlib.device_status()
    assert st == 0, (st, detail)


def test_noalloc_rejects_problems_beyond_the_fixed_scratch(rzlib):
    pb, X, h, bias = _case(rzlib, 256, 512, 512, (1 << 20) + 64, 128, 128, torch.bfloat16, 3)
    assert 8 * 2 * ((1 << 20) + 64) > rzlib.NOALLOC_SCRATCH_BYTES     # the shifted copies alone do not fit
    Y = torch.zeros((256, 512), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(rzlib.RzLinearError) as e:
        rzlib.forward_noalloc(pb, X, h, bias, Y)
    assert e.value.status == -10 and "capacity" in str(e.value)
    torch.cuda.synchronize()
    assert float(Y.float().abs().sum()) == 0.0      # nothing was launched


def test_noalloc_runs_without_the_workspace_when_only_the_copies_fit(rzlib):
    # few output blocks and a long contraction: the ordinary entry point splits the contraction and keeps fp32
    # partial sums in a workspace behind the copies.  Here the copies nearly fill the fixed array, so the
    # no-alloc call runs whole contractions per block instead: same result up to summation order.
    H = (1 << 20) - 64
    pb, X, h, bias = _case(rzlib, 32, 4096, 4096, H, 64, 64, torch.bfloat16, 5)
    copies = 8 * 2 * H
    assert copies <= rzlib.NOALLOC_SCRATCH_BYTES < rzlib.shadow_bytes(pb)
    want = _reference_forward(rzlib, pb, X, h, bias)
    for _ in range(2):
        got = torch.zeros_like(want)
        rzlib.forward_noalloc(pb, X, h, bias, got)
        torch.cuda.synchronize()
        err = float((got.float() - want.float()).norm() / want.float().norm())
        assert err < 2e-3, err                                # the tolerance of the bf16 tensor-core tests
    # with room for both, the no-alloc call splits the contraction like the ordinary one (the partial sums meet in
    # the workspace through atomic adds, so the order of summation, and with it the last bit, varies from run to run)
    pb2, X2, h2, bias2 = _case(rzlib, 32, 4096, 4096, 300007, 64, 64, torch.bfloat16, 6)
    assert 8 * 2 * 300032 < rzlib.shadow_bytes(pb2) <= rzlib.NOALLOC_SCRATCH_BYTES
    want2 = _reference_forward(rzlib, pb2, X2, h2, bias2)
    for _ in range(2):
        got2 = torch.zeros_like(want2)
        rzlib.forward_noalloc(pb2, X2, h2, bias2, got2)
        torch.cuda.synchronize()
        err = float((got2.float() - want2.float()).norm() / want2.float().norm())
        assert err < 2e-3, err
    assert rzlib.device_status() == (0, 0)


def test_noalloc_refuses_fp32_precision_that_needs_its_workspace(rzlib):
    # fp32 precision bounds its accumulation chains by splitting contractions longer than 2048: without room for
    # the workspace the call is refused rather than run at lower accuracy
    rs = np.random.RandomState(8)
    R = [PRIME] + [int(v) for v in rs.randint(1, 2**31 - 1, 7)]
    H = (1 << 20) - 64
    pb = rzlib.make_problem(256, 4096, 1024, H, 64, 64, R, rzlib.HASH_SINGLE, rzlib.F32, rzlib.PREC_FP32, 1.0)
    assert rzlib.plan(pb, 0) == rzlib.PATH_TCGEN05 and rzlib.shadow_bytes(pb) > rzlib.NOALLOC_SCRATCH_BYTES
    X = torch.randn(256, 4096, device=DEV)
    h = torch.rand(H, device=DEV)
    Y = torch.zeros(256, 1024, device=DEV)
    with pytest.raises(rzlib.RzLinearError) as e:
        rzlib.forward_noalloc(pb, X, h, None, Y)
    assert e.value.status == rzlib.RZ_ERR_TOO_LARGE
    torch.cuda.synchronize()
    assert float(Y.abs().sum()) == 0.0


def test_noalloc_fp32_path_needs_no_scratch(rzlib):
    # problems that run the FMA kernels have no shadow; the entry point then is the ordinary forward
    rs = np.random.RandomState(4)
    R = [PRIME] + [int(v) for v in rs.randint(1, 2**31 - 1, 7)]
    pb = rzlib.make_problem(64, 96, 160, 4000, 32, 32, R, rzlib.HASH_SINGLE, rzlib.F32, rzlib.PREC_FP32, 1.0)
    g = torch.Generator().manual_seed(4)
    X = torch.randn(64, 96, generator=g).to(DEV)
    h = torch.rand(4000, generator=g).to(DEV)
    want = _reference_forward(rzlib, pb, X, h, None)
    got = torch.empty_like(want)
    rzlib.forward_noalloc(pb, X, h, None, got)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
