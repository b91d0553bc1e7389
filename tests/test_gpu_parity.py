"""Parity of the CUDA kernels (through the C ABI) with the CPU oracle and the reference fixtures.

Tolerances (rel-L2): 1e-5 for the fp32 path, 2e-3 for the tf32 and bf16 tensor-core paths (for
bf16 the oracle consumes the same bf16-rounded operands the kernels see and accumulates in fp64);
hash offsets and the materialised weight are bit-exact.
"""
import os

import numpy as np
import pytest
import torch

from oracle import rz_oracle as o

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
LARGE_PRIME = 2038074743
TOL_FP32 = 1e-5
TOL_TC = 2e-3


@pytest.fixture(scope="module")
def L(rzlib):
    assert torch.cuda.is_available(), "these tests need a GPU"
    rzlib.load()
    from rzlinear_b200.impl import launchers
    return launchers


def seeded_R(seed, prime=LARGE_PRIME):
    rs = np.random.RandomState(seed)
    if prime == LARGE_PRIME:
        return [prime] + [int(v) for v in rs.randint(1, 2**31 - 1, 7)]
    return [prime] + [int(v) for v in rs.randint(0, prime, 7)]


def run_three(L, X, dY, h, N, BK, BN, R, mode, alpha=1.0, allow_tf32=False):
    M, K = X.shape
    H = h.shape[0]
    Rargs = (R[7], R[6], R[5], R[4], R[3], R[2], R[1], R[0])
    kw = dict(allow_tf32=allow_tf32, allow_autotune=False, BLOCK_SIZE_K=BK, BLOCK_SIZE_N=BN, hash_mode=mode)
    Y = L.rz_linear_forward_tl(X, h, alpha, M, K, N, H, *Rargs, **kw)
    dX = L.rz_linear_backward_input_grad_tl(dY, h, alpha, M, K, N, H, *Rargs, **kw)
    dH = L.rz_linear_backward_weight_grad_tl(X, dY, alpha, M, K, N, H, *Rargs, **kw)
    torch.cuda.synchronize()
    return Y.float().cpu().numpy(), dX.float().cpu().numpy(), dH.cpu().numpy()


def check_status(rzlib):
    st, detail = rzlib.device_status()
    assert st == 0, f"device pipeline reported status {st}, wait code {detail}"


# ---------------------------------------------------------------------------------------------
# hash
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("K,N,H,BK,BN,mode,prime", [
    (1024, 1024, 65536, 32, 32, 0, LARGE_PRIME),
    (4096, 4096, 1 << 20, 64, 64, 0, LARGE_PRIME),
    (8192, 32768, 1 << 22, 128, 128, 0, LARGE_PRIME),
    (8192, 8192, 1 << 22, 128, 128, 0, LARGE_PRIME),
    (1000, 777, 5000, 16, 24, 0, LARGE_PRIME),
    (1024, 1024, 65536, 32, 64, 1, 45007),
    (256, 256, 1025, 32, 32, 0, LARGE_PRIME),
])
def test_device_hash_offsets_bit_exact(rzlib, L, K, N, H, BK, BN, mode, prime):
    for seed in (1, 2):
        R = seeded_R(seed + K, prime)
        pb = rzlib.make_problem(1, K, N, H, BK, BN, R, mode, 0, 0)
        got = rzlib.hash_indices_device(pb, DEV).cpu().numpy()
        want = o.tile_offsets(K, N, H, BK, BN, R, mode)
        assert np.array_equal(got, want)
        assert np.array_equal(rzlib.hash_indices_host(pb), want)


@pytest.mark.parametrize("tag", ["idx_a", "idx_b"])
def test_materialize_matches_reference_idx_kernel(L, golden_dir, tag):
    d = np.load(os.path.join(golden_dir, tag + ".npz"))
    K, N, H, BK, BN = (int(v) for v in d["dims"])
    R = [int(v) for v in d["R"]]
    W = L.rz_linear_idx_tl(torch.from_numpy(d["hashed"]).to(DEV), K, N, H, R[3], R[2], R[1], R[0], BK, BN)
    assert np.array_equal(W.cpu().numpy(), d["W"])


def test_materialize_large_prime_and_ragged(L):
    K, N, H, BK, BN = 200, 300, 9000, 32, 64
    R = seeded_R(5)
    h = torch.rand(H, generator=torch.Generator().manual_seed(1))
    W = L.rz_linear_idx_tl(h.to(DEV), K, N, H, R[3], R[2], R[1], R[0], BK, BN)
    assert np.array_equal(W.cpu().numpy(), o.materialize(h.numpy(), K, N, BK, BN, R, 0))


# ---------------------------------------------------------------------------------------------
# fp32 path against the reference's own outputs and the oracle
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["k_full", "k_ragged", "k_small_tiles"])
def test_fp32_kernels_match_reference_fixtures(rzlib, L, golden_dir, tag):
    d = np.load(os.path.join(golden_dir, tag + ".npz"))
    M, K, N, H, BK, BN = (int(v) for v in d["dims"])
    R, a = [int(v) for v in d["R"]], float(d["alpha"])
    X, dY, h = (torch.from_numpy(d[k]).to(DEV) for k in ("X", "dY", "hashed"))
    Y, dX, dH = run_three(L, X, dY, h, N, BK, BN, R, 1, a)
    for got, key in ((Y, "Y"), (dX, "dX"), (dH, "dH")):
        assert o.rel_l2(got, d[key]) < TOL_FP32, key
    assert o.rel_l2(Y, o.forward(d["X"], d["hashed"], N, BK, BN, R, 1, a)) < TOL_FP32
    assert o.rel_l2(dX, o.backward_input(d["dY"], d["hashed"], K, BK, BN, R, 1, a)) < TOL_FP32
    assert o.rel_l2(dH, o.backward_weight(d["X"], d["dY"], H, BK, BN, R, 1, a)) < TOL_FP32
    check_status(rzlib)


def make_inputs(M, K, N, H, seed, dtype=torch.float32, h_scale=None):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(M, K, generator=g).to(dtype)
    dY = torch.randn(M, N, generator=g).to(dtype)
    s = h_scale if h_scale is not None else 1.0 / np.sqrt(K)
    h = (torch.rand(H, generator=g) * 2 - 1) * s
    return X, dY, h


def test_fp32_config_1024_cubed_single_level(rzlib, L):
    # fp32, M=K=N=1024, H=65536, 32x32 tiles, large prime, seeded R in [1, 2^31)
    M = K = N = 1024
    H, BK, BN = 65536, 32, 32
    R = seeded_R(1234)
    X, dY, h = make_inputs(M, K, N, H, 1001, h_scale=1 / 32)
    Y, dX, dH = run_three(L, X.to(DEV), dY.to(DEV), h.to(DEV), N, BK, BN, R, 0)
    assert o.rel_l2(Y, o.forward(X.numpy(), h.numpy(), N, BK, BN, R, 0)) < TOL_FP32
    assert o.rel_l2(dX, o.backward_input(dY.numpy(), h.numpy(), K, BK, BN, R, 0)) < TOL_FP32
    assert o.rel_l2(dH, o.backward_weight(X.numpy(), dY.numpy(), H, BK, BN, R, 0)) < TOL_FP32
    check_status(rzlib)


@pytest.mark.parametrize("R", [
    [LARGE_PRIME, 99, LARGE_PRIME, 12345, 0, 0, 0, 0],   # R2 = 0 mod P: rows of tiles collide exactly
    [LARGE_PRIME, 99, 0, 0, 0, 0, 0, 0],                 # every tile on one slice
    [LARGE_PRIME, 7, 3, 5, 0, 0, 0, 0],                  # small multipliers: neighbouring slices overlap partly
])
def test_fp32_colliding_tiles(L, R):
    M, K, N, H, BK, BN = 96, 128, 256, 3000, 32, 32
    X, dY, h = make_inputs(M, K, N, H, 7)
    Y, dX, dH = run_three(L, X.to(DEV), dY.to(DEV), h.to(DEV), N, BK, BN, R, 0, alpha=0.5)
    assert o.rel_l2(Y, o.forward(X.numpy(), h.numpy(), N, BK, BN, R, 0, 0.5)) < TOL_FP32
    assert o.rel_l2(dX, o.backward_input(dY.numpy(), h.numpy(), K, BK, BN, R, 0, 0.5)) < TOL_FP32
    assert o.rel_l2(dH, o.backward_weight(X.numpy(), dY.numpy(), H, BK, BN, R, 0, 0.5)) < TOL_FP32


def test_fp32_odd_shapes_and_single_row(L):
    for (M, K, N, H, BK, BN) in [(1, 7, 5, 100, 3, 4), (33, 65, 129, 777, 16, 24), (5, 300, 70, 5000, 64, 8)]:
        R = seeded_R(M + K)
        X, dY, h = make_inputs(M, K, N, H, 3)
        Y, dX, dH = run_three(L, X.to(DEV), dY.to(DEV), h.to(DEV), N, BK, BN, R, 0)
        assert o.rel_l2(Y, o.forward(X.numpy(), h.numpy(), N, BK, BN, R, 0)) < TOL_FP32
        assert o.rel_l2(dX, o.backward_input(dY.numpy(), h.numpy(), K, BK, BN, R, 0)) < TOL_FP32
        assert o.rel_l2(dH, o.backward_weight(X.numpy(), dY.numpy(), H, BK, BN, R, 0)) < TOL_FP32


def test_accumulate_flag_and_relu_bias(rzlib, L):
    M, K, N, H, BK, BN = 64, 96, 160, 4000, 32, 32
    R = seeded_R(11)
    X, dY, h = make_inputs(M, K, N, H, 5)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(2))
    Rargs = (R[7], R[6], R[5], R[4], R[3], R[2], R[1], R[0])
    Y = L.rz_linear_forward_tl(X.to(DEV), h.to(DEV), 1.0, M, K, N, H, *Rargs, allow_tf32=False, BLOCK_SIZE_K=BK,
                               BLOCK_SIZE_N=BN, hash_mode=0, bias=bias.to(DEV), relu=True)
    want = np.maximum(o.forward(X.numpy(), h.numpy(), N, BK, BN, R, 0) + bias.numpy().astype(np.float64), 0)
    assert o.rel_l2(Y.cpu().numpy(), want) < TOL_FP32
    # accumulate: two calls into the same dH give twice the gradient
    pb = rzlib.make_problem(M, K, N, H, BK, BN, R, 0, 0, 0, 1.0, rzlib.FLAG_ACCUMULATE_DH)
    dh = torch.zeros(H, device=DEV)
    rzlib.backward_weight(pb, X.to(DEV), dY.to(DEV), dh)
    rzlib.backward_weight(pb, X.to(DEV), dY.to(DEV), dh)
    assert o.rel_l2(dh.cpu().numpy(), 2 * o.backward_weight(X.numpy(), dY.numpy(), H, BK, BN, R, 0)) < TOL_FP32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N", [(257, 512), (64, 100), (1, 8), (3000, 4096)])
def test_grad_prepare_masks_and_sums(rzlib, dtype, M, N):
    # backward of the fused bias + ReLU epilogue: masked gradient bit-identical to the elementwise definition,
    # bias gradient = fp64 column sums within fp32 accumulation error
    g = torch.Generator().manual_seed(M * 7 + N)
    dY = torch.randn(M, N, generator=g).to(dtype)
    Y = torch.relu(torch.randn(M, N, generator=g)).to(dtype)
    pb = rzlib.make_problem(M, 64, N, 70000, 32, 32, seeded_R(1), 0, rzlib.torch_io_dtype(dtype),
                            rzlib.PREC_BF16 if dtype == torch.bfloat16 else rzlib.PREC_FP32)
    dYd, Yd = dY.to(DEV), Y.to(DEV)
    masked = torch.full((M, N), 7.0, device=DEV, dtype=dtype)
    bg = torch.full((N,), 7.0, device=DEV)
    rzlib.grad_prepare(pb, dYd, Yd, masked, bg)
    want = torch.where(Y > 0, dY, torch.zeros_like(dY))
    assert torch.equal(masked.cpu(), want)
    ref = want.double().sum(0).numpy()
    assert np.abs(bg.cpu().numpy() - ref).max() <= 1e-5 * max(1.0, np.abs(want.double()).sum(0).max())
    # bias gradient alone (no mask, nothing written)
    bg2 = torch.empty((N,), device=DEV)
    rzlib.grad_prepare(pb, dYd, None, None, bg2)
    ref2 = dY.double().sum(0).numpy()
    assert np.abs(bg2.cpu().numpy() - ref2).max() <= 1e-5 * max(1.0, dY.double().abs().sum(0).max().item())
    # mask alone; a misaligned view takes the scalar path
    if N > 8:
        flat = torch.empty(M * N + 1, device=DEV, dtype=dtype)
        dv = flat[1:].view(M, N)
        dv.copy_(dYd)
        m2 = torch.empty((M, N), device=DEV, dtype=dtype)
        rzlib.grad_prepare(pb, dv, Yd, m2, None)
        assert torch.equal(m2.cpu(), want)


# ---------------------------------------------------------------------------------------------
# module / autograd
# ---------------------------------------------------------------------------------------------
def test_module_matches_reference_fixture(golden_dir):
    from rzlinear_b200 import RzLinear
    d = np.load(os.path.join(golden_dir, "module.npz"))
    rz = RzLinear(input_dim=64, output_dim=128, seed=1024, compress_ratio=0.75, init_factor=0.125)
    assert [int(v) for v in rz._random_numbers] == [int(v) for v in d["R"]]
    with torch.no_grad():
        rz._hashed_weight.copy_(torch.from_numpy(d["hashed"]))
        rz._bias.copy_(torch.from_numpy(d["bias"]))
    rz = rz.to(DEV)
    x = torch.from_numpy(d["x"]).to(DEV).requires_grad_(True)
    y = rz(x)
    assert y.shape == (3, 10, 128)
    y.backward(torch.from_numpy(d["gy"]).to(DEV))
    assert o.rel_l2(y.detach().cpu().numpy(), d["y"]) < TOL_FP32
    assert o.rel_l2(x.grad.cpu().numpy(), d["dx"]) < TOL_FP32
    assert o.rel_l2(rz._hashed_weight.grad.cpu().numpy(), d["dh"]) < TOL_FP32
    assert o.rel_l2(rz._bias.grad.cpu().numpy(), d["dbias"]) < TOL_FP32


def test_default_module_on_bf16_activations_runs_the_tensor_core_path(rzlib):
    # RzLinear with nothing but its dimensions: the reference's defaults (two-level hash, prime 45007, 32 x 64 hash
    # tile, compress_ratio 1/16).  On bf16 activations all three products take the tcgen05 kernels.
    from rzlinear_b200 import RzLinear
    torch.manual_seed(11)
    K, N, M = 512, 768, 320
    rz = RzLinear(K, N, seed=7).to(DEV)
    H = rz._hashed_weight.numel()
    with torch.no_grad():
        rz._hashed_weight.copy_((torch.rand(H, device=DEV) * 2 - 1) / K ** 0.5)
        rz._bias.copy_(torch.randn(N, device=DEV) * 0.1)
    R = [int(v) for v in rz._random_numbers]
    pb = rzlib.make_problem(M, K, N, H, 32, 64, R, rzlib.HASH_TWO_LEVEL, rzlib.BF16, rzlib.PREC_BF16)
    assert all(rzlib.plan(pb, op) == rzlib.PATH_TCGEN05 for op in (0, 1, 2))
    x = torch.randn(M, K, device=DEV).bfloat16().requires_grad_(True)
    gy = torch.randn(M, N, device=DEV).bfloat16()
    n0 = rzlib.launch_count()
    y = rz(x)
    y.backward(gy)
    torch.cuda.synchronize()
    check_status(rzlib)
    assert rzlib.launch_count() - n0 <= 8            # refresh, forward, bias-gradient pass, dX, memset-free dH ...
    hf = o.bf16_round(rz._hashed_weight.detach().cpu().numpy())
    xf, gf = x.detach().float().cpu().numpy(), gy.float().cpu().numpy()
    want_y = o.forward(xf, hf, N, 32, 64, R, 1) + rz._bias.detach().cpu().numpy().astype(np.float64)
    assert o.rel_l2(y.detach().float().cpu().numpy(), want_y) < TOL_TC
    assert o.rel_l2(x.grad.float().cpu().numpy(), o.backward_input(gf, hf, K, 32, 64, R, 1)) < TOL_TC
    assert o.rel_l2(rz._hashed_weight.grad.cpu().numpy(), o.backward_weight(xf, gf, H, 32, 64, R, 1)) < TOL_TC
    assert o.rel_l2(rz._bias.grad.cpu().numpy(), gf.sum(0)) < 1e-5


def test_module_accepts_float16_activations():
    # float16 is not a kernel dtype: the layer computes in float32 (tf32 allowed by default) and casts back
    from rzlinear_b200 import RzLinear
    torch.manual_seed(3)
    hw = torch.nn.Parameter((torch.rand(12288) * 2 - 1) / 128 ** 0.5)   # (the default initialisation is far outside float16's range)
    rz = RzLinear(128, 192, hashed_weight=hw, seed=5, bias=True).to(DEV)
    x16 = torch.randn(40, 128, device=DEV).half().requires_grad_(True)
    y16 = rz(x16)
    assert y16.dtype == torch.float16 and y16.shape == (40, 192)
    y16.float().pow(2).sum().backward()
    g16, gh16 = x16.grad.clone(), rz._hashed_weight.grad.clone()
    assert g16.dtype == torch.float16
    rz._hashed_weight.grad = None
    x32 = x16.detach().float().requires_grad_(True)
    y32 = rz(x32)
    y32.pow(2).sum().backward()
    errs = (o.rel_l2(y16.detach().float().cpu().numpy(), y32.detach().cpu().numpy()),
            o.rel_l2(g16.float().cpu().numpy(), x32.grad.cpu().numpy()),
            o.rel_l2(gh16.cpu().numpy(), rz._hashed_weight.grad.cpu().numpy()))
    # float16 rounding of the output and of the incoming gradient (2^-11 per element) is all that separates the two runs
    assert max(errs) < 2e-3, errs


def test_module_shape_smoke_like_reference_test_module():
    from rzlinear_b200 import RzLinear
    rz = RzLinear(input_dim=1024, output_dim=1024).to(DEV)
    out = rz(torch.rand((1024, 1024), device=DEV))
    assert out.shape == (1024, 1024)


def test_module_skips_input_grad_and_shares_weight():
    from rzlinear_b200 import RzLinear
    shared = torch.nn.Parameter(torch.randn(20000, device=DEV) * 0.05)
    a = RzLinear(128, 128, hashed_weight=shared, seed=1).to(DEV)
    b = RzLinear(128, 64, hashed_weight=shared, seed=2, relu=True).to(DEV)
    x = torch.randn(32, 128, device=DEV)            # no grad needed for the input
    loss = b(a(x)).square().mean()
    loss.backward()
    assert shared.grad is not None and shared.grad.shape == shared.shape and x.grad is None
    # compare with autograd through the materialised weights
    from rzlinear_b200.impl.launchers import rz_linear_idx_tl
    Ra, Rb = a._random_numbers.tolist(), b._random_numbers.tolist()
    sh = shared.detach().clone().requires_grad_(True)
    idx_a = torch.from_numpy(o.element_index(128, 128, 20000, 32, 64, Ra, 1)).to(DEV)
    idx_b = torch.from_numpy(o.element_index(128, 64, 20000, 32, 64, Rb, 1)).to(DEV)
    ref = torch.relu((x @ sh[idx_a] + a._bias.detach()) @ sh[idx_b] + b._bias.detach()).square().mean()
    ref.backward()
    assert o.rel_l2(shared.grad.cpu().numpy(), sh.grad.cpu().numpy()) < 1e-4
    assert abs(float(loss) - float(ref)) < 1e-4 * abs(float(ref))


# ---------------------------------------------------------------------------------------------
# tensor-core paths
# ---------------------------------------------------------------------------------------------
def tc_case(rzlib, L, M, K, N, H, BK, BN, dtype, seed, alpha=1.0, mode=0, allow_tf32=None):
    if allow_tf32 is None:
        allow_tf32 = dtype == torch.float32
    R = seeded_R(seed) if mode == 0 else seeded_R(seed, 45007)
    X, dY, h = make_inputs(M, K, N, H, seed, dtype)
    pb = rzlib.make_problem(M, K, N, H, BK, BN, R, mode, 1 if dtype == torch.bfloat16 else 0,
                            2 if dtype == torch.bfloat16 else (1 if allow_tf32 else 0), alpha)
    for op in (0, 1, 2):
        assert rzlib.plan(pb, op) == rzlib.PATH_TCGEN05
    Y, dX, dH = run_three(L, X.to(DEV), dY.to(DEV), h.to(DEV), N, BK, BN, R, mode, alpha, allow_tf32)
    check_status(rzlib)
    Xf, dYf = X.float().numpy(), dY.float().numpy()
    hf = o.bf16_round(h.numpy()) if dtype == torch.bfloat16 else h.numpy()
    eY = o.rel_l2(Y, o.forward(Xf, hf, N, BK, BN, R, mode, alpha))
    eX = o.rel_l2(dX, o.backward_input(dYf, hf, K, BK, BN, R, mode, alpha))
    eH = o.rel_l2(dH, o.backward_weight(Xf, dYf, H, BK, BN, R, mode, alpha))
    return eY, eX, eH


@pytest.mark.parametrize("M,K,N,H,BK,BN", [
    (256, 512, 512, 1 << 17, 128, 128),
    (256, 512, 512, 1 << 17, 64, 64),
    (384, 256, 768, 100003, 64, 128),      # odd H, rectangular tile
    (300, 320, 328, 1 << 16, 64, 64),      # ragged M, K, N (multiples of 8 only)
    (128, 1024, 256, 1 << 18, 256, 64),
    (256, 512, 512, 1 << 16, 32, 64),      # the module's default hash tile: two hash tiles per 64-row stage
    (520, 328, 1032, 50001, 32, 128),      # the same, ragged, pair blocks
])
def test_bf16_tensor_core_path(rzlib, L, M, K, N, H, BK, BN):
    eY, eX, eH = tc_case(rzlib, L, M, K, N, H, BK, BN, torch.bfloat16, seed=M + K + BK, alpha=0.75)
    assert eY < TOL_TC and eX < TOL_TC and eH < TOL_TC, (eY, eX, eH)


@pytest.mark.parametrize("M,K,N,H,BK,BN", [
    (256, 256, 512, 1 << 17, 64, 64),
    (256, 512, 256, 1 << 16, 32, 32),
    (200, 132, 260, 50001, 32, 64),        # ragged (multiples of 4 only), odd H
])
def test_tf32_tensor_core_path(rzlib, L, M, K, N, H, BK, BN):
    eY, eX, eH = tc_case(rzlib, L, M, K, N, H, BK, BN, torch.float32, seed=M + K + BK)
    assert eY < TOL_TC and eX < TOL_TC and eH < TOL_TC, (eY, eX, eH)


@pytest.mark.parametrize("M,K,N,H,BK,BN", [
    (256, 256, 512, 1 << 17, 64, 64),      # CTA pair
    (1024, 1024, 1024, 65536, 32, 32),     # the fp32 baseline configuration
    (200, 132, 260, 50001, 32, 64),        # single CTA, ragged
    (640, 512, 384, 1 << 16, 128, 32),
])
def test_fp32_precision_on_tensor_cores(rzlib, L, M, K, N, H, BK, BN):
    # fp32 in, fp32-grade out: split operands (hi + lo), three tf32 MMAs per product; the fp32 bar applies
    eY, eX, eH = tc_case(rzlib, L, M, K, N, H, BK, BN, torch.float32, seed=M + N + BN, alpha=1.25, allow_tf32=False)
    assert eY < TOL_FP32 and eX < TOL_FP32 and eH < TOL_FP32, (eY, eX, eH)


def test_tensor_core_two_level_hash_and_collisions(rzlib, L):
    eY, eX, eH = tc_case(rzlib, L, 256, 512, 512, 1 << 16, 64, 64, torch.bfloat16, seed=9, mode=1)
    assert eY < TOL_TC and eX < TOL_TC and eH < TOL_TC, (eY, eX, eH)
    # colliding tiles, merged in registers by the weight-gradient epilogue before the reductions:
    #   R2 = 0 mod P           -> all tiles of a tile row share one slice
    #   R2 = (H - BK*BN) / 2   -> every second tile of a tile row shares a slice
    #   R2 = 100               -> neighbouring slices overlap partly (left to the L2 atomics)
    M, K, N, H, BK, BN = 512, 256, 768, 40000, 64, 64
    for R2 in (LARGE_PRIME, (H - BK * BN) // 2, 100):
        R = [LARGE_PRIME, 99, R2, 12345, 0, 0, 0, 0]
        off = o.tile_offsets(K, N, H, BK, BN, R, 0)
        if R2 == LARGE_PRIME:
            assert (off == off[:, :1]).all()
        elif R2 != 100:
            assert (off[:, 0] == off[:, 2]).all() and (off[:, 0] != off[:, 1]).all()
        X, dY, h = make_inputs(M, K, N, H, 4, torch.bfloat16)
        Y, dX, dH = run_three(L, X.to(DEV), dY.to(DEV), h.to(DEV), N, BK, BN, R, 0)
        hf = o.bf16_round(h.numpy())
        assert o.rel_l2(Y, o.forward(X.float().numpy(), hf, N, BK, BN, R, 0)) < TOL_TC
        assert o.rel_l2(dX, o.backward_input(dY.float().numpy(), hf, K, BK, BN, R, 0)) < TOL_TC
        assert o.rel_l2(dH, o.backward_weight(X.float().numpy(), dY.float().numpy(), H, BK, BN, R, 0)) < TOL_TC
    check_status(rzlib)


# ---------------------------------------------------------------------------------------------
# failure detection: a device-side wait that runs out is reported, nothing hangs or faults
# ---------------------------------------------------------------------------------------------
def test_bounded_wait_reports_timeout_and_context_survives(rzlib, L):
    assert rzlib.device_status() == (0, 0)
    rzlib.selftest_bounded_wait(2_000_000, DEV)          # about a millisecond of waiting on a flag nothing sets
    st, detail = rzlib.device_status()
    assert st == -8 and detail == 6                      # RZ_ERR_PIPELINE, wait code of the self-test
    assert "pipeline" in rzlib.load().rz_status_string(st).decode()
    assert rzlib.device_status() == (0, 0)               # reading the status clears it
    # the context is still usable: a tensor-core problem runs and matches the oracle
    eY, eX, eH = tc_case(rzlib, L, 256, 512, 512, 1 << 17, 128, 128, torch.bfloat16, seed=3)
    assert max(eY, eX, eH) < TOL_TC
    with pytest.raises(rzlib.RzLinearError):
        rzlib.selftest_bounded_wait(0, DEV)
