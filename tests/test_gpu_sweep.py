"""Seeded sweep over shapes, hash tiles, hash modes and precisions: every tensor-core configuration
(single CTA, CTA pair, pair with two row blocks, split-precision fp32) against the fp32 FMA kernels of the
same library on the same inputs.  The FMA kernels are pinned to the oracle in test_gpu_parity.py."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PRIME = 2038074743


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def one_case(rzlib, rs, prec):
    bf16 = prec == rzlib.PREC_BF16
    unit = 8 if bf16 else 4                      # leading dimensions in multiples of 16 bytes
    tile_unit = 64 if bf16 else 32
    M = int(rs.choice([8, 32, 72, 128, 136, 200, 256, 384, 520, 640, 1024, 1500]))
    K = int(rs.randint(tile_unit // unit, 96)) * unit
    N = int(rs.randint(tile_unit // unit, 96)) * unit
    BK = int(rs.choice([32, 64, 128, 256]))
    BN = int(rs.choice([tile_unit, 2 * tile_unit, 3 * tile_unit, 128, 256]))
    if BK <= 128 and 128 % BK:
        BK = 128
    H = int(BK * BN + rs.randint(1, 200000))
    mode = int(rs.randint(0, 2))
    if mode == 0:
        R = [PRIME] + [int(v) for v in rs.randint(1, 2**31 - 1, 7)]
    else:
        R = [45007] + [int(v) for v in rs.randint(0, 45007, 7)]
    alpha = float(rs.choice([1.0, 0.5, 2.0]))
    dtype = torch.bfloat16 if bf16 else torch.float32
    io = rzlib.BF16 if bf16 else rzlib.F32
    g = torch.Generator(device=DEV).manual_seed(int(rs.randint(1 << 30)))
    X = torch.randn((M, K), generator=g, device=DEV).to(dtype)
    dY = torch.randn((M, N), generator=g, device=DEV).to(dtype)
    h = (torch.rand(H, generator=g, device=DEV) * 2 - 1) / K ** 0.5
    bias = torch.randn(N, generator=g, device=DEV)
    relu = bool(rs.randint(0, 2))
    flags = rzlib.FLAG_RELU if relu else 0
    pb = rzlib.make_problem(M, K, N, H, BK, BN, R, mode, io, prec, alpha, flags)
    ref = rzlib.make_problem(M, K, N, H, BK, BN, R, mode, io, prec, alpha, flags | rzlib.FLAG_FORCE_SIMT)
    desc = dict(M=M, K=K, N=N, H=H, BK=BK, BN=BN, mode=mode, prec=prec, relu=relu)
    if rzlib.plan(pb, 0) != rzlib.PATH_TCGEN05:
        return None, desc
    outs = []
    for p in (pb, ref):
        nbytes = rzlib.shadow_bytes(p)
        shadow = torch.empty(nbytes, dtype=torch.uint8, device=DEV) if nbytes else None
        hh = h
        if p is ref and bf16:
            hh = h.bfloat16().float()            # the tensor-core path rounds the weights to bf16
        if shadow is not None:
            rzlib.shadow_refresh(p, hh, shadow)
        Y = torch.empty((M, N), dtype=dtype, device=DEV)
        dX = torch.empty((M, K), dtype=dtype, device=DEV)
        dH = torch.empty(H, dtype=torch.float32, device=DEV)
        rzlib.forward(p, X, hh, shadow, bias, Y)
        rzlib.backward_input(p, dY, hh, shadow, dX)
        rzlib.backward_weight(p, X, dY, dH)
        outs.append((Y.float(), dX.float(), dH))
    torch.cuda.synchronize()
    errs = tuple(rel(a, b) for a, b in zip(outs[0], outs[1]))
    return errs, desc


@pytest.mark.parametrize("prec_name,tol,seed", [("bf16", 2e-3, 11), ("tf32", 2e-3, 12), ("fp32", 1e-5, 13)])
def test_sweep_tensor_core_vs_fma_kernels(rzlib, prec_name, tol, seed):
    prec = {"bf16": rzlib.PREC_BF16, "tf32": rzlib.PREC_TF32, "fp32": rzlib.PREC_FP32}[prec_name]
    rs = np.random.RandomState(seed)
    ran = 0
    for _ in range(24):
        errs, desc = one_case(rzlib, rs, prec)
        if errs is None:
            continue
        ran += 1
        assert max(errs) < tol, (errs, desc)
    assert ran >= 12
    st, detail = rzlib.device_status()
    assert st == 0, (st, detail)


def test_configs_forced(rzlib, monkeypatch):
    # the same problem through each of the three block shapes must agree with the FMA kernels
    rs = np.random.RandomState(5)
    for config in ("1", "2", "3"):
        monkeypatch.setenv("RZ_TC_CONFIG", config)
        rzlib.reload_env()          # the knobs are read once; this reads them again
        rs2 = np.random.RandomState(99)
        errs, desc = None, None
        while errs is None:
            errs, desc = one_case(rzlib, rs2, rzlib.PREC_BF16)
        assert max(errs) < 2e-3, (config, errs, desc)
    monkeypatch.delenv("RZ_TC_CONFIG")
    rzlib.reload_env()


@pytest.mark.parametrize("prec_name,tol", [("bf16", 2e-3), ("tf32", 2e-3), ("fp32", 1e-5)])
@pytest.mark.parametrize("M,K,N", [(32, 4096, 4096), (128, 4096, 2560), (8, 8192, 4096), (256, 8192, 4096)])
def test_split_contraction_small_batches(rzlib, prec_name, tol, M, K, N):
    # few output blocks and a long contraction: the contraction is split over CTAs, fp32 partial sums go
    # through the workspace that rz_shadow_bytes() adds to the scratch, a finalize kernel scales/biases/converts
    prec = {"bf16": rzlib.PREC_BF16, "tf32": rzlib.PREC_TF32, "fp32": rzlib.PREC_FP32}[prec_name]
    bf16 = prec == rzlib.PREC_BF16
    dtype = torch.bfloat16 if bf16 else torch.float32
    io = rzlib.BF16 if bf16 else rzlib.F32
    H, BK, BN = 300007, 64, 64
    R = [PRIME] + [int(v) for v in np.random.RandomState(M + K).randint(1, 2**31 - 1, 7)]
    g = torch.Generator(device=DEV).manual_seed(M * 7 + N)
    X = torch.randn((M, K), generator=g, device=DEV).to(dtype)
    dY = torch.randn((M, N), generator=g, device=DEV).to(dtype)
    h = (torch.rand(H, generator=g, device=DEV) * 2 - 1) / K ** 0.5
    bias = torch.randn(N, generator=g, device=DEV)
    pb = rzlib.make_problem(M, K, N, H, BK, BN, R, 0, io, prec, 0.5, rzlib.FLAG_RELU)
    ref = rzlib.make_problem(M, K, N, H, BK, BN, R, 0, io, prec, 0.5, rzlib.FLAG_RELU | rzlib.FLAG_FORCE_SIMT)
    assert rzlib.plan(pb, 0) == rzlib.PATH_TCGEN05
    copies = (16 // (2 if bf16 else 4)) * (-(-H // 64) * 64) * (2 if bf16 else 4)
    assert rzlib.shadow_bytes(pb) > copies          # the workspace is part of the scratch for these shapes
    nbytes = rzlib.shadow_bytes(pb)
    shadow = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    rzlib.shadow_refresh(pb, h, shadow)
    Y = torch.empty((M, N), dtype=dtype, device=DEV)
    dX = torch.empty((M, K), dtype=dtype, device=DEV)
    dH = torch.empty(H, dtype=torch.float32, device=DEV)
    rzlib.forward(pb, X, h, shadow, bias, Y)
    rzlib.backward_input(pb, dY, h, shadow, dX)
    rzlib.backward_weight(pb, X, dY, dH)
    dH_ref = torch.empty(H, dtype=torch.float32, device=DEV)
    rzlib.backward_weight(ref, X, dY, dH_ref)          # short contraction (M rows): the FMA kernels are exact enough
    torch.cuda.synchronize()
    assert rzlib.device_status() == (0, 0)
    # long contractions: fp64 matmul over the materialised weight (bit-exact gather) is the reference
    from rzlinear_b200.impl.launchers import rz_linear_idx_tl
    hw = h.bfloat16().float() if bf16 else h
    W = rz_linear_idx_tl(hw, K, N, H, R[3], R[2], R[1], R[0], BK, BN).double()
    Y_ref = torch.relu(0.5 * (X.double() @ W) + bias.double())
    dX_ref = 0.5 * (dY.double() @ W.t())
    errs = (rel(Y.float(), Y_ref), rel(dX.float(), dX_ref), rel(dH, dH_ref))
    assert max(errs) < tol, errs
