"""Parity at the full sizes of the baseline configurations, where a full CPU oracle pass is too slow.

Three witnesses.  (1) The oracle on a sample: forward on sampled rows x sampled column tiles and input gradient
on sampled rows x sampled row tiles of the virtual weight (oracle index arithmetic, fp64 products of exactly the
operands the kernels see), and the hashed-weight gradient on sampled words - for word j the oracle enumerates
every (k, n) whose element lands on j and the test sums X[:, k] . dY[:, n] in fp64.  (2) The fp32 FMA kernels of
the same library on the same inputs (themselves pinned to the oracle and to the reference's fixtures at small
sizes).  (3) Properties that do not depend on size: the sum of the hashed-weight gradient equals
alpha * sum_m (sum_k X[m,k]) (sum_n dY[m,n]) because every element of X^T.dY is added exactly once, and the
gradient is additive over row blocks.
"""
import numpy as np
import pytest
import torch

from oracle import rz_oracle as o

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
PRIME = 2038074743
TOL_TC = 2e-3


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm())


def run(rzlib, pb, X, dY, h, ops=("fwd", "dx", "dw")):
    nbytes = rzlib.shadow_bytes(pb)
    shadow = torch.empty(nbytes, dtype=torch.uint8, device=DEV) if nbytes else None
    if shadow is not None:
        rzlib.shadow_refresh(pb, h, shadow)
    out = {}
    if "fwd" in ops:
        out["fwd"] = torch.empty((pb.M, pb.N), dtype=X.dtype, device=DEV)
        rzlib.forward(pb, X, h, shadow, None, out["fwd"])
    if "dx" in ops:
        out["dx"] = torch.empty((pb.M, pb.K), dtype=X.dtype, device=DEV)
        rzlib.backward_input(pb, dY, h, shadow, out["dx"])
    if "dw" in ops:
        out["dw"] = torch.empty(pb.H, dtype=torch.float32, device=DEV)
        rzlib.backward_weight(pb, X, dY, out["dw"])
    torch.cuda.synchronize()
    return out


def case(rzlib, M, K, N, H, BK, BN, dtype, seed, h_scale, alpha=1.0):
    R = [PRIME] + [int(v) for v in np.random.RandomState(seed).randint(1, 2**31 - 1, 3)] + [0, 0, 0, 0]
    g = torch.Generator(device=DEV).manual_seed(seed)
    X = torch.randn((M, K), generator=g, device=DEV).to(dtype)
    dY = torch.randn((M, N), generator=g, device=DEV).to(dtype)
    h = (torch.rand(H, generator=g, device=DEV) * 2 - 1) * h_scale
    io, prec = (rzlib.BF16, rzlib.PREC_BF16) if dtype == torch.bfloat16 else (rzlib.F32, rzlib.PREC_TF32)
    pb = rzlib.make_problem(M, K, N, H, BK, BN, R, rzlib.HASH_SINGLE, io, prec, alpha)
    pb_ref = rzlib.make_problem(M, K, N, H, BK, BN, R, rzlib.HASH_SINGLE, io, prec, alpha, rzlib.FLAG_FORCE_SIMT)
    for op in (0, 1, 2):
        assert rzlib.plan(pb, op) == rzlib.PATH_TCGEN05 and rzlib.plan(pb_ref, op) == rzlib.PATH_SIMT
    return pb, pb_ref, X, dY, h


def check_against_oracle_sample(pb, X, dY, h, got, rows=256, words=320):
    """The oracle's index arithmetic and fp64 products on a sample of the outputs (tolerance TOL_TC, rel-L2)."""
    M, K, N, H, BK, BN = pb.M, pb.K, pb.N, pb.H, pb.BK, pb.BN
    R, mode, alpha = list(pb.R), pb.hash_mode, float(pb.alpha)
    rs = np.random.RandomState(7)
    bf16 = X.dtype == torch.bfloat16
    hw = (h.bfloat16() if bf16 else h).double()                       # the weights as the tensor cores see them
    ridx = torch.from_numpy(np.sort(rs.choice(M, rows, replace=False))).to(DEV)
    Xs, dYs = X[ridx].double(), dY[ridx].double()
    # forward: all of K, a few column tiles
    ns = np.concatenate([np.arange(t * BN, min(N, (t + 1) * BN)) for t in np.sort(rs.choice(-(-N // BN), 3, replace=False))])
    idx = torch.from_numpy(o.element_index_block(K, N, H, BK, BN, R, mode, np.arange(K), ns)).to(DEV)
    want = alpha * (Xs @ hw[idx])
    assert rel(got["fwd"][ridx][:, torch.from_numpy(ns).to(DEV)].float(), want) < TOL_TC
    # input gradient: all of N, a few row tiles of the virtual weight
    ks = np.concatenate([np.arange(t * BK, min(K, (t + 1) * BK)) for t in np.sort(rs.choice(-(-K // BK), 3, replace=False))])
    idx = torch.from_numpy(o.element_index_block(K, N, H, BK, BN, R, mode, ks, np.arange(N))).to(DEV)
    want = alpha * (dYs @ hw[idx].t())
    assert rel(got["dx"][ridx][:, torch.from_numpy(ks).to(DEV)].float(), want) < TOL_TC
    # hashed-weight gradient: sampled words, every virtual element that lands on them, all rows
    js = np.sort(rs.choice(H, words, replace=False))
    pairs = [o.elements_of_word(int(j), K, N, H, BK, BN, R, mode) for j in js]
    owner = np.concatenate([np.full(len(k), i) for i, (k, _) in enumerate(pairs)])
    kall = torch.from_numpy(np.concatenate([k for k, _ in pairs])).to(DEV)
    nall = torch.from_numpy(np.concatenate([n for _, n in pairs])).to(DEV)
    dots = torch.empty(len(owner), dtype=torch.float64, device=DEV)
    for c0 in range(0, len(owner), 1024):                             # M x 1024 fp64 products at a time
        sl = slice(c0, c0 + 1024)
        dots[sl] = (X[:, kall[sl]].double() * dY[:, nall[sl]].double()).sum(0)
    want = torch.zeros(words, dtype=torch.float64, device=DEV).index_add_(0, torch.from_numpy(owner).to(DEV), dots) * alpha
    assert len(owner) > words                                         # (compression: several elements per word)
    assert rel(got["dw"][torch.from_numpy(js).to(DEV)], want) < TOL_TC


def check_against_fma_kernels(rzlib, pb, pb_ref, X, dY, h, rows=256):
    got = run(rzlib, pb, X, dY, h)
    st, detail = rzlib.device_status()
    assert st == 0, (st, detail)
    check_against_oracle_sample(pb, X, dY, h, got)
    # forward / input gradient are row-independent: the FMA kernels redo a sample of rows
    idx = torch.randperm(pb.M, generator=torch.Generator().manual_seed(1))[:rows].sort().values.to(DEV)
    R = list(pb.R)
    sub = rzlib.make_problem(rows, pb.K, pb.N, pb.H, pb.BK, pb.BN, R, pb.hash_mode, pb.io_dtype, pb.precision, pb.alpha,
                             rzlib.FLAG_FORCE_SIMT)
    h_used = h.bfloat16().float() if X.dtype == torch.bfloat16 else h   # the tensor-core path rounds the weights
    ref = run(rzlib, sub, X[idx].contiguous(), dY[idx].contiguous(), h_used, ops=("fwd", "dx"))
    assert rel(got["fwd"][idx].float(), ref["fwd"].float()) < TOL_TC
    assert rel(got["dx"][idx].float(), ref["dx"].float()) < TOL_TC
    # the hashed-weight gradient contracts over all rows: redo all of it with the FMA kernels
    ref_dw = run(rzlib, pb_ref, X, dY, h, ops=("dw",))["dw"]
    assert rel(got["dw"], ref_dw) < TOL_TC
    # size-independent properties
    want_sum = float(pb.alpha) * float((X.double().sum(1) * dY.double().sum(1)).sum())
    scale = float(got["dw"].double().abs().sum())
    assert abs(float(got["dw"].double().sum()) - want_sum) < 1e-4 * scale
    half = pb.M // 2
    Rl = list(pb.R)
    pb_half = rzlib.make_problem(half, pb.K, pb.N, pb.H, pb.BK, pb.BN, Rl, pb.hash_mode, pb.io_dtype, pb.precision, pb.alpha)
    a = run(rzlib, pb_half, X[:half].contiguous(), dY[:half].contiguous(), h, ops=("dw",))["dw"]
    b = run(rzlib, pb_half, X[half:].contiguous(), dY[half:].contiguous(), h, ops=("dw",))["dw"]
    assert rel(a + b, got["dw"]) < 1e-4
    assert torch.isfinite(got["fwd"].float()).all() and torch.isfinite(got["dx"].float()).all()


def test_tf32_layer_16384x4096x4096(rzlib):
    # X[16384,4096] fp32, virtual W[4096,4096] from H = 2^20 (16x), 64x64 tiles, tf32 tensor cores
    args = case(rzlib, 16384, 4096, 4096, 1 << 20, 64, 64, torch.float32, 1002, 1 / 64)
    check_against_fma_kernels(rzlib, *args)


def test_bf16_layer_8192x8192x32768(rzlib):
    # X[8192,8192] bf16, virtual W[8192,32768] from H = 2^22 (64x), 128x128 tiles: many tiles per slice
    args = case(rzlib, 8192, 8192, 32768, 1 << 22, 128, 128, torch.bfloat16, 1003, 1 / 90.5)
    check_against_fma_kernels(rzlib, *args)


def test_bf16_data_parallel_shard_16384x8192x8192(rzlib):
    # one eighth of the global batch of the data-parallel configuration
    args = case(rzlib, 16384, 8192, 8192, 1 << 22, 128, 128, torch.bfloat16, 1005, 1 / 90.5, alpha=0.5)
    check_against_fma_kernels(rzlib, *args, rows=128)
