"""The CPU oracle against the fixtures produced by the reference's own kernels (tests/golden/)."""
import ctypes
import os

import numpy as np
import pytest

from oracle import rz_oracle as o


def _load(golden_dir, tag):
    return np.load(os.path.join(golden_dir, tag + ".npz"))


def test_random_numbers_match_reference(golden_dir):
    d = _load(golden_dir, "random_numbers")
    for seed in d.files:
        assert o.reference_random_numbers(int(seed)) == [int(v) for v in d[seed]]


@pytest.mark.parametrize("tag", ["idx_a", "idx_b"])
def test_materialize_single_level_matches_reference_idx_kernel(golden_dir, tag):
    d = _load(golden_dir, tag)
    K, N, H, BK, BN = (int(v) for v in d["dims"])
    W = o.materialize(d["hashed"], K, N, BK, BN, d["R"], o.HASH_SINGLE)
    assert np.array_equal(W, d["W"])
    assert np.array_equal(o.materialize_loops(d["hashed"], K, N, BK, BN, d["R"], o.HASH_SINGLE), d["W"])


@pytest.mark.parametrize("tag", ["k_full", "k_ragged", "k_small_tiles"])
def test_kernels_two_level_match_reference(golden_dir, tag):
    d = _load(golden_dir, tag)
    M, K, N, H, BK, BN = (int(v) for v in d["dims"])
    a = float(d["alpha"])
    Y = o.forward(d["X"], d["hashed"], N, BK, BN, d["R"], o.HASH_TWO_LEVEL, a)
    dX = o.backward_input(d["dY"], d["hashed"], K, BK, BN, d["R"], o.HASH_TWO_LEVEL, a)
    dH = o.backward_weight(d["X"], d["dY"], H, BK, BN, d["R"], o.HASH_TWO_LEVEL, a)
    # the reference accumulates in fp32; the oracle in fp64
    assert o.rel_l2(Y, d["Y"]) < 1e-6
    assert o.rel_l2(dX, d["dX"]) < 1e-6
    assert o.rel_l2(dH, d["dH"]) < 1e-6


def test_module_fixture(golden_dir):
    d = _load(golden_dir, "module")
    R, a = d["R"], float(d["alpha"])
    x = d["x"].reshape(-1, 64)
    gy = d["gy"].reshape(-1, 128)
    H = d["hashed"].shape[0]
    y = o.forward(x, d["hashed"], 128, 32, 64, R, o.HASH_TWO_LEVEL, a) + d["bias"]
    assert o.rel_l2(y, d["y"].reshape(-1, 128)) < 1e-6
    assert o.rel_l2(o.backward_input(gy, d["hashed"], 64, 32, 64, R, o.HASH_TWO_LEVEL, a), d["dx"].reshape(-1, 64)) < 1e-6
    assert o.rel_l2(o.backward_weight(x, gy, H, 32, 64, R, o.HASH_TWO_LEVEL, a), d["dh"]) < 1e-6
    assert o.rel_l2(gy.sum(0), d["dbias"]) < 1e-6


def _i64(a):
    a = np.ascontiguousarray(a, dtype=np.int64)
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))


@pytest.mark.parametrize("mode", [o.HASH_SINGLE, o.HASH_TWO_LEVEL])
def test_c_oracle_agrees_with_numpy_oracle(oracle_c, mode):
    rng = np.random.RandomState(3)
    M, K, N, H, BK, BN = 9, 40, 56, 700, 16, 24
    R = [2038074743] + [int(v) for v in rng.randint(1, 2**31 - 1, 7)]
    if mode == o.HASH_TWO_LEVEL:
        R = [45007] + [int(v) for v in rng.randint(0, 45007, 7)]
    Rarr, Rp = _i64(R)
    nk, nn = o.cdiv(K, BK), o.cdiv(N, BN)
    out = np.zeros((nk, nn), dtype=np.int64)
    assert oracle_c.rzo_tile_offsets(ctypes.c_int64(K), ctypes.c_int64(N), ctypes.c_int64(H), ctypes.c_int64(BK),
                                     ctypes.c_int64(BN), Rp, mode,
                                     out.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))) == 0
    assert np.array_equal(out, o.tile_offsets(K, N, H, BK, BN, R, mode))

    X = rng.randn(M, K).astype(np.float32)
    dY = rng.randn(M, N).astype(np.float32)
    h = rng.rand(H).astype(np.float32)
    fp = ctypes.POINTER(ctypes.c_float)
    dp = ctypes.POINTER(ctypes.c_double)
    dims = [ctypes.c_int64(v) for v in (M, K, N, H, BK, BN)]
    Y = np.zeros((M, N)); dX = np.zeros((M, K)); dH = np.zeros(H)
    assert oracle_c.rzo_forward(X.ctypes.data_as(fp), h.ctypes.data_as(fp), *dims, Rp, mode, ctypes.c_double(0.5),
                                Y.ctypes.data_as(dp)) == 0
    assert oracle_c.rzo_backward_input(dY.ctypes.data_as(fp), h.ctypes.data_as(fp), *dims, Rp, mode,
                                       ctypes.c_double(0.5), dX.ctypes.data_as(dp)) == 0
    assert oracle_c.rzo_backward_weight(X.ctypes.data_as(fp), dY.ctypes.data_as(fp), *dims, Rp, mode,
                                        ctypes.c_double(0.5), dH.ctypes.data_as(dp)) == 0
    assert o.rel_l2(Y, o.forward(X, h, N, BK, BN, R, mode, 0.5)) < 1e-12
    assert o.rel_l2(dX, o.backward_input(dY, h, K, BK, BN, R, mode, 0.5)) < 1e-12
    assert o.rel_l2(dH, o.backward_weight(X, dY, H, BK, BN, R, mode, 0.5)) < 1e-12


def test_colliding_tiles_sum():
    # R2 = R3 = 0: every tile hashes to the same slice; the gradient of that slice is the sum over tiles
    K, N, H, BK, BN = 32, 48, 300, 16, 16
    R = [45007, 11, 0, 0, 5, 0, 0, 0]
    off = o.tile_offsets(K, N, H, BK, BN, R, o.HASH_SINGLE)
    assert (off == off[0, 0]).all()
    rng = np.random.RandomState(0)
    X = rng.randn(7, K); dY = rng.randn(7, N)
    dH = o.backward_weight(X, dY, H, BK, BN, R, o.HASH_SINGLE)
    G = X.T @ dY
    want = sum(G[i * BK:(i + 1) * BK, j * BN:(j + 1) * BN] for i in range(2) for j in range(3)).ravel()
    s = int(off[0, 0])
    assert np.allclose(dH[s:s + BK * BN], want)
    assert np.count_nonzero(dH) == BK * BN


def test_hash_range_guard():
    with pytest.raises(ValueError):
        o.tile_offsets(32, 32, 256, 16, 16, [45007] * 8)
