"""Host-side checks of the C ABI that need no GPU: exports, argument validation, the host hash."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle import rz_oracle as o

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LARGE_PRIME = 2038074743


def test_library_exports_every_declared_symbol(rzlib):
    header = open(os.path.join(ROOT, "include", "rzlinear_b200.h")).read()
    declared = set(re.findall(r"\b(rz_[a-z0-9_]+)\s*\(", header))
    assert {"rz_linear_forward", "rz_linear_backward_input", "rz_linear_backward_weight",
            "rz_hash_indices_host"} <= declared
    lib = rzlib.load()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(rzlib.EXPORTS) <= declared
    assert lib.rz_version() >= 100


def _pb(rzlib, M=64, K=128, N=192, H=8192, BK=32, BN=64, R=None, mode=0, io=0, prec=0, alpha=1.0, flags=0, sm_reserve=0):
    R = R if R is not None else [LARGE_PRIME, 5, 7, 11, 13, 17, 19, 23]
    return rzlib.make_problem(M, K, N, H, BK, BN, R, mode, io, prec, alpha, flags, sm_reserve)


CASES = [
    # K, N, H, BK, BN, R, mode
    (1024, 1024, 65536, 32, 32, None, 0),
    (4096, 4096, 1 << 20, 64, 64, None, 0),
    (8192, 32768, 1 << 22, 128, 128, None, 0),
    (100, 77, 500, 16, 24, None, 0),            # ragged tiles
    (99999, 64, 1 << 16, 1, 64, None, 0),       # largest layer edge the module accepts, BK = 1
    (256, 256, 32 * 32 + 1, 32, 32, None, 0),   # range = 1: every tile at offset 0
    (1024, 1024, 65536, 32, 64, "small", 1),    # the reference's two-level hash
    (512, 2048, 70000, 64, 128, "small", 1),
    (512, 512, 40000, 32, 32, "maxr", 0),       # all R at 2^31 - 1
]


@pytest.mark.parametrize("K,N,H,BK,BN,Rkind,mode", CASES)
def test_host_hash_is_bit_exact(rzlib, K, N, H, BK, BN, Rkind, mode):
    rng = np.random.RandomState(K + N + BK)
    for trial in range(3):
        if Rkind == "small":
            R = [45007] + [int(v) for v in rng.randint(0, 45007, 7)]
        elif Rkind == "maxr":
            R = [LARGE_PRIME] + [2**31 - 1] * 7
        else:
            R = [LARGE_PRIME] + [int(v) for v in rng.randint(1, 2**31 - 1, 7)]
        pb = _pb(rzlib, K=K, N=N, H=H, BK=BK, BN=BN, R=R, mode=mode)
        got = rzlib.hash_indices_host(pb)
        want = o.tile_offsets(K, N, H, BK, BN, R, mode)
        assert got.dtype == np.int64 and got.shape == want.shape
        assert np.array_equal(got, want)
        assert got.min() >= 0 and got.max() < H - BK * BN


def test_host_hash_reference_seed_numbers(rzlib, golden_dir):
    d = np.load(os.path.join(golden_dir, "random_numbers.npz"))
    for seed in d.files:
        R = [int(v) for v in d[seed]]
        pb = _pb(rzlib, K=1024, N=1024, H=65536, BK=32, BN=64, R=R, mode=1)
        assert np.array_equal(rzlib.hash_indices_host(pb), o.tile_offsets(1024, 1024, 65536, 32, 64, R, 1))


def test_adversarial_collisions(rzlib):
    # R2 = 0 (mod P): all tiles in a row of tiles collide; R2 = R3 = 0: all tiles collide
    R = [LARGE_PRIME, 99, LARGE_PRIME, 12345, 0, 0, 0, 0]
    pb = _pb(rzlib, K=256, N=512, H=50000, BK=32, BN=32, R=R)
    off = rzlib.hash_indices_host(pb)
    assert (off == off[:, :1]).all() and len(np.unique(off[:, 0])) > 1
    R = [LARGE_PRIME, 99, 0, 0, 0, 0, 0, 0]
    off = rzlib.hash_indices_host(_pb(rzlib, K=256, N=512, H=50000, BK=32, BN=32, R=R))
    assert (off == 99 % (50000 - 1024)).all()


@pytest.mark.parametrize("kw,status", [
    (dict(M=0), -2), (dict(K=-1), -2), (dict(BK=0), -2), (dict(M=1 << 31), -2),
    (dict(H=32 * 64), -3), (dict(H=100), -3),
    (dict(mode=2), -6), (dict(R=[0, 1, 2, 3, 4, 5, 6, 7]), -6), (dict(R=[7, -1, 2, 3, 4, 5, 6, 7]), -6),
    (dict(R=[7, 1 << 31, 2, 3, 4, 5, 6, 7]), -6),
    (dict(io=2), -4), (dict(prec=3), -4), (dict(io=1, prec=1), -4), (dict(io=0, prec=2), -4),
    (dict(sm_reserve=-1), -2),
])
def test_validation_statuses(rzlib, kw, status):
    pb = _pb(rzlib, **kw)
    out = (ctypes.c_int64 * 64)()
    assert rzlib.load().rz_hash_indices_host(ctypes.byref(pb), out) == status
    assert rzlib.load().rz_plan(ctypes.byref(pb), 0) == status
    with pytest.raises(rzlib.RzLinearError):
        rzlib.check(status)


def test_null_pointers_are_rejected_before_any_launch(rzlib):
    lib = rzlib.load()
    pb = _pb(rzlib)
    assert lib.rz_hash_indices_host(ctypes.byref(pb), None) == -1
    assert lib.rz_linear_forward(ctypes.byref(pb), None, None, None, 0, None, None, None) == -1
    assert lib.rz_linear_backward_input(ctypes.byref(pb), None, None, None, 0, None, None) == -1
    assert lib.rz_linear_backward_weight(ctypes.byref(pb), None, None, None, None) == -1
    assert lib.rz_linear_materialize(ctypes.byref(pb), None, None, None) == -1
    assert lib.rz_grad_prepare(ctypes.byref(pb), None, None, None, None, None) == -1
    assert lib.rz_hash_indices_host(None, None) == -1
    assert lib.rz_status_string(-3).decode().startswith("hashed array too small")


def test_plan_selects_kernel_family(rzlib):
    # fp32 precision on fp32 data: tensor cores with split (hi/lo) operands when the shape is tile-aligned,
    # FMA kernels otherwise (hash tile not a multiple of 32, rows shorter than 128 bytes, forced)
    assert rzlib.plan(_pb(rzlib, M=1024, K=1024, N=1024, H=65536, BK=32, BN=32), 0) == rzlib.PATH_TCGEN05
    assert rzlib.plan(_pb(rzlib, M=64, K=1024, N=1024, H=65536, BK=32, BN=32), 0) == rzlib.PATH_TCGEN05   # small batch too
    assert rzlib.plan(_pb(rzlib, M=1024, K=16, N=1024, H=65536, BK=32, BN=32), 0) == rzlib.PATH_SIMT       # K below one 128-byte row
    assert rzlib.plan(_pb(rzlib, M=1024, K=1024, N=1024, H=65536, BK=16, BN=32), 0) == rzlib.PATH_SIMT
    assert rzlib.plan(_pb(rzlib, M=1024, K=1024, N=1024, H=65536, BK=32, BN=32, flags=rzlib.FLAG_FORCE_SIMT), 0) == rzlib.PATH_SIMT
    # tile-aligned bf16 / tf32 problems take the tensor-core kernels
    big = dict(M=8192, K=8192, N=8192, H=1 << 22, BK=128, BN=128)
    for op in (0, 1, 2):
        assert rzlib.plan(_pb(rzlib, io=1, prec=2, **big), op) == rzlib.PATH_TCGEN05
        assert rzlib.plan(_pb(rzlib, io=0, prec=1, M=16384, K=4096, N=4096, H=1 << 20, BK=64, BN=64), op) == rzlib.PATH_TCGEN05
    assert rzlib.plan(_pb(rzlib, io=1, prec=2, flags=rzlib.FLAG_FORCE_SIMT, **big), 0) == rzlib.PATH_SIMT
    # the module's default hash tile (32 x 64, the reference's BLOCK_SIZE_K / BLOCK_SIZE_N) runs on the tensor
    # cores in every precision: a bf16 pipeline stage of 64 contraction rows is then made of two hash tiles
    for op in (0, 1, 2):
        assert rzlib.plan(_pb(rzlib, io=1, prec=2, M=1024, K=1024, N=1024, H=65536, BK=32, BN=64), op) == rzlib.PATH_TCGEN05
        assert rzlib.plan(_pb(rzlib, io=0, prec=1, M=1024, K=1024, N=1024, H=65536, BK=32, BN=64), op) == rzlib.PATH_TCGEN05
    # hash tiles narrower than a 128-byte row, or odd leading dimensions, fall to the FMA kernels
    assert rzlib.plan(_pb(rzlib, io=1, prec=2, M=1024, K=1024, N=1024, H=65536, BK=32, BN=32), 0) == rzlib.PATH_SIMT
    assert rzlib.plan(_pb(rzlib, io=1, prec=2, M=1024, K=1024, N=1024, H=65536, BK=48, BN=64), 0) == rzlib.PATH_SIMT
    assert rzlib.plan(_pb(rzlib, io=1, prec=2, M=1024, K=1020, N=1024, H=1 << 20, BK=64, BN=64), 0) == rzlib.PATH_SIMT
    # shadow scratch: NS shifted copies (8 for bf16, 4 for tf32), none for the FMA kernels
    assert rzlib.shadow_bytes(_pb(rzlib, io=1, prec=2, **big)) == 8 * (1 << 22) * 2
    assert rzlib.shadow_bytes(_pb(rzlib, io=0, prec=1, M=16384, K=4096, N=4096, H=1 << 20, BK=64, BN=64)) == 4 * (1 << 20) * 4
    assert rzlib.shadow_bytes(_pb(rzlib, flags=rzlib.FLAG_FORCE_SIMT)) == 0
    assert rzlib.shadow_bytes(_pb(rzlib, BK=16)) == 0


def test_scratch_size_rules(rzlib):
    # the scratch = shifted copies + the workspace of split-contraction launches, which depends on the rows of the
    # launch and on the SMs it may use: a buffer that serves several problems must be sized for the largest
    big = dict(io=1, prec=2, K=8192, N=8192, H=1 << 22, BK=128, BN=128)
    copies = 8 * (1 << 22) * 2
    assert rzlib.shadow_bytes(_pb(rzlib, M=131072, **big)) == copies                      # full waves only
    small = rzlib.shadow_bytes(_pb(rzlib, M=128, **big))
    assert small > copies                                                                  # few blocks: split contraction
    assert rzlib.shadow_bytes(_pb(rzlib, M=7232, **big)) > rzlib.shadow_bytes(_pb(rzlib, M=40000, **big)) > copies
    # reserving SMs changes the wave structure, hence possibly the workspace
    assert rzlib.shadow_bytes(_pb(rzlib, M=16384, sm_reserve=8, **big)) >= copies
    # copying a problem and changing fields
    pb = _pb(rzlib, M=40000, **big)
    q = rzlib.with_fields(pb, M=7232, flags=rzlib.FLAG_ACCUMULATE_DH)
    assert (q.M, q.K, q.H, q.flags, list(q.R)) == (7232, 8192, 1 << 22, 1, list(pb.R)) and pb.M == 40000
    assert rzlib.load().rz_status_string(-11).decode().startswith("scratch buffer smaller")
