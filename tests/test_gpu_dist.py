"""The data-parallel training step on real GPUs: one rank against the oracle, and (when the box has
two or more GPUs) two NCCL ranks against the single-device full-batch result."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import rz_oracle as o

pytestmark = pytest.mark.gpu

PRIME = 2038074743
M, K, N, H, BK, BN = 1024, 512, 768, 1 << 17, 128, 128
LR = 0.01
R = [PRIME] + [int(v) for v in np.random.RandomState(77).randint(1, 2**31 - 1, 3)] + [0, 0, 0, 0]


def _inputs():
    g = torch.Generator().manual_seed(77)
    X = torch.randn(M, K, generator=g).bfloat16()
    dY = torch.randn(M, N, generator=g).bfloat16()
    h = (torch.rand(H, generator=g) * 2 - 1) / K ** 0.5
    return X, dY, h


def _expected():
    X, dY, h = _inputs()
    hb = o.bf16_round(h.numpy())
    Xf, dYf = X.float().numpy(), dY.float().numpy()
    dH = o.backward_weight(Xf, dYf, H, BK, BN, R, 0)
    return (o.forward(Xf, hb, N, BK, BN, R, 0), o.backward_input(dYf, hb, K, BK, BN, R, 0), dH,
            h.numpy().astype(np.float64) - LR * dH)


def test_single_rank_step_matches_oracle(rzlib):
    from rzlinear_b200.dist import RzDataParallelStep
    X, dY, h = _inputs()
    step = RzDataParallelStep(M, K, N, H, BK, BN, R, rzlib.HASH_SINGLE, torch.bfloat16, LR, "cuda:0")
    step.load_weights(h.cuda())
    step.step(X.cuda(), dY.cuda())
    torch.cuda.synchronize()
    st, detail = rzlib.device_status()
    assert st == 0, (st, detail)
    Y, dX, dH, h_new = _expected()
    assert o.rel_l2(step.Y.float().cpu().numpy(), Y) < 2e-3
    assert o.rel_l2(step.dX.float().cpu().numpy(), dX) < 2e-3
    assert o.rel_l2(step.dH.cpu().numpy(), dH) < 2e-3
    assert o.rel_l2(step.hashed.cpu().numpy(), h_new) < 1e-5
    # a second step reads the refreshed shadow: forward now equals the oracle on the updated weights
    step.step(X.cuda(), dY.cuda())
    torch.cuda.synchronize()
    Y2 = o.forward(X.float().numpy(), o.bf16_round(h_new.astype(np.float32)), N, BK, BN, R, 0)
    assert o.rel_l2(step.Y.float().cpu().numpy(), Y2) < 2e-3


def test_momentum_update_matches_reference(rzlib):
    from rzlinear_b200.dist import RzDataParallelStep
    X, dY, h = _inputs()
    step = RzDataParallelStep(M, K, N, H, BK, BN, R, rzlib.HASH_SINGLE, torch.bfloat16, LR, "cuda:0", momentum=0.9)
    step.load_weights(h.cuda())
    dH = _expected()[2]
    hh, v = h.numpy().astype(np.float64), np.zeros(H)
    for _ in range(2):      # dY is given, so the hashed-weight gradient is the same in both steps
        step.step(X.cuda(), dY.cuda())
        v = 0.9 * v + dH
        hh = hh - LR * v
    torch.cuda.synchronize()
    assert o.rel_l2(step.velocity.cpu().numpy(), v) < 2e-3
    assert o.rel_l2(step.hashed.cpu().numpy(), hh) < 1e-5


def test_step_from_host_buffers(rzlib):
    from rzlinear_b200.dist import RzDataParallelStep
    X, dY, h = _inputs()
    step = RzDataParallelStep(M, K, N, H, BK, BN, R, rzlib.HASH_SINGLE, torch.bfloat16, LR, "cuda:0")
    step.load_weights(h.cuda())
    out = torch.empty(H, dtype=torch.float32).pin_memory()
    step.step_host(X.pin_memory(), dY.pin_memory(), out)
    torch.cuda.synchronize()
    assert o.rel_l2(out.numpy(), _expected()[3]) < 1e-5


def test_step_from_host_buffers_with_a_remainder_chunk(rzlib):
    # Rows not a multiple of the chunk, contraction long enough (64 pipeline stages) that the small remainder chunk
    # splits its contraction and so needs a larger workspace inside the scratch than the whole shard does: the step
    # must size the scratch for its largest launch (a scratch that is too small is refused by the library).
    from rzlinear_b200.dist import RzDataParallelStep
    Mr, Kr, Nr, Hr, chunk = 8784, 4096, 4096, 1 << 17, 4096
    g = torch.Generator().manual_seed(5)
    X = torch.randn(Mr, Kr, generator=g).bfloat16()
    dY = torch.randn(Mr, Nr, generator=g).bfloat16()
    h = (torch.rand(Hr, generator=g) * 2 - 1) / Kr ** 0.5
    step = RzDataParallelStep(Mr, Kr, Nr, Hr, 64, 64, R, rzlib.HASH_SINGLE, torch.bfloat16, LR, "cuda:0")
    step.load_weights(h.cuda())
    whole = rzlib.shadow_bytes(step.pb)
    tail = rzlib.shadow_bytes(rzlib.with_fields(step.pb, M=Mr - chunk))
    assert tail > whole                                         # the case this test is about
    out = torch.empty(Hr, dtype=torch.float32).pin_memory()
    step.step_host(X.pin_memory(), dY.pin_memory(), out, chunk_rows=chunk)
    torch.cuda.synchronize()
    assert rzlib.device_status() == (0, 0)
    assert step.kernels.shadow.numel() >= tail
    hb = o.bf16_round(h.numpy())
    Xf, dYf = X.float().numpy(), dY.float().numpy()
    dH = o.backward_weight(Xf, dYf, Hr, 64, 64, R, 0)
    assert o.rel_l2(step.Y.float().cpu().numpy(), o.forward(Xf, hb, Nr, 64, 64, R, 0)) < 2e-3
    assert o.rel_l2(step.dX.float().cpu().numpy(), o.backward_input(dYf, hb, Kr, 64, 64, R, 0)) < 2e-3
    assert o.rel_l2(step.dH.cpu().numpy(), dH) < 2e-3
    assert o.rel_l2(out.numpy(), h.numpy().astype(np.float64) - LR * dH) < 1e-5


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    from rzlinear_b200 import _lib
    from rzlinear_b200.dist import RzDataParallelStep, shard_rows
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    X, dY, h = _inputs()
    lo, hi = shard_rows(M, rank, world)
    dev = torch.device("cuda", rank)
    step = RzDataParallelStep(hi - lo, K, N, H, BK, BN, R, _lib.HASH_SINGLE, torch.bfloat16, LR, dev)
    step.load_weights(h.to(dev))
    step.step(X[lo:hi].contiguous().to(dev), dY[lo:hi].contiguous().to(dev))
    torch.cuda.synchronize()
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), h=step.hashed.cpu().numpy(), dH=step.dH.cpu().numpy(),
             Y=step.Y.float().cpu().numpy(), lo=lo, hi=hi, status=np.array(_lib.device_status()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_equal_full_batch(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    Y, dX, dH, h_new = _expected()
    outs = [np.load(tmp_path / f"r{r}.npz") for r in range(2)]
    assert np.array_equal(outs[0]["h"], outs[1]["h"])      # replicas identical after the all-reduce
    for r in range(2):
        assert tuple(outs[r]["status"]) == (0, 0)
        lo, hi = int(outs[r]["lo"]), int(outs[r]["hi"])
        assert o.rel_l2(outs[r]["Y"], Y[lo:hi]) < 2e-3
        assert o.rel_l2(outs[r]["dH"], dH) < 2e-3
        assert o.rel_l2(outs[r]["h"], h_new) < 1e-5
