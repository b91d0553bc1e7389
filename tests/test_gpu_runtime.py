"""Host-runtime behaviour around the kernels, on a GPU: the fused optimiser + shadow pass, the per-parameter shadow
cache of the autograd path, scratch-size checking, reserved SMs, and what happens after a device-side wait gave up."""
import numpy as np
import pytest
import torch

from oracle import rz_oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PRIME = 2038074743
R = [PRIME] + [int(v) for v in np.random.RandomState(21).randint(1, 2**31 - 1, 7)]


def _problem(rzlib, M, K, N, H, BK, BN, prec, **kw):
    io = rzlib.BF16 if prec == rzlib.PREC_BF16 else rzlib.F32
    return rzlib.make_problem(M, K, N, H, BK, BN, R, rzlib.HASH_SINGLE, io, prec, 1.0, **kw)


@pytest.mark.parametrize("prec_name", ["bf16", "tf32", "fp32"])
@pytest.mark.parametrize("H", [1 << 17, 100003, 64 * 64 + 1, 2055, 3 * 1024 * 8 + 5])   # (2055: one word more than a 32 x 64 tile)
@pytest.mark.parametrize("momentum", [0.0, 0.9])
def test_optimiser_step_rewrites_the_shadow_in_the_same_launch(rzlib, prec_name, H, momentum):
    # hashed / velocity against fp64 arithmetic; the shadow bit-identical to a refresh from the updated array
    prec = {"bf16": rzlib.PREC_BF16, "tf32": rzlib.PREC_TF32, "fp32": rzlib.PREC_FP32}[prec_name]
    BK, BN = (64, 64) if H > 64 * 64 else (32, 64)
    pb = _problem(rzlib, 256, 256, 256, H, BK, BN, prec)
    assert rzlib.plan(pb, 0) == rzlib.PATH_TCGEN05
    g = torch.Generator().manual_seed(H)
    h0, dh, v0 = torch.rand(H, generator=g) - 0.5, torch.randn(H, generator=g), torch.randn(H, generator=g)
    h, vel = h0.to(DEV), v0.to(DEV)
    nbytes = rzlib.shadow_bytes(pb)
    shadow = torch.full((nbytes,), 0x5A, dtype=torch.uint8, device=DEV)
    want_shadow = torch.full((nbytes,), 0x5A, dtype=torch.uint8, device=DEV)
    lr = 0.05
    n0 = rzlib.launch_count()
    if momentum:
        rzlib.sgd_momentum_step(pb, h, dh.to(DEV), vel, lr, momentum, shadow)
    else:
        rzlib.sgd_step(pb, h, dh.to(DEV), lr, shadow)
    assert rzlib.launch_count() - n0 == 1                      # one kernel: update and shadow together
    v_new = momentum * v0.double() + dh.double() if momentum else dh.double()
    assert o.rel_l2(h.cpu().numpy(), (h0.double() - lr * v_new).numpy()) < 1e-6
    if momentum:
        assert o.rel_l2(vel.cpu().numpy(), v_new.numpy()) < 1e-6
    rzlib.shadow_refresh(pb, h, want_shadow)
    torch.cuda.synchronize()
    assert torch.equal(shadow, want_shadow)
    # twice in a row (the ticket word of the first launch has been handed back)
    if momentum:
        rzlib.sgd_momentum_step(pb, h, dh.to(DEV), vel, lr, momentum, shadow)
    else:
        rzlib.sgd_step(pb, h, dh.to(DEV), lr, shadow)
    rzlib.shadow_refresh(pb, h, want_shadow)
    torch.cuda.synchronize()
    assert torch.equal(shadow, want_shadow)


def test_many_optimiser_steps_share_the_ticket_words(rzlib):
    # more launches than ticket words, back to back on one stream
    H = 70001
    pb = _problem(rzlib, 256, 256, 256, H, 64, 64, rzlib.PREC_BF16)
    h = torch.zeros(H, device=DEV)
    dh = torch.ones(H, device=DEV)
    shadow = torch.empty(rzlib.shadow_bytes(pb), dtype=torch.uint8, device=DEV)
    for _ in range(150):
        rzlib.sgd_step(pb, h, dh, 0.5, shadow)
    want = torch.empty_like(shadow)
    rzlib.shadow_refresh(pb, h, want)
    torch.cuda.synchronize()
    assert torch.equal(h, torch.full((H,), -75.0, device=DEV)) and torch.equal(shadow, want)


def test_autograd_path_rebuilds_the_shadow_only_when_weights_change(rzlib):
    from rzlinear_b200 import RzLinear
    from rzlinear_b200.impl import launchers
    torch.manual_seed(0)
    hw = torch.nn.Parameter(((torch.rand(1 << 16) * 2 - 1) / 16).to(DEV))
    a = RzLinear(256, 512, hashed_weight=hw, seed=1, block_size_k=64, block_size_n=64).to(DEV)
    b = RzLinear(256, 512, hashed_weight=hw, seed=2, block_size_k=64, block_size_n=64).to(DEV)   # shares the array
    x = torch.randn(128, 256, device=DEV).bfloat16()
    with torch.no_grad():
        y0 = a(x)
        n0 = rzlib.launch_count()
        y1 = a(x)
        yb = b(x)
        assert rzlib.launch_count() - n0 == 2                  # two forward kernels, no refresh
        assert torch.equal(y0, y1) and not torch.equal(y0, yb)
        hw.mul_(2.0)                                           # in-place update: the version counter moves
        n0 = rzlib.launch_count()
        y2 = a(x)
        assert rzlib.launch_count() - n0 == 2                  # refresh + forward
        assert o.rel_l2(y2.float().cpu().numpy(), 2 * y0.float().cpu().numpy()) < 2e-3
        hw.data.mul_(0.5)                                      # a write the counter does not see ...
        launchers.drop_shadow_cache(hw)                        # ... has to be announced
        assert torch.equal(a(x), y0)
    # training: forward, backward, optimiser step, forward - the second forward sees the new weights
    opt = torch.optim.SGD([hw], lr=0.5)
    a(x).float().square().mean().backward()
    opt.step()
    y3 = a(x)
    ref = RzLinear(256, 512, hashed_weight=torch.nn.Parameter(hw.detach().clone()), seed=1, block_size_k=64,
                   block_size_n=64).to(DEV)
    assert torch.equal(y3, ref(x)) and not torch.equal(y3, y0)


def test_scratch_smaller_than_the_problem_needs_is_refused(rzlib):
    # a problem whose scratch includes a workspace (few blocks, long contraction) given the copies alone
    pb = _problem(rzlib, 128, 4096, 4096, 300007, 64, 64, rzlib.PREC_BF16)
    copies = 8 * 2 * (-(-300007 // 64) * 64)
    assert rzlib.shadow_bytes(pb) > copies
    X = torch.randn(128, 4096, device=DEV).bfloat16()
    h = torch.rand(300007, device=DEV)
    Y = torch.zeros(128, 4096, device=DEV, dtype=torch.bfloat16)
    short = torch.empty(copies, dtype=torch.uint8, device=DEV)
    rzlib.shadow_refresh(pb, h, short)
    for call in (lambda: rzlib.forward(pb, X, h, short, None, Y), lambda: rzlib.backward_input(pb, X, h, short, Y)):
        with pytest.raises(rzlib.RzLinearError) as e:
            call()
        assert e.value.status == rzlib.RZ_ERR_SCRATCH
    torch.cuda.synchronize()
    assert float(Y.float().abs().sum()) == 0.0                 # nothing was launched


@pytest.mark.parametrize("prec_name,M,K,N", [("bf16", 2048, 1024, 2048), ("bf16", 128, 4096, 2048), ("tf32", 1024, 512, 1024)])
def test_reserved_sms_do_not_change_results(rzlib, prec_name, M, K, N):
    prec = {"bf16": rzlib.PREC_BF16, "tf32": rzlib.PREC_TF32}[prec_name]
    dtype = torch.bfloat16 if prec_name == "bf16" else torch.float32
    H = 1 << 18
    g = torch.Generator(device=DEV).manual_seed(5)
    X = torch.randn((M, K), generator=g, device=DEV).to(dtype)
    dY = torch.randn((M, N), generator=g, device=DEV).to(dtype)
    h = (torch.rand(H, generator=g, device=DEV) - 0.5) / 16
    outs = []
    for reserve in (0, 8, 40):
        pb = _problem(rzlib, M, K, N, H, 64, 64, prec, sm_reserve=reserve)
        shadow = torch.empty(rzlib.shadow_bytes(pb), dtype=torch.uint8, device=DEV)
        rzlib.shadow_refresh(pb, h, shadow)
        Y = torch.empty((M, N), dtype=dtype, device=DEV)
        dX = torch.empty((M, K), dtype=dtype, device=DEV)
        dH = torch.empty(H, device=DEV)
        rzlib.forward(pb, X, h, shadow, None, Y)
        rzlib.backward_input(pb, dY, h, shadow, dX)
        rzlib.backward_weight(pb, X, dY, dH)
        outs.append((Y.float(), dX.float(), dH))
    torch.cuda.synchronize()
    assert rzlib.device_status() == (0, 0)
    for other in outs[1:]:
        for a, b in zip(outs[0], other):                       # (split contractions may sum in another order)
            assert o.rel_l2(b.cpu().numpy(), a.cpu().numpy()) < 1e-3


def test_launches_are_refused_after_a_wait_gave_up_until_acknowledged(rzlib):
    # a kernel whose wait ran out leaves partial results: nothing may silently continue on them
    pb = _problem(rzlib, 256, 512, 512, 1 << 17, 128, 128, rzlib.PREC_BF16)
    X = torch.randn(256, 512, device=DEV).bfloat16()
    h = torch.rand(1 << 17, device=DEV) - 0.5
    shadow = torch.empty(rzlib.shadow_bytes(pb), dtype=torch.uint8, device=DEV)
    rzlib.shadow_refresh(pb, h, shadow)
    Y = torch.empty(256, 512, device=DEV, dtype=torch.bfloat16)
    rzlib.forward(pb, X, h, shadow, None, Y)
    torch.cuda.synchronize()
    good = Y.clone()
    assert rzlib.device_status() == (0, 0)
    rzlib.selftest_bounded_wait(1_000_000, DEV)               # a wait on a flag nothing sets: gives up, reports
    torch.cuda.synchronize()
    Y.zero_()
    for call in (lambda: rzlib.forward(pb, X, h, shadow, None, Y),
                 lambda: rzlib.backward_weight(pb, X, X, torch.empty(1 << 17, device=DEV))):
        with pytest.raises(rzlib.RzLinearError) as e:
            call()
        assert e.value.status == rzlib.RZ_ERR_PIPELINE
    torch.cuda.synchronize()
    assert float(Y.float().abs().sum()) == 0.0                 # refused before anything was launched
    assert rzlib.device_status() == (rzlib.RZ_ERR_PIPELINE, 6)
    assert rzlib.device_status() == (0, 0)
    rzlib.forward(pb, X, h, shadow, None, Y)                   # acknowledged: back to normal
    torch.cuda.synchronize()
    assert torch.equal(Y, good) and rzlib.device_status() == (0, 0)


def test_training_step_replayed_from_a_cuda_graph(rzlib):
    # forward, backward and an in-place SGD update of a small layer captured once and replayed: every replay must see
    # the weights the previous one wrote (the shadow refresh has to be a node of the graph, not a cached buffer)
    from rzlinear_b200 import RzLinear
    torch.manual_seed(2)
    K, N, M, lr = 256, 512, 256, 0.05

    def make():
        hw = torch.nn.Parameter(((torch.rand(1 << 16, generator=torch.Generator().manual_seed(3)) * 2 - 1) / 16).to(DEV))
        return RzLinear(K, N, hashed_weight=hw, seed=5, bias=False, block_size_k=64, block_size_n=64).to(DEV), hw

    x = torch.randn(M, K, device=DEV).bfloat16()
    t = torch.randn(M, N, device=DEV).bfloat16()

    def step(layer, hw):
        hw.grad = None
        loss = (layer(x).float() - t.float()).square().mean()
        loss.backward()
        with torch.no_grad():
            hw.add_(hw.grad, alpha=-lr)
        return loss

    eager, hw_e = make()
    losses_e = [float(step(eager, hw_e)) for _ in range(4)]

    graphed, hw_g = make()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):          # warm-up outside the capture: first-use set-up of the library, autograd
        step(graphed, hw_g)
    torch.cuda.current_stream().wait_stream(side)
    with torch.no_grad():
        hw_g.copy_(make()[1])              # back to the initial weights
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        loss_g = step(graphed, hw_g)
    losses_g = []
    with torch.no_grad():
        hw_g.copy_(make()[1])
    for _ in range(4):
        g.replay()
        losses_g.append(float(loss_g))
    torch.cuda.synchronize()
    assert rzlib.device_status() == (0, 0)
    assert losses_e[0] > losses_e[-1]                                   # it trains
    for a, b in zip(losses_e, losses_g):
        assert abs(a - b) < 2e-3 * abs(a), (losses_e, losses_g)
    assert o.rel_l2(hw_g.detach().cpu().numpy(), hw_e.detach().cpu().numpy()) < 1e-4
