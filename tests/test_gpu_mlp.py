"""Three RzLinear layers with ReLU and an MSE loss (the MLP configuration of the baseline, scaled down),
through the module / autograd API, against autograd over the materialised weights in fp64."""
import numpy as np
import pytest
import torch

from oracle import rz_oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PRIME = 2038074743


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_three_layer_mlp_step(dtype, tol):
    from rzlinear_b200 import RzLinear
    dims = [256, 512, 512, 64]
    batch, H, BK, BN = 512, 1 << 16, 64, 64
    layers = []
    rs = np.random.RandomState(4)
    for i in range(3):
        R = [PRIME] + [int(v) for v in rs.randint(1, 2**31 - 1, 3)] + [0, 0, 0, 0]
        g = torch.Generator().manual_seed(10 + i)
        hw = torch.nn.Parameter(((torch.rand(H, generator=g) * 2 - 1) / dims[i] ** 0.5))
        layers.append(RzLinear(dims[i], dims[i + 1], hashed_weight=hw, bias=True, hash_mode="single",
                               random_numbers=R, block_size_k=BK, block_size_n=BN, relu=(i < 2)))
    model = torch.nn.Sequential(*layers).to(DEV)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(batch, dims[0], generator=g)
    target = torch.randn(batch, dims[-1], generator=g)
    for i, l in enumerate(layers):
        with torch.no_grad():
            l._bias.copy_(torch.randn(dims[i + 1], generator=g) * 0.1)

    out = model(x.to(DEV).to(dtype))
    loss = torch.nn.functional.mse_loss(out.float(), target.to(DEV))
    loss.backward()

    # reference: same network over materialised weights, autograd on the CPU.  fp32 case: fp64 arithmetic.
    # bf16 case: the same rounding points as the kernels (bf16 weights, bf16 activations and gradients
    # between layers, fp32 accumulation), so that the comparison isolates the kernels.
    bf = dtype == torch.bfloat16
    wd = torch.float32 if bf else torch.float64
    hs = [l._hashed_weight.detach().cpu().to(wd).requires_grad_(True) for l in layers]
    bs = [l._bias.detach().cpu().to(wd).requires_grad_(True) for l in layers]
    a = x.bfloat16() if bf else x.double()
    for i, l in enumerate(layers):
        idx = torch.from_numpy(o.element_index(dims[i], dims[i + 1], H, BK, BN, l._random_numbers.tolist(), 0))
        W = hs[i][idx]
        if bf:
            a = (a.float() @ W.bfloat16().float() + bs[i])
        else:
            a = a @ W + bs[i]
        if i < 2:
            a = torch.relu(a)
        if bf:
            a = a.bfloat16()
    ref_loss = torch.nn.functional.mse_loss(a.float() if bf else a, target.to(torch.float32 if bf else torch.float64))
    ref_loss.backward()
    assert abs(float(loss) - float(ref_loss)) < tol * abs(float(ref_loss)), (float(loss), float(ref_loss))
    for i, l in enumerate(layers):
        eh = o.rel_l2(l._hashed_weight.grad.cpu().numpy(), hs[i].grad.numpy())
        eb = o.rel_l2(l._bias.grad.cpu().numpy(), bs[i].grad.numpy())
        assert eh < tol and eb < tol, (i, eh, eb)
