"""Three RzLinear layers with ReLU and an MSE loss (the MLP configuration of the baseline) through the module /
autograd API, against autograd over the materialised weights: scaled down with the reference computed on the CPU,
and at the configuration's full size (1024 -> 4096 -> 4096 -> 256, batch 65536, H = 2^18 per layer, bf16 compute)
with the reference's own method - torch matmuls over the materialised weight on the GPU
(python/tests/test_rz_linear.py:68-71), fp32, the weight gathered with the oracle's index table.

Bar: loss and all three hashed-weight gradients within 2e-3 (1e-4 in fp32).  In the bf16 case the reference takes
the same rounding points as the kernels (bf16 weights, bf16 activations and gradients between layers, fp32
accumulation), so that the comparison isolates the kernels."""
import numpy as np
import pytest
import torch

from oracle import rz_oracle as o

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PRIME = 2038074743


def build_layers(dims, H, BK, BN):
    from rzlinear_b200 import RzLinear
    layers = []
    rs = np.random.RandomState(4)
    for i in range(3):
        R = [PRIME] + [int(v) for v in rs.randint(1, 2**31 - 1, 3)] + [0, 0, 0, 0]
        g = torch.Generator().manual_seed(10 + i)
        hw = torch.nn.Parameter(((torch.rand(H, generator=g) * 2 - 1) / dims[i] ** 0.5))
        layers.append(RzLinear(dims[i], dims[i + 1], hashed_weight=hw, bias=True, hash_mode="single",
                               random_numbers=R, block_size_k=BK, block_size_n=BN, relu=(i < 2)))
    return layers


def run_case(dims, batch, H, BK, BN, dtype, tol, ref_dev):
    layers = build_layers(dims, H, BK, BN)
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
    torch.cuda.synchronize()
    from rzlinear_b200 import _lib
    assert _lib.device_status() == (0, 0)

    bf = dtype == torch.bfloat16
    wd = torch.float32 if bf else torch.float64
    assert not torch.backends.cuda.matmul.allow_tf32          # the reference's GEMMs are plain fp32 / fp64
    hs = [l._hashed_weight.detach().to(ref_dev).to(wd).requires_grad_(True) for l in layers]
    bs = [l._bias.detach().to(ref_dev).to(wd).requires_grad_(True) for l in layers]
    a = (x.bfloat16() if bf else x.double()).to(ref_dev)
    for i, l in enumerate(layers):
        idx = torch.from_numpy(o.element_index(dims[i], dims[i + 1], H, BK, BN, l._random_numbers.tolist(), 0)).to(ref_dev)
        W = hs[i][idx]
        if bf:
            a = (a.float() @ W.bfloat16().float() + bs[i])
        else:
            a = a @ W + bs[i]
        if i < 2:
            a = torch.relu(a)
        if bf:
            a = a.bfloat16()
    ref_loss = torch.nn.functional.mse_loss(a.float() if bf else a, target.to(ref_dev).to(torch.float32 if bf else torch.float64))
    ref_loss.backward()
    errs = {"loss": abs(float(loss) - float(ref_loss)) / abs(float(ref_loss))}
    for i, l in enumerate(layers):
        errs[f"dH{i}"] = o.rel_l2(l._hashed_weight.grad.cpu().numpy(), hs[i].grad.cpu().numpy())
        errs[f"db{i}"] = o.rel_l2(l._bias.grad.cpu().numpy(), bs[i].grad.cpu().numpy())
    print("mlp errors", dims, batch, dtype, {k: f"{v:.2e}" for k, v in errs.items()})
    assert max(errs.values()) < tol, errs


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-3)])
def test_three_layer_mlp_step(dtype, tol):
    run_case([256, 512, 512, 64], 512, 1 << 16, 64, 64, dtype, tol, "cpu")


def test_three_layer_mlp_step_full_size_bf16():
    # the MLP baseline configuration itself; the tensor-core path runs every product (hash tile 64 x 64)
    run_case([1024, 4096, 4096, 256], 65536, 1 << 18, 64, 64, torch.bfloat16, 2e-3, DEV)
