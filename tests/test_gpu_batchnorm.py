"""FusedBatchNorm2d (batch norm + residual add + ReLU, training mode) against torch.nn.BatchNorm2d
evaluated in float64 on the CPU: outputs, running statistics and all gradients."""
import pytest
import torch
import torch.nn as nn

from oracle import adder_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SHAPES = [(64, 16, 32, 32), (8, 5, 7, 7), (4, 64, 8, 8), (3, 3, 1, 1), (2, 7, 5, 3), (16, 32, 16, 16)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("mode", ["plain", "relu", "residual_relu"])
def test_fused_batchnorm_matches_torch(shape, mode):
    from addernetcuda_b200.batchnorm import FusedBatchNorm2d
    torch.manual_seed(sum(shape) * 3 + ["plain", "relu", "residual_relu"].index(mode))
    n, c, h, w = shape
    y = torch.randn(shape) * 3 + 1.5
    res = torch.randn(shape) if mode == "residual_relu" else None
    relu = mode != "plain"
    dz = torch.randn(shape)
    ref = nn.BatchNorm2d(c).double()
    with torch.no_grad():
        ref.weight.copy_(torch.rand(c) + 0.5)
        ref.bias.copy_(torch.randn(c) * 0.3)
    if relu:
        # Whether a pre-activation within rounding of zero passes the ReLU is a coin toss between fp32 and
        # fp64; no gradient is sent through those (few) elements, so that the mask does not enter the comparison.
        with torch.no_grad():
            probe = nn.BatchNorm2d(c).double()
            probe.load_state_dict(ref.state_dict())
            pre = probe.train()(y.double()) + (res.double() if res is not None else 0.0)
            dz[pre.abs() < 1e-4] = 0.0
    bn = FusedBatchNorm2d(c).to(DEV)
    bn.load_state_dict({k: v.float() for k, v in ref.state_dict().items()})
    ref.train(); bn.train()
    for step in range(2):       # two steps: running statistics accumulate
        yr = y.double().requires_grad_()
        rr = res.double().requires_grad_() if res is not None else None
        zr = ref(yr)
        if rr is not None:
            zr = zr + rr
        if relu:
            zr = torch.relu(zr)
        zr.backward(dz.double())
        yg = y.to(DEV).requires_grad_()
        rg = res.to(DEV).requires_grad_() if res is not None else None
        ref_grads = (ref.weight.grad.clone(), ref.bias.grad.clone())
        ref.zero_grad()
        bn.zero_grad()
        zg = bn(yg, residual=rg, relu=relu)
        zg.backward(dz.to(DEV))
        torch.cuda.synchronize()
        checks = [("z", zg, zr), ("dy", yg.grad, yr.grad), ("dgamma", bn.weight.grad, ref_grads[0]),
                  ("dbeta", bn.bias.grad, ref_grads[1]), ("running_mean", bn.running_mean, ref.running_mean),
                  ("running_var", bn.running_var, ref.running_var)]
        if rg is not None:
            checks.append(("dresidual", rg.grad, rr.grad))
        for name, got, want in checks:
            scale = max(1.0, float(want.detach().abs().max()))
            ok, err, msg = O.compare(f"{name} step{step}", got.double().cpu() / scale, want.detach() / scale, rel=1e-5, abs_=2e-5)
            assert ok, msg
    assert int(bn.num_batches_tracked) == 2


def test_eval_mode_and_state_dict_are_plain_batchnorm():
    from addernetcuda_b200.batchnorm import FusedBatchNorm2d
    bn = FusedBatchNorm2d(6).to(DEV)
    ref = nn.BatchNorm2d(6).to(DEV)
    assert list(bn.state_dict().keys()) == list(ref.state_dict().keys())
    ref.load_state_dict(bn.state_dict())
    x = torch.randn(4, 6, 5, 5, device=DEV)
    bn.eval(); ref.eval()
    assert torch.allclose(bn(x), ref(x))
