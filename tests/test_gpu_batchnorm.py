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


# (n, ci, co, hw, k, stride, pad): every register tile of the forward kernel, ragged planes, 1x1 layers
STAT_LAYERS = [(32, 16, 16, 32, 3, 1, 1), (16, 32, 32, 16, 3, 1, 1), (8, 64, 64, 8, 3, 1, 1), (8, 16, 32, 32, 3, 2, 1),
               (4, 24, 40, 14, 3, 1, 1), (3, 5, 7, 9, 3, 1, 1), (4, 64, 256, 14, 1, 1, 0), (2, 8, 12, 7, 1, 2, 0),
               (1, 3, 4, 5, 3, 1, 0)]


@pytest.mark.parametrize("layer", STAT_LAYERS, ids=lambda l: "n%d_c%dto%d_%d_k%ds%dp%d" % l)
def test_forward_statistics_epilogue_feeds_the_batchnorm(layer):
    """The adder layer's forward with the statistics epilogue: same output bits as the plain forward; the
    slices add up to the per-channel sums of the output and of its squares; and batch norm fed by them gives
    what batch norm that measures the output itself gives (z, saved statistics, running estimates, gradients)."""
    from addernetcuda_b200 import adder_cuda as ac
    from addernetcuda_b200.adder import adder2d
    from addernetcuda_b200.batchnorm import FusedBatchNorm2d
    n, ci, co, hw, k, s, p = layer
    torch.manual_seed(n * 7 + co)
    x = torch.randn(n, ci, hw, hw, device=DEV)
    conv = adder2d(ci, co, k, stride=s, padding=p).to(DEV)
    plain = ac.forward(x, conv.adder.detach(), s, p)
    out, st = ac.forward(x, conv.adder.detach(), s, p, stats=True)
    assert torch.equal(out, plain)
    if st.shape[1] == 0:
        pytest.skip("this geometry's forward kernel has no statistics epilogue")
    assert st.shape == (co, st.shape[1], 2) and st.dtype == torch.float64
    tot = st.sum(dim=1).cpu()
    yd = plain.double().cpu()
    want_s = yd.sum(dim=(0, 2, 3))
    want_q = (yd * yd).sum(dim=(0, 2, 3))
    scale = yd.abs().sum(dim=(0, 2, 3))
    assert torch.all((tot[:, 0] - want_s).abs() <= 1e-6 * scale), (tot[:, 0] - want_s).abs().max()
    assert torch.all((tot[:, 1] - want_q).abs() <= 1e-6 * want_q), ((tot[:, 1] - want_q).abs() / want_q).max()

    # the layer pair, once with the statistics handed over and once measured by the batch norm itself
    res = torch.randn_like(plain)
    dz = torch.randn_like(plain)
    gamma, beta = torch.rand(co) + 0.5, torch.randn(co) * 0.3
    ref64 = nn.BatchNorm2d(co).double()
    with torch.no_grad():
        ref64.weight.copy_(gamma); ref64.bias.copy_(beta)
        # gates of pre-activations within rounding of zero may differ between the two statistics paths:
        # no gradient is sent through those elements
        pre = ref64.train()(yd) + res.double().cpu()
        dz[(pre.abs() < 1e-4).to(DEV)] = 0.0

    def run(fused):
        bn = FusedBatchNorm2d(co).to(DEV)
        with torch.no_grad():
            bn.weight.copy_(gamma); bn.bias.copy_(beta)
        conv.zero_grad()
        xr = x.clone().requires_grad_()
        if fused:
            y, st_ = conv.forward_with_stats(xr)
            assert st_ is not None
            z = bn(y, residual=res, relu=True, stats=st_)
        else:
            z = bn(conv(xr), residual=res, relu=True)
        z.backward(dz)
        torch.cuda.synchronize()
        assert int(bn.num_batches_tracked) == 1
        return {"z": z.detach(), "running_mean": bn.running_mean.clone(), "running_var": bn.running_var.clone(),
                "dx": xr.grad.clone(), "dw": conv.adder.grad.clone(), "dgamma": bn.weight.grad.clone(),
                "dbeta": bn.bias.grad.clone()}

    got, want = run(True), run(False)
    for name in want:
        ok, worst, msg = O.compare(name, got[name], want[name])
        print("   ", msg)
        assert ok, msg
