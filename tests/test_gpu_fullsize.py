"""Full-size checks (batch 256, the per-layer shapes of the benchmark definition) through properties
that do not need a full-size CPU result:
  * images are independent in the forward and in the input gradient, so a few images cut out of the
    full batch must match the oracle run on just those images;
  * the unscaled weight gradient is additive over the batch: halves sum to the whole;
  * the rescaled weight gradient has L2 norm eta * sqrt(numel) (adder.py:78);
  * the result for a sub-batch is bitwise the same whether computed alone or inside the big batch, and the
    same call twice gives the same bits.
"""
import math

import numpy as np
import pytest
import torch

from oracle import adder_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# (Ci, Co, H, W, stride, k, pad) at batch 256
SHAPES = [
    (16, 16, 32, 32, 1, 3, 1),
    (16, 32, 32, 32, 2, 3, 1),
    (32, 32, 16, 16, 1, 3, 1),
    (64, 64, 8, 8, 1, 3, 1),
    (256, 256, 14, 14, 1, 3, 1),
    (512, 512, 7, 7, 1, 3, 1),
    (1024, 256, 14, 14, 1, 1, 0),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "c%dto%d_%dx%d_s%d_k%d" % s[:6])
def test_full_batch_properties(shape):
    from addernetcuda_b200 import adder_cuda as ac
    ci, co, h, w, s, k, p = shape
    n = 256
    gen = torch.Generator(device=DEV).manual_seed(1234 + 300 + ci + co + h)
    x = torch.randn((n, ci, h, w), device=DEV, generator=gen)
    wt = torch.randn((co, ci, k, k), device=DEV, generator=gen) * math.sqrt(2.0 / (ci * k * k))
    ho, wo = O.out_hw(h, w, k, s, p)
    g = torch.randn((n, co, ho, wo), device=DEV, generator=gen)

    out = ac.forward(x, wt, s, p)
    gx = ac.backward_input(g, x, wt, s, p)
    gx_fast = ac.backward_input(g, x, wt, s, p, fast_clamp=True)
    gw = ac.backward_weight(g, x, wt, s, p)
    gw_raw = ac.backward_weight(g, x, wt, s, p, eta=0.0)

    # (1) a few images against the oracle (unfold form, fp32 on the CPU like the reference path)
    pick = [0, 101, 255] if ci * co <= 64 * 64 else [255]
    xs, gs = x[pick].cpu(), g[pick].cpu()
    want_out = O.adder2d_forward_unfold(xs, wt.cpu(), s, p)
    want_gx, _, _ = O.adder2d_backward_unfold(gs, xs, wt.cpu(), s, p)
    for name, got, want in (("out", out[pick], want_out), ("grad_x", gx[pick], want_gx),
                            ("grad_x(fast)", gx_fast[pick], want_gx)):
        ok, worst, msg = O.compare(name, got, want)
        print("   ", msg)
        assert ok, msg

    # (2) additivity of the unscaled weight gradient over the batch
    half = n // 2
    a = ac.backward_weight(g[:half].contiguous(), x[:half].contiguous(), wt, s, p, eta=0.0)
    b = ac.backward_weight(g[half:].contiguous(), x[half:].contiguous(), wt, s, p, eta=0.0)
    scale = float(gw_raw.abs().max())
    ok, worst, msg = O.compare("grad_w halves/scale", (a + b) / scale, gw_raw / scale)
    print("   ", msg)
    assert ok, msg

    # (3) rescale: direction of the raw gradient, norm eta*sqrt(numel)
    numel = gw.numel()
    assert abs(float(gw.double().norm()) - 0.2 * math.sqrt(numel)) <= 1e-5 * math.sqrt(numel)
    want_scaled = gw_raw.double() / gw_raw.double().norm() * math.sqrt(numel) * 0.2
    ok, worst, msg = O.compare("grad_w rescaled", gw, want_scaled)
    print("   ", msg)
    assert ok, msg

    # (4) sub-batch alone == sub-batch inside the big batch, bit for bit (forward and input gradient are
    # per-image sums whose chunking does not depend on the batch size)
    sub = slice(64, 72)
    assert torch.equal(ac.forward(x[sub].contiguous(), wt, s, p), out[sub])
    assert torch.equal(ac.backward_input(g[sub].contiguous(), x[sub].contiguous(), wt, s, p), gx[sub])
    # (5) and the same call twice gives the same bits
    assert torch.equal(ac.forward(x, wt, s, p), out)
    assert torch.equal(ac.backward_input(g, x, wt, s, p), gx)
    assert torch.equal(ac.backward_weight(g, x, wt, s, p), gw)
