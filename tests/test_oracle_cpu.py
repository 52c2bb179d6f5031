"""CPU checks of the oracle against the committed reference outputs (no GPU, no reference checkout)."""
import numpy as np
import pytest
import torch

from oracle import adder_oracle as O, adder_unfold
from tests.cases import COL_CASES, LAYER_CASES, draw_cols, draw_layer, resnet20_batch

# keep the CPU suite to a few minutes: the biggest ResNet-50 cases are checked in float32 only
_BIG = {"r50_n2_c256to256_14x14_k3s1p1", "r50_n2_c512to512_7x7_k3s1p1"}


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


@pytest.mark.parametrize("case", LAYER_CASES, ids=lambda c: c["name"])
def test_unfold_forms_match_reference_outputs(case, golden):
    x, w, g = (_t(a) for a in draw_layer(case))
    s, p = case["stride"], case["pad"]
    out = O.adder2d_forward_unfold(x, w, s, p)
    gx, gws, gw = O.adder2d_backward_unfold(g, x, w, s, p)
    for key, got in (("out", out), ("grad_x", gx), ("grad_w", gws), ("grad_w_unscaled", gw)):
        ok, worst, msg = golden.check(case["name"], key, got)
        assert ok, msg


@pytest.mark.parametrize("case", [c for c in LAYER_CASES if c["name"] not in _BIG], ids=lambda c: c["name"])
def test_direct_float64_forms_match_reference_outputs(case, golden):
    x, w, g = (_t(a) for a in draw_layer(case))
    s, p = case["stride"], case["pad"]
    out = O.adder2d_forward_direct(x, w, s, p)
    gx, gws, gw = O.adder2d_backward_direct(g, x, w, s, p)
    for key, got in (("out", out), ("grad_x", gx), ("grad_w", gws)):
        ok, worst, msg = golden.check(case["name"], key, got)
        assert ok, msg
    # the rescaled gradient has norm eta * sqrt(numel) by construction (adder.py:78)
    assert abs(float(gws.norm()) - 0.2 * np.sqrt(gws.numel())) < 1e-6 * np.sqrt(gws.numel())


@pytest.mark.parametrize("case", COL_CASES, ids=lambda c: c["name"])
def test_column_forms_match_reference_outputs(case, golden):
    W, X, g = (_t(a) for a in draw_cols(case))
    for key, got in (("y", O.forward_col(W, X)), ("grad_W", O.rescale(O.grad_w_col(W, X, g))),
                     ("grad_X", O.grad_x_col(W, X, g)), ("grad_W_unscaled", O.grad_w_col(W, X, g))):
        ok, worst, msg = golden.check(case["name"], key, got)
        assert ok, msg


def test_output_size_truncates_like_the_reference():
    assert O.out_hw(9, 8, 3, 2, 1) == (5, 4)      # (8 - 3 + 2) / 2 + 1 = 4.5 -> 4   (adder.py:26-31)
    assert O.out_hw(32, 32, 1, 2, 0) == (16, 16)
    assert O.out_hw(7, 7, 3, 2, 1) == (4, 4)


def test_padding_counts_as_zero_input():
    # one pixel, 3x3 kernel, pad 1: eight of the nine taps read padding and contribute |0 - w|
    x = torch.tensor([[[[2.0]]]])
    w = torch.arange(9, dtype=torch.float32).view(1, 1, 3, 3) / 10
    out = O.adder2d_forward_direct(x, w, 1, 1, dtype=torch.float32)
    want = -(w.abs().sum() - w[0, 0, 1, 1].abs() + (2.0 - w[0, 0, 1, 1]).abs())
    assert abs(float(out) - float(want)) < 1e-6


def test_empty_batch():
    x = torch.zeros((0, 3, 5, 5))
    w = torch.randn(4, 3, 3, 3)
    assert O.adder2d_forward_direct(x, w, 1, 1).shape == (0, 4, 5, 5)


def test_resnet20_step_matches_reference_fixture():
    """The oracle network (this repository's builder + the oracle layer) reproduces the reference's
    resnet20.py training step stored in the fixture (batch 16)."""
    from addernetcuda_b200 import resnet as R
    z = np.load("tests/golden/resnet20_b16.npz")
    net = R.resnet20(conv=adder_unfold.adder2d)
    R.init_seeded(net, 1434)
    images, labels = resnet20_batch(16, 1434)
    net.train()
    logits = net(_t(images))
    loss = torch.nn.functional.cross_entropy(logits, _t(labels))
    loss.backward()
    ok, worst, msg = O.compare("logits", logits, _t(z["logits"]))
    assert ok, msg
    assert abs(float(loss.detach()) - float(z["loss"])) < 1e-5
    grads = dict(net.named_parameters())
    assert [str(k) for k in z["keys"]] == list(grads.keys())
    for k, p in grads.items():
        ok, worst, msg = O.compare(k, p.grad, _t(z["grad/" + k]))
        assert ok, msg


@pytest.mark.parametrize("stride,padding", [(1, 1), (2, 1), (1, 0)])
def test_general_geometry_oracle_agrees_with_the_direct_one_on_square_kernels(stride, padding):
    """adder2d_general (any kernel extent / dilation) restates the same three expressions: on a 3x3 layer
    it must give what the direct float64 sums give."""
    torch.manual_seed(5 + stride)
    x, w = torch.randn(3, 5, 9, 9), torch.randn(7, 5, 3, 3)
    ho, wo = O.out_hw(9, 9, 3, stride, padding)
    g = torch.randn(3, 7, ho, wo)
    out, gx, gw = O.adder2d_general(g, x, w, stride, padding)
    gx_d, gws_d, _ = O.adder2d_backward_direct(g, x, w, stride, padding)
    for name, a, b in (("out", out, O.adder2d_forward_direct(x, w, stride, padding)), ("grad_x", gx, gx_d),
                       ("grad_w", gw, gws_d)):
        ok, worst, msg = O.compare(name, a, b, 1e-9, 1e-9)
        assert ok, msg
