"""adder2d for the geometries the fused kernels are not built for (5x5, 7x7, 2x2 and rectangular kernels,
stride 3, dilation): they run through the column-matrix kernels behind an explicit im2col, as the reference
runs every layer (adder.py:22-41), and must agree with the float64 oracle like any other layer."""
import pytest
import torch

from oracle import adder_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# (n, ci, co, h, w, kernel, stride, padding, dilation)
CASES = [(4, 6, 10, 16, 16, 5, 1, 2, 1), (2, 3, 16, 33, 33, 7, 2, 3, 1), (3, 8, 12, 12, 20, (3, 5), 1, (1, 2), 1),
         (2, 16, 8, 17, 17, 3, 3, 1, 1), (2, 8, 8, 14, 14, 3, 1, 2, 2), (5, 4, 6, 8, 8, 2, 2, 0, 1),
         (1, 1, 1, 5, 5, 5, 1, 0, 1)]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "n%d_c%dto%d_%dx%d_k%s_s%s_p%s_d%s" % c)
def test_general_geometry_layer_matches_float64_oracle(case):
    from addernetcuda_b200.adder import adder2d, _fused_geometry
    n, ci, co, h, w, k, s, p, d = case
    torch.manual_seed(ci * 31 + co)
    layer = adder2d(ci, co, k, stride=s, padding=p, dilation=d).to(DEV)
    assert not _fused_geometry(layer.adder, s, p, d)
    x = torch.randn(n, ci, h, w)
    xg = x.to(DEV).requires_grad_()
    out = layer(xg)
    g = torch.randn(out.shape)
    out.backward(g.to(DEV))
    torch.cuda.synchronize()
    want_out, want_gx, want_gw = O.adder2d_general(g, x, layer.adder.detach().cpu(), s, p, d)
    for name, got, want in (("out", out, want_out), ("grad_x", xg.grad, want_gx), ("grad_w", layer.adder.grad, want_gw)):
        assert got.shape == want.shape, (name, got.shape, want.shape)
        ok, worst, msg = O.compare(name, got, want)
        print("   ", msg)
        assert ok, msg


def test_fused_geometries_do_not_take_the_column_path():
    from addernetcuda_b200.adder import adder2d, _fused_geometry
    for k, s in ((1, 1), (1, 2), (3, 1), (3, 2)):
        layer = adder2d(4, 4, k, stride=s, padding=k // 2)
        assert _fused_geometry(layer.adder, layer.stride, layer.padding, layer.dilation)
