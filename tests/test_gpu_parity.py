"""Parity of the CUDA kernels (called through the C ABI) with the reference outputs and the oracle.

Tolerance: |got - want| <= 1e-4 + 1e-5 * |want| per element in fp32, the bound the benchmark
definition states; the maximum absolute error per tensor is printed (run with -s to see it).
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import adder_oracle as O
from tests.cases import COL_CASES, LAYER_CASES, draw_cols, draw_layer

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _gpu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _assert(ok_msg):
    ok, worst, msg = ok_msg
    print("   ", msg)
    assert ok, msg


@pytest.fixture(scope="module")
def ac():
    from addernetcuda_b200 import adder_cuda
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return adder_cuda


@pytest.mark.parametrize("case", LAYER_CASES, ids=lambda c: c["name"])
def test_layer_matches_reference_outputs(case, golden, ac):
    x, w, g = (_gpu(a) for a in draw_layer(case))
    s, p = case["stride"], case["pad"]
    out = ac.forward(x, w, s, p)
    _assert(golden.check(case["name"], "out", out))
    gx = ac.backward_input(g, x, w, s, p)
    _assert(golden.check(case["name"], "grad_x", gx))
    gx_fast = ac.backward_input(g, x, w, s, p, fast_clamp=True)
    _assert(golden.check(case["name"], "grad_x", gx_fast))
    gw = ac.backward_weight(g, x, w, s, p)                        # eta = 0.2, rescaled
    _assert(golden.check(case["name"], "grad_w", gw))
    gw_raw, norm = ac.backward_weight(g, x, w, s, p, eta=0.0, return_norm=True)
    # unscaled sums grow with the number of pixels: compare relative to their own scale
    got_s, want_s = golden.pair(case["name"], "grad_w_unscaled", gw_raw)
    scale = max(1.0, float(want_s.abs().max()))
    _assert(O.compare("grad_w_unscaled/scale", got_s / scale, want_s / scale))
    assert abs(float(norm) - float(gw_raw.double().norm())) <= 1e-5 * float(norm) + 1e-6
    torch.cuda.synchronize()


@pytest.mark.parametrize("case", [c for c in LAYER_CASES if c["n"] * c["ci"] * c["co"] * c["h"] * c["w"] <= 1 << 22],
                         ids=lambda c: c["name"])
def test_layer_matches_float64_oracle(case, ac):
    """Against the independent float64 direct form computed now (no stored numbers involved)."""
    x, w, g = draw_layer(case)
    s, p = case["stride"], case["pad"]
    xt, wt, gt = (torch.from_numpy(a) for a in (x, w, g))
    want_out = O.adder2d_forward_direct(xt, wt, s, p)
    want_gx, want_gws, _ = O.adder2d_backward_direct(gt, xt, wt, s, p)
    xg, wg, gg = _gpu(x), _gpu(w), _gpu(g)
    _assert(O.compare("out", ac.forward(xg, wg, s, p), want_out))
    _assert(O.compare("grad_x", ac.backward_input(gg, xg, wg, s, p), want_gx))
    _assert(O.compare("grad_x(fast)", ac.backward_input(gg, xg, wg, s, p, fast_clamp=True), want_gx))
    _assert(O.compare("grad_w", ac.backward_weight(gg, xg, wg, s, p), want_gws))


@pytest.mark.parametrize("case", COL_CASES, ids=lambda c: c["name"])
def test_reference_extension_entry_points(case, golden, ac):
    """ADDER_CONV / ADDER_CONV_WEIGHT / ADDER_CONV_INPUT / ADDER_BACKWARD with the reference's
    argument order and buffer semantics (overwrite y, accumulate into gradients)."""
    W, X, g = (_gpu(a) for a in draw_cols(case))
    Co, K = W.shape
    P = X.shape[1]
    y = torch.full((Co, P), 7.0, device=DEV)                 # ADDER_CONV must overwrite, not add
    ac.ADDER_CONV(X, W, y)
    _assert(golden.check(case["name"], "y", y))
    gw = torch.zeros((Co, K), device=DEV)
    gi = torch.zeros((K, P), device=DEV)
    ac.ADDER_BACKWARD(g, X, W, gw, gi)
    _assert(golden.check(case["name"], "grad_X", gi))
    got_s, want_s = golden.pair(case["name"], "grad_W_unscaled", gw)
    scale = max(1.0, float(want_s.abs().max()))
    _assert(O.compare("grad_W_unscaled/scale", got_s / scale, want_s / scale))
    # accumulate semantics: a second call doubles the buffers
    ac.ADDER_CONV_WEIGHT(g, X, W, gw)
    ac.ADDER_CONV_INPUT(g, X, W, gi)
    got_s, want_s = golden.pair(case["name"], "grad_W_unscaled", gw)
    _assert(O.compare("2*grad_W/scale", got_s / scale, 2 * want_s / scale))
    got_s, want_s = golden.pair(case["name"], "grad_X", gi)
    _assert(O.compare("2*grad_X", got_s, 2 * want_s, abs_=2e-4))
    # the column-level autograd Function of adder.py:43-80
    from addernetcuda_b200 import adder as A
    Wr, Xr = W.clone().requires_grad_(), X.clone().requires_grad_()
    A.adder.apply(Wr, Xr).backward(g)
    _assert(golden.check(case["name"], "grad_W", Wr.grad))
    _assert(golden.check(case["name"], "grad_X", Xr.grad))


@pytest.mark.parametrize("tile", [(8, 8), (8, 4), (4, 4)], ids=lambda t: "px%d_ch%d" % t)
@pytest.mark.parametrize("name", ["r20_n4_c16to16_32x32_k3s1p1", "r20_n4_c16to32_32x32_k3s2p1", "r20_n4_c32to64_16x16_k1s2p0",
                                  "odd_n1_c6to10_3x70_k3s1p1", "odd_n2_c7to5_9x9_k1s1p0"])
def test_every_register_tile(name, tile, golden, ac):
    """The launcher picks the per-thread register tile from the layer size; force each one in turn so
    that all compiled variants are checked on small cases too."""
    from addernetcuda_b200 import _lib
    from tests.cases import LAYER_BY_NAME
    case = LAYER_BY_NAME[name]
    x, w, g = (_gpu(a) for a in draw_layer(case))
    s, p = case["stride"], case["pad"]
    with _lib.tuning() as lib:
        assert lib.adder_b200_set_micro_tile(0, tile[0], tile[1]) == 0
        assert lib.adder_b200_set_micro_tile(1, tile[0], 4) == 0
        _assert(golden.check(name, "out", ac.forward(x, w, s, p)))
        _assert(golden.check(name, "grad_x", ac.backward_input(g, x, w, s, p)))
        _assert(golden.check(name, "grad_x", ac.backward_input(g, x, w, s, p, fast_clamp=True)))


@pytest.mark.parametrize("variant", [1, 2], ids=["pixel-lane kernel", "warp-tile kernel with cp.async"])
@pytest.mark.parametrize("case", [c for c in LAYER_CASES if c["k"] == 3 and c["ci"] % 16 == 0 and c["co"] % 16 == 0],
                         ids=lambda c: c["name"])
def test_weight_gradient_kernel_families(case, variant, golden, ac):
    """3x3 layers with channels in sixteens take the warp-tile weight-gradient kernel fed by tiled bulk copies
    (stride 1) or by cp.async (stride 2, unaligned tensors).  The other two families, which remain the path
    of every geometry the default does not cover, must give the reference's gradient on the same layers."""
    from addernetcuda_b200 import _lib
    x, w, g = (_gpu(a) for a in draw_layer(case))
    s, p = case["stride"], case["pad"]
    shape = (case["n"], case["ci"], case["h"], case["w"], case["co"], case["k"], s, p)
    default_plan = _lib.describe_plan(2, *shape, 0)
    with _lib.tuning() as lib:
        assert lib.adder_b200_set_variant(2, variant) == 0
        plan = _lib.describe_plan(2, *shape, 0)
        assert "tma" not in plan, plan
        if s == 1 and "tma" in default_plan:
            assert plan != default_plan
        if variant == 1:
            assert "warp-tile" not in plan, plan
        _assert(golden.check(case["name"], "grad_w", ac.backward_weight(g, x, w, s, p)))
        gw_raw = ac.backward_weight(g, x, w, s, p, eta=0.0)
        got_s, want_s = golden.pair(case["name"], "grad_w_unscaled", gw_raw)
        scale = max(1.0, float(want_s.abs().max()))
        _assert(O.compare("grad_w_unscaled/scale", got_s / scale, want_s / scale))


@pytest.mark.parametrize("geom", [(4, 32, 48, 14, 14, 1), (6, 16, 32, 7, 7, 1), (3, 32, 32, 28, 28, 1), (4, 32, 16, 28, 28, 2),
                                  (5, 16, 64, 14, 14, 2), (2, 64, 32, 13, 27, 2)],
                         ids=lambda t: "n%d_c%dto%d_%dx%d_s%d" % t)
def test_warp_tile_weight_gradient_on_imagenet_planes(geom, ac):
    """Output planes 7, 14 and 28 wide (resnet50.py's stages 2-4) take the warp-tile weight-gradient kernel
    with 7- or 4-pixel segments; against the float64 oracle, and equal to what the pixel-lane kernel gives."""
    from addernetcuda_b200 import _lib
    n, ci, co, h, w_, s = geom
    plan = _lib.describe_plan(2, n, ci, h, w_, co, 3, s, 1, 0)
    assert "warp-tile" in plan, plan
    gen = torch.Generator().manual_seed(311 + n + ci + co + h + s)
    x = torch.randn(n, ci, h, w_, generator=gen)
    w = torch.randn(co, ci, 3, 3, generator=gen) * 0.4
    ho, wo = (h + 2 - 3) // s + 1, (w_ + 2 - 3) // s + 1
    g = torch.randn(n, co, ho, wo, generator=gen)
    _, want_gws, want_gw = O.adder2d_backward_direct(g, x, w, s, 1)
    xg, wg, gg = x.to(DEV), w.to(DEV), g.to(DEV)
    got = ac.backward_weight(gg, xg, wg, s, 1)
    _assert(O.compare("grad_w", got, want_gws))
    raw = ac.backward_weight(gg, xg, wg, s, 1, eta=0.0)
    scale = max(1.0, float(want_gw.abs().max()))
    _assert(O.compare("grad_w_unscaled/scale", raw.cpu() / scale, want_gw / scale))
    assert torch.equal(ac.backward_weight(gg, xg, wg, s, 1), got)        # same bits twice
    with _lib.tuning() as lib:
        assert lib.adder_b200_set_variant(2, 1) == 0
        assert "warp-tile" not in _lib.describe_plan(2, n, ci, h, w_, co, 3, s, 1, 0)
        _assert(O.compare("pixel-lane kernel", ac.backward_weight(gg, xg, wg, s, 1), want_gws))


def test_module_autograd_and_bias(ac):
    from addernetcuda_b200 import adder as A
    from oracle import adder_unfold as U
    torch.manual_seed(3)
    m = A.adder2d(5, 7, 3, stride=1, padding=1, bias=True).to(DEV)
    mo = U.adder2d(5, 7, 3, stride=1, padding=1, bias=True)
    mo.load_state_dict({k: v.cpu() for k, v in m.state_dict().items()})
    x = torch.randn(3, 5, 9, 6)
    xg = x.to(DEV).requires_grad_()
    xo = x.clone().requires_grad_()
    yg = m(xg)
    yo = mo(xo)
    _assert(O.compare("module out", yg, yo))
    gy = torch.randn_like(yo)
    yg.backward(gy.to(DEV))
    yo.backward(gy)
    _assert(O.compare("module grad_x", xg.grad, xo.grad))
    _assert(O.compare("module grad adder", m.adder.grad, mo.adder.grad))
    _assert(O.compare("module grad b", m.b.grad, mo.b.grad))


def test_run_twice_is_bitwise_identical(ac):
    """The kernels use no atomics: any run-to-run difference would be a race."""
    case = next(c for c in LAYER_CASES if c["name"].startswith("r20_n4_c16to32_32x32_k3s2"))
    x, w, g = (_gpu(a) for a in draw_layer(case))
    s, p = case["stride"], case["pad"]
    a = [ac.forward(x, w, s, p), ac.backward_input(g, x, w, s, p), ac.backward_weight(g, x, w, s, p)]
    b = [ac.forward(x, w, s, p), ac.backward_input(g, x, w, s, p), ac.backward_weight(g, x, w, s, p)]
    for u, v in zip(a, b):
        assert torch.equal(u, v)


def test_no_write_outside_the_outputs(ac):
    """Outputs are carved out of larger buffers pre-filled with a NaN pattern; after the kernels the
    guard bands on both sides must be untouched (catches out-of-bounds stores)."""
    from addernetcuda_b200 import _lib
    lib = _lib.load()
    case = next(c for c in LAYER_CASES if c["name"] == "odd_n3_c4to6_9x8_k3s2p1")
    x, w, g = (_gpu(a) for a in draw_layer(case))
    n, ci, co, h, wd, k, s, p = (case[q] for q in ("n", "ci", "co", "h", "w", "k", "stride", "pad"))
    ho, wo = O.out_hw(h, wd, k, s, p)
    GUARD = 256
    stream = torch.cuda.current_stream().cuda_stream

    def guarded(numel):
        buf = torch.full((numel + 2 * GUARD,), float("nan"), device=DEV)
        return buf, buf[GUARD:GUARD + numel]

    geom = (n, ci, h, wd, co, k, s, p)
    b_out, v_out = guarded(n * co * ho * wo)
    assert lib.adder_b200_forward(x.data_ptr(), w.data_ptr(), v_out.data_ptr(), *geom, stream) == 0
    b_gx, v_gx = guarded(x.numel())
    assert lib.adder_b200_backward_input(g.data_ptr(), x.data_ptr(), w.data_ptr(), v_gx.data_ptr(), *geom, 0, stream) == 0
    b_gw, v_gw = guarded(w.numel())
    nbytes = lib.adder_b200_backward_weight_workspace_bytes(*geom)
    ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=DEV)
    assert ws.data_ptr() % 256 == 0
    assert lib.adder_b200_backward_weight(g.data_ptr(), x.data_ptr(), w.data_ptr(), v_gw.data_ptr(), ctypes.c_float(0.2),
                                          None, ws.data_ptr(), nbytes, *geom, 0, stream) == 0
    torch.cuda.synchronize()
    for buf, view in ((b_out, v_out), (b_gx, v_gx), (b_gw, v_gw)):
        assert torch.isnan(buf[:GUARD]).all() and torch.isnan(buf[-GUARD:]).all()
        assert torch.isfinite(view).all()
    # too-small workspace is refused, not overrun
    assert lib.adder_b200_backward_weight(g.data_ptr(), x.data_ptr(), w.data_ptr(), v_gw.data_ptr(), ctypes.c_float(0.2),
                                          None, ws.data_ptr(), 16, *geom, 0, stream) == 5


def test_errors_are_statuses_not_aborts(ac):
    x = torch.randn(2, 3, 8, 8, device=DEV)
    w = torch.randn(4, 3, 5, 5, device=DEV)
    with pytest.raises(ValueError):
        ac.forward(x, w, 1, 2)                      # k = 5: unsupported, reported as an exception
    with pytest.raises(RuntimeError, match="contiguous"):
        ac.forward(x.permute(0, 1, 3, 2), torch.randn(4, 3, 3, 3, device=DEV), 1, 1)
    with pytest.raises(TypeError):
        ac.forward(x.double(), torch.randn(4, 3, 3, 3, device=DEV).double(), 1, 1)
    # shapes the reference aborts on (Co, P not multiples of 16/12/8; adder.cu:294-297) just work
    y = torch.empty(5, 50, device=DEV)
    ac.ADDER_CONV(torch.randn(27, 50, device=DEV), torch.randn(5, 27, device=DEV), y)
    assert torch.isfinite(y).all()
    assert ac.forward(torch.zeros(0, 3, 8, 8, device=DEV), torch.randn(4, 3, 3, 3, device=DEV), 1, 1).shape == (0, 4, 8, 8)


@pytest.mark.parametrize("geom", [(16, 32, 32, 32, 1, 2, 0), (16, 32, 32, 16, 3, 1, 1), (64, 14, 14, 128, 1, 1, 0)],
                         ids=lambda t: "c%d_%dx%d_to%d_k%ds%dp%d" % t)
def test_weight_gradient_of_an_empty_batch_is_zero(geom, ac):
    """n = 0 through the C ABI: no pixels, so grad_w is all zeros (and stays finite under the rescale)."""
    from addernetcuda_b200 import _lib
    lib = _lib.load()
    ci, h, wd, co, k, s, p = geom
    g8 = (0, ci, h, wd, co, k, s, p)
    w = torch.randn(co, ci, k, k, device=DEV)
    gw = torch.full_like(w, float("nan"))
    nbytes = lib.adder_b200_backward_weight_workspace_bytes(*g8)
    assert nbytes > 0
    ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=DEV)
    st = lib.adder_b200_backward_weight(None, None, w.data_ptr(), gw.data_ptr(), ctypes.c_float(0.2), None,
                                        ws.data_ptr(), nbytes, *g8, 0, torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.adder_b200_status_string(st)
    torch.cuda.synchronize()
    assert torch.equal(gw, torch.zeros_like(gw))


@pytest.mark.parametrize("geom", [(3, 16, 32, 32, 32), (2, 32, 64, 16, 16), (2, 5, 7, 9, 11), (1, 33, 20, 6, 5), (2, 64, 64, 8, 8)],
                         ids=lambda t: "n%d_c%dto%d_%dx%d" % t)
def test_pointwise_stride2_kernels(geom, ac):
    """1x1 stride-2 layers with few channels take the one-thread-per-position kernels.  They must agree
    with the float64 oracle, write every input pixel (zeros where no output reads), honour the
    accumulate flag, and agree with the tiled kernels that a tile hint selects instead."""
    from addernetcuda_b200 import _lib
    lib = _lib.load()
    n, ci, co, h, w_ = geom
    assert "pointwise" in _lib.describe_plan(0, n, ci, h, w_, co, 1, 2, 0, 0)
    assert "pointwise" in _lib.describe_plan(1, n, ci, h, w_, co, 1, 2, 0, 1)
    gen = torch.Generator().manual_seed(77 + n + ci + co + h)
    x = torch.randn(n, ci, h, w_, generator=gen)
    w = torch.randn(co, ci, 1, 1, generator=gen) * 0.7
    ho, wo = (h - 1) // 2 + 1, (w_ - 1) // 2 + 1
    g = torch.randn(n, co, ho, wo, generator=gen)
    want_out = O.adder2d_forward_direct(x, w, 2, 0)
    want_gx, want_gws, want_gw = O.adder2d_backward_direct(g, x, w, 2, 0)
    xg, wg, gg = x.to(DEV), w.to(DEV), g.to(DEV)
    out = ac.forward(xg, wg, 2, 0)
    _assert(O.compare("out", out, want_out))
    assert "pointwise=1" in _lib.describe_plan(2, n, ci, h, w_, co, 1, 2, 0, 0)
    _assert(O.compare("grad_w", ac.backward_weight(gg, xg, wg, 2, 0), want_gws))
    gw_raw = ac.backward_weight(gg, xg, wg, 2, 0, eta=0.0)
    scale = max(1.0, float(want_gw.abs().max()))
    _assert(O.compare("grad_w_unscaled/scale", gw_raw.cpu() / scale, want_gw / scale))
    for fast in (False, True):
        gx = ac.backward_input(gg, xg, wg, 2, 0, fast_clamp=fast)
        _assert(O.compare("grad_x fast=%d" % fast, gx, want_gx))
        # every element is written: a poisoned buffer comes back finite, zeros off the sampled grid
        buf = torch.full_like(xg, float("nan"))
        flags = _lib.FLAG_FAST_CLAMP if fast else 0
        args = (gg.data_ptr(), xg.data_ptr(), wg.data_ptr(), buf.data_ptr(), n, ci, h, w_, co, 1, 2, 0)
        stream = torch.cuda.current_stream().cuda_stream
        assert lib.adder_b200_backward_input(*args, flags, stream) == 0
        assert torch.isfinite(buf).all()
        mask = torch.zeros(h, w_, dtype=torch.bool, device=DEV)
        mask[::2, ::2] = True
        assert (buf[:, :, ~mask] == 0).all()
        assert torch.equal(buf, gx)
        # accumulate: adds on the sampled grid, leaves the rest alone
        base = torch.randn_like(xg)
        acc = base.clone()
        args = args[:3] + (acc.data_ptr(),) + args[4:]
        assert lib.adder_b200_backward_input(*args, flags | _lib.FLAG_ACCUMULATE, stream) == 0
        _assert(O.compare("accumulated", acc, (base + gx).cpu()))
        assert torch.equal(acc[:, :, ~mask], base[:, :, ~mask])
    with _lib.tuning() as tlib:    # the tiled kernels on the same inputs
        assert tlib.adder_b200_set_micro_tile(0, 8, 4) == 0
        assert tlib.adder_b200_set_micro_tile(1, 4, 4) == 0
        assert "pointwise" not in _lib.describe_plan(0, n, ci, h, w_, co, 1, 2, 0, 0)
        _assert(O.compare("tiled out", ac.forward(xg, wg, 2, 0), out.cpu()))
        _assert(O.compare("tiled grad_x", ac.backward_input(gg, xg, wg, 2, 0, fast_clamp=True), want_gx))
        assert tlib.adder_b200_set_tile_hint(2, 256, 0, 0, 0, 0, 0) == 0
        assert "pointwise=0" in _lib.describe_plan(2, n, ci, h, w_, co, 1, 2, 0, 0)
        _assert(O.compare("tiled grad_w", ac.backward_weight(gg, xg, wg, 2, 0), want_gws))


@pytest.mark.parametrize("geom", [(4, 256, 512, 28, 28), (2, 128, 96, 14, 14), (3, 72, 130, 15, 13), (2, 512, 1024, 8, 6),
                                  (1, 65, 64, 9, 9)],
                         ids=lambda t: "n%d_c%dto%d_%dx%d" % t)
def test_wide_strided_1x1_layers_run_on_the_sampled_grid(geom, ac):
    """1x1 stride-2 layers too wide for the pointwise kernels (the downsample branches of resnet50.py:84-90):
    forward, input gradient and weight gradient run their stride-1 forms on the grid of sampled pixels (gather
    in the fills, scatter with zero fill in the input gradient).  Against the float64 oracle; every input pixel
    written; accumulate flag; odd plane sizes."""
    from addernetcuda_b200 import _lib
    lib = _lib.load()
    n, ci, co, h, w_ = geom
    assert "pointwise" not in _lib.describe_plan(0, n, ci, h, w_, co, 1, 2, 0, 0)
    assert "gemm1x1=1" in _lib.describe_plan(2, n, ci, h, w_, co, 1, 2, 0, 0)
    gen = torch.Generator().manual_seed(177 + n + ci + co + h)
    x = torch.randn(n, ci, h, w_, generator=gen)
    w = torch.randn(co, ci, 1, 1, generator=gen) * 0.7
    ho, wo = (h - 1) // 2 + 1, (w_ - 1) // 2 + 1
    g = torch.randn(n, co, ho, wo, generator=gen)
    want_out = O.adder2d_forward_direct(x, w, 2, 0)
    want_gx, want_gws, want_gw = O.adder2d_backward_direct(g, x, w, 2, 0)
    xg, wg, gg = x.to(DEV), w.to(DEV), g.to(DEV)
    _assert(O.compare("out", ac.forward(xg, wg, 2, 0), want_out))
    out_s, st = ac.forward(xg, wg, 2, 0, stats=True)
    _assert(O.compare("out (statistics epilogue)", out_s, want_out))
    if st.shape[1]:
        tot = st.sum(1).cpu()
        ref = want_out.double()
        assert torch.allclose(tot[:, 0], ref.sum((0, 2, 3)), rtol=1e-5, atol=1e-2)
    _assert(O.compare("grad_w", ac.backward_weight(gg, xg, wg, 2, 0), want_gws))
    gw_raw = ac.backward_weight(gg, xg, wg, 2, 0, eta=0.0)
    scale = max(1.0, float(want_gw.abs().max()))
    _assert(O.compare("grad_w_unscaled/scale", gw_raw.cpu() / scale, want_gw / scale))
    mask = torch.zeros(h, w_, dtype=torch.bool, device=DEV)
    mask[::2, ::2] = True
    stream = torch.cuda.current_stream().cuda_stream
    for fast in (False, True):
        gx = ac.backward_input(gg, xg, wg, 2, 0, fast_clamp=fast)
        _assert(O.compare("grad_x fast=%d" % fast, gx, want_gx))
        buf = torch.full_like(xg, float("nan"))
        flags = _lib.FLAG_FAST_CLAMP if fast else 0
        args = (gg.data_ptr(), xg.data_ptr(), wg.data_ptr(), buf.data_ptr(), n, ci, h, w_, co, 1, 2, 0)
        assert lib.adder_b200_backward_input(*args, flags, stream) == 0
        assert torch.isfinite(buf).all()
        assert (buf[:, :, ~mask] == 0).all()
        assert torch.equal(buf, gx)
        base = torch.randn_like(xg)
        acc = base.clone()
        args = args[:3] + (acc.data_ptr(),) + args[4:]
        assert lib.adder_b200_backward_input(*args, flags | _lib.FLAG_ACCUMULATE, stream) == 0
        _assert(O.compare("accumulated", acc, (base + gx).cpu()))
        assert torch.equal(acc[:, :, ~mask], base[:, :, ~mask])
    # a misaligned gradient buffer takes the element-wise scatter
    pool = torch.full((xg.numel() + 1,), float("nan"), device=DEV)
    odd = pool[1:].view_as(xg)
    args = (gg.data_ptr(), xg.data_ptr(), wg.data_ptr(), odd.data_ptr(), n, ci, h, w_, co, 1, 2, 0)
    assert lib.adder_b200_backward_input(*args, 0, stream) == 0
    _assert(O.compare("grad_x into a 4-byte aligned buffer", odd, want_gx))


@pytest.mark.parametrize("geom", [(3, 16, 32, 32, 32), (5, 32, 64, 16, 16), (2, 6, 5, 12, 24), (2, 6, 5, 12, 20), (2, 9, 3, 10, 7)],
                         ids=lambda t: "n%d_c%dto%d_%dx%d" % t)
def test_stride2_paired_input_gradient(geom, ac):
    """3x3 stride-2 layers: the kernel in which a thread owns two segments of complementary tap classes
    (the default where the tile allows whole row pairs) and the one-class-per-thread kernel that a
    tile hint selects must both match the float64 oracle, exact and saturating-add forms."""
    from addernetcuda_b200 import _lib
    lib = _lib.load()
    n, ci, co, h, w_ = geom
    gen = torch.Generator().manual_seed(91 + n + ci + co + h)
    x = torch.randn(n, ci, h, w_, generator=gen)
    w = torch.randn(co, ci, 3, 3, generator=gen) * 0.5
    ho, wo = (h + 2 - 3) // 2 + 1, (w_ + 2 - 3) // 2 + 1
    g = torch.randn(n, co, ho, wo, generator=gen)
    want_gx, _, _ = O.adder2d_backward_direct(g, x, w, 2, 1)
    xg, wg, gg = x.to(DEV), w.to(DEV), g.to(DEV)
    plan = _lib.describe_plan(1, n, ci, h, w_, co, 3, 2, 1, 1)
    print("   ", plan)
    if h % 2 == 0 and "RW=4" in plan:      # whole row pairs and 4-pixel segments: the paired kernel
        assert "segs/thread=2" in plan
    results = []
    for fast in (False, True):
        got = ac.backward_input(gg, xg, wg, 2, 1, fast_clamp=fast)
        _assert(O.compare("paired grad_x fast=%d" % fast, got, want_gx))
        results.append(got)
    with _lib.tuning() as tlib:
        assert tlib.adder_b200_set_tile_hint(1, 256, 0, 0, 0, 0, 0) == 0
        assert "segs/thread=1" in _lib.describe_plan(1, n, ci, h, w_, co, 3, 2, 1, 1)
        for fast in (False, True):
            _assert(O.compare("one-class grad_x fast=%d" % fast, ac.backward_input(gg, xg, wg, 2, 1, fast_clamp=fast), want_gx))
