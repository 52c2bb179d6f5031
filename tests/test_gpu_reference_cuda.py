"""The reference's own CUDA kernels as a third oracle, on the GPU itself.

baseline/_ref/ holds the reference's adder.py and its `adder_cuda` extension built for sm_100 from the
unmodified sources (four `x.type()` -> `x.scalar_type()` tokens aside, which PyTorch >= 2 needs to compile
it; baseline/install_ref.py).  Its forward + autograd backward (unfold, CONV, CONV_BACKWARD, col2im, rescale)
must agree with this library on the same tensors at the usual tolerance.  Agreement is not bitwise: the
reference accumulates with atomics in arbitrary order and Kahan-sums its forward.

Only shapes with K, Co and P in multiples of 16 are used.  The reference kernels guard nothing beyond that
divisibility (adder_cuda/adder.cu:19-70, :194-272 index X, W and both gradients with unguarded
k0 + threadIdx terms), so other shapes would read and write outside their buffers; its standalone
CONV_WEIGHT / CONV_INPUT exports (adder.cu:72-192) have no bounds guard at all and are never called.
"""
import math
import sys
from pathlib import Path

import pytest
import torch

from oracle import adder_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent

# (n, ci, co, h, w, k, stride, pad): K = ci*k*k, Co and P = n*ho*wo all multiples of 16
SHAPES = [(8, 16, 16, 32, 32, 3, 1, 1), (4, 32, 32, 16, 16, 3, 1, 1), (4, 64, 64, 8, 8, 3, 1, 1),
          (4, 16, 32, 32, 32, 3, 2, 1), (4, 16, 32, 32, 32, 1, 2, 0), (4, 64, 128, 14, 14, 1, 1, 0)]


@pytest.fixture(scope="module")
def reference_adder():
    sys.path.insert(0, str(ROOT))
    import bench
    mod, why = bench.load_reference_cuda()
    if mod is None:
        pytest.skip(why)
    return mod


@pytest.mark.parametrize("shape", SHAPES, ids=lambda t: "n%d_c%dto%d_%dx%d_k%ds%dp%d" % t)
def test_reference_cuda_kernels_agree(shape, reference_adder):
    from addernetcuda_b200 import adder_cuda as ac
    n, ci, co, h, w, k, s, p = shape
    ho, wo = (h - k + 2 * p) // s + 1, (w - k + 2 * p) // s + 1
    assert (ci * k * k) % 16 == 0 and co % 16 == 0 and (n * ho * wo) % 16 == 0
    gen = torch.Generator().manual_seed(600 + n + ci + co + h)
    x = torch.randn((n, ci, h, w), generator=gen).to(DEV)
    wt = (torch.randn((co, ci, k, k), generator=gen) * math.sqrt(2.0 / (ci * k * k))).to(DEV)
    g = torch.randn((n, co, ho, wo), generator=gen).to(DEV)
    xr, wr = x.clone().requires_grad_(), wt.clone().requires_grad_()
    y = reference_adder.adder2d_function(xr, wr, s, p)
    y.backward(g)
    torch.cuda.synchronize()
    for what, got, want in (("out", ac.forward(x, wt, s, p), y.detach()),
                            ("grad_x", ac.backward_input(g, x, wt, s, p), xr.grad),
                            ("grad_x (saturating-add form)", ac.backward_input(g, x, wt, s, p, fast_clamp=True), xr.grad),
                            ("grad_w", ac.backward_weight(g, x, wt, s, p), wr.grad)):
        ok, err, msg = O.compare(f"{what} vs reference CUDA", got, want)
        print("   ", msg)
        assert ok, msg
