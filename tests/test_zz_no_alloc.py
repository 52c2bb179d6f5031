"""The weight-gradient entry point that allocates nothing (scratch inside the library).

Some callers cannot give the library a workspace: hosts whose memory manager owns the whole GPU and
forbids cudaMalloc inside plugins, and bindings that only ever receive input and output pointers.
For them `adder_b200_backward_weight_static` keeps its scratch in a fixed 8 MiB device array.  This
test calls it through the C ABI and requires bit-identical gradients to the workspace-taking entry
point (and agreement with the float64 oracle at the tolerance of the other parity tests), on two calls
in a row with different inputs (the shared array still holds the first call's partial sums when the
second call starts), and checks that an oversized layer is refused, not overrun.

The file sorts last on purpose: a run that stops at the first failure has then already executed
every other test.  It also passes when run alone in a fresh process, where its first call is the
one that resolves the array's device address.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(seed, n, ci, co, h, w, k, s, p):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    ho, wo = (h - k + 2 * p) // s + 1, (w - k + 2 * p) // s + 1
    x = torch.randn((n, ci, h, w), generator=gen).to(DEV)
    wt = (torch.randn((co, ci, k, k), generator=gen) * math.sqrt(2.0 / (ci * k * k))).to(DEV)
    g = torch.randn((n, co, ho, wo), generator=gen).to(DEV)
    return x, wt, g


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from addernetcuda_b200 import _lib
    lib = _lib.load()
    assert torch.cuda.is_available()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.adder_b200_static_scratch_bytes() == 8 << 20
    # two different layers back to back: the second finds the first one's partial sums in the array
    for seed, geom in ((5, (32, 16, 32, 32, 16, 3, 1, 1)), (6, (24, 32, 16, 16, 64, 3, 2, 1)), (7, (8, 16, 32, 32, 32, 1, 2, 0))):
        n, ci, h, w, co, k, s, p = geom
        x, wt, g = _inputs(seed, n, ci, co, h, w, k, s, p)
        need = lib.adder_b200_backward_weight_workspace_bytes(*geom)
        assert 0 < need <= 8 << 20
        ws = torch.empty(need, dtype=torch.uint8, device=DEV)
        want = torch.empty_like(wt)
        want_norm = torch.zeros(1, device=DEV)
        st = lib.adder_b200_backward_weight(g.data_ptr(), x.data_ptr(), wt.data_ptr(), want.data_ptr(), ctypes.c_float(0.2),
                                            want_norm.data_ptr(), ws.data_ptr(), need, *geom, 0, stream)
        assert st == 0
        got = torch.full_like(wt, float("nan"))
        got_norm = torch.zeros(1, device=DEV)
        for _ in range(2):   # and the same layer twice in a row
            st = lib.adder_b200_backward_weight_static(g.data_ptr(), x.data_ptr(), wt.data_ptr(), got.data_ptr(),
                                                       ctypes.c_float(0.2), got_norm.data_ptr(), *geom, stream)
            assert st == 0, lib.adder_b200_status_string(st)
            torch.cuda.synchronize()
            # same kernels, same plan, same summation order: the two entry points agree bit for bit
            assert torch.equal(got, want), f"geom {geom}: max_abs_err {(got - want).abs().max().item():.3e}"
            assert float(got_norm) == float(want_norm)
        # and the result is the reference's: rescaled weight gradient from the float64 oracle
        from oracle import adder_oracle as O
        _, want_oracle, _ = O.adder2d_backward_direct(g.cpu(), x.cpu(), wt.cpu(), s, p)
        ok, err, msg = O.compare(f"static-scratch grad_w {geom}", got, want_oracle)
        assert ok, msg


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from addernetcuda_b200 import _lib
    lib = _lib.load()
    geom = (64, 512, 7, 7, 512, 3, 1, 1)               # partial sums of a 512x512x3x3 gradient: > 8 MiB
    assert lib.adder_b200_backward_weight_workspace_bytes(*geom) > 8 << 20
    dummy = torch.zeros(16, device=DEV)
    st = lib.adder_b200_backward_weight_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                               ctypes.c_float(0.2), None, *geom, None)
    assert st == 8 and b"scratch" in lib.adder_b200_status_string(st)
    # argument errors are reported like everywhere else
    assert lib.adder_b200_backward_weight_static(None, None, None, None, ctypes.c_float(0.2), None,
                                                 4, 16, 8, 8, 16, 3, 1, 1, None) == 1
    assert lib.adder_b200_backward_weight_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                                 ctypes.c_float(0.2), None, 4, 16, 8, 8, 16, 5, 1, 2, None) == 3
