"""Seeded random small geometries (every kernel size, stride, padding; odd channel counts, ragged
widths and heights, tiny batches) against the float64 direct oracle."""
import math
import random

import numpy as np
import pytest
import torch

from oracle import adder_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cases():
    rnd = random.Random(20240607)
    out = []
    while len(out) < 36:
        k = rnd.choice([1, 3])
        s = rnd.choice([1, 2])
        p = rnd.choice([0, 1]) if k == 3 else 0
        n = rnd.choice([1, 2, 3, 5])
        ci = rnd.choice([1, 2, 3, 5, 7, 8, 12, 17, 24, 33])
        co = rnd.choice([1, 2, 3, 5, 8, 9, 16, 19, 32, 40, 65])
        h = rnd.choice([1, 2, 3, 4, 5, 7, 8, 9, 13, 16, 21])
        w = rnd.choice([1, 2, 3, 4, 5, 7, 8, 9, 13, 16, 28, 37, 70])
        if h + 2 * p < k or w + 2 * p < k:
            continue
        out.append((n, ci, co, h, w, k, s, p, 1000 + len(out)))
    return out


@pytest.mark.parametrize("case", _cases(), ids=lambda c: "n%d_c%dto%d_%dx%d_k%ds%dp%d" % c[:8])
def test_random_geometry_matches_float64_oracle(case):
    from addernetcuda_b200 import adder_cuda as ac
    n, ci, co, h, w, k, s, p, seed = case
    rng = np.random.default_rng(seed)
    ho, wo = O.out_hw(h, w, k, s, p)
    x = torch.from_numpy(rng.standard_normal((n, ci, h, w)).astype(np.float32))
    wt = torch.from_numpy((rng.standard_normal((co, ci, k, k)) * math.sqrt(2.0 / (ci * k * k))).astype(np.float32))
    g = torch.from_numpy(rng.standard_normal((n, co, ho, wo)).astype(np.float32))
    want_out = O.adder2d_forward_direct(x, wt, s, p)
    want_gx, want_gws, want_gw = O.adder2d_backward_direct(g, x, wt, s, p)
    xg, wg, gg = x.to(DEV), wt.to(DEV), g.to(DEV)
    scale = max(1.0, float(want_gw.abs().max()))
    for name, got, want in (("out", ac.forward(xg, wg, s, p), want_out),
                            ("grad_x", ac.backward_input(gg, xg, wg, s, p), want_gx),
                            ("grad_x(fast)", ac.backward_input(gg, xg, wg, s, p, fast_clamp=True), want_gx),
                            ("grad_w", ac.backward_weight(gg, xg, wg, s, p), want_gws),
                            ("grad_w_unscaled/scale", ac.backward_weight(gg, xg, wg, s, p, eta=0.0) / scale, want_gw / scale)):
        ok, err, msg = O.compare(name, got, want)
        assert ok, f"{case}: {msg}"
