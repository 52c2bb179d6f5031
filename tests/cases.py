"""Shared parity cases and seeded input generators (NumPy PCG64: identical on every platform)."""
from __future__ import annotations

import math

import numpy as np


def _case(name, n, ci, co, h, w, k, stride, pad, seed):
    return dict(name=name, n=n, ci=ci, co=co, h=h, w=w, k=k, stride=stride, pad=pad, seed=seed)


# name, N, Ci, Co, H, W, k, stride, pad, seed
LAYER_CASES = [
    # configuration 1 of the benchmark definition: one adder2d layer, N=32, 16->16, 32x32, k3 s1 p1
    _case("cfg1_n32_c16_32x32_k3s1p1", 32, 16, 16, 32, 32, 3, 1, 1, 1334),
    # small odd shapes: every tail (channels, rows, columns, batch) and both paddings
    _case("odd_n2_c3to5_7x6_k3s1p1", 2, 3, 5, 7, 6, 3, 1, 1, 11),
    _case("odd_n3_c4to6_9x8_k3s2p1", 3, 4, 6, 9, 8, 3, 2, 1, 12),
    _case("odd_n2_c8to4_5x5_k1s2p0", 2, 8, 4, 5, 5, 1, 2, 0, 13),
    _case("odd_n1_c2to3_6x6_k3s1p0", 1, 2, 3, 6, 6, 3, 1, 0, 14),
    _case("odd_n2_c3to4_8x8_k3s2p0", 2, 3, 4, 8, 8, 3, 2, 0, 15),
    _case("odd_n1_c1to17_11x13_k3s1p1", 1, 1, 17, 11, 13, 3, 1, 1, 16),      # K = 9
    _case("odd_n2_c3to12_10x10_k3s1p1", 2, 3, 12, 10, 10, 3, 1, 1, 17),      # K = 27 (VGG first layer)
    _case("odd_n3_c84to3_4x9_k1s1p0", 3, 84, 3, 4, 9, 1, 1, 0, 18),          # K = 84
    _case("odd_n2_c5to9_40x3_k3s1p1", 2, 5, 9, 40, 3, 3, 1, 1, 19),          # tall and narrow
    _case("odd_n1_c6to10_3x70_k3s1p1", 1, 6, 10, 3, 70, 3, 1, 1, 20),        # wide rows (column tiling)
    _case("odd_n2_c7to5_9x9_k1s1p0", 2, 7, 5, 9, 9, 1, 1, 0, 21),
    _case("odd_n2_c4to4_7x7_k3s2p1", 2, 4, 4, 7, 7, 3, 2, 1, 22),
    # the layer shapes of ResNet-20 (CIFAR) at a small batch
    _case("r20_n4_c16to16_32x32_k3s1p1", 4, 16, 16, 32, 32, 3, 1, 1, 31),
    _case("r20_n4_c16to32_32x32_k3s2p1", 4, 16, 32, 32, 32, 3, 2, 1, 32),
    _case("r20_n4_c32to32_16x16_k3s1p1", 4, 32, 32, 16, 16, 3, 1, 1, 33),
    _case("r20_n4_c32to64_16x16_k3s2p1", 4, 32, 64, 16, 16, 3, 2, 1, 34),
    _case("r20_n4_c64to64_8x8_k3s1p1", 4, 64, 64, 8, 8, 3, 1, 1, 35),
    _case("r20_n4_c16to32_32x32_k1s2p0", 4, 16, 32, 32, 32, 1, 2, 0, 36),
    _case("r20_n4_c32to64_16x16_k1s2p0", 4, 32, 64, 16, 16, 1, 2, 0, 37),
    # the distinct layer classes of ResNet-50 (ImageNet) at batch 1-2; outputs stored as samples
    _case("r50_n1_c64to64_56x56_k3s1p1", 1, 64, 64, 56, 56, 3, 1, 1, 41),
    _case("r50_n1_c128to128_56x56_k3s2p1", 1, 128, 128, 56, 56, 3, 2, 1, 42),
    _case("r50_n2_c256to256_14x14_k3s1p1", 2, 256, 256, 14, 14, 3, 1, 1, 43),
    _case("r50_n2_c512to512_7x7_k3s1p1", 2, 512, 512, 7, 7, 3, 1, 1, 44),
    _case("r50_n2_c1024to256_14x14_k1s1p0", 2, 1024, 256, 14, 14, 1, 1, 0, 45),
    _case("r50_n1_c256to512_56x56_k1s2p0", 1, 256, 512, 56, 56, 1, 2, 0, 46),
    _case("r50_n2_c64to256_28x28_k1s1p0", 2, 64, 256, 28, 28, 1, 1, 0, 47),
]

# column-matrix cases for the reference extension's own entry points: W[Co,K], X[K,P], g[Co,P]
COL_CASES = [
    # the shape of the reference's test script (adder_cuda/test_cuda.py:165-172): N=16, Co=Ci=32, k=3, 8x8
    dict(name="col_testcuda_k288_p1024_co32", K=288, P=1024, Co=32, seed=51, scale=1.0),
    dict(name="col_testcuda_x5_k288_p1024_co32", K=288, P=1024, Co=32, seed=52, scale=5.0),  # test_cuda.py:64-66
    dict(name="col_ragged_k27_p50_co5", K=27, P=50, Co=5, seed=53, scale=1.0),
    dict(name="col_tiny_k7_p1_co1", K=7, P=1, Co=1, seed=54, scale=1.0),
    dict(name="col_k84_p36_co12", K=84, P=36, Co=12, seed=55, scale=1.0),
]

LAYER_BY_NAME = {c["name"]: c for c in LAYER_CASES}
COL_BY_NAME = {c["name"]: c for c in COL_CASES}


def draw_layer(case):
    """x ~ N(0,1), w Kaiming-normal (std sqrt(2/fan_in)), grad_out ~ N(0,1), drawn in that order."""
    rng = np.random.default_rng(case["seed"])
    n, ci, co, h, w, k, s, p = (case[q] for q in ("n", "ci", "co", "h", "w", "k", "stride", "pad"))
    ho = (h - k + 2 * p) // s + 1
    wo = (w - k + 2 * p) // s + 1
    x = rng.standard_normal((n, ci, h, w)).astype(np.float32)
    wt = (rng.standard_normal((co, ci, k, k)) * math.sqrt(2.0 / (ci * k * k))).astype(np.float32)
    g = rng.standard_normal((n, co, ho, wo)).astype(np.float32)
    return x, wt, g


def draw_cols(case):
    rng = np.random.default_rng(case["seed"])
    K, P, Co, sc = case["K"], case["P"], case["Co"], case["scale"]
    W = (rng.standard_normal((Co, K)) * sc).astype(np.float32)
    X = (rng.standard_normal((K, P)) * sc).astype(np.float32)
    g = rng.standard_normal((Co, P)).astype(np.float32)
    return W, X, g


from addernetcuda_b200.synthetic import resnet20_batch  # noqa: E402,F401  (re-exported for the tests)
