"""Tile planners of the three kernel families, exercised without a GPU.

`adder_b200_describe_plan` runs the same host code that precedes a launch and returns the plan as text.
For a seeded sample of layer geometries (the benchmark shapes plus random ones) every plan must be
launchable: status 0, at most 256 threads in whole warps, shared memory within the 227 KB a CTA can
have, a non-empty grid, and the special-case kernels chosen exactly where they apply.
"""
import random
import re

import pytest

from addernetcuda_b200 import _lib

SMEM_LIMIT = 227 * 1024

BENCH_SHAPES = [  # (n, ci, h, w, co, k, stride, pad)
    (256, 16, 32, 32, 16, 3, 1, 1), (256, 16, 32, 32, 32, 3, 2, 1), (256, 32, 16, 16, 32, 3, 1, 1),
    (256, 64, 8, 8, 64, 3, 1, 1), (256, 256, 14, 14, 256, 3, 1, 1), (256, 512, 7, 7, 512, 3, 1, 1),
    (256, 1024, 14, 14, 256, 1, 1, 0), (256, 16, 32, 32, 32, 1, 2, 0), (256, 32, 16, 16, 64, 1, 2, 0),
    (64, 64, 56, 56, 64, 3, 1, 1), (64, 128, 56, 56, 128, 3, 2, 1), (64, 256, 56, 56, 512, 1, 2, 0),
    (64, 2048, 7, 7, 512, 1, 1, 0), (32, 16, 32, 32, 16, 3, 1, 1), (1, 3, 224, 224, 64, 3, 1, 1),
]


def _random_shapes(count, seed):
    rng = random.Random(seed)
    out = []
    while len(out) < count:
        k = rng.choice((1, 3))
        s = rng.choice((1, 2))
        p = rng.randrange(0, k)
        h, w = rng.randrange(1, 70), rng.randrange(1, 70)
        if h + 2 * p < k or w + 2 * p < k:
            continue
        out.append((rng.randrange(1, 40), rng.randrange(1, 200), h, w, rng.randrange(1, 200), k, s, p))
    return out


def _field(plan, name):
    m = re.search(r"\b%s=(\d+)" % re.escape(name), plan)
    return int(m.group(1)) if m else None


@pytest.mark.parametrize("op", [0, 1, 2], ids=["forward", "grad_x", "grad_w"])
def test_plans_are_launchable(op):
    for shape in BENCH_SHAPES + _random_shapes(150, 20 + op):
        for flags in ((0, 1) if op == 1 else (0,)):
            plan = _lib.describe_plan(op, *shape, flags)
            assert "status=0" in plan, (shape, plan)
            threads = _field(plan, "threads")
            assert threads is not None and 32 <= threads <= 256 and threads % 32 == 0, (shape, plan)
            smem = _field(plan, "smem")
            if smem is not None:          # the one-thread-per-position kernels use static shared memory
                assert smem <= SMEM_LIMIT, (shape, plan)
            grid = re.search(r"grid=\((\d+),(\d+)\)", plan)
            if grid:
                assert int(grid.group(1)) >= 1 and 1 <= int(grid.group(2)) <= 65535, (shape, plan)
            splits = _field(plan, "splits")
            if splits is not None:
                assert splits >= 1, (shape, plan)


def test_special_case_kernels_are_chosen_where_they_apply():
    # 1x1 stride-2, few channels: one thread per output position, all three passes
    for op in (0, 1):
        assert "pointwise" in _lib.describe_plan(op, 256, 16, 32, 32, 32, 1, 2, 0, 1)
        assert "pointwise" not in _lib.describe_plan(op, 64, 256, 56, 56, 512, 1, 2, 0, 1)     # too many channels
        assert "pointwise" not in _lib.describe_plan(op, 256, 16, 32, 32, 32, 1, 1, 0, 1)      # stride 1
    assert "pointwise=1" in _lib.describe_plan(2, 256, 16, 32, 32, 32, 1, 2, 0, 0)
    assert "pointwise=0" in _lib.describe_plan(2, 64, 256, 56, 56, 512, 1, 2, 0, 0)
    # 1x1 stride-1 with many channels: the GEMM-style weight gradient
    assert "gemm1x1=1" in _lib.describe_plan(2, 256, 1024, 14, 14, 256, 1, 1, 0, 0)
    assert "gemm1x1=0" in _lib.describe_plan(2, 256, 16, 32, 32, 16, 3, 1, 1, 0)
    # 3x3 stride-2 input gradient: two segments per thread with 4-pixel segments and whole row pairs
    assert "segs/thread=2" in _lib.describe_plan(1, 256, 16, 32, 32, 32, 3, 2, 1, 1)
    assert "segs/thread=1" in _lib.describe_plan(1, 256, 16, 32, 32, 16, 3, 1, 1, 1)
    assert "segs/thread=2" in _lib.describe_plan(1, 64, 256, 28, 28, 256, 3, 2, 1, 1)          # ragged last segment


def test_chunking_does_not_depend_on_the_batch():
    """Sub-batches must be computed with the same chunk boundaries in the input gradient, whose two-level
    summation folds one partial sum per chunk (bitwise-equal results per image).  The forward keeps one running
    sum per output over all input channels, so its bits do not depend on where the chunks are cut; its chunk
    size may follow the CTA shape, which follows the size of the launch."""
    for shape in ((64, 8, 8, 64), (32, 16, 16, 32), (256, 14, 14, 256)):
        ci, h, w, co = shape
        values = {_field(_lib.describe_plan(1, n, ci, h, w, co, 3, 1, 1, 1), "CKO") for n in (1, 2, 3, 8, 64, 256)}
        assert len(values) == 1, (shape, values)


def test_unsupported_geometry_is_reported_not_planned():
    lib = _lib.load()
    import ctypes
    buf = ctypes.create_string_buffer(256)
    assert lib.adder_b200_describe_plan(0, 4, 8, 16, 16, 8, 5, 1, 2, 0, buf, 256) != 0       # 5x5 kernel
    assert lib.adder_b200_describe_plan(0, 4, 8, 16, 16, 8, 3, 3, 1, 0, buf, 256) != 0       # stride 3
    assert lib.adder_b200_describe_plan(0, 4, 0, 16, 16, 8, 3, 1, 1, 0, buf, 256) != 0       # no channels


def test_empty_batch_plans_have_at_least_one_split():
    """An empty batch still defines the weight gradient (all zeros): the plan must keep one CTA per output
    tile to write the zero slices, also on the geometry that otherwise takes the pointwise kernels."""
    for shape in ((0, 16, 32, 32, 32, 1, 2, 0), (0, 16, 32, 32, 16, 3, 1, 1), (0, 1024, 14, 14, 256, 1, 1, 0)):
        plan = _lib.describe_plan(2, *shape, 0)
        assert "status=0" in plan and "pointwise=0" in plan, plan
        assert _field(plan, "splits") >= 1, plan


def test_imagenet_plane_rules():
    """Planner rules for the ResNet-50 shapes (resnet50.py:84-90 and the 7/14/28-wide stages): which kernel
    family and which segment width a geometry gets.  Host-side only: the plans are computed without a GPU."""
    # 3x3 weight gradient on 28-, 14- and 7-wide planes: warp-tile kernel with 4- or 7-pixel segments
    for hw, rw in ((28, 4), (14, 7), (7, 7)):
        plan = _lib.describe_plan(2, 64, 128, hw, hw, 128, 3, 1, 1, 0)
        assert "warp-tile" in plan and f"RW={rw} " in plan, plan
    # 56-wide planes take the bulk-copy form
    assert "tma" in _lib.describe_plan(2, 64, 64, 56, 56, 64, 3, 1, 1, 0)
    # strided 1x1 layers too wide for the pointwise kernels: stride-1 forms on the sampled grid
    fwd = _lib.describe_plan(0, 64, 256, 56, 56, 512, 1, 2, 0, 0)
    assert "pointwise" not in fwd and "s=1" in fwd, fwd
    assert "gemm1x1=1" in _lib.describe_plan(2, 64, 256, 56, 56, 512, 1, 2, 0, 0)
    gx = _lib.describe_plan(1, 64, 256, 56, 56, 512, 1, 2, 0, 1)
    assert "k=1 s=1" in gx and "cols=28" in gx, gx                # tiled over the 28x28 sampled grid
    # 1x1 stride-1 layers: one row of H*W pixels per image unless the plane is 7n wide
    assert "cols=3136" in _lib.describe_plan(1, 64, 256, 56, 56, 64, 1, 1, 0, 1) or \
        "rows=1 " in _lib.describe_plan(1, 64, 256, 56, 56, 64, 1, 1, 0, 1)
    assert "RW=7" in _lib.describe_plan(1, 64, 1024, 14, 14, 256, 1, 1, 0, 1)
    # every 3x3 stride-2 input gradient: two complementary segments per thread
    for hw in (32, 56, 28, 14):
        assert "segs/thread=2" in _lib.describe_plan(1, 64, 128, hw, hw, 128, 3, 2, 1, 1)
