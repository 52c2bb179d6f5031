"""Run and time the three adder kernels of one layer (forward, input gradient, weight gradient).

    python -m addernetcuda_b200.layer_bench --ci 16 --co 16 --hw 32 --k 3 --stride 1 --pad 1 --batch 256

Prints the tile plan of each kernel and its device time (CUDA events around a CUDA-graph replay of
several launches, L2 flushed before each replay), Gop/s by the 3-ops-per-triple rule and the share of
the FP32 CUDA-core peak.  With --plain the kernels are launched eagerly `--reps` times and nothing is
timed: that form is the target for `ncu -k regex:adder_` captures.
"""
from __future__ import annotations

import argparse
import math
import statistics

import torch

from . import _lib, adder_cuda as ac


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ci", type=int, required=True)
    ap.add_argument("--co", type=int, required=True)
    ap.add_argument("--hw", type=int, required=True, help="input height = width")
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--pad", type=int, default=1)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--exact-clamp", action="store_true")
    ap.add_argument("--plain", action="store_true", help="launch only (profiling target)")
    ap.add_argument("--reps", type=int, default=1)
    ap.add_argument("--legacy", action="store_true", help="weight gradient by the older pixel-lane tiled kernel (variant 1, through the tuning library)")
    ap.add_argument("--gw-variant", type=int, default=0, help="weight-gradient kernel family (1 pixel-lane, 2 warp-tile with cp.async)")
    ap.add_argument("--hint", action="append", default=[], metavar="OP:THREADS:CG:TH:TI:CK:SMEMKB",
                    help="tile override for one op (0 forward, 1 grad_x, 2 grad_w), through the tuning library")
    ap.add_argument("--tile", action="append", default=[], metavar="OP:PIXELS:CHANNELS", help="register tile override")
    a = ap.parse_args()
    if a.legacy or a.hint or a.tile or a.gw_variant:
        ctx = _lib.tuning()
        tlib = ctx.__enter__()
        if a.legacy:
            tlib.adder_b200_set_variant(2, 1)
        if a.gw_variant:
            tlib.adder_b200_set_variant(2, a.gw_variant)
        for h in a.hint:
            v = [int(t) for t in h.split(":")]
            assert tlib.adder_b200_set_tile_hint(*v) == 0
        for t in a.tile:
            v = [int(q) for q in t.split(":")]
            assert tlib.adder_b200_set_micro_tile(*v) == 0
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    n, ci, co, h, k, s, p = a.batch, a.ci, a.co, a.hw, a.k, a.stride, a.pad
    ho, wo = ac.output_size(h, h, k, s, p)
    x = torch.randn(n, ci, h, h, device=dev)
    w = torch.randn(co, ci, k, k, device=dev) * math.sqrt(2.0 / (ci * k * k))
    g = torch.randn(n, co, ho, wo, device=dev)
    fast = not a.exact_clamp
    ops = {"forward": lambda: ac.forward(x, w, s, p),
           "grad_x": lambda: ac.backward_input(g, x, w, s, p, fast_clamp=fast),
           "grad_w": lambda: ac.backward_weight(g, x, w, s, p)}
    if a.plain:
        for _ in range(a.reps):
            for f in ops.values():
                f()
        torch.cuda.synchronize()
        print("ok")
        return
    T = n * ho * wo * co * ci * k * k
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    peak = 2 * 128 * sms * 1.965e9
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    total = 0.0
    times = {}
    ops["bwd"] = lambda: ac.backward(g, x, w, s, p, fast_clamp=fast)   # both gradients, weight gradient on a side stream
    for i, (name, f) in enumerate(ops.items()):
        if i < 3:
            print(_lib.describe_plan(i, n, ci, h, h, co, k, s, p, 1 if fast else 0))
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            f(); f()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(4):
                f()
        ts = []
        for _ in range(7):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); graph.replay(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / 4)
        ms = statistics.median(ts)
        times[name] = ms
        if name == "bwd":
            break
        total += ms
        print(f"  {name:8s} {ms * 1e3:9.1f} us   {3 * T / ms / 1e6:9.0f} Gop/s   {100 * 3 * T / (ms * 1e-3) / peak:5.1f} % of FP32 peak")
    both = times["forward"] + times["bwd"]
    print(f"  bwd (grad_w beside grad_x) {times['bwd'] * 1e3:9.1f} us;  forward + that: {both * 1e3:9.1f} us   "
          f"{9 * T / both / 1e6:9.0f} Gop/s   {100 * 9 * T / (both * 1e-3) / peak:5.1f} % of FP32 peak")
    print(f"  fwd+bwd  {total * 1e3:9.1f} us   {9 * T / total / 1e6:9.0f} Gop/s   {100 * 9 * T / (total * 1e-3) / peak:5.1f} % of FP32 peak")


if __name__ == "__main__":
    main()
