#!/usr/bin/env python
"""Benchmark of the adder-convolution hot path: ResNet-20 adder training throughput (fp32).

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this library, CUDA kernels
    python bench.py --impl reference [--steps K] [--warmup W]      # the CPU path (oracle port)

Workload (N = 1): one SGD training step of ResNet-20 (18 adder 3x3 + 2 adder 1x1 layers, BatchNorm,
cross-entropy, momentum 0.9, lr 0.1) on a synthetic CIFAR-shaped batch of 256 images ~ N(0,1) with
uniform random labels.  N > 1: the same per-GPU batch on every rank (weak scaling), gradients
averaged by a bucketed all-reduce overlapped with backward.  One JSON line is printed by rank 0.

Timing: W warm-up steps, then exactly K steps between a barrier + device synchronisation on both
sides, CUDA events on the launching stream, maximum over ranks.  `value` has the batch resident in
device memory; `e2e` copies every batch from pinned host memory and reads the loss back each step.
The working set of one step (hundreds of MB of activations) is larger than L2, so no explicit L2
flush is needed between steps; the per-layer kernel timings flush L2 explicitly.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# reference: 0.3158 s per batch, ResNet-20 / CIFAR-10 on an RTX 2080Ti (its README.md:22); the batch
# size is not stated there; 3920 backward calls / 20 layers = 196 batches per epoch implies 256.
PUBLISHED_STEPS_PER_S = 1.0 / 0.3158

# (Ci, Co, H, W, stride, k, pad): the per-layer sweep of the benchmark definition (batch 256)
SWEEP_SHAPES = [
    (16, 16, 32, 32, 1, 3, 1), (16, 32, 32, 32, 2, 3, 1), (32, 32, 16, 16, 1, 3, 1), (64, 64, 8, 8, 1, 3, 1),
    (256, 256, 14, 14, 1, 3, 1), (512, 512, 7, 7, 1, 3, 1), (1024, 256, 14, 14, 1, 1, 0),
]
# the 20 adder layers of ResNet-20 as (shape, multiplicity)
RESNET20_LAYERS = [
    ((16, 16, 32, 32, 1, 3, 1), 6), ((16, 32, 32, 32, 2, 3, 1), 1), ((32, 32, 16, 16, 1, 3, 1), 5),
    ((32, 64, 16, 16, 2, 3, 1), 1), ((64, 64, 8, 8, 1, 3, 1), 5), ((16, 32, 32, 32, 2, 1, 0), 1),
    ((32, 64, 16, 16, 2, 1, 0), 1),
]


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of each adder kernel on the 16->16 32x32 k3
# layer at batch 256 (ncu capture summarised in profiles/adder_kernels_c16to16_32x32_b256.txt), and the
# algorithmic bytes of that launch: 4(|x|+|w|+|out|), 4(|g|+|x|+|w|+|gx|), 4(|g|+|x|+|w|+|gw|).
NCU_CAPTURE = "profiles/adder_kernels_c16to16_32x32_b256.txt"
NCU_DRAM_BYTES = {"fwd": 16824832, "grad_x": 33615616, "grad_w": 33592064}
ALGO_BYTES_16x16 = {"fwd": 33563648, "grad_x": 50340864, "grad_w": 33572864}
KERNEL_NAMES = {"fwd": "adder_fwd_kernel", "grad_x": "adder_gx_kernel", "grad_w": "adder_gw_tma_kernel"}


def triples(n, shape):
    ci, co, h, w, s, k, p = shape
    ho, wo = (h - k + 2 * p) // s + 1, (w - k + 2 * p) // s + 1
    return n * ho * wo * co * ci * k * k


# ------------------------------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [v.strip() for v in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------ CPU arm

def cpu_step_factory(batch: int, seed: int = 1434):
    """ResNet-20 training step on the host through the oracle port of the reference's adder.py
    (unfold + column matrices), all host threads."""
    import torch
    from addernetcuda_b200 import resnet as R
    from oracle import adder_unfold as U
    from addernetcuda_b200.synthetic import resnet20_batch
    torch.set_num_threads(os.cpu_count() or 1)
    net = R.resnet20(conv=U.adder2d)
    R.init_seeded(net, seed)
    net.train()
    opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
    images, labels = resnet20_batch(batch, seed)
    images, labels = torch.from_numpy(images), torch.from_numpy(labels)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.cross_entropy(net(images), labels)
        loss.backward()
        opt.step()
        return float(loss.detach())
    return step


def cpu_images_per_s(budget_s: float, steps: int, warmup: int):
    """Times `steps` CPU training steps on a batch chosen so that warmup+steps fits the budget."""
    probe = cpu_step_factory(4)
    probe()
    t0 = time.perf_counter(); probe(); t_img = (time.perf_counter() - t0) / 4
    batch = int(budget_s / max(1e-9, (steps + warmup) * t_img))
    batch = max(4, min(256, batch // 4 * 4))
    step = cpu_step_factory(batch)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return batch * steps / dt, batch, dt / steps


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # the CPU path is ~4000x slower: cap the number of timed steps so the run ends within a few minutes
    steps, warmup = max(1, min(args.steps, 5)), max(0, min(args.warmup, 1))
    ips, batch, s_per_step = cpu_images_per_s(args.cpu_budget_s, steps, warmup)
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": "resnet20_adder_train_throughput", "value": ips, "unit": "images/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": s_per_step * 1e3,
        "steps_per_s_at_batch_256": ips / 256.0, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "resnet20_adder_train_step_fp32", "per_gpu_batch": 256, "sample_batch": batch},
        "cpu_baseline": {"value": ips, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": f"{steps} training steps of ResNet-20 at batch {batch} (of 256) through the CPU port "
                                   f"of the reference's adder.py unfold path, {cores} host threads"},
        "e2e": {"value": ips, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ GPU arm

def time_layer_ops(n, shape, iters=9):
    """Device time (ms) of the three adder kernels of one layer, and of the two gradient kernels issued
    together as the layer's backward does.  Every sample is ONE launch (a CUDA-graph replay, so that the
    host is out of the picture) between CUDA events on the current stream, with L2 flushed (a 256 MB
    write) before it: cold-cache numbers.  Median of `iters` samples."""
    import torch
    from addernetcuda_b200 import adder_cuda as ac
    dev = torch.device("cuda", torch.cuda.current_device())
    ci, co, h, w, s, k, p = shape
    ho, wo = (h - k + 2 * p) // s + 1, (w - k + 2 * p) // s + 1
    x = torch.randn(n, ci, h, w, device=dev)
    wt = torch.randn(co, ci, k, k, device=dev) * math.sqrt(2.0 / (ci * k * k))
    g = torch.randn(n, co, ho, wo, device=dev)
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    out = {}
    ops = {"fwd": lambda: ac.forward(x, wt, s, p),
           "grad_x": lambda: ac.backward_input(g, x, wt, s, p, fast_clamp=True),
           "grad_w": lambda: ac.backward_weight(g, x, wt, s, p),
           # both gradients the way the layer's backward issues them: weight gradient on a side stream
           "bwd": lambda: ac.backward(g, x, wt, s, p, fast_clamp=True)}
    for name, f in ops.items():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                f()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            f()
        ts = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); graph.replay(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        out[name] = statistics.median(ts)
    return out


# ------------------------------------------------------------------------------------------ the reference's kernels

def load_reference_cuda():
    """The reference's own adder.py on top of its own CUDA extension, both as installed (unmodified apart
    from four `x.type()` -> `x.scalar_type()` tokens the current PyTorch needs to compile it) in
    baseline/_ref/ by baseline/install_ref.py.  Returns the module, or None with the reason."""
    import importlib.util
    ref = ROOT / "baseline" / "_ref"
    so = sorted(ref.glob("adder_cuda*.so"))
    if not so or not (ref / "adder.py").exists():
        return None, "baseline/_ref holds no reference build (run baseline/install_ref.py where the reference checkout is)"
    saved = sys.modules.get("adder_cuda")
    try:
        spec = importlib.util.spec_from_file_location("adder_cuda", so[0])
        ext = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ext)
        sys.modules["adder_cuda"] = ext               # adder.py does `import adder_cuda`
        spec = importlib.util.spec_from_file_location("reference_adder", ref / "adder.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod, None
    except Exception as e:  # noqa: BLE001  (an extension that does not load is reported, not fatal)
        return None, f"reference extension did not load: {e!r}"[:200]
    finally:
        if saved is not None:
            sys.modules["adder_cuda"] = saved
        else:
            sys.modules.pop("adder_cuda", None)


def reference_cuda_in_bounds(n, shape):
    """The reference kernels guard nothing beyond their launch-time divisibility test: CONV needs K, Co and
    P in multiples of 16 to stay inside its buffers, CONV_BACKWARD in multiples of 8 (adder.cu:19-70,
    :194-272).  Only such shapes are ever handed to it."""
    ci, co, h, w, s, k, p = shape
    ho, wo = (h - k + 2 * p) // s + 1, (w - k + 2 * p) // s + 1
    K, P = ci * k * k, n * ho * wo
    return K % 16 == 0 and co % 16 == 0 and P % 16 == 0


def time_reference_cuda(ref_adder, n, shape, iters=3):
    """fwd and bwd device time (ms) of one layer through the reference's adder2d_function (F.unfold, permute
    copies, its CONV / CONV_BACKWARD kernels, col2im, the rescale): the path its README profiles."""
    import torch
    dev = torch.device("cuda", torch.cuda.current_device())
    ci, co, h, w, s, k, p = shape
    ho, wo = (h - k + 2 * p) // s + 1, (w - k + 2 * p) // s + 1
    x = torch.randn(n, ci, h, w, device=dev, requires_grad=True)
    wt = (torch.randn(co, ci, k, k, device=dev) * math.sqrt(2.0 / (ci * k * k))).requires_grad_()
    g = torch.randn(n, co, ho, wo, device=dev)
    tf, tb = [], []
    for i in range(iters + 1):
        x.grad = wt.grad = None
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        torch.cuda.synchronize()
        e[0].record()
        y = ref_adder.adder2d_function(x, wt, s, p)
        e[1].record()
        y.backward(g)
        e[2].record()
        torch.cuda.synchronize()
        if i > 0:
            tf.append(e[0].elapsed_time(e[1])); tb.append(e[1].elapsed_time(e[2]))
    return statistics.median(tf), statistics.median(tb)


# ------------------------------------------------------------------------------------------ CPU timings of single layers

def time_layer_cpu(n, shape, iters=3):
    """fwd+bwd seconds of one adder2d layer on the host through the port of the reference's adder.py (unfold,
    column matrices, rescale), all host threads; 1 warm-up + `iters` timed runs, median."""
    import torch
    from oracle import adder_unfold as U
    torch.set_num_threads(os.cpu_count() or 1)
    ci, co, h, w, s, k, p = shape
    ho, wo = (h - k + 2 * p) // s + 1, (w - k + 2 * p) // s + 1
    gen = torch.Generator().manual_seed(1234 + 100)
    x = torch.randn((n, ci, h, w), generator=gen).requires_grad_()
    wt = (torch.randn((co, ci, k, k), generator=gen) * math.sqrt(2.0 / (ci * k * k))).requires_grad_()
    g = torch.randn((n, co, ho, wo), generator=gen)
    ts = []
    for i in range(iters + 1):
        x.grad = wt.grad = None
        t0 = time.perf_counter()
        U.adder2d_function(x, wt, s, p).backward(g)
        if i > 0:
            ts.append(time.perf_counter() - t0)
    return statistics.median(ts)


def resnet50_block(dev, fp32_peak):
    """ResNet-50 adder training step at batch 64 (224x224 synthetic images, 1000 classes, fp32, SGD momentum):
    ms per step over a few CUDA-graph replays, and how much of it the adder kernels are."""
    import numpy as np
    import torch
    from addernetcuda_b200 import resnet as R
    from addernetcuda_b200.synthetic import image_batch
    from addernetcuda_b200.train import TrainStep
    B = 64
    net = R.resnet50()
    R.init_seeded(net, 1434)
    net = net.to(dev).train()
    ts = TrainStep(net, (B, 3, 224, 224), 1000, lr=0.1, momentum=0.9, use_graph=True, device=dev)
    images, labels = image_batch(B, 224, 1000, 1434)
    ts.load_batch(torch.from_numpy(images).to(dev), torch.from_numpy(labels).to(dev))
    for _ in range(2):
        ts.run()
    torch.cuda.synchronize()
    K = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        ts.run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / K
    out = {"workload": "resnet50_adder_train_step_fp32", "per_gpu_batch": B, "steps": K, "ms_per_step": ms,
           "images_per_s": B / (ms * 1e-3), "final_loss": float(ts.loss)}
    T = resnet50_triples(B)
    out["adder_triples_per_forward"] = T
    if fp32_peak:
        # the whole step against the roofline of its adder work alone (9 ops per triple): a lower bound on
        # what the adder kernels reach, since the step also holds BatchNorm, the stem and the optimiser
        out["step_pct_fp32_peak_lower_bound"] = 100 * 9 * T / (ms * 1e-3) / fp32_peak
    del ts, net
    torch.cuda.empty_cache()
    return out


def resnet50_triples(batch):
    """(co, k, pixel) triples of the 52 adder layers of ResNet-50 in one forward pass at 224x224."""
    import torch
    from addernetcuda_b200 import resnet as R, adder as A
    total = [0]
    orig = A.adder2d.forward

    def fwd(self, x):
        n, c, h, w = x.shape
        k, s, p = self.kernel_size, self.stride, self.padding
        ho, wo = (h - k + 2 * p) // s + 1, (w - k + 2 * p) // s + 1
        total[0] += n * ho * wo * self.output_channel * c * k * k
        return x.new_empty((n, self.output_channel, ho, wo))

    A.adder2d.forward = fwd
    try:
        with torch.device("meta"):
            net = R.resnet50(fused_bn=False)
            net(torch.empty(batch, 3, 224, 224))
    finally:
        A.adder2d.forward = orig
    return total[0]


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    import addernetcuda_b200 as ab
    from addernetcuda_b200 import resnet as R, adder as A
    from addernetcuda_b200.train import TrainStep
    from addernetcuda_b200.ddp import BucketedDDP

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback; use --impl reference for the CPU arm)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != max(1, args.gpus) and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    ab.strict_fp32()
    A.FAST_CLAMP = not args.exact_clamp

    B = args.batch
    if args.workload == "resnet20":
        net, shape, classes = R.resnet20(), (B, 3, 32, 32), 10
    else:
        net, shape, classes = R.resnet50(), (B, 3, 224, 224), 1000
    R.init_seeded(net, 1434)
    net = net.to(dev).train()
    if args.sync_bn and world > 1:
        net = torch.nn.SyncBatchNorm.convert_sync_batchnorm(net)
    peer_reduce = {"auto": None, "on": True, "off": False}[args.exchange]
    ddp = BucketedDDP(net, bucket_mb=args.bucket_mb, peer_reduce=peer_reduce) if world > 1 else None
    ts = TrainStep(net, shape, classes, lr=0.1, momentum=0.9, ddp=ddp, use_graph=not args.no_graph, device=dev)

    import numpy as np
    rng = np.random.default_rng(1434 + 1000 * rank)
    host_images = torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).pin_memory()
    host_labels = torch.from_numpy(rng.integers(0, classes, size=(B,)).astype(np.int64)).pin_memory()
    ts.load_batch(host_images, host_labels)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    W, K = max(3, args.warmup), max(1, args.steps)
    for _ in range(W):
        ts.run()
    barrier()
    if ddp is not None:
        ddp.check()      # a peer exchange that gave up waiting must not be timed as if it had worked

    # ---- value: K steps, batch resident in device memory
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        ts.run()
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else None
    final_loss = float(ts.loss)

    # ---- e2e: every step copies its batch from pinned host memory (prefetched one step ahead on a copy
    # stream, as a data loader would) and reads the loss back
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    ts.prefetch(host_images, host_labels)
    for i in range(K):
        loss = ts.step_prefetched()
        if i + 1 < K:
            ts.prefetch(host_images, host_labels)      # the next batch's copy overlaps this step
        _ = loss.item()
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))
    if ddp is not None:
        ddp.check()
    h2d = host_images.numel() * 4 + host_labels.numel() * 8
    d2h = 4

    n_adder = sum(1 for m in net.modules() if isinstance(m, A.adder2d))
    # kernels of this library per step: counted by the library across one eager forward + backward
    # (a graph replay runs the same kernels without passing through the host-side counter)
    from addernetcuda_b200 import _lib
    before = _lib.load().adder_b200_launch_count()
    ts.forward_backward_only()
    torch.cuda.synchronize()
    launches_per_step = int(_lib.load().adder_b200_launch_count() - before)

    line = None
    if rank == 0:
        images_per_s = world * B * K / (ms_total * 1e-3)
        steps_per_s = K / (ms_total * 1e-3)
        line = {
            "metric": "resnet20_adder_train_throughput" if args.workload == "resnet20" else "resnet50_adder_train_throughput",
            "value": images_per_s, "unit": "images/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_total / K, "steps_per_s": steps_per_s, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (steps_per_s / PUBLISHED_STEPS_PER_S) if (args.workload == "resnet20" and B == 256 and world == 1) else None,
            "vs_baseline_note": "reference README: 0.3158 s/batch, ResNet-20 on an RTX 2080Ti (batch 256 inferred)",
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}_adder_train_step_fp32", "per_gpu_batch": B, "global_batch": B * world,
                       "optimizer": "sgd(lr=0.1,momentum=0.9)", "cuda_graph": not args.no_graph,
                       "input_grad_clamp": "exact" if args.exact_clamp else "saturating-add form",
                       "batchnorm": "sync" if (args.sync_bn and world > 1) else "per-rank",
                       "parallelism": f"dp{world}", "buckets": len(ddp.buckets) if ddp is not None else 0,
                       "exchange": ("none" if ddp is None else
                                    "one-kernel push/wait/add over peer memory" if all(b.peer is not None for b in ddp.buckets)
                                    else "nccl all-reduce" if all(b.peer is None for b in ddp.buckets) else "mixed"),
                       "l2": "not flushed between steps: one step streams far more than the 126 MB L2"},
            "e2e": {"value": world * B * K / (ms_e2e * 1e-3), "unit": "images/s", "ms_per_step": ms_e2e / K,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * K,
            "clocks": clocks, "final_loss": final_loss,
        }

    # ---- kernel-level numbers (rank 0, one GPU's view): ResNet-20 layer set + the per-layer sweep
    if rank == 0 and not args.skip_layers:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        peaks = {}
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except (OSError, ValueError):
            pass
        f_max = (clocks or {}).get("sm_max_mhz") or peaks.get("sm_max_mhz") or 1965.0
        fp32_peak = 2 * 128 * sms * f_max * 1e6            # FLOP/s of the FP32 CUDA cores (FMA = 2)
        hbm_peak = peaks.get("hbm_gbs", 6650.0)
        tot = {"fwd": 0.0, "grad_x": 0.0, "grad_w": 0.0, "bwd": 0.0}
        tot_T = 0.0
        per_layer = []
        for shp, mult in RESNET20_LAYERS:
            t = time_layer_ops(256, shp)
            T = triples(256, shp)
            tot_T += T * mult
            for k in tot:
                tot[k] += t[k] * mult
        dom = max(("fwd", "grad_x", "grad_w"), key=tot.get)
        achieved = 3 * tot_T / (tot[dom] * 1e-3)
        all_ms = tot["fwd"] + tot["grad_x"] + tot["grad_w"]
        pass_ms = tot["fwd"] + tot["bwd"]
        line["roofline"] = {
            "bound": "fp32", "kernel": KERNEL_NAMES[dom],
            "achieved": achieved / 1e12, "peak": fp32_peak / 1e12, "unit": "TFLOP/s", "frac": achieved / fp32_peak,
            "peak_source": f"2*128*{sms} SMs*{f_max:.0f} MHz (FP32 CUDA-core FMA peak; MEASURED_PEAKS.json holds no SIMT figure)",
            "ops_rule": "3 ops per (co,k,pixel) triple per pass", "launches": 20, "ms_total": tot[dom],
            "traffic": NCU_DRAM_BYTES.get(dom),
            "traffic_note": "dram read+write bytes of ONE launch of this kernel on the 16->16 32x32 layer at batch 256, "
                            f"ncu capture summarised in {NCU_CAPTURE}; algorithmic bytes of that launch: "
                            f"{ALGO_BYTES_16x16.get(dom, 0)}",
            "per_kernel": {KERNEL_NAMES[k]: {"ms_total": tot[k], "frac": 3 * tot_T / (tot[k] * 1e-3) / fp32_peak,
                                             "traffic": NCU_DRAM_BYTES.get(k), "algorithmic_bytes": ALGO_BYTES_16x16.get(k)}
                           for k in ("fwd", "grad_x", "grad_w")},
        }
        line["adder_conv"] = {
            "workload": "the 20 adder layers of ResNet-20 at batch 256, every kernel timed alone, one launch per sample, L2 flushed before each",
            "fwd_ms": tot["fwd"], "grad_x_ms": tot["grad_x"], "grad_w_ms": tot["grad_w"],
            "fwd_bwd_gops": 9 * tot_T / (all_ms * 1e-3) / 1e9, "pct_fp32_peak": 100 * 9 * tot_T / (all_ms * 1e-3) / fp32_peak,
            "bwd_ms": tot["bwd"], "bwd_note": "both gradient kernels issued as the layer's backward does (weight gradient on a side stream)",
            "pass_gops": 9 * tot_T / (pass_ms * 1e-3) / 1e9, "pass_pct_fp32_peak": 100 * 9 * tot_T / (pass_ms * 1e-3) / fp32_peak,
            "share_of_step": pass_ms / (ms_total / K),
        }
        # the per-layer sweep of the benchmark definition, with two columns beside it: the reference's own
        # CUDA path (its adder.py + its kernels built for sm_100, from baseline/_ref) timed on this GPU with
        # the same events, and its CPU path (the port of adder.py) on the host cores
        ref_adder, ref_why = load_reference_cuda() if not args.skip_reference_cuda else (None, "skipped by flag")
        cpu_cols = world == 1 and not args.skip_cpu_baseline
        cores = os.cpu_count() or 1
        sweep = []
        for shp in SWEEP_SHAPES:
            t = time_layer_ops(256, shp)
            T = triples(256, shp)
            ms = t["fwd"] + t["grad_x"] + t["grad_w"]
            ci, co, h, w, s, k, p = shp
            x_b, w_b, o_b = 256 * ci * h * w * 4, co * ci * k * k * 4, T // (ci * k * k) * 4
            row = {"shape": {"ci": ci, "co": co, "h": h, "w": w, "stride": s, "k": k}, "fwd_ms": t["fwd"],
                   "grad_x_ms": t["grad_x"], "grad_w_ms": t["grad_w"], "bwd_ms": t["bwd"],
                   "pass_pct_fp32_peak": 100 * 9 * T / ((t["fwd"] + t["bwd"]) * 1e-3) / fp32_peak,
                   "fwd_bwd_gops": 9 * T / (ms * 1e-3) / 1e9, "pct_fp32_peak": 100 * 9 * T / (ms * 1e-3) / fp32_peak,
                   "fwd_gbs": (x_b + w_b + o_b) / (t["fwd"] * 1e-3) / 1e9}
            if ref_adder is not None and reference_cuda_in_bounds(256, shp):
                rf, rb = time_reference_cuda(ref_adder, 256, shp)
                row["reference_cuda"] = {"fwd_ms": rf, "bwd_ms": rb, "fwd_bwd_gops": 9 * T / ((rf + rb) * 1e-3) / 1e9}
                row["vs_reference_cuda"] = (rf + rb) / (t["fwd"] + t["bwd"])
            if cpu_cols:
                # CIFAR-size layers in full; the ImageNet-size ones (3e10 triples) on a batch-16 slice, scaled x16
                nb = 256 if T < 2e9 else 16
                sec = time_layer_cpu(nb, shp, iters=2 if nb == 256 else 1) * (256 / nb)
                row["cpu"] = {"fwd_bwd_s": sec, "fwd_bwd_gops": 9 * T / sec / 1e9, "cores": cores, "batch_timed": nb}
            sweep.append(row)
        line["reference_cuda"] = {"available": ref_adder is not None, "why_not": ref_why,
                                  "what": "the reference's adder2d_function forward + autograd backward (unfold, permutes, "
                                          "CONV / CONV_BACKWARD built for sm_100, col2im, rescale), same CUDA events, batch 256"}
        line["layers"] = sweep
        # the two 1x1 stride-2 downsample layers (about 6 op/B): bound by memory traffic, reported as GB/s of
        # algorithmic bytes (each tensor once; only the sampled quarter of x) against the measured HBM peak
        hbm_layers = []
        for shp in ((16, 32, 32, 32, 2, 1, 0), (32, 64, 16, 16, 2, 1, 0)):
            t = time_layer_ops(256, shp)
            ci, co, h, w, s, k, p = shp
            x_b, g_b, w_b = 256 * ci * h * w * 4, 256 * co * (h // 2) * (w // 2) * 4, co * ci * 4
            by = {"fwd": x_b // 4 + w_b + g_b, "grad_x": g_b + x_b // 4 + w_b + x_b, "grad_w": g_b + x_b // 4 + 2 * w_b}
            hbm_layers.append({"shape": {"ci": ci, "co": co, "h": h, "w": w, "stride": s, "k": k},
                               **{f"{op}_ms": t[op] for op in ("fwd", "grad_x", "grad_w", "bwd")},
                               **{f"{op}_gbs": by[op] / (t[op] * 1e-3) / 1e9 for op in by},
                               **{f"{op}_frac_hbm": by[op] / (t[op] * 1e-3) / 1e9 / hbm_peak for op in by}})
        line["hbm_layers"] = hbm_layers
        line["hbm"] = {"peak_gbs": hbm_peak, "note": "the 3x3 and the wide 1x1 adder layers are FP32-issue bound (54-1460 op/B against a "
                       "machine balance of ~11 op/B); the 1x1 stride-2 downsample layers are in hbm_layers"}

    # ---- ResNet-50 (ImageNet shapes, batch 64 per GPU): a few steps of the other network the benchmark names
    if rank == 0 and world == 1 and args.workload == "resnet20" and not args.skip_resnet50:
        line["resnet50"] = resnet50_block(dev, fp32_peak if not args.skip_layers else None)

    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        ips, b, s_per_step = cpu_images_per_s(args.cpu_budget_s, 2, 1)
        cores = os.cpu_count() or 1
        line["cpu_baseline"] = {"value": ips, "unit": "images/s", "cores": cores, "kind": "port",
                                "sample": f"2 training steps of ResNet-20 at batch {b} (of 256) through the CPU port of the "
                                          f"reference's adder.py unfold path, {cores} host threads, {s_per_step:.1f} s/step"}
        # configuration 1 of the benchmark definition: one adder2d layer, N=32, 16->16, 32x32, fwd+bwd on the host
        cfg1 = (16, 16, 32, 32, 1, 3, 1)
        sec = time_layer_cpu(32, cfg1, iters=3)
        t1 = time_layer_ops(32, cfg1)
        line["config1_single_layer"] = {
            "shape": "N=32 Ci=16 Co=16 32x32 k3 s1 p1", "cpu_fwd_bwd_s": sec, "cpu_gops": 9 * triples(32, cfg1) / sec / 1e9,
            "cpu_cores": cores, "cpu_sample": "1 warm-up + 3 timed forward+backward passes, median",
            "gpu_fwd_ms": t1["fwd"], "gpu_bwd_ms": t1["bwd"], "gpu_gops": 9 * triples(32, cfg1) / ((t1["fwd"] + t1["bwd"]) * 1e-3) / 1e9}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the communicator down: CUDA graphs that captured collectives on it are
        # still alive, and destroying it under them can block.  Everything is flushed and every rank has
        # passed the barrier, so a hard exit loses nothing.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["resnet20", "resnet50"], default="resnet20")
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch (default 256 for resnet20, 64 for resnet50)")
    ap.add_argument("--bucket-mb", type=float, default=None,
                    help="gradient bucket size; default: a third of the model's gradients, at most 25 MB")
    ap.add_argument("--sync-bn", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--exchange", choices=["auto", "on", "off"], default="auto",
                    help="gradient exchange at N > 1: this library's peer-memory kernel where it applies (auto), "
                         "required (on), or NCCL only (off)")
    ap.add_argument("--exact-clamp", action="store_true", help="input gradient with min/max instead of the saturating add")
    ap.add_argument("--skip-layers", action="store_true")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-resnet50", action="store_true")
    ap.add_argument("--skip-reference-cuda", action="store_true")
    ap.add_argument("--cpu-budget-s", type=float, default=150.0,
                    help="time budget of the CPU arm: the sample batch is the largest (up to 256) that fits it")
    args = ap.parse_args()
    if args.batch is None:
        args.batch = 256 if args.workload == "resnet20" else 64
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
