"""Bucketed data-parallel gradient averaging on two CPU ranks (gloo): the host-side logic of the
multi-GPU path — bucket assignment, readiness hooks, overlap bookkeeping, averaging, parameter
broadcast — with the oracle adder layer standing in for the CUDA one."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _make_model(seed):
    from oracle import adder_unfold as U
    torch.manual_seed(seed)
    m = nn.Sequential(
        nn.Conv2d(3, 4, 3, padding=1, bias=False), nn.BatchNorm2d(4), nn.ReLU(),
        U.adder2d(4, 6, 3, stride=2, padding=1), nn.BatchNorm2d(6), nn.ReLU(),
        U.adder2d(6, 5, 1, stride=1, padding=0), nn.BatchNorm2d(5),
        nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(5, 3))
    return m


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from addernetcuda_b200.ddp import BucketedDDP
        torch.set_num_threads(1)
        model = _make_model(seed=100 + rank)          # different init per rank: broadcast must fix it
        ddp = BucketedDDP(model, bucket_mb=0.0005)     # ~131 floats per bucket -> several buckets
        ref = _make_model(seed=100)                    # rank 0's init, used for the manual average
        for (k, a), (_, b) in zip(model.state_dict().items(), ref.state_dict().items()):
            assert torch.equal(a, b), f"parameter {k} was not broadcast from rank 0"
        g = torch.Generator().manual_seed(7 + rank)
        x = torch.randn(4, 3, 8, 8, generator=g)
        y = torch.randint(0, 3, (4,), generator=g)
        # data-parallel gradients
        ddp.zero_grad()
        nn.functional.cross_entropy(model(x), y).backward()
        ddp.finish()
        # manual: local gradients of an identical replica, gathered and averaged
        nn.functional.cross_entropy(ref(x), y).backward()
        for (k, p), (_, pr) in zip(model.named_parameters(), ref.named_parameters()):
            gathered = [torch.zeros_like(pr.grad) for _ in range(world)]
            dist.all_gather(gathered, pr.grad)
            want = sum(gathered) / world
            assert torch.allclose(p.grad, want, rtol=1e-6, atol=1e-7), f"{k}: averaged gradient differs"
        assert len(ddp.buckets) >= 3
        # buckets hold parameters in reverse registration order and are reduced roughly last-layer first
        assert ddp.launch_order[0] == 0 and sorted(ddp.launch_order) == list(range(len(ddp.buckets)))
        # every gradient is now a view into its bucket
        for b in ddp.buckets:
            for p, v in zip(b.params, b.views):
                assert p.grad.data_ptr() == v.data_ptr()
        # a second step reuses the buckets
        ddp.zero_grad()
        nn.functional.cross_entropy(model(x), y).backward()
        ddp.finish()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        import traceback
        q.put((rank, "".join(traceback.format_exception(e))))
    finally:
        dist.destroy_process_group()


def test_bucketed_allreduce_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_requires_initialised_process_group():
    from addernetcuda_b200.ddp import BucketedDDP
    if dist.is_initialized():
        pytest.skip("a process group is already initialised in this process")
    with pytest.raises(RuntimeError):
        BucketedDDP(nn.Linear(2, 2))
