"""Two-GPU data-parallel step over NCCL: averaged gradients equal the mean of the per-rank gradients,
and a CUDA-graph-captured step with the collectives inside the graph trains like the eager one.
Skipped on a single-GPU box (the host-side logic is covered on CPU ranks in test_ddp_gloo.py)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q, peer):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import numpy as np
        import addernetcuda_b200 as ab
        from addernetcuda_b200 import resnet as R
        from addernetcuda_b200.ddp import BucketedDDP
        from addernetcuda_b200.train import TrainStep
        ab.strict_fp32()
        rng = np.random.default_rng(50 + rank)
        images = torch.from_numpy(rng.standard_normal((32, 3, 32, 32)).astype(np.float32)).to(dev)
        labels = torch.from_numpy(rng.integers(0, 10, size=(32,)).astype(np.int64)).to(dev)

        def build():
            net = R.resnet20()
            R.init_seeded(net, 77)
            return net.to(dev).train()

        # local gradients of an identical replica, averaged by hand
        ref = build()
        torch.nn.functional.cross_entropy(ref(images), labels).backward()
        want = {}
        for k, p in ref.named_parameters():
            t = p.grad.clone()
            dist.all_reduce(t)
            want[k] = t / world
        # bucketed, overlapped reduction; the bucket size comes from the model: three or more buckets
        net = build()
        ddp = BucketedDDP(net, peer_reduce=peer)
        assert len(ddp.buckets) >= 3, len(ddp.buckets)
        # peer=True: every bucket is exchanged by this library's one-kernel push/wait/add over peer memory;
        # peer=False: NCCL's all-reduce
        assert all((b.peer is not None) == peer for b in ddp.buckets)
        ddp.zero_grad()
        torch.nn.functional.cross_entropy(net(images), labels).backward()
        ddp.finish()
        torch.cuda.synchronize()
        ddp.check()
        for k, p in net.named_parameters():
            err = (p.grad - want[k]).abs().max().item()
            assert err <= 1e-6 + 1e-5 * want[k].abs().max().item(), f"{k}: {err}"
        # the averaged gradients against the CPU oracle: every rank steps the oracle network (the port of
        # the reference's adder.py) on its own shard in float32 and float64, the per-shard results are
        # averaged over the ranks, and the data-parallel gradients must match that mean
        from oracle import adder_unfold as U
        from tests import netcheck
        worst = 0.0
        for dtype in (torch.float32, torch.float64):
            ora = R.resnet20(conv=U.adder2d)
            R.init_seeded(ora, 77)
            ora = ora.to(dtype).train()
            torch.nn.functional.cross_entropy(ora(images.cpu().to(dtype)), labels.cpu()).backward()
            mean = {}
            for k, p in ora.named_parameters():
                t = p.grad.to(dev, torch.float64)
                dist.all_reduce(t)
                mean[k] = (t / world).cpu()
            if dtype == torch.float32:
                mean32 = mean
            else:
                mean64 = mean
        anchored = 0
        for k, p in net.named_parameters():
            ok, used64, msg = netcheck.grad_ok(k, p.grad, mean32[k], mean64[k])
            anchored += int(used64)
            worst = max(worst, (p.grad.double().cpu() - mean32[k]).abs().max().item())
            assert ok, msg
        assert anchored <= 3, anchored
        print(f"rank {rank}: {len(mean32)} averaged gradients match the mean of the per-shard CPU oracle "
              f"gradients, worst max_abs_err {worst:.3e}, {anchored} judged against float64", flush=True)
        # adder weight gradients were written straight into their bucket slots
        for b in ddp.buckets:
            for p, v in zip(b.params, b.views):
                assert p.grad.data_ptr() == v.data_ptr()
        # graph-captured training steps with the all-reduce inside the graph: loss goes down, ranks agree
        ts = TrainStep(net, (32, 3, 32, 32), 10, ddp=ddp, use_graph=True, device=dev)
        ts.load_batch(images, labels)
        losses = [float(ts.run()) for _ in range(6)]
        assert losses[-1] < losses[0], losses
        w = net.layer1[0].conv1.adder.detach().clone()
        gathered = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(gathered, w)
        assert torch.equal(gathered[0], gathered[1]), "replicas diverged"
        ddp.check()
        print(f"rank {rank}: 6 graph-captured steps, exchange by {'peer-memory kernel' if peer else 'NCCL'}, "
              f"losses {losses[0]:.4f} -> {losses[-1]:.4f}, replicas identical", flush=True)
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, "".join(traceback.format_exception(e))))
    finally:
        torch.cuda.synchronize()
        q.close()
        q.join_thread()  # the result must have left the feeder thread before the hard exit below
        os._exit(0)      # leave without communicator teardown (live CUDA graphs hold captured collectives)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("peer", [False, True], ids=["nccl", "peer_memory"])
def test_two_gpu_bucketed_allreduce_and_graph_step(peer):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, peer)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
