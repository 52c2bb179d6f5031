"""Batch-sharded data parallelism for adder networks: one process per GPU, replicated weights,
flat fp32 gradient buckets all-reduced over NCCL while the rest of the backward pass still runs.

The reference has no multi-process training (its only multi-GPU construct is nn.DataParallel for
evaluation, test.py:37); this module supplies the capability the benchmark configurations ask for.
Semantics follow the reference op: the adaptive rescale (adder.py:78) happens inside each replica's
backward, *before* the reduction, so ranks average per-rank-normalised adder gradients.

Mechanics
  * parameters are assigned to buckets in reverse registration order (roughly the order their
    gradients become ready); every bucket is one contiguous fp32 buffer;
  * a post-accumulate hook on each parameter counts arrivals; when a bucket is complete its gradients
    are packed into the flat buffer with one multi-tensor copy, `.grad` is re-pointed at the views,
    and the all-reduce is enqueued on a side stream that waits for the packing only;
  * `finish()` makes the compute stream wait for the side stream and divides by the world size.
Everything is stream-ordered (no host synchronisation), so a whole training step, collectives
included, can be captured in a CUDA graph.  Works on CPU tensors with the gloo backend (tests).
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist


class _Bucket:
    def __init__(self, params: List[torch.nn.Parameter], device, dtype):
        self.params = params
        self.numel = sum(p.numel() for p in params)
        self.flat = torch.zeros(self.numel, device=device, dtype=dtype)
        self.views = []
        off = 0
        for p in params:
            self.views.append(self.flat[off:off + p.numel()].view_as(p))
            off += p.numel()
        self.pending = len(params)
        self.work = None


class BucketedDDP:
    """Gradient bucketing + overlapped all-reduce around an existing module.

        ddp = BucketedDDP(model, bucket_mb=25)
        loss = criterion(ddp.module(x), y); loss.backward(); ddp.finish(); optimizer.step()
    """

    def __init__(self, module: torch.nn.Module, bucket_mb: float = 25.0, process_group=None,
                 broadcast_from_rank0: bool = True):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised before BucketedDDP")
        self.module = module
        self.group = process_group
        self.world = dist.get_world_size(process_group)
        params = [p for p in module.parameters() if p.requires_grad]
        if not params:
            raise ValueError("module has no trainable parameters")
        self.device = params[0].device
        self.is_cuda = self.device.type == "cuda"
        if broadcast_from_rank0:
            with torch.no_grad():
                for t in list(module.parameters()) + list(module.buffers()):
                    dist.broadcast(t, src=0, group=process_group)
        cap = max(1, int(bucket_mb * 1024 * 1024 / 4))
        self.buckets: List[_Bucket] = []
        cur: List[torch.nn.Parameter] = []
        size = 0
        for p in reversed(params):
            if cur and size + p.numel() > cap:
                self.buckets.append(_Bucket(cur, self.device, p.dtype))
                cur, size = [], 0
            cur.append(p)
            size += p.numel()
        if cur:
            self.buckets.append(_Bucket(cur, self.device, cur[0].dtype))
        self._where = {}
        for b in self.buckets:
            for p, v in zip(b.params, b.views):
                self._where[p] = b
                p._grad_slot = v      # adder layers write their weight gradient straight into the bucket
                p.register_post_accumulate_grad_hook(self._on_grad)
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        self.launch_order: List[int] = []   # bucket indices in the order their all-reduce was enqueued

    # ------------------------------------------------------------------ hooks
    def _on_grad(self, p: torch.nn.Parameter) -> None:
        b = self._where[p]
        b.pending -= 1
        if b.pending == 0:
            self._launch(b)

    def _launch(self, b: _Bucket) -> None:
        with torch.no_grad():
            srcs = [p.grad for p in b.params]
            need = [(v, s) for v, s in zip(b.views, srcs) if s.data_ptr() != v.data_ptr()]
            if need:
                torch._foreach_copy_([v for v, _ in need], [s for _, s in need])
            for p, v in zip(b.params, b.views):
                p.grad = v
        self.launch_order.append(self.buckets.index(b))
        if self.world == 1:
            return
        if self.is_cuda:
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.comm_stream):
                dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group)
        else:
            b.work = dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    # ------------------------------------------------------------------ step boundary
    def finish(self) -> None:
        """Call after backward(): waits (on the stream, not the host) for the reductions and averages."""
        for b in self.buckets:
            if b.pending != 0:
                raise RuntimeError("backward() did not produce a gradient for every parameter of a bucket")
        if self.world > 1:
            if self.is_cuda:
                torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
            else:
                for b in self.buckets:
                    if b.work is not None:
                        b.work.wait()
                        b.work = None
            with torch.no_grad():
                torch._foreach_mul_([b.flat for b in self.buckets], 1.0 / self.world)
        for b in self.buckets:
            b.pending = len(b.params)

    def zero_grad(self) -> None:
        """Drop gradients so that the next backward writes fresh ones (set-to-none semantics)."""
        for b in self.buckets:
            for p in b.params:
                p.grad = None
        self.launch_order.clear()
