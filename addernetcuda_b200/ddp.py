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
  * the reduction averages (NCCL's AVG operator), so no scaling pass follows it; `finish()` only makes
    the compute stream wait for the side stream (with gloo, which can only sum, it also scales);
  * on one node with NVLink peers, buckets of up to 8 MB skip NCCL: one kernel of this library pushes the
    bucket into a receive area on every rank, waits (bounded) for the others' pushes and adds them in rank
    order (`peer.PeerAllReduce`) - one launch and one NVLink round per bucket instead of a ring.
Everything is stream-ordered (no host synchronisation), so a whole training step, collectives
included, can be captured in a CUDA graph.  Works on CPU tensors with the gloo backend (tests).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class _Bucket:
    def __init__(self, params: List[torch.nn.Parameter], device, dtype):
        self.params = params
        self.numel = sum(p.numel() for p in params)
        # padded to whole 128-bit words (the peer all-reduce moves quads); the pad stays zero
        self.flat = torch.zeros((self.numel + 3) // 4 * 4, device=device, dtype=dtype)
        self.views = []
        off = 0
        for p in params:
            self.views.append(self.flat[off:off + p.numel()].view_as(p))
            off += p.numel()
        self.pending = len(params)
        self.work = None
        self.peer = None          # peer.PeerAllReduce when the bucket is exchanged over peer memory


class BucketedDDP:
    """Gradient bucketing + overlapped all-reduce around an existing module.

        ddp = BucketedDDP(model)            # bucket size chosen from the model
        loss = criterion(ddp.module(x), y); loss.backward(); ddp.finish(); optimizer.step()

    `bucket_mb=None` picks the bucket size from the model: a third of the gradient bytes, at most
    25 MB.  A small network (ResNet-20: 1.09 MB of gradients) then still has three buckets, so the
    gradients of its last stage are on the wire while the first stage is still in backward; with one
    big bucket the whole reduction would start after the last gradient and be fully exposed.
    """

    def __init__(self, module: torch.nn.Module, bucket_mb: Optional[float] = None, process_group=None,
                 broadcast_from_rank0: bool = True, peer_reduce: Optional[bool] = None, peer_max_polls: Optional[int] = None):
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
        total_bytes = sum(p.numel() * p.element_size() for p in params)
        if bucket_mb is None:
            cap_bytes = min(25 * 1024 * 1024, -(-total_bytes // 3))
        else:
            cap_bytes = int(bucket_mb * 1024 * 1024)
        cap_bytes = max(cap_bytes, 1)
        # reverse registration order (roughly the order gradients become ready); a bucket holds one dtype
        self.buckets: List[_Bucket] = []
        cur: List[torch.nn.Parameter] = []
        size = 0
        for p in reversed(params):
            nbytes = p.numel() * p.element_size()
            if cur and (size + nbytes > cap_bytes or p.dtype != cur[0].dtype):
                self.buckets.append(_Bucket(cur, self.device, cur[0].dtype))
                cur, size = [], 0
            cur.append(p)
            size += nbytes
        if cur:
            self.buckets.append(_Bucket(cur, self.device, cur[0].dtype))
        self._where = {}
        self._seen = set()       # parameters whose gradient has arrived in the current backward
        for b in self.buckets:
            for p, v in zip(b.params, b.views):
                self._where[p] = b
                p._grad_slot = v      # adder layers write their weight gradient straight into the bucket
                p.register_post_accumulate_grad_hook(self._on_grad)
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        # NCCL averages inside the reduction; gloo only sums, so its buckets are scaled in finish()
        self._avg_in_reduce = self.is_cuda and dist.get_backend(process_group) == "nccl"
        self.launch_order: List[int] = []   # bucket indices in the order their all-reduce was enqueued
        # peer_reduce: None = use the one-kernel exchange where it applies, False = NCCL only, True = require it
        self.peer_arena = None
        if peer_reduce is not False and self.world > 1:
            self._setup_peer_reduce(required=bool(peer_reduce), max_polls=peer_max_polls)

    def _setup_peer_reduce(self, required: bool, max_polls: Optional[int]) -> None:
        """All ranks decide together: either every eligible bucket goes over peer memory on every rank, or none."""
        from . import peer
        eligible = [b for b in self.buckets
                    if b.flat.dtype == torch.float32 and b.flat.numel() * 4 <= peer.MAX_BUCKET_BYTES]
        ok = self._avg_in_reduce and bool(eligible)
        err: Optional[Exception] = None
        if ok:
            ok = peer.same_host(self.group)
        if ok:
            try:
                sizes = [peer.PeerAllReduce.area_bytes(b.flat.numel(), self.world) for b in eligible]
                self.peer_arena = peer.PeerArena(sum(sizes), self.device, self.group)
            except Exception as e:          # no IPC / no peer access on this machine
                ok, err = False, e
        flag = torch.tensor([1 if ok else 0], device=self.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self.peer_arena = None
            if required:
                raise RuntimeError(f"peer_reduce=True but the peer-memory exchange cannot be set up here: {err}")
            return
        off = 0
        kw = {} if max_polls is None else {"max_polls": int(max_polls)}
        for b, sz in zip(eligible, sizes):
            b.peer = peer.PeerAllReduce(b.flat, self.peer_arena, off, **kw)
            off += sz
        dist.barrier(group=self.group)
        # Self-test before the first real step: every bucket is exchanged once by the kernel and once by NCCL on
        # rank-dependent values; unless both agree on every rank, all ranks go back to NCCL together.
        good = True
        rank = dist.get_rank(self.group)
        with torch.no_grad():
            for b in eligible:
                probe = torch.arange(b.flat.numel(), device=self.device, dtype=torch.float32).remainder_(251.0)
                probe = probe * (0.25 + 0.5 * rank) + rank
                want = probe.clone()
                dist.all_reduce(want, op=dist.ReduceOp.SUM, group=self.group)
                want /= self.world
                b.flat.copy_(probe)
                b.peer.launch()
                torch.cuda.synchronize(self.device)
                good = good and b.peer.status(reset=True) == 0 and bool(torch.allclose(b.flat, want, rtol=1e-6, atol=1e-6))
                b.flat.zero_()
        flag = torch.tensor([1 if good else 0], device=self.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            for b in eligible:
                b.peer = None
            if required:
                raise RuntimeError("peer_reduce=True but the peer-memory exchange failed its self-test against NCCL")

    def check(self) -> None:
        """Raises if a peer exchange gave up waiting for another rank (synchronises the device).  Call it
        where a host synchronisation is acceptable: after a validation pass, every so many steps, at the end."""
        for i, b in enumerate(self.buckets):
            if b.peer is not None:
                st = b.peer.status(reset=True)
                if st != 0:
                    raise RuntimeError(f"BucketedDDP: the peer exchange of bucket {i} timed out waiting for another "
                                       f"rank (status {st}); its gradients were not averaged")

    # ------------------------------------------------------------------ hooks
    def _on_grad(self, p: torch.nn.Parameter) -> None:
        if p in self._seen:
            # A weight used twice in one forward accumulates twice: the bucket would be reduced after the
            # first arrival, and an adder layer's direct write into the bucket slot would overwrite it.
            raise RuntimeError("BucketedDDP: a parameter received two gradients in one backward pass "
                               "(shared weights are not supported)")
        self._seen.add(p)
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
                if b.peer is not None:
                    b.peer.launch(self.comm_stream)
                else:
                    dist.all_reduce(b.flat, op=dist.ReduceOp.AVG if self._avg_in_reduce else dist.ReduceOp.SUM,
                                    group=self.group)
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
            if not self._avg_in_reduce:
                with torch.no_grad():
                    torch._foreach_mul_([b.flat for b in self.buckets], 1.0 / self.world)
        for b in self.buckets:
            b.pending = len(b.params)
        self._seen.clear()

    def sync_buffers(self) -> None:
        """Average the floating-point buffers (BatchNorm running statistics) over the ranks.  Batch
        statistics are per rank during training, so the running averages drift apart; call this before
        evaluating or writing a checkpoint if every rank's copy should be the same."""
        if self.world == 1:
            return
        with torch.no_grad():
            for t in self.module.buffers():
                if torch.is_floating_point(t):
                    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
                    t.div_(self.world)

    def zero_grad(self) -> None:
        """Drop gradients so that the next backward writes fresh ones (set-to-none semantics)."""
        for b in self.buckets:
            for p in b.params:
                p.grad = None
        self.launch_order.clear()
        self._seen.clear()
