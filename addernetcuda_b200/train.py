"""Training-step harness: forward, loss, backward, (all-reduce,) SGD step — optionally captured in
one CUDA graph so that the ~300 small kernels of a ResNet-20 step are launched with one call.

It replaces, for benchmarking and parity, the per-batch body of the reference's training loop
(main.py:86-101: zero_grad, net(images), CrossEntropyLoss, backward, optimizer.step) without its
per-step host synchronisation (`loss.data.item()`, main.py:92): the loss stays on the device until
the caller asks for it.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn


class TrainStep:
    """One SGD training step on static device buffers.

    step(images, labels) copies the batch into the static buffers (from pinned host memory when the
    inputs are CPU tensors), runs the step (graph replay when `use_graph`), and returns the loss as
    a 0-dim device tensor.
    """

    def __init__(self, model: nn.Module, batch_shape, num_classes: int, lr: float = 0.1, momentum: float = 0.9,
                 weight_decay: float = 0.0, ddp=None, use_graph: bool = True, device="cuda:0"):
        from . import strict_fp32
        strict_fp32()          # the benchmark configurations are fp32 end to end
        self.model = model
        self.ddp = ddp
        self.device = torch.device(device)
        self.images = torch.zeros(batch_shape, device=self.device)
        self.labels = torch.zeros(batch_shape[0], dtype=torch.long, device=self.device)
        self.num_classes = num_classes
        self.opt = torch.optim.SGD(model.parameters(), lr=lr, momentum=momentum, weight_decay=weight_decay)
        self.criterion = nn.CrossEntropyLoss()
        self.loss = torch.zeros((), device=self.device)
        self.logits: Optional[torch.Tensor] = None
        self.use_graph = use_graph
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.stream = torch.cuda.Stream(device=self.device)
        self._stage = None      # staging buffers, copy stream and events of prefetch()

    def _body(self, update: bool = True) -> None:
        if self.ddp is not None:
            self.ddp.zero_grad()
        else:
            self.opt.zero_grad(set_to_none=True)
        logits = self.model(self.images)
        loss = self.criterion(logits, self.labels)
        loss.backward()
        if self.ddp is not None:
            self.ddp.finish()
        if update:
            self.opt.step()
        self.logits = logits.detach()
        self.loss.copy_(loss.detach())

    def warmup(self, iters: int = 3) -> None:
        """Eager iterations on a side stream (required before capture); they do update the weights."""
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            for _ in range(iters):
                self._body()
        torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def capture(self) -> None:
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.stream):
            self._body()

    def load_batch(self, images: torch.Tensor, labels: torch.Tensor) -> None:
        self.images.copy_(images, non_blocking=True)
        self.labels.copy_(labels, non_blocking=True)

    def prefetch(self, images: torch.Tensor, labels: torch.Tensor) -> None:
        """Start copying the NEXT batch (pinned host memory) into staging buffers on a copy stream, so
        that the transfer overlaps the step that is running; `step_prefetched` consumes it."""
        if self._stage is None:
            self._stage = (torch.empty_like(self.images), torch.empty_like(self.labels))
            self._copy_stream = torch.cuda.Stream(device=self.device)
            self._copied = torch.cuda.Event()
            self._consumed = torch.cuda.Event()
            self._consumed.record(torch.cuda.current_stream(self.device))
        self._copy_stream.wait_event(self._consumed)      # the previous batch has left the staging buffers
        with torch.cuda.stream(self._copy_stream):
            self._stage[0].copy_(images, non_blocking=True)
            self._stage[1].copy_(labels, non_blocking=True)
            self._copied.record(self._copy_stream)

    def step_prefetched(self) -> torch.Tensor:
        """Run one step on the batch last given to `prefetch`."""
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(self._copied)
        self.images.copy_(self._stage[0], non_blocking=True)
        self.labels.copy_(self._stage[1], non_blocking=True)
        self._consumed.record(cur)
        return self.run()

    def run(self) -> torch.Tensor:
        """Run one step on whatever the static buffers hold."""
        if self.use_graph:
            if self.graph is None:
                self.warmup()
                self.capture()
            self.graph.replay()
        else:
            self._body()
        return self.loss

    def step(self, images: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        self.load_batch(images, labels)
        return self.run()

    def forward_backward_only(self) -> None:
        """Forward + backward without the optimizer update (parity checks of gradients)."""
        self._body(update=False)
