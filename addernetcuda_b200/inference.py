"""Inference with adder networks: reference checkpoints, folded batch norm, top-k accuracy.

What the reference's test.py does around a trained network, without its dataset plumbing:
  * `load_reference_checkpoint` accepts a state dict written by the reference scripts, including the
    `module.` prefix nn.DataParallel adds (test.py:37-39);
  * `fold_batchnorm` turns every BatchNorm2d of a network in evaluation mode into the per-channel affine
    map it is (running statistics are constants), applied together with the residual add and ReLU of the
    block in ONE kernel behind each adder layer (the adder output is not linear in the weights, so the
    affine map cannot move into them; it becomes the layer's epilogue instead);
  * `accuracy` / `validate` are test.py:68-126: top-1 / top-5 over batches, no gradients.
"""
from __future__ import annotations

from typing import Iterable, Sequence, Tuple

import torch
import torch.nn as nn

from . import _lib, adder_cuda


def load_reference_checkpoint(model: nn.Module, state_dict: dict, strict: bool = True):
    """Load a checkpoint saved by the reference (plain, or from an nn.DataParallel wrapper)."""
    if "state_dict" in state_dict and isinstance(state_dict["state_dict"], dict):
        state_dict = state_dict["state_dict"]
    cleaned = {(k[len("module."):] if k.startswith("module.") else k): v for k, v in state_dict.items()}
    return model.load_state_dict(cleaned, strict=strict)


class FoldedBatchNorm2d(nn.Module):
    """Evaluation-mode BatchNorm2d as z = y*scale + shift [+ residual] [ReLU], one kernel on CUDA."""

    def __init__(self, bn: nn.BatchNorm2d):
        super().__init__()
        if bn.running_mean is None or bn.running_var is None:
            raise ValueError("batch norm without running statistics cannot be folded")
        with torch.no_grad():
            gamma = bn.weight if bn.affine else torch.ones_like(bn.running_mean)
            beta = bn.bias if bn.affine else torch.zeros_like(bn.running_mean)
            scale = gamma.float() / torch.sqrt(bn.running_var.float() + bn.eps)
            shift = beta.float() - bn.running_mean.float() * scale
        self.register_buffer("scale", scale.contiguous())
        self.register_buffer("shift", shift.contiguous())

    def forward(self, y, residual=None, relu=False):
        if not (y.is_cuda and y.dtype == torch.float32):
            out = y * self.scale.view(1, -1, 1, 1) + self.shift.view(1, -1, 1, 1)
            if residual is not None:
                out = out + residual
            return torch.relu(out) if relu else out
        y = y.contiguous()
        res = residual.contiguous() if residual is not None else None
        n, c, h, w = y.shape
        z = torch.empty_like(y)
        with torch.cuda.device(y.device):
            _lib.check(_lib.load().adder_b200_affine_forward(
                y.data_ptr(), self.scale.data_ptr(), self.shift.data_ptr(), res.data_ptr() if res is not None else None,
                z.data_ptr(), int(relu), n, c, h * w, adder_cuda._stream(y.device)), "adder_b200_affine_forward")
        return z


def fold_batchnorm(model: nn.Module) -> nn.Module:
    """Replace, in place, every 2-d batch norm of `model` by its folded form and put the model in
    evaluation mode.  The blocks of `addernetcuda_b200.resnet` then run BN + residual + ReLU as one kernel;
    any other container (the reference's own model files) still gets the one-kernel affine map and keeps
    its separate add / ReLU."""
    model.eval()

    def convert(module: nn.Module):
        for name, child in list(module.named_children()):
            if isinstance(child, nn.BatchNorm2d):
                setattr(module, name, FoldedBatchNorm2d(child))
            else:
                convert(child)

    convert(model)
    return model


def accuracy(output: torch.Tensor, target: torch.Tensor, topk: Sequence[int] = (1,)):
    """Precision@k in percent for each k (test.py:112-126)."""
    maxk = max(topk)
    batch = target.size(0)
    _, pred = output.topk(maxk, 1, True, True)
    correct = pred.t().eq(target.view(1, -1).expand(maxk, batch))
    return [correct[:k].reshape(-1).float().sum() * (100.0 / batch) for k in topk]


@torch.no_grad()
def validate(batches: Iterable[Tuple[torch.Tensor, torch.Tensor]], model: nn.Module, device=None, topk=(1, 5)):
    """Average top-k accuracy of `model` over (images, labels) batches (test.py:68-90).  Returns a tuple of
    floats, one per k, weighted by batch size."""
    model.eval()
    device = device if device is not None else next(model.parameters()).device
    sums = [0.0 for _ in topk]
    seen = 0
    for images, labels in batches:
        images, labels = images.to(device, non_blocking=True), labels.to(device, non_blocking=True)
        out = model(images)
        for i, a in enumerate(accuracy(out, labels, topk)):
            sums[i] += float(a) * labels.size(0)
        seen += labels.size(0)
    return tuple(s / max(seen, 1) for s in sums)
