"""BatchNorm2d for adder networks with the residual add and ReLU folded in (CUDA, training mode).

`FusedBatchNorm2d` is an nn.BatchNorm2d (same parameters, buffers and state-dict keys) whose
training-mode forward on CUDA runs this library's kernels: per-channel reductions split over many
CTAs instead of the one-CTA-per-channel library kernels that dominate a ResNet-20 step on a B200.
`forward(y, residual=None, relu=False)` computes relu?(bn(y) + residual?) in one pass; plain
`forward(y)` is ordinary batch norm.  Evaluation mode and CPU tensors fall through to nn.BatchNorm2d
(those are not the training hot path and torch's implementation is the reference for them).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib, adder_cuda


class _BNFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, gamma, beta, residual, running_mean, running_var, num_batches, eps, momentum, relu, stats=None):
        y = y.contiguous()
        n, c, h, w = y.shape
        dev = y.device
        lib = _lib.load()
        z = torch.empty_like(y)
        mean = torch.empty(c, device=dev, dtype=torch.float32)
        invstd = torch.empty(c, device=dev, dtype=torch.float32)
        res = residual.contiguous() if residual is not None else None
        common = (gamma.data_ptr(), beta.data_ptr(), res.data_ptr() if res is not None else None,
                  z.data_ptr(), mean.data_ptr(), invstd.data_ptr(),
                  running_mean.data_ptr() if running_mean is not None else None,
                  running_var.data_ptr() if running_var is not None else None,
                  num_batches.data_ptr() if num_batches is not None else None,
                  float(eps), float(momentum), int(relu))
        with torch.cuda.device(dev):
            if stats is not None:
                if stats.dtype != torch.float64 or stats.dim() != 3 or stats.shape[0] != c or stats.shape[2] != 2 \
                        or not stats.is_contiguous() or stats.device != dev:
                    raise ValueError("stats must be a contiguous float64 [C, slices, 2] tensor on y's device")
                _lib.check(lib.adder_b200_batchnorm_forward_from_stats(
                    y.data_ptr(), stats.data_ptr(), int(stats.shape[1]), *common, n, c, h * w,
                    adder_cuda._stream(dev)), "adder_b200_batchnorm_forward_from_stats")
            else:
                ws = adder_cuda._workspace(dev, lib.adder_b200_batchnorm_workspace_bytes(n, c, h * w))
                _lib.check(lib.adder_b200_batchnorm_forward(
                    y.data_ptr(), *common, ws.data_ptr(), ws.numel(), n, c, h * w,
                    adder_cuda._stream(dev)), "adder_b200_batchnorm_forward")
        ctx.save_for_backward(y, z if relu else None, gamma, mean, invstd)
        ctx.relu = bool(relu)
        ctx.has_res = residual is not None
        return z

    @staticmethod
    def backward(ctx, dz):
        y, z, gamma, mean, invstd = ctx.saved_tensors
        dz = dz.contiguous()
        n, c, h, w = y.shape
        dev = y.device
        lib = _lib.load()
        dy = torch.empty_like(y)
        dres = torch.empty_like(y) if ctx.has_res else None
        dgamma = torch.empty_like(gamma)
        dbeta = torch.empty_like(gamma)
        with torch.cuda.device(dev):
            ws = adder_cuda._workspace(dev, lib.adder_b200_batchnorm_workspace_bytes(n, c, h * w))
            _lib.check(lib.adder_b200_batchnorm_backward(
                dz.data_ptr(), y.data_ptr(), z.data_ptr() if z is not None else None, gamma.data_ptr(),
                mean.data_ptr(), invstd.data_ptr(), dy.data_ptr(), dres.data_ptr() if dres is not None else None,
                dgamma.data_ptr(), dbeta.data_ptr(), int(ctx.relu), ws.data_ptr(), ws.numel(), n, c, h * w,
                adder_cuda._stream(dev)), "adder_b200_batchnorm_backward")
        return dy, dgamma, dbeta, dres, None, None, None, None, None, None, None


class FusedBatchNorm2d(nn.BatchNorm2d):
    """nn.BatchNorm2d with `forward(y, residual=None, relu=False, stats=None)`; `stats` are the per-channel
    sums the adder layer that produced `y` wrote (`adder2d.forward_with_stats`), which save the statistics pass."""

    def forward(self, y, residual=None, relu=False, stats=None):
        fused = (self.training and y.is_cuda and y.dtype == torch.float32 and self.affine
                 and self.track_running_stats and self.momentum is not None)
        if not fused:
            out = super().forward(y)
            if residual is not None:
                out = out + residual
            return torch.relu(out) if relu else out
        return _BNFunction.apply(y, self.weight, self.bias, residual, self.running_mean, self.running_var,
                                 self.num_batches_tracked, self.eps, self.momentum, relu, stats)
