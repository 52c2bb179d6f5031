"""Drop-in for the reference's `adder` module (adder.py): `adder2d`, `adder2d_function`, `adder`.

Same names, constructor arguments, attributes and state-dict keys (`adder`, `b`), so the
reference's resnet20.py, resnet50.py and vgg.py run unchanged on top of it and its checkpoints
load.  What differs is underneath: `adder2d_function` calls one fused CUDA kernel per direction on
NCHW tensors instead of unfold + permute + a kernel on column matrices + permute.  The column
level autograd Function `adder` is kept for code written against adder.py:43-80.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
from torch.autograd import Function

from . import adder_cuda

# Global switch for the one-instruction clamp in the input gradient (see adder_b200.h).
FAST_CLAMP = False
# Run the weight gradient of a layer on a side stream, concurrently with its input gradient
# (see adder_cuda.backward).
OVERLAP_BACKWARD = True


class _Adder2dNCHW(Function):
    """out = -sum|x_patch - w| with the reference's two surrogate gradients (adder.py:62-80)."""

    @staticmethod
    def forward(ctx, x, w, stride, padding, want_stats=False):
        # A data-parallel wrapper may attach `_grad_slot` to the parameter: a view into its flat
        # gradient bucket.  The weight-gradient kernel then writes the rescaled gradient there
        # directly, so no pack copy precedes the all-reduce.
        ctx.grad_slot = getattr(w, "_grad_slot", None)
        x = x.contiguous()
        w = w.contiguous()
        ctx.save_for_backward(x, w)
        ctx.stride, ctx.padding = stride, padding
        if want_stats:
            out, st = adder_cuda.forward(x, w, stride, padding, stats=True)
            ctx.mark_non_differentiable(st)
            ctx.set_materialize_grads(False)     # no zero-filled "gradient" of the statistics in backward
            return out, st
        return adder_cuda.forward(x, w, stride, padding)

    @staticmethod
    def backward(ctx, grad_out, *_unused):
        if grad_out is None:
            return None, None, None, None, None
        x, w = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0] and ctx.needs_input_grad[1]:
            gx, gw = adder_cuda.backward(grad_out, x, w, ctx.stride, ctx.padding, adder_cuda.ETA, FAST_CLAMP,
                                         out_w=ctx.grad_slot, overlap=OVERLAP_BACKWARD)
            return gx, gw, None, None, None
        if ctx.needs_input_grad[0]:
            gx = adder_cuda.backward_input(grad_out, x, w, ctx.stride, ctx.padding, FAST_CLAMP)
        if ctx.needs_input_grad[1]:
            gw = adder_cuda.backward_weight(grad_out, x, w, ctx.stride, ctx.padding, adder_cuda.ETA,
                                            out=ctx.grad_slot)
        return gx, gw, None, None, None


def _fused_geometry(W, stride, padding, dilation) -> bool:
    """The geometries the fused NCHW kernels are built for: square 1x1 / 3x3 kernels, stride 1 or 2."""
    return (W.dim() == 4 and W.shape[2] == W.shape[3] and W.shape[2] in (1, 3) and isinstance(stride, int)
            and stride in (1, 2) and isinstance(padding, int) and dilation in (1, (1, 1)))


def _adder2d_columns(X, W, stride, padding, dilation):
    """Every other geometry (5x5, 7x7, rectangular kernels, stride 3, dilation ...): the layer as the
    reference itself computes it, an explicit im2col around the column-matrix op (adder.py:22-41), with this
    library's column kernels underneath (`adder`) and autograd's fold as col2im.  Columns are ordered
    (image, position), which the op does not care about."""
    n, co = X.shape[0], W.shape[0]
    cols = torch.nn.functional.unfold(X, (W.shape[2], W.shape[3]), dilation=dilation, padding=padding, stride=stride)
    k, positions = cols.shape[1], cols.shape[2]
    Y = adder.apply(W.reshape(co, k), cols.transpose(0, 1).reshape(k, n * positions))
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)
    (sh, _), (ph, _), (dh, _) = pair(stride), pair(padding), pair(dilation)
    ho = (X.shape[2] + 2 * ph - dh * (W.shape[2] - 1) - 1) // sh + 1
    return Y.view(co, n, ho, positions // ho).transpose(0, 1).contiguous()


def adder2d_function(X, W, stride=1, padding=0, dilation=1):
    """Same contract as adder.py:22-41: X[N,Ci,H,W], W[Co,Ci,kh,kw] -> [N,Co,Ho,Wo], differentiable.
    `dilation` is an extension (the reference fixes it to 1)."""
    if _fused_geometry(W, stride, padding, dilation):
        return _Adder2dNCHW.apply(X, W, stride, padding)
    return _adder2d_columns(X, W, stride, padding, dilation)


class adder(Function):
    """Column-matrix op of adder.py:43-80: `adder.apply(W_col[Co,K], X_col[K,P]) -> [Co,P]`,
    backward returning (rescaled grad_W_col, grad_X_col)."""

    @staticmethod
    def forward(ctx, W_col, X_col):
        W_col = W_col.contiguous()
        X_col = X_col.contiguous()
        ctx.save_for_backward(W_col, X_col)
        output = torch.empty((W_col.size(0), X_col.size(1)), device=W_col.device, dtype=torch.float32)
        adder_cuda.ADDER_CONV(X_col, W_col, output)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        W_col, X_col = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        grad_W_col = torch.zeros_like(W_col)
        grad_X_col = torch.zeros_like(X_col)
        adder_cuda.ADDER_BACKWARD(grad_output, X_col, W_col, grad_W_col, grad_X_col)
        grad_W_col = grad_W_col / grad_W_col.norm(p=2).clamp(min=1e-12) * math.sqrt(W_col.size(1) * W_col.size(0)) / 5
        return grad_W_col, grad_X_col


class adder2d(nn.Module):
    """adder.py:83-108.  `depth_wise=True` is rejected: the reference allocates [Co,1,k,k] weights for
    it but its forward ignores the flag, so no caller can rely on it.  3x3 and 1x1 kernels at stride 1 or 2 run
    on the fused kernels; any other kernel size or stride (and the extensions: a (kh, kw) tuple, `dilation`)
    runs through the column-matrix kernels behind an explicit im2col."""

    def __init__(self, input_channel, output_channel, kernel_size, stride=1, padding=0, bias=False,
                 depth_wise=False, dilation=1):
        super().__init__()
        if depth_wise:
            raise NotImplementedError("depth_wise adder2d is not implemented (nor computed by the reference)")
        self.stride = stride
        self.padding = padding
        self.dilation = dilation          # extension: the reference has no dilation (adder.py:32)
        self.input_channel = input_channel
        self.output_channel = output_channel
        self.kernel_size = kernel_size
        self.depth_wise = depth_wise
        kh, kw = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size   # (kh, kw): extension
        self.adder = torch.nn.Parameter(nn.init.normal_(torch.randn(output_channel, input_channel, kh, kw)))
        self.bias = bias
        if bias:
            self.b = torch.nn.Parameter(nn.init.uniform_(torch.zeros(output_channel)))

    def forward(self, x):
        output = adder2d_function(x, self.adder, self.stride, self.padding, self.dilation)
        if self.bias:
            output = output + self.b.unsqueeze(0).unsqueeze(2).unsqueeze(3)
        return output

    def forward_with_stats(self, x):
        """`(forward(x), st)` where `st` holds the per-channel sums a following batch norm needs
        (`adder_cuda.forward(..., stats=True)`), or None where the layer cannot provide them."""
        if self.bias or not x.is_cuda or not _fused_geometry(self.adder, self.stride, self.padding, self.dilation):
            return self.forward(x), None
        out, st = _Adder2dNCHW.apply(x, self.adder, self.stride, self.padding, True)
        return out, (st if st.shape[1] > 0 else None)
