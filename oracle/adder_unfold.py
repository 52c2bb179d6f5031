"""CPU port of the reference's Python layer (adder.py).  TEST INFRASTRUCTURE ONLY.

`adder2d_function`, the `adder` autograd Function and the `adder2d` module, restated so that a whole
network can be stepped on the CPU where the reference's sources are not present (the timed CPU
baseline and the network-level parity check).  Same structure as the reference: unfold + permute to
column matrices (adder.py:32-34), the op on columns (adder.py:44-60), the backward with the
adaptive rescale inside it (adder.py:62-80), the module with parameter `adder` and optional `b`
(adder.py:83-108).  `tests/golden/make_golden.py` checks it bit-for-bit against the reference file.
"""
import torch
import torch.nn as nn

from . import adder_oracle as _o


class adder(torch.autograd.Function):
    @staticmethod
    def forward(ctx, W_col, X_col):
        ctx.save_for_backward(W_col, X_col)
        return _o.forward_col(W_col, X_col)

    @staticmethod
    def backward(ctx, grad_output):
        W_col, X_col = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        gw = _o.grad_w_col(W_col, X_col, grad_output)
        gx = _o.grad_x_col(W_col, X_col, grad_output)
        return _o.rescale(gw), gx


def adder2d_function(X, W, stride=1, padding=0):
    co, _, k, _ = W.size()
    n, _, h, w = X.size()
    ho, wo = _o.out_hw(h, w, k, stride, padding)
    X_col = torch.nn.functional.unfold(X.view(1, -1, h, w), k, dilation=1, padding=padding,
                                       stride=stride).view(n, -1, ho * wo)
    X_col = X_col.permute(1, 2, 0).contiguous().view(X_col.size(1), -1)
    out = adder.apply(W.view(co, -1), X_col)
    return out.view(co, ho, wo, n).permute(3, 0, 1, 2).contiguous()


class adder2d(nn.Module):
    def __init__(self, input_channel, output_channel, kernel_size, stride=1, padding=0, bias=False,
                 depth_wise=False):
        super().__init__()
        if depth_wise:
            raise NotImplementedError("depth_wise adder2d is not computed by the reference either")
        self.stride, self.padding = stride, padding
        self.input_channel, self.output_channel = input_channel, output_channel
        self.kernel_size, self.depth_wise, self.bias = kernel_size, depth_wise, bias
        self.adder = nn.Parameter(nn.init.normal_(torch.randn(output_channel, input_channel,
                                                              kernel_size, kernel_size)))
        if bias:
            self.b = nn.Parameter(nn.init.uniform_(torch.zeros(output_channel)))

    def forward(self, x):
        out = adder2d_function(x, self.adder, self.stride, self.padding)
        if self.bias:
            out = out + self.b.view(1, -1, 1, 1)
        return out
