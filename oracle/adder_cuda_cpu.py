"""CPU stand-in for the reference's `adder_cuda` extension.  TEST INFRASTRUCTURE ONLY.

Same four entry points, argument order and buffer semantics as the pybind module of
adder_cuda/adder_cuda.cpp:88-93: `ADDER_CONV` overwrites `y` (adder.cu:67 stores, does not add);
the three gradient entry points accumulate into caller-zeroed buffers (atomicAdd at adder.cu:125,
:186, :266-267).  The arithmetic is the reference's own ground-truth expressions
(adder_cuda/test_cuda.py:21, :39-40, :58-59).  With this module registered as `adder_cuda`, the
reference's adder.py, resnet20.py, resnet50.py and vgg.py import and run unchanged on the CPU,
which is how the golden fixtures are produced and how the oracle is pinned.
"""
from . import adder_oracle as _o


def ADDER_CONV(x, w, y):
    y.copy_(_o.forward_col(w, x))


def ADDER_CONV_WEIGHT(grad_y, x, w, grad_w):
    grad_w.add_(_o.grad_w_col(w, x, grad_y))


def ADDER_CONV_INPUT(grad_y, x, w, grad_i):
    grad_i.add_(_o.grad_x_col(w, x, grad_y))


def ADDER_BACKWARD(grad_y, x, w, grad_w, grad_i):
    grad_w.add_(_o.grad_w_col(w, x, grad_y))
    grad_i.add_(_o.grad_x_col(w, x, grad_y))
