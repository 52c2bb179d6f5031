"""Drop-in for the reference's `adder_cuda` extension module, on top of libadder_b200.so.

The four column-matrix entry points keep the reference's names, argument order and buffer
semantics (adder_cuda/adder_cuda.cpp:37-93): `ADDER_CONV(x, w, y)` overwrites `y`; the gradient
entry points add into caller-zeroed buffers.  `forward` / `backward` are the fused NCHW
operations that `adder.adder2d` uses: no unfold, no permute copies, no column matrices.

Every tensor must be a contiguous float32 CUDA tensor; anything else raises (the reference raises
for non-CUDA or non-contiguous tensors, adder_cuda.cpp:33-35, and silently misreads other dtypes).
There is no CPU path.
"""
from __future__ import annotations

import torch

from . import _lib

ETA = 0.2  # adaptive learning-rate constant of adder.py:78 ("/5")

_workspaces: dict = {}


def _check(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32, got {t.dtype}")


def _same_device(*ts: torch.Tensor) -> torch.device:
    dev = ts[0].device
    for t in ts[1:]:
        if t.device != dev:
            raise RuntimeError(f"tensors are on different devices ({dev} and {t.device})")
    return dev


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


_retired: list = []


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Per-(device, stream) scratch for the weight-gradient kernels, grown on demand.  Calls on one
    stream are ordered, so they can share it; allocation goes through torch's caching allocator.

    A buffer that has to grow is replaced, never freed: a captured CUDA graph may have baked the old
    buffer's address into its kernel nodes, and handing that memory back to the allocator would let a
    later replay write partial sums into someone else's tensor.  Growth is geometric, so the retired
    buffers of a stream add up to less than the live one."""
    key = (dev.index, _stream(dev))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired.append(ws)
            nbytes = max(nbytes, 2 * ws.numel())
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def output_size(h: int, w: int, k: int, stride: int, padding: int):
    import ctypes
    ho, wo = ctypes.c_int(), ctypes.c_int()
    _lib.check(_lib.load().adder_b200_output_size(h, w, k, stride, padding, ctypes.byref(ho), ctypes.byref(wo)),
               "output_size")
    return ho.value, wo.value


def _geom(x: torch.Tensor, w: torch.Tensor, stride: int, padding: int):
    if x.dim() != 4 or w.dim() != 4:
        raise ValueError("x must be [N,Ci,H,W] and w [Co,Ci,k,k]")
    n, ci, h, wd = x.shape
    co, ci_w, kh, kw = w.shape
    if ci_w != ci:
        raise ValueError(f"w has {ci_w} input channels, x has {ci}")
    if kh != kw:
        raise ValueError("only square kernels are supported (as in adder.py:32)")
    return (n, ci, h, wd, co, kh, int(stride), int(padding))


# ---------------------------------------------------------------------------- fused NCHW path

def forward(x: torch.Tensor, w: torch.Tensor, stride: int = 1, padding: int = 0, stats: bool = False):
    """out[N,Co,Ho,Wo] = -sum |x_patch - w|: adder2d_function's forward (adder.py:22-41) in one kernel.

    With `stats=True` returns `(out, st)`: `st` is a float64 tensor [Co, slices, 2] holding, per pixel
    tile of the launch, the sum of each channel's outputs and of their squares - what the batch norm
    after the layer (resnet20.py:28-29) needs, so that it does not have to read `out` twice.  `st` is
    empty (0 slices) for the geometries whose kernel has no such epilogue."""
    _check(x, "x"); _check(w, "w")
    dev = _same_device(x, w)
    g = _geom(x, w, stride, padding)
    ho, wo = output_size(g[2], g[3], g[5], g[6], g[7])
    out = torch.empty((g[0], g[4], ho, wo), dtype=torch.float32, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        slices = lib.adder_b200_forward_stat_slices(*g) if stats else 0
        if slices > 0:
            st = torch.empty((g[4], slices, 2), dtype=torch.float64, device=dev)
            _lib.check(lib.adder_b200_forward_with_stats(x.data_ptr(), w.data_ptr(), out.data_ptr(), st.data_ptr(),
                                                         slices, *g, _stream(dev)), "adder_b200_forward_with_stats")
            return out, st
        _lib.check(lib.adder_b200_forward(x.data_ptr(), w.data_ptr(), out.data_ptr(), *g, _stream(dev)),
                   "adder_b200_forward")
    if stats:
        return out, torch.empty((g[4], 0, 2), dtype=torch.float64, device=dev)
    return out


def backward_input(grad_out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stride: int = 1, padding: int = 0,
                   fast_clamp: bool = False) -> torch.Tensor:
    """grad_x[N,Ci,H,W] = sum over taps of clamp(w - x, -1, 1) * grad_out (adder.py:74 + col2im)."""
    _check(grad_out, "grad_out"); _check(x, "x"); _check(w, "w")
    dev = _same_device(grad_out, x, w)
    g = _geom(x, w, stride, padding)
    _expect_grad_shape(grad_out, g)
    gx = torch.empty_like(x)
    flags = _lib.FLAG_FAST_CLAMP if fast_clamp else 0
    with torch.cuda.device(dev):
        _lib.check(_lib.load().adder_b200_backward_input(grad_out.data_ptr(), x.data_ptr(), w.data_ptr(),
                                                         gx.data_ptr(), *g, flags, _stream(dev)),
                   "adder_b200_backward_input")
    return gx


def backward_weight(grad_out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stride: int = 1, padding: int = 0,
                    eta: float = ETA, out: torch.Tensor | None = None, return_norm: bool = False):
    """grad_w[Co,Ci,k,k] = sum (x_patch - w) * grad_out, rescaled by eta*sqrt(numel)/||grad_w||
    when eta > 0 (adder.py:70,78).  `out` lets the caller have it written in place (e.g. into a
    gradient bucket)."""
    _check(grad_out, "grad_out"); _check(x, "x"); _check(w, "w")
    dev = _same_device(grad_out, x, w)
    g = _geom(x, w, stride, padding)
    _expect_grad_shape(grad_out, g)
    if out is None:
        out = torch.empty_like(w)
    else:
        _check(out, "out")
        if out.shape != w.shape:
            raise ValueError("out must have the shape of w")
    norm = torch.empty(1, dtype=torch.float32, device=dev) if return_norm else None
    lib = _lib.load()
    with torch.cuda.device(dev):
        nbytes = lib.adder_b200_backward_weight_workspace_bytes(*g)
        ws = _workspace(dev, nbytes)
        _lib.check(lib.adder_b200_backward_weight(grad_out.data_ptr(), x.data_ptr(), w.data_ptr(), out.data_ptr(),
                                                  float(eta), norm.data_ptr() if return_norm else None,
                                                  ws.data_ptr(), ws.numel(), *g, 0, _stream(dev)),
                   "adder_b200_backward_weight")
    return (out, norm) if return_norm else out


_side_streams: dict = {}


def _side_stream(dev: torch.device) -> torch.cuda.Stream:
    s = _side_streams.get(dev.index)
    if s is None:
        s = torch.cuda.Stream(device=dev)
        _side_streams[dev.index] = s
    return s


def backward(grad_out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stride: int = 1, padding: int = 0,
             eta: float = ETA, fast_clamp: bool = False, out_w: torch.Tensor | None = None, overlap: bool = True):
    """(grad_x, grad_w rescaled): what adder.backward returns (adder.py:62-80), on NCHW tensors.

    The two gradients are independent.  With `overlap` the weight gradient is enqueued on a side stream
    and the input gradient on the current one, and the current stream then waits for the side stream:
    the kernels fill each other's idle SMs (first and last waves), and under CUDA-graph capture they
    become two parallel branches of the graph.  Results are identical either way."""
    if not overlap:
        return (backward_input(grad_out, x, w, stride, padding, fast_clamp),
                backward_weight(grad_out, x, w, stride, padding, eta, out=out_w))
    dev = x.device
    cur = torch.cuda.current_stream(dev)
    side = _side_stream(dev)
    gw = out_w if out_w is not None else torch.empty_like(w)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        backward_weight(grad_out, x, w, stride, padding, eta, out=gw)
    gx = backward_input(grad_out, x, w, stride, padding, fast_clamp)
    cur.wait_stream(side)
    return gx, gw


def _expect_grad_shape(grad_out, g):
    ho, wo = output_size(g[2], g[3], g[5], g[6], g[7])
    want = (g[0], g[4], ho, wo)
    if tuple(grad_out.shape) != want:
        raise ValueError(f"grad_out has shape {tuple(grad_out.shape)}, expected {want}")


# ---------------------------------------------------------------- reference extension entry points

def _col_dims(x, w, *others):
    if x.dim() != 2 or w.dim() != 2:
        raise ValueError("x must be [K,P] and w [Co,K]")
    K, P = x.shape
    Co, Kw = w.shape
    if Kw != K:
        raise ValueError(f"w has K={Kw}, x has K={K}")
    return K, P, Co


def ADDER_CONV(x, w, y):
    """y[Co,P] <- -sum_k |w[co,k] - x[k,p]| (adder_cuda.cpp:37-46).  Returns None."""
    for t, nm in ((x, "x"), (w, "w"), (y, "y")):
        _check(t, nm)
    dev = _same_device(x, w, y)
    K, P, Co = _col_dims(x, w)
    if tuple(y.shape) != (Co, P):
        raise ValueError(f"y must be [{Co},{P}]")
    with torch.cuda.device(dev):
        _lib.check(_lib.load().adder_b200_conv_col(x.data_ptr(), w.data_ptr(), y.data_ptr(), K, P, Co, _stream(dev)),
                   "adder_b200_conv_col")


def ADDER_CONV_WEIGHT(grad_y, x, w, grad_w):
    """grad_w[Co,K] += sum_p (x - w) * grad_y (adder_cuda.cpp:48-59)."""
    for t, nm in ((grad_y, "grad_y"), (x, "x"), (w, "w"), (grad_w, "grad_w")):
        _check(t, nm)
    dev = _same_device(grad_y, x, w, grad_w)
    K, P, Co = _col_dims(x, w)
    if tuple(grad_y.shape) != (Co, P) or tuple(grad_w.shape) != (Co, K):
        raise ValueError("grad_y must be [Co,P] and grad_w [Co,K]")
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws = _workspace(dev, lib.adder_b200_col_workspace_bytes(K, P, Co))
        _lib.check(lib.adder_b200_conv_weight_col(grad_y.data_ptr(), x.data_ptr(), w.data_ptr(), grad_w.data_ptr(),
                                                  K, P, Co, ws.data_ptr(), ws.numel(), _stream(dev)),
                   "adder_b200_conv_weight_col")


def ADDER_CONV_INPUT(grad_y, x, w, grad_i):
    """grad_i[K,P] += sum_co clamp(w - x, -1, 1) * grad_y (adder_cuda.cpp:61-72)."""
    for t, nm in ((grad_y, "grad_y"), (x, "x"), (w, "w"), (grad_i, "grad_i")):
        _check(t, nm)
    dev = _same_device(grad_y, x, w, grad_i)
    K, P, Co = _col_dims(x, w)
    if tuple(grad_y.shape) != (Co, P) or tuple(grad_i.shape) != (K, P):
        raise ValueError("grad_y must be [Co,P] and grad_i [K,P]")
    with torch.cuda.device(dev):
        _lib.check(_lib.load().adder_b200_conv_input_col(grad_y.data_ptr(), x.data_ptr(), w.data_ptr(),
                                                         grad_i.data_ptr(), K, P, Co, _stream(dev)),
                   "adder_b200_conv_input_col")


def ADDER_BACKWARD(grad_y, x, w, grad_w, grad_i):
    """Both gradient accumulations in one call (adder_cuda.cpp:74-86)."""
    for t, nm in ((grad_y, "grad_y"), (x, "x"), (w, "w"), (grad_w, "grad_w"), (grad_i, "grad_i")):
        _check(t, nm)
    dev = _same_device(grad_y, x, w, grad_w, grad_i)
    K, P, Co = _col_dims(x, w)
    if tuple(grad_y.shape) != (Co, P) or tuple(grad_w.shape) != (Co, K) or tuple(grad_i.shape) != (K, P):
        raise ValueError("grad_y must be [Co,P], grad_w [Co,K] and grad_i [K,P]")
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws = _workspace(dev, lib.adder_b200_col_workspace_bytes(K, P, Co))
        _lib.check(lib.adder_b200_backward_col(grad_y.data_ptr(), x.data_ptr(), w.data_ptr(), grad_w.data_ptr(),
                                               grad_i.data_ptr(), K, P, Co, ws.data_ptr(), ws.numel(), _stream(dev)),
                   "adder_b200_backward_col")
