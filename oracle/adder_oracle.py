"""CPU oracle for the adder-convolution hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, what LingYeAI/AdderNetCUDA computes for one
adder2d layer.  It is the checker for the CUDA kernels; only the tests, the
smoke check and the CPU-baseline leg of the benchmark may import it.  The
product package never does, and it has no CPU fallback.

Parity is PINNED: `tests/golden/make_golden.py` imports the reference's own
`adder.py` (unchanged) behind the CPU stand-in for its extension that lives in
`oracle/adder_cuda_cpu.py`, checks that every function here reproduces it, and
stores the reference's outputs as fixtures under `tests/golden/`.

Two independent restatements are kept on purpose:

* the *column* forms (`*_col`) are the three closed-form expressions the
  reference itself uses as ground truth (adder_cuda/test_cuda.py:21, :39-40,
  :58-59; repeated in adder.py:55, :70, :74), evaluated in chunks so the
  [Co, K, P] temporary stays small, plus the adaptive-eta rescale of
  adder.py:78 and the unfold/permute layout contract of adder.py:32-33,38-39;
* the *direct* forms (`*_direct`) evaluate the same sums on NCHW tensors by
  looping over (kh, kw) taps, without any im2col matrix, in float64.  They do
  not share code with the column forms, so a layout mistake in one shows up as
  a disagreement with the other.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

ETA = 0.2  # adder.py:78 divides by 5


# --------------------------------------------------------------------------
# column forms (layout of the reference extension: W_col[Co,K], X_col[K,P])
# --------------------------------------------------------------------------

def _chunk(P: int, Co: int, K: int, budget_elems: int = 1 << 26) -> int:
    return max(1, min(P, budget_elems // max(1, Co * K)))


def forward_col(W_col: torch.Tensor, X_col: torch.Tensor) -> torch.Tensor:
    """Y[co,p] = -sum_k |W[co,k] - X[k,p]|   (adder_cuda/test_cuda.py:21, adder.py:55)."""
    Co, K = W_col.shape
    P = X_col.shape[1]
    out = torch.empty((Co, P), dtype=W_col.dtype)
    step = _chunk(P, Co, K)
    for p0 in range(0, P, step):
        xs = X_col[:, p0:p0 + step]
        out[:, p0:p0 + step] = -(W_col.unsqueeze(2) - xs.unsqueeze(0)).abs().sum(1)
    return out


def grad_w_col(W_col: torch.Tensor, X_col: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """gW[co,k] = sum_p (X[k,p] - W[co,k]) * g[co,p]   (test_cuda.py:39-40, adder.py:70). Unscaled."""
    Co, K = W_col.shape
    P = X_col.shape[1]
    acc = torch.zeros((Co, K), dtype=W_col.dtype)
    step = _chunk(P, Co, K)
    for p0 in range(0, P, step):
        xs = X_col[:, p0:p0 + step]
        gs = g[:, p0:p0 + step]
        acc += ((xs.unsqueeze(0) - W_col.unsqueeze(2)) * gs.unsqueeze(1)).sum(2)
    return acc


def grad_x_col(W_col: torch.Tensor, X_col: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """gX[k,p] = sum_co clamp(W[co,k] - X[k,p], -1, 1) * g[co,p]   (test_cuda.py:58-59, adder.py:74)."""
    Co, K = W_col.shape
    P = X_col.shape[1]
    out = torch.empty((K, P), dtype=W_col.dtype)
    step = _chunk(P, Co, K)
    for p0 in range(0, P, step):
        xs = X_col[:, p0:p0 + step]
        gs = g[:, p0:p0 + step]
        out[:, p0:p0 + step] = (-(xs.unsqueeze(0) - W_col.unsqueeze(2)).clamp(-1, 1)
                                * gs.unsqueeze(1)).sum(0)
    return out


def rescale(grad_W_col: torch.Tensor, eta: float = ETA) -> torch.Tensor:
    """Adaptive learning-rate scaling: eta * sqrt(numel) * gW / max(||gW||_2, 1e-12)   (adder.py:78)."""
    k = grad_W_col.numel()
    # same operation order as the reference line: g / norm * sqrt(k) / 5   (1 / 0.2 == 5.0 exactly)
    return grad_W_col / grad_W_col.norm(p=2).clamp(min=1e-12) * math.sqrt(k) / (1.0 / eta)


def out_hw(h: int, w: int, k: int, stride: int, padding: int) -> tuple[int, int]:
    """Output size with the reference's int() truncation (adder.py:26-31)."""
    return int((h - k + 2 * padding) / stride + 1), int((w - k + 2 * padding) / stride + 1)


def im2col(X: torch.Tensor, k: int, stride: int, padding: int) -> torch.Tensor:
    """X[N,Ci,H,W] -> X_col[Ci*k*k, Ho*Wo*N]; row = ci*k*k + kh*k + kw, column = (ho*Wo+wo)*N + n
    (adder.py:32-33)."""
    n, c, h, w = X.shape
    ho, wo = out_hw(h, w, k, stride, padding)
    cols = F.unfold(X.reshape(1, -1, h, w), k, dilation=1, padding=padding, stride=stride)
    cols = cols.view(n, -1, ho * wo)
    return cols.permute(1, 2, 0).contiguous().view(cols.size(1), -1)


def col2im(gX_col: torch.Tensor, x_shape, k: int, stride: int, padding: int) -> torch.Tensor:
    """Adjoint of `im2col` (what autograd does for adder.py:32-33): overlapping taps add up,
    taps that fall into the zero padding are dropped."""
    n, c, h, w = x_shape
    ho, wo = out_hw(h, w, k, stride, padding)
    t = gX_col.view(c * k * k, ho * wo, n).permute(2, 0, 1).contiguous()       # [N, K, L]
    t = t.view(1, n * c * k * k, ho * wo)
    img = F.fold(t, (h, w), k, dilation=1, padding=padding, stride=stride)        # [1, N*Ci, H, W]
    return img.view(n, c, h, w)


def cols_to_nchw(Y: torch.Tensor, n: int, co: int, ho: int, wo: int) -> torch.Tensor:
    """[Co, Ho*Wo*N] -> [N,Co,Ho,Wo]   (adder.py:38-39)."""
    return Y.view(co, ho, wo, n).permute(3, 0, 1, 2).contiguous()


def nchw_to_cols(G: torch.Tensor) -> torch.Tensor:
    """[N,Co,Ho,Wo] -> [Co, Ho*Wo*N]: the adjoint of `cols_to_nchw`."""
    n, co, ho, wo = G.shape
    return G.permute(1, 2, 3, 0).contiguous().view(co, -1)


def adder2d_forward_unfold(X: torch.Tensor, W: torch.Tensor, stride: int = 1, padding: int = 0) -> torch.Tensor:
    """The reference's forward path end to end (adder.py:22-41) on NCHW tensors."""
    co, ci, k, _ = W.shape
    n, _, h, w = X.shape
    ho, wo = out_hw(h, w, k, stride, padding)
    Y = forward_col(W.reshape(co, -1), im2col(X, k, stride, padding))
    return cols_to_nchw(Y, n, co, ho, wo)


def adder2d_backward_unfold(G: torch.Tensor, X: torch.Tensor, W: torch.Tensor, stride: int = 1,
                            padding: int = 0, eta: float = ETA):
    """The reference's backward path end to end (adder.py:62-80 plus the autograd adjoints of
    :32-33 and :38-39).  Returns (grad_x[N,Ci,H,W], grad_w[Co,Ci,k,k] rescaled, grad_w unscaled)."""
    co, ci, k, _ = W.shape
    W_col = W.reshape(co, -1)
    X_col = im2col(X, k, stride, padding)
    g = nchw_to_cols(G)
    gw = grad_w_col(W_col, X_col, g)
    gx = col2im(grad_x_col(W_col, X_col, g), X.shape, k, stride, padding)
    return gx, rescale(gw, eta).view_as(W), gw.view_as(W)


# --------------------------------------------------------------------------
# direct forms (NCHW, no im2col, float64): the independent second opinion
# --------------------------------------------------------------------------

def _taps(X: torch.Tensor, k: int, stride: int, padding: int, ho: int, wo: int):
    """Yield (kh, kw, window) where window[n,ci,i,j] = Xpad[n,ci,i*stride+kh,j*stride+kw]."""
    Xp = F.pad(X, (padding, padding, padding, padding))
    for kh in range(k):
        for kw in range(k):
            yield kh, kw, Xp[:, :, kh:kh + (ho - 1) * stride + 1:stride, kw:kw + (wo - 1) * stride + 1:stride]


def adder2d_forward_direct(X: torch.Tensor, W: torch.Tensor, stride: int = 1, padding: int = 0,
                           dtype=torch.float64) -> torch.Tensor:
    """out[n,co,i,j] = -sum_{ci,kh,kw} |x_pad[n,ci,i*s+kh,j*s+kw] - w[co,ci,kh,kw]|, padding counted
    as zero-valued inputs (what F.unfold feeds the reference kernel, adder.py:32)."""
    X = X.to(dtype)
    W = W.to(dtype)
    co, ci, k, _ = W.shape
    n, _, h, w = X.shape
    ho, wo = out_hw(h, w, k, stride, padding)
    out = torch.zeros((n, co, ho, wo), dtype=dtype)
    for kh, kw, win in _taps(X, k, stride, padding, ho, wo):
        for c in range(ci):
            # [n,1,ho,wo] - [1,co,1,1]
            out -= (win[:, c:c + 1] - W[None, :, c, kh, kw, None, None]).abs()
    return out


def adder2d_backward_direct(G: torch.Tensor, X: torch.Tensor, W: torch.Tensor, stride: int = 1,
                            padding: int = 0, eta: float = ETA, dtype=torch.float64):
    """grad_x[n,ci,y,x] = sum over the taps that read that pixel of clamp(w - x, -1, 1) * g;
    grad_w[co,ci,kh,kw] = sum_{n,i,j} (x_pad - w) * g  (padding contributes (0 - w) * g);
    then the rescale of adder.py:78.  Returns (grad_x, grad_w rescaled, grad_w unscaled)."""
    X = X.to(dtype)
    W = W.to(dtype)
    G = G.to(dtype)
    co, ci, k, _ = W.shape
    n, _, h, w = X.shape
    ho, wo = out_hw(h, w, k, stride, padding)
    gw = torch.zeros_like(W)
    gxp = torch.zeros((n, ci, h + 2 * padding, w + 2 * padding), dtype=dtype)
    for kh, kw, win in _taps(X, k, stride, padding, ho, wo):
        for o in range(co):
            d = win - W[o, :, kh, kw].view(1, ci, 1, 1)            # x - w   [n,ci,ho,wo]
            go = G[:, o:o + 1]                                      # [n,1,ho,wo]
            gw[o, :, kh, kw] += (d * go).sum(dim=(0, 2, 3))
            gxp[:, :, kh:kh + (ho - 1) * stride + 1:stride,
                kw:kw + (wo - 1) * stride + 1:stride] += (-d).clamp(-1, 1) * go
    gx = gxp[:, :, padding:padding + h, padding:padding + w].contiguous()
    return gx, rescale(gw, eta), gw


# --------------------------------------------------------------------------
# tolerance rule shared by every parity test
# --------------------------------------------------------------------------

REL_TOL = 1e-5
ABS_TOL = 1e-4


def adder2d_general(G, X, W, stride=1, padding=0, dilation=1, eta: float = ETA):
    """Float64 layer for ANY kernel extent, stride, padding and dilation: (out, grad_x, rescaled grad_w).
    The same three expressions as the column op (adder.py:58, :70-74, :76-78) on an explicit im2col
    (adder.py:32-33 generalised by F.unfold's kernel-size / dilation arguments), col2im by F.fold.
    G may be None (forward only).  Small cases only: materialises [N, Co, K, L]."""
    F = torch.nn.functional
    X64, W64 = X.double(), W.double()
    n, co = X.shape[0], W.shape[0]
    ksz = (W.shape[2], W.shape[3])
    cols = F.unfold(X64, ksz, dilation=dilation, padding=padding, stride=stride)           # [N, K, L]
    D = cols.unsqueeze(1) - W64.reshape(1, co, -1, 1)                                       # x - w, [N, Co, K, L]
    out_cols = -D.abs().sum(2)                                                              # [N, Co, L]
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)
    (sh, _), (ph, _), (dh, _) = pair(stride), pair(padding), pair(dilation)
    ho = (X.shape[2] + 2 * ph - dh * (ksz[0] - 1) - 1) // sh + 1
    out = out_cols.reshape(n, co, ho, -1)
    if G is None:
        return out, None, None
    g = G.double().reshape(n, co, 1, -1)
    gw = (D * g).sum((0, 3)).reshape(W.shape)
    gw = gw / gw.norm(p=2).clamp(min=1e-12) * math.sqrt(W.numel()) * eta
    gx_cols = ((-D).clamp(-1.0, 1.0) * g).sum(1)                                            # [N, K, L]
    gx = F.fold(gx_cols, (X.shape[2], X.shape[3]), ksz, dilation=dilation, padding=padding, stride=stride)
    return out, gx, gw


def compare(name: str, got: torch.Tensor, want: torch.Tensor, rel: float = REL_TOL, abs_: float = ABS_TOL):
    """Return (ok, max_abs_err, report) under |got - want| <= abs + rel * |want|."""
    got = got.detach().to("cpu", torch.float64)
    want = want.detach().to("cpu", torch.float64)
    if got.shape != want.shape:
        return False, float("inf"), f"{name}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    if got.numel() == 0:
        return True, 0.0, f"{name}: empty"
    err = (got - want).abs()
    bound = abs_ + rel * want.abs()
    ok = bool((err <= bound).all()) and bool(torch.isfinite(got).all())
    worst = float(err.max())
    return ok, worst, f"{name}: max_abs_err={worst:.3e} (max |want|={float(want.abs().max()):.3e}) {'ok' if ok else 'FAIL'}"
