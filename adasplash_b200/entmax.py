"""Row-wise entmax over the last dimension (host side of the CUDA kernels).

Mirrors the interface of the reference's adasplash/triton_entmax_v2.py:
`triton_entmax` (:690-716), `triton_sparsemax` (:724-726), `triton_entmax15`
(:729-731) and the autograd wrapper `_entmax_triton` (:620-687).
"""
from __future__ import annotations

import torch

from . import _lib


def _ptr(t):
    return None if t is None else t.data_ptr()


class _EntmaxFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, alpha=1.5, n_iter=10, use_histogram=True, fast_math=False):
        assert x.is_contiguous(), "x must be contiguous"
        assert x.is_cuda, "x must be a CUDA tensor (there is no CPU path)"
        lib = _lib.load()
        cols = x.shape[-1] if x.dim() > 0 else 1
        rows = x.numel() // cols if cols > 0 else 0
        y = torch.empty_like(x)
        with torch.cuda.device(x.device):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.adasplash_entmax_fwd(
                _ptr(x), _ptr(y), None, rows, cols, float(alpha), int(n_iter),
                int(bool(use_histogram)), int(bool(fast_math)), _lib.dtype_code(x.dtype), st))
        ctx.save_for_backward(y)
        ctx.alpha = float(alpha)
        ctx.fast_math = bool(fast_math)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        if not dy.is_contiguous():
            dy = dy.contiguous()
        if dy.dtype != y.dtype:
            dy = dy.to(y.dtype)
        lib = _lib.load()
        cols = y.shape[-1] if y.dim() > 0 else 1
        rows = y.numel() // cols if cols > 0 else 0
        dx = torch.empty_like(y)
        with torch.cuda.device(y.device):
            st = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.adasplash_entmax_bwd(
                _ptr(y), _ptr(dy), _ptr(dx), rows, cols, ctx.alpha, int(ctx.fast_math),
                _lib.dtype_code(y.dtype), st))
        return dx, None, None, None, None


def triton_entmax(x, alpha=1.5, n_iter=2, use_histogram=True, fast_math=False):
    """alpha-entmax over the last dim.  alpha outside {1.5, 2.0} disables the
    histogram start and uses at least 10 refinements (triton_entmax_v2.py:713-715)."""
    if alpha not in (1.5, 2.0):
        use_histogram = False
        n_iter = max(n_iter, 10)
    return _EntmaxFunction.apply(x, alpha, n_iter, use_histogram, fast_math)


def triton_sparsemax(x, **kwargs):
    return triton_entmax(x, alpha=2.0, **kwargs)


def triton_entmax15(x, **kwargs):
    return triton_entmax(x, alpha=1.5, **kwargs)


def entmax_with_tau(x, alpha=1.5, n_iter=2, use_histogram=True, fast_math=False):
    """Forward only; also returns the per-row threshold (fp32).  Test hook."""
    assert x.is_contiguous() and x.is_cuda
    if alpha not in (1.5, 2.0):
        use_histogram = False
        n_iter = max(n_iter, 10)
    lib = _lib.load()
    cols = x.shape[-1]
    rows = x.numel() // cols
    y = torch.empty_like(x)
    tau = torch.empty(x.shape[:-1], device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.adasplash_entmax_fwd(
            _ptr(x), _ptr(y), _ptr(tau), rows, cols, float(alpha), int(n_iter),
            int(bool(use_histogram)), int(bool(fast_math)), _lib.dtype_code(x.dtype), st))
    return y, tau
