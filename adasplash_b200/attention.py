"""AdaSplash-2 causal entmax-1.5 sparse attention (host side of the CUDA kernels).

Mirrors `_sparse_attention` / `sparse_attn` of the reference's
adasplash/adasplash_v2.py (:1241-1591): same argument checks (raised as
AssertionError), same saved-tensor tuple (q, k, v, out2, taus, bmask), same
bitmap layout.  All device work goes through the C ABI on the current stream;
nothing here synchronises the host.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

BMASK_TILE = 64


def _ptr(t):
    return None if t is None else t.data_ptr()


def _check_inputs(q, k, v, varlen, require_pow2=True, min_len=BMASK_TILE):
    assert q.dim() == 4, "q must have shape (batch, heads, seq_len, head_dim)"
    B, N_H, N_CTX, H_DIM = q.shape
    assert H_DIM in {16, 32, 64, 128, 256}
    assert k.shape == v.shape, (
        f"K and V must share shape; got k.shape={tuple(k.shape)} v.shape={tuple(v.shape)}")
    N_KV_H = k.shape[1]
    assert N_KV_H >= 1 and N_H % N_KV_H == 0, (
        f"N_H ({N_H}) must be a positive multiple of N_KV_H ({N_KV_H}).")
    assert k.shape[0] == B and k.shape[2] == N_CTX and k.shape[3] == H_DIM, (
        f"K/V must have shape (B={B}, N_KV_H, N_CTX={N_CTX}, H_DIM={H_DIM}); got {tuple(k.shape)}.")
    assert N_CTX >= min_len, f"N_CTX={N_CTX} must be at least {min_len}."
    if varlen is None:
        assert not require_pow2 or (N_CTX & (N_CTX - 1)) == 0, "If varlen is None, N_CTX must be a power of two."
    else:
        assert varlen.dim() == 1 and varlen.shape[0] == B, (
            f"varlen must be a 1-D tensor of shape (B={B},); got {tuple(varlen.shape)}.")
        assert varlen.dtype in (torch.int32, torch.int64), (
            f"varlen must be int32/int64; got {varlen.dtype}.")
        assert varlen.device == q.device, "varlen must be on the same device as q."
        assert varlen.is_contiguous(), "varlen must be contiguous."
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous(), (
        "Q, K and/or V are not contiguous.")
    assert q.dtype == k.dtype == v.dtype, "q, k and v must share a dtype"
    assert q.is_cuda and k.device == q.device and v.device == q.device, (
        "q, k and v must be CUDA tensors on one device (there is no CPU path)")


def make_shape(q, k, niter, varlen, path=None, alpha=1.5, is_causal=True):
    B, Hq, N, D = q.shape
    return _lib.AttnShape(
        B=B, Hq=Hq, Hkv=k.shape[1], N=N, D=D, dtype=_lib.dtype_code(q.dtype), niter=int(niter),
        varlen_is_i64=int(varlen is not None and varlen.dtype == torch.int64),
        path=_lib.kernel_path() if path is None else path,
        alpha=float(alpha), non_causal=int(not is_causal))


def bitmap_extent(shape):
    rows, words = ctypes.c_int32(), ctypes.c_int32()
    _lib.load().adasplash2_bitmap_words(ctypes.byref(shape), ctypes.byref(rows), ctypes.byref(words))
    return rows.value, words.value


def _workspace(shape, device, full=False):
    """Scratch of one call: the 256-byte status word; `full` (a backward with a support buffer)
    adds the room for its key-sorted copy of the supports."""
    nbytes = int(_lib.load().adasplash2_workspace_bytes(ctypes.byref(shape)))
    if nbytes == 0:
        _lib.check(_lib.load().adasplash2_resolved_path(ctypes.byref(shape)) < 0)
    if not full:
        nbytes = min(nbytes, 256)
    return torch.empty(max(nbytes, 256), device=device, dtype=torch.uint8), nbytes


ROW_SUPPORTS = True   # let the solver export the rows' supports, so that sparse heads run as gathers
ROW_SUPPORTS_MIN_N = 1024  # the autograd Function asks for supports from this sequence length on:
#                            below it a step is a few tiles per head and the extra launches cost more


def support_buffer(shape, device):
    """Buffer for the rows' supports of one problem (None where the library has no such route)."""
    nbytes = int(_lib.load().adasplash2_support_bytes(ctypes.byref(shape)))
    if nbytes == 0 or not ROW_SUPPORTS:
        return None
    return torch.empty(nbytes, device=device, dtype=torch.uint8)


def _sup_args(support):
    return (None, 0) if support is None else (support.data_ptr(), support.numel())


DEBUG_STATUS = False  # tests set this: check the device status word after every call (synchronises)


def _maybe_check(ws, st):
    if DEBUG_STATUS:
        _lib.check(_lib.load().adasplash2_check_status(_ptr(ws), st))


def solve(q, k, niter=1, varlen=None, path=None, alpha=1.5, is_causal=True, support=None):
    """Thresholds and block mask only: (taus (B,Hq,N) fp32, bmask int32).  `support`: a buffer
    from `support_buffer` that receives the rows' supports."""
    lib = _lib.load()
    shape = make_shape(q, k, niter, varlen, path, alpha, is_causal)
    rows, words = bitmap_extent(shape)
    B, Hq, N, _ = q.shape
    taus = torch.empty((B, Hq, N), device=q.device, dtype=torch.float32)
    bmask = torch.empty((B, Hq, rows, words), device=q.device, dtype=torch.int32)
    with torch.cuda.device(q.device):
        ws, nbytes = _workspace(shape, q.device)
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.adasplash2_solve(_ptr(q), _ptr(k), _ptr(varlen), _ptr(taus), _ptr(bmask),
                                        ctypes.byref(shape), _ptr(ws), nbytes, *_sup_args(support), st))
        _maybe_check(ws, st)
    return taus, bmask


def mask_from_tau(q, k, taus, varlen=None, path=None):
    """Block mask for caller-supplied thresholds (bit = any(z > tau) per 64x64 tile)."""
    lib = _lib.load()
    shape = make_shape(q, k, 0, varlen, path)
    rows, words = bitmap_extent(shape)
    B, Hq, N, _ = q.shape
    assert taus.shape == (B, Hq, N) and taus.dtype == torch.float32 and taus.is_contiguous()
    bmask = torch.empty((B, Hq, rows, words), device=q.device, dtype=torch.int32)
    with torch.cuda.device(q.device):
        ws, nbytes = _workspace(shape, q.device)
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.adasplash2_mask_from_tau(_ptr(q), _ptr(k), _ptr(varlen), _ptr(taus),
                                                _ptr(bmask), ctypes.byref(shape), _ptr(ws),
                                                nbytes, st))
        _maybe_check(ws, st)
    return bmask


class _SparseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, niter=10, varlen=None):
        _check_inputs(q, k, v, varlen)
        lib = _lib.load()
        shape = make_shape(q, k, niter, varlen)
        rows, words = bitmap_extent(shape)
        B, Hq, N, _ = q.shape
        dev = q.device
        taus = torch.empty((B, Hq, N), device=dev, dtype=torch.float32)
        bmask = torch.empty((B, Hq, rows, words), device=dev, dtype=torch.int32)
        out = torch.empty_like(q)
        out2 = torch.empty_like(q)
        with torch.cuda.device(dev):
            ws, nbytes = _workspace(shape, dev)
            support = support_buffer(shape, dev) if N >= ROW_SUPPORTS_MIN_N else None
            st = torch.cuda.current_stream().cuda_stream
            sp = ctypes.byref(shape)
            _lib.check(lib.adasplash2_solve(_ptr(q), _ptr(k), _ptr(varlen), _ptr(taus),
                                            _ptr(bmask), sp, _ptr(ws), nbytes, *_sup_args(support), st))
            _maybe_check(ws, st)
            _lib.check(lib.adasplash2_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(varlen), _ptr(taus),
                                          _ptr(bmask), _ptr(out), _ptr(out2), sp, _ptr(ws),
                                          nbytes, *_sup_args(support), st))
            _maybe_check(ws, st)
        ctx.save_for_backward(q, k, v, out2, taus, bmask)
        ctx.support = support
        ctx.varlen = varlen
        ctx.niter = niter
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out2, taus, bmask = ctx.saved_tensors
        do = do.contiguous()
        if do.dtype != q.dtype:
            do = do.to(q.dtype)
        dq, dk, dv, _, _ = backward_raw(q, k, v, do, out2, taus, bmask, ctx.varlen, ctx.niter,
                                        support=ctx.support)
        return dq, dk, dv, None, None


def forward_raw(q, k, v, taus, bmask, varlen=None, path=None, alpha=1.5, is_causal=True, support=None):
    """`adasplash2_fwd` alone for given thresholds and block mask: (out, out2).  `support`: the
    buffer a `solve` of the same problem filled."""
    lib = _lib.load()
    shape = make_shape(q, k, 0, varlen, path, alpha, is_causal)
    out = torch.empty_like(q)
    out2 = torch.empty_like(q)
    with torch.cuda.device(q.device):
        ws, nbytes = _workspace(shape, q.device)
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.adasplash2_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(varlen), _ptr(taus),
                                      _ptr(bmask), _ptr(out), _ptr(out2), ctypes.byref(shape),
                                      _ptr(ws), nbytes, *_sup_args(support), st))
        _maybe_check(ws, st)
    return out, out2


def backward_raw(q, k, v, do, out2, taus, bmask, varlen=None, niter=1, stages=0, buffers=None,
                 path=None, alpha=1.5, is_causal=True, support=None):
    """`adasplash2_bwd`: returns (dq, dk, dv, delta, bmask_t).  `stages` != 0 runs only
    the named kernels (ADS_BWD_* mask; a measurement aid), reusing `buffers` =
    (dq, dk, dv, delta, bmask_t) from an earlier full call."""
    lib = _lib.load()
    shape = make_shape(q, k, niter, varlen, path, alpha, is_causal)
    shape.bwd_stages = int(stages)
    dev = q.device
    if buffers is None:
        buffers = (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v),
                   torch.empty(taus.shape, device=dev, dtype=torch.float32), torch.empty_like(bmask))
    dq, dk, dv, delta, bmask_t = buffers
    with torch.cuda.device(dev):
        ws, nbytes = _workspace(shape, dev, full=support is not None)
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.adasplash2_bwd(_ptr(q), _ptr(k), _ptr(v), _ptr(do), _ptr(out2),
                                      _ptr(varlen), _ptr(taus), _ptr(bmask), _ptr(bmask_t),
                                      _ptr(delta), _ptr(dq), _ptr(dk), _ptr(dv),
                                      ctypes.byref(shape), _ptr(ws), nbytes, *_sup_args(support), st))
        _maybe_check(ws, st)
    return dq, dk, dv, delta, bmask_t


def sparse_attn(q, k, v, niter=1, varlen=None):
    """Causal entmax-1.5 sparse attention with GQA and right-padded varlen.

    q (batch, n_heads, seq_len, head_dim); k, v (batch, n_kv_heads, seq_len,
    head_dim) with n_heads % n_kv_heads == 0.  `niter` = refinements after the
    histogram start.  `varlen` (batch,) int32/int64 = valid length per batch
    item; padded output rows are zero.  Returns a tensor like q.
    """
    return _SparseAttention.apply(q, k, v, niter, varlen)
