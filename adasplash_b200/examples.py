"""Dense entmax attention helper and the one-line flash wrapper of the reference's examples.

Mirrors examples/attention.py of deep-spin/adasplash: `slow_entmax_attention` (:34-91) builds
the full score matrix with torch, applies ALiBi (:17-31), the causal mask and left- or
right-padded lengths (:8-14), runs this library's row-wise `triton_entmax` on it and multiplies
by v; `flash_entmax_attention` (:94-96) forwards to the `adasplash` dispatcher.  The dense
helper exists for examples and small checks: it materialises (B, H, Nq, Nk) scores.
"""
from __future__ import annotations

import math

import torch


def _length_mask(varlen, size, padding):
    """(B, size) bool: True on the valid positions of each sequence."""
    pos = torch.arange(size, device=varlen.device).unsqueeze(0)
    n = varlen.unsqueeze(1)
    if padding == "right":
        return pos < n
    if padding == "left":
        return pos >= (size - n)
    raise ValueError("padding must be either 'right' or 'left'.")


def _alibi(n_heads, q_len, k_len, slopes, device):
    """slopes[h] * (key position - query position); a single query is the last position."""
    if slopes.shape != (n_heads,):
        raise ValueError(f"alibi_slopes must have shape ({n_heads},); got {tuple(slopes.shape)}.")
    kpos = torch.arange(k_len, device=device)
    if q_len == 1 and k_len > 1:
        rel = (kpos - (k_len - 1)).view(1, 1, 1, k_len)
    else:
        qpos = torch.arange(q_len, device=device)
        rel = (kpos.unsqueeze(0) - qpos.unsqueeze(1)).view(1, 1, q_len, k_len)
    return slopes.to(device).view(1, n_heads, 1, 1) * rel


def slow_entmax_attention(q, k, v, alpha=1.5, varlen=None, is_causal=False, padding="right",
                          niter=2, alibi_slopes=None):
    """Dense alpha-entmax attention from `triton_entmax`; differentiable through torch autograd.

    q (B, H, Nq, D); k, v (B, H, Nk, D).  `varlen` (B,) masks keys outside each sequence
    (`padding` = 'right' or 'left'); when Nq == Nk the padded query rows get score 0 before the
    entmax (so that no row is empty) and their output rows are zeroed.
    """
    for t in (q, k, v):
        if t.dim() != 4:
            raise ValueError("q, k and v must have shape (batch, heads, seq_len, head_dim).")
    if k.shape != v.shape:
        raise ValueError(f"k and v must have the same shape; got {tuple(k.shape)} and {tuple(v.shape)}.")
    if (q.shape[0], q.shape[1], q.shape[3]) != (k.shape[0], k.shape[1], k.shape[3]):
        raise ValueError("q, k and v must agree on batch, heads and head_dim.")
    B, H, q_len, D = q.shape
    k_len = k.shape[2]
    scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(D)
    if alibi_slopes is not None:
        scores = scores + _alibi(H, q_len, k_len, alibi_slopes, q.device)
    neg = float("-inf")
    if is_causal:
        # query i sits at key position i + (Nk - Nq)
        qpos = torch.arange(q_len, device=q.device) + (k_len - q_len)
        visible = qpos.unsqueeze(1) >= torch.arange(k_len, device=q.device).unsqueeze(0)
        scores = scores.masked_fill(~visible.view(1, 1, q_len, k_len), neg)
    rows_valid = None
    if varlen is not None:
        if varlen.dim() != 1 or varlen.shape[0] != B:
            raise ValueError(f"varlen must be a 1-D tensor of shape ({B},).")
        lens = varlen.to(q.device)
        scores = scores.masked_fill(~_length_mask(lens, k_len, padding)[:, None, None, :], neg)
        if q_len == k_len:
            rows_valid = _length_mask(lens, q_len, padding)[:, None, :, None]
            scores = scores.masked_fill(~rows_valid, 0.0)
    from .entmax import triton_entmax

    probs = triton_entmax(scores.contiguous(), alpha=alpha, n_iter=niter, fast_math=False)
    out = torch.matmul(probs, v)
    if rows_valid is not None:
        out = out.masked_fill(~rows_valid, 0)
    return out


def flash_entmax_attention(q, k, v, alpha=1.5, varlen=None, is_causal=True, niter=None):
    """The fused path: the `adasplash` dispatcher."""
    from . import adasplash

    return adasplash(q, k, v, alpha=alpha, is_causal=is_causal, varlen=varlen, niter=niter)
