"""First-generation AdaSplash semantics: any alpha in (1, 2], causal or full attention,
right-padded varlen, no grouped-query heads.

Mirrors `sparse_attn(q, k, v, alpha, is_causal, varlen, niter)` of the reference's
adasplash/adasplash_block_mask.py (:938-1232).  The reference runs its own 16x16-tile
Triton kernels for this; here the same entry points of the CUDA library are used as for
AdaSplash-2, with `alpha` / `non_causal` set in the shape: threshold by Halley steps with
bisection fallback on [max-1, max-n^(1-alpha)] (:170-176), 64x64 block mask taken at the
lower end of the final bracket, p = [(alpha-1)s - tau]_+^(1/(alpha-1)), backward through
the entmax Jacobian with weights p^(2-alpha).  Causal alpha = 1.5 calls take the AdaSplash-2
kernels.
"""
from __future__ import annotations

import torch

from . import attention as att


class _SparseAttentionV1(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, alpha=1.5, is_causal=False, varlen=None, niter=10):
        att._check_inputs(q, k, v, varlen, require_pow2=False, min_len=1)   # the v1 kernels take any length
        assert k.shape[1] == q.shape[1], "adasplash_v1 does not support grouped-query attention"
        assert 1.0 < alpha <= 2.0, f"alpha must be in (1, 2]; got {alpha}"
        support = None
        if q.shape[2] >= att.ROW_SUPPORTS_MIN_N:
            # rows' supports from the solver: sparse heads run as gathers (see attention.py)
            with torch.cuda.device(q.device):
                support = att.support_buffer(att.make_shape(q, k, niter, varlen, None, alpha, is_causal), q.device)
        taus, bmask = att.solve(q, k, niter, varlen, None, alpha, is_causal, support=support)
        out, out2 = att.forward_raw(q, k, v, taus, bmask, varlen, None, alpha, is_causal, support=support)
        ctx.save_for_backward(q, k, v, out2, taus, bmask)
        ctx.support = support
        ctx.args = (alpha, is_causal, varlen, niter)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out2, taus, bmask = ctx.saved_tensors
        alpha, is_causal, varlen, niter = ctx.args
        do = do.contiguous()
        if do.dtype != q.dtype:
            do = do.to(q.dtype)
        dq, dk, dv, _, _ = att.backward_raw(q, k, v, do, out2, taus, bmask, varlen, niter,
                                            alpha=alpha, is_causal=is_causal, support=ctx.support)
        return dq, dk, dv, None, None, None, None


def sparse_attn(q, k, v, alpha=1.5, is_causal=False, varlen=None, niter=10):
    """alpha-entmax attention; q, k, v (batch, heads, seq_len, head_dim); `varlen` (batch,)
    valid lengths (padded output rows are zero); `niter` solver iterations."""
    return _SparseAttentionV1.apply(q, k, v, alpha, is_causal, varlen, niter)
