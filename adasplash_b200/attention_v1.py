"""v1 semantics (any alpha in (1, 2], causal or not, no GQA) of
adasplash/adasplash_block_mask.py:1213-1232.

Not built yet: the CUDA kernels of this package cover the causal alpha = 1.5
path.  Calls fail loudly instead of falling back to another implementation.
"""


def sparse_attn(q, k, v, alpha=1.5, is_causal=False, varlen=None, niter=10):
    if alpha == 1.5 and is_causal:
        from .attention import sparse_attn as v2

        assert k.shape[1] == q.shape[1], "adasplash_v1 does not support grouped-query attention"
        return v2(q, k, v, niter=niter, varlen=varlen)
    raise NotImplementedError(
        "adasplash_b200 implements causal alpha=1.5 attention; "
        f"alpha={alpha}, is_causal={is_causal} is not available")
