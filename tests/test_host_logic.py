"""Host-side argument checks mirror the reference's AssertionErrors
(adasplash_v2.py:1248-1276, triton_entmax_v2.py:645)."""
import pytest
import torch

import adasplash_b200 as adasplash


def _qkv(B=1, Hq=2, Hkv=2, N=64, D=32, dtype=torch.float32):
    return (torch.zeros(B, Hq, N, D, dtype=dtype), torch.zeros(B, Hkv, N, D, dtype=dtype),
            torch.zeros(B, Hkv, N, D, dtype=dtype))


@pytest.mark.parametrize("kw", [
    dict(D=48), dict(Hq=3, Hkv=2), dict(N=32), dict(N=96),
])
def test_shape_asserts(kw):
    q, k, v = _qkv(**kw)
    with pytest.raises(AssertionError):
        adasplash.adasplash_v2(q, k, v)


def test_kv_shape_mismatch():
    q, k, v = _qkv()
    with pytest.raises(AssertionError):
        adasplash.adasplash_v2(q, k, v[:, :, :32])


def test_varlen_asserts():
    q, k, v = _qkv(N=96)
    with pytest.raises(AssertionError):
        adasplash.adasplash_v2(q, k, v, varlen=torch.tensor([[96]], dtype=torch.int32))
    with pytest.raises(AssertionError):
        adasplash.adasplash_v2(q, k, v, varlen=torch.tensor([96.0]))
    with pytest.raises(AssertionError):
        adasplash.adasplash_v2(q, k, v, varlen=torch.tensor([96, 96], dtype=torch.int32))


def test_contiguity_and_device_asserts():
    q, k, v = _qkv()
    with pytest.raises(AssertionError):
        adasplash.adasplash_v2(torch.zeros(1, 2, 32, 64).transpose(2, 3), k, v)
    with pytest.raises(AssertionError, match="CUDA"):
        adasplash.adasplash_v2(q, k, v)        # CPU tensors: no CPU path
    with pytest.raises(AssertionError, match="contiguous"):
        adasplash.triton_entmax(torch.zeros(4, 8).t())
    with pytest.raises(AssertionError, match="CUDA"):
        adasplash.triton_entmax(torch.zeros(4, 8))


def test_dispatcher_defaults(monkeypatch):
    calls = {}
    import adasplash_b200.attention as att

    def fake(q, k, v, niter=1, varlen=None):
        calls["niter"] = niter
        return q
    monkeypatch.setattr(att, "sparse_attn", fake)
    q, k, v = _qkv()
    adasplash.adasplash(q, k, v)
    assert calls["niter"] == 1
    adasplash.adasplash(q, k, v, niter=7)
    assert calls["niter"] == 7


def test_entmax_wrapper_rule(monkeypatch):
    # alpha outside {1.5, 2.0}: histogram off, n_iter >= 10 (triton_entmax_v2.py:713-715)
    import adasplash_b200.entmax as em
    seen = {}

    class Fake:
        @staticmethod
        def apply(x, alpha, n_iter, use_histogram, fast_math):
            seen.update(alpha=alpha, n_iter=n_iter, use_histogram=use_histogram)
            return x
    monkeypatch.setattr(em, "_EntmaxFunction", Fake)
    em.triton_entmax(torch.zeros(2, 4), alpha=1.333)
    assert seen == dict(alpha=1.333, n_iter=10, use_histogram=False)
    em.triton_entmax(torch.zeros(2, 4), alpha=2.0)
    assert seen == dict(alpha=2.0, n_iter=2, use_histogram=True)
    em.triton_sparsemax(torch.zeros(2, 4), n_iter=5)
    assert seen == dict(alpha=2.0, n_iter=5, use_histogram=True)
