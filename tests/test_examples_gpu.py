"""The example helpers (`slow_entmax_attention`, `flash_entmax_attention`) against the exact
definition.  Cases and tolerances follow the reference's tests/test_attention.py:50-107: one
sequence of 64 positions with 48 valid, ALiBi slopes (0.1, 0.2), left and right padding, causal
and full attention; forward 1e-4, gradients 1e-3 (fp32, niter = 10)."""
import math

import pytest
import torch

from adasplash_b200.examples import flash_entmax_attention, slow_entmax_attention
from oracle import entmax_oracle as O

pytestmark = pytest.mark.gpu


def _randn(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g)


def _valid(varlen, size, padding):
    pos = torch.arange(size)[None, :]
    return pos < varlen[:, None] if padding == "right" else pos >= size - varlen[:, None]


def _exact(q, k, v, do, alpha, varlen, is_causal, padding, slopes):
    """Dense fp64 attention with tau by bisection and the analytic entmax Jacobian."""
    q, k, v, do = (t.double() for t in (q, k, v, do))
    B, H, N, D = q.shape
    s = q @ k.transpose(-1, -2) / math.sqrt(D)
    if slopes is not None:
        rel = (torch.arange(N)[None, :] - torch.arange(N)[:, None]).double()
        s = s + slopes.double().view(1, H, 1, 1) * rel
    if is_causal:
        s = s.masked_fill(~torch.ones(N, N, dtype=torch.bool).tril(), float("-inf"))
    rows = torch.ones(B, 1, N, 1, dtype=torch.bool)
    if varlen is not None:
        s = s.masked_fill(~_valid(varlen, N, padding)[:, None, None, :], float("-inf"))
        rows = _valid(varlen, N, padding)[:, None, :, None]
        s = s.masked_fill(~rows, 0.0)
    p, _ = O.entmax_bisect_exact(s, alpha)
    out = (p @ v) * rows
    do = do * rows
    ds = O.entmax_backward_exact(p, do @ v.transpose(-1, -2), alpha) * rows
    return out, ds @ k / math.sqrt(D), ds.transpose(-1, -2) @ q / math.sqrt(D), p.transpose(-1, -2) @ do


@pytest.mark.parametrize("padding", ["left", "right"])
@pytest.mark.parametrize("is_causal", [False, True])
@pytest.mark.parametrize("alpha", [1.5, 2.0])
def test_slow_entmax_attention_matches_exact_definition(padding, is_causal, alpha):
    q, k, v, do = (_randn((1, 2, 64, 32), 60 + i) for i in range(4))
    varlen = torch.tensor([48], dtype=torch.int32)
    slopes = torch.tensor([0.1, 0.2])
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = slow_entmax_attention(qc, kc, vc, alpha=alpha, varlen=varlen.cuda(), is_causal=is_causal,
                                padding=padding, niter=10, alibi_slopes=slopes.cuda())
    dq, dk, dv = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
    ref = _exact(q, k, v, do, alpha, varlen, is_causal, padding, slopes)
    assert (out.detach().cpu().double() - ref[0]).abs().max() < 1e-4
    for got, want, name in zip((dq, dk, dv), ref[1:], ("dq", "dk", "dv")):
        assert (got.cpu().double() - want).abs().max() < 1e-3, name
    invalid = ~_valid(varlen, 64, padding)[0]
    assert out.detach().cpu()[0, :, invalid].abs().max() == 0


def test_slow_entmax_attention_argument_errors():
    q = torch.zeros(1, 2, 8, 4)
    with pytest.raises(ValueError):
        slow_entmax_attention(q[0], q, q)
    with pytest.raises(ValueError):
        slow_entmax_attention(q, q, q[:, :, :4])
    with pytest.raises(ValueError):
        slow_entmax_attention(q.cuda(), q.cuda(), q.cuda(), varlen=torch.tensor([8]).cuda(), padding="middle")
    with pytest.raises(ValueError):
        slow_entmax_attention(q.cuda(), q.cuda(), q.cuda(), alibi_slopes=torch.ones(3).cuda())


def test_flash_entmax_attention_matches_exact_definition():
    # tests/test_attention.py:84-100: N = 128, D = 32, fp32, causal, niter = 10, 1e-4
    q, k, v, do = (_randn((1, 1, 128, 32), 70 + i) for i in range(4))
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = flash_entmax_attention(qc, kc, vc, is_causal=True, niter=10)
    dq, dk, dv = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
    ref = _exact(q, k, v, do, 1.5, None, True, "right", None)
    assert (out.detach().cpu().double() - ref[0]).abs().max() < 1e-4
    for got, want, name in zip((dq, dk, dv), ref[1:], ("dq", "dk", "dv")):
        assert (got.cpu().double() - want).abs().max() < 1e-4, name
