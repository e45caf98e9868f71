"""GPU parity of the row-wise entmax kernels (through the C ABI) against the
CPU oracle and the reference's golden outputs."""
import os

import pytest
import torch

import adasplash_b200 as adasplash
from adasplash_b200 import entmax as em
from oracle import entmax_oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _randn(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


# tolerances of the reference's tests/test_triton_entmax.py:17-20
def _fwd_tol(dtype, alpha):
    if dtype != torch.float32:
        return 2e-2 if alpha == 1.333 else 1e-2
    return 5e-4 if alpha == 1.333 else 1e-4


@pytest.mark.parametrize("shape", [(2,), (2, 4), (2, 4, 8), (2, 4, 8, 16), (3, 100), (5, 513),
                                   (4, 1000), (3, 2050), (2, 4096), (2, 5000), (2, 9000),
                                   (1, 20000), (1, 40000)])
@pytest.mark.parametrize("alpha", [1.333, 1.5, 2.0])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_forward_backward_vs_exact(shape, alpha, dtype):
    if dtype != torch.float32 and shape[-1] > 5000:
        pytest.skip("16-bit inputs: long rows covered by fp32")
    x = _randn(shape, 11, 2.0, dtype)
    dy = _randn(shape, 12, 1.0, dtype)
    xc = x.cuda().requires_grad_(True)
    y = adasplash.triton_entmax(xc, alpha=alpha, n_iter=10)
    (dx,) = torch.autograd.grad(y, xc, dy.cuda())
    p, _ = O.entmax_bisect_exact(x.float(), alpha)
    tol = _fwd_tol(dtype, alpha)
    assert y.dtype == dtype and y.shape == x.shape
    assert (y.float().cpu().double() - p).abs().max() < tol
    assert abs(y.float().sum(-1).cpu() - 1).max() < 1e-2
    dxe = O.entmax_backward_exact(y.float().cpu(), dy.float(), alpha)
    gtol = 1e-2 if dtype == torch.float32 else 5e-2
    assert (dx.float().cpu().double() - dxe).abs().max() < gtol


@pytest.mark.parametrize("alpha,n_iter,hist", [(1.5, 2, True), (2.0, 2, True), (1.333, 2, True),
                                               (1.5, 3, False), (2.0, 0, True), (1.5, 0, True)])
def test_trajectory_matches_oracle(alpha, n_iter, hist):
    x = _randn((64, 4096), 21, 4.0)
    y, tau = em.entmax_with_tau(x.cuda(), alpha, n_iter, hist)
    yo, to = O.rowwise_entmax_v2(x, alpha, n_iter, hist, return_tau=True)
    # with no refinement the result is the raw quadratic start, whose Lagrange
    # coefficients cancel catastrophically in fp32: only loosely comparable
    tol = 2e-6 if n_iter > 0 else 2e-3
    if alpha not in (1.5, 2.0):
        tol = 1e-5  # generic alpha goes through the approximate lg2 / ex2 units
    assert (tau.cpu() - to).abs().max() < tol
    assert (y.cpu() - yo).abs().max() < tol


@pytest.mark.parametrize("cols", [100, 1000, 4096, 9000, 40000])
@pytest.mark.parametrize("alpha", [1.5, 2.0, 1.333])
def test_nearly_flat_rows_take_the_full_passes(cols, alpha):
    # Rows with a small spread have most of their elements within 1 of the maximum: more than
    # the kernel's candidate list holds, so it sweeps the whole row at every step instead.
    # Peaked rows of the same batch use the list; both must follow the oracle's trajectory.
    flat = _randn((3, cols), 31, 0.2)
    peaked = _randn((3, cols), 32, 4.0)
    x = torch.cat([flat, peaked], 0)
    for n_iter in (2, 6):   # 6 steps: the list is built (and overflows for the flat rows)
        y, tau = em.entmax_with_tau(x.cuda(), alpha, n_iter, True)
        yo, to = O.rowwise_entmax_v2(x, alpha, n_iter, True, return_tau=True)
        tol = 2e-6 if alpha in (1.5, 2.0) else 1e-5
        assert (tau.cpu() - to).abs().max() < tol
        assert (y.cpu() - yo).abs().max() < tol


def test_forward_is_reproducible():
    # the candidate list is filled by atomics in arbitrary order and then sorted: two runs
    # must agree bit for bit
    x = _randn((256, 4096), 33, 4.0).cuda()
    for alpha, n_iter in ((1.5, 8), (1.333, 10)):
        a = adasplash.triton_entmax(x, alpha=alpha, n_iter=n_iter)
        for _ in range(3):
            assert torch.equal(a, adasplash.triton_entmax(x, alpha=alpha, n_iter=n_iter))


def test_unaligned_rows_use_scalar_path():
    x = _randn((7, 1001), 31, 3.0)
    base = torch.zeros(7 * 1001 + 1, device="cuda")
    xv = base[1:].view(7, 1001)
    xv.copy_(x)
    assert xv.data_ptr() % 16 != 0
    y = adasplash.triton_entmax(xv, n_iter=10)
    p, _ = O.entmax_bisect_exact(x, 1.5)
    assert (y.cpu().double() - p).abs().max() < 1e-5


def test_aliases_and_histogram_toggle():
    x = _randn((8, 300), 41, 2.0).cuda()
    a = adasplash.triton_entmax(x, alpha=2.0)
    b = adasplash.triton_sparsemax(x)
    assert torch.equal(a, b)
    a = adasplash.triton_entmax(x, alpha=1.5)
    b = adasplash.triton_entmax15(x)
    assert torch.equal(a, b)
    c = adasplash.triton_entmax(x, alpha=1.5, n_iter=10, use_histogram=False)
    assert (a - c).abs().max() < 1e-4
    d = adasplash.triton_entmax_v1(x)
    assert (d - c).abs().max() < 1e-5


def test_large_magnitude_inputs_stay_finite():
    x = (_randn((4, 777), 51) * 100).cuda().requires_grad_(True)
    for alpha in (1.333, 1.5, 2.0):
        y = adasplash.triton_entmax(x, alpha=alpha)
        (g,) = torch.autograd.grad(y.sum(), x)
        assert torch.isfinite(y).all() and (y >= 0).all() and torch.isfinite(g).all()


def test_empty_and_single_column():
    assert adasplash.triton_entmax(torch.zeros(0, 8, device="cuda")).shape == (0, 8)
    y = adasplash.triton_entmax(torch.randn(5, 1, device="cuda"))
    assert torch.allclose(y, torch.ones_like(y))


def test_reference_golden():
    path = os.path.join(GOLD, "rowwise.pt")
    if not os.path.exists(path):
        pytest.fail("tests/golden/rowwise.pt missing")
    fx = torch.load(path, weights_only=False)
    x = fx["x"].cuda().requires_grad_(True)
    for tag in ("a15_hist", "a2_default", "a1333", "a15_nohist_it10"):
        y = adasplash.triton_entmax(x, **fx[tag]["kwargs"])
        (dx,) = torch.autograd.grad(y, x, fx["dy"].cuda())
        assert (y.detach().cpu() - fx[tag]["y"]).abs().max() < (1e-5 if tag == "a1333" else 2e-6), tag
        assert (dx.cpu() - fx[tag]["dx"]).abs().max() < 1e-4, tag
    xs = fx["x_small_f16"].cuda().requires_grad_(True)
    for tag in ("small_a15", "small_a2", "small_a1333"):
        y = adasplash.triton_entmax(xs, **fx[tag]["kwargs"])
        (dx,) = torch.autograd.grad(y, xs, fx["dy_small_f16"].cuda())
        assert (y.detach().float().cpu() - fx[tag]["y"].float()).abs().max() < 1e-2, tag
        assert torch.isfinite(dx).all()


@pytest.mark.slow
def test_full_size_properties():
    # the 16384 x 4096 benchmark matrix: rows sum to one, support is preserved by
    # the backward, and a row permutation commutes with the operator
    g = torch.Generator(device="cuda").manual_seed(20261)
    x = torch.randn(16384, 4096, device="cuda", generator=g) * 4
    y = adasplash.triton_entmax(x, alpha=1.5, n_iter=2)
    assert (y.sum(-1) - 1).abs().max() < 1e-4
    assert (y >= 0).all()
    perm = torch.randperm(16384, device="cuda", generator=g)
    y2 = adasplash.triton_entmax(x[perm].contiguous(), alpha=1.5, n_iter=2)
    assert torch.equal(y2, y[perm])
    ys, tau = em.entmax_with_tau(x[:64].contiguous(), 1.5, 2, True)
    yo, to = O.rowwise_entmax_v2(x[:64].cpu(), 1.5, 2, True, return_tau=True)
    assert (ys.cpu() - yo).abs().max() < 2e-6


@pytest.mark.parametrize("alpha", [1.5, 2.0, 1.333])
@pytest.mark.parametrize("rows,cols,dtype", [(8197, 516, torch.float32), (9001, 4096, torch.float32),
                                             (8200, 260, torch.bfloat16), (16384, 100, torch.float16)])
def test_many_rows_take_the_pipelined_kernel(rows, cols, dtype, alpha):
    # From 8192 rows on, vectorisable matrices run the kernel that prefetches the next row of a
    # group into shared memory; row counts that do not fill the last groups, several groups per
    # CTA (short rows) and 16-bit inputs all go through it.  Same trajectory as the oracle.
    x = _randn((rows, cols), 41, 4.0, dtype)
    y, tau = em.entmax_with_tau(x.cuda(), alpha, 2, True)
    sel = torch.cat([torch.arange(0, 40), torch.arange(rows // 2, rows // 2 + 40), torch.arange(rows - 40, rows)])
    yo, to = O.rowwise_entmax_v2(x[sel].float(), alpha, 2, True, return_tau=True)
    if dtype == torch.float32:
        tol = 2e-6 if alpha in (1.5, 2.0) else 1e-5
        assert (tau.cpu()[sel] - to).abs().max() < tol
        assert (y.cpu()[sel] - yo).abs().max() < tol
    else:
        assert (y.float().cpu()[sel] - yo).abs().max() < 1e-2   # the reference's 16-bit tolerance
    # no row was left unwritten (two refinement steps do not fully converge sparsemax on wide
    # inputs, so the row sums are only near 1)
    sums = y.float().sum(-1)
    assert sums.min() > 0.8 and sums.max() < 1.2
