"""CPU checks of the oracle itself: the trajectory restatements against the
exact (bisection) definition, and both against the golden outputs of the
reference stored under tests/golden/."""
import os

import pytest
import torch

from oracle import entmax_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    path = os.path.join(GOLD, name + ".pt")
    if not os.path.exists(path):
        pytest.fail(f"golden fixture {name}.pt is missing; see tests/golden/make_reference_fixtures.py")
    return torch.load(path, weights_only=False)


@pytest.mark.parametrize("alpha,n_iter,hist,tol", [(1.5, 2, True, 2e-5), (2.0, 10, True, 1e-5),
                                                    (1.333, 2, False, 1e-5), (1.5, 10, False, 1e-5)])
def test_rowwise_trajectory_matches_exact(alpha, n_iter, hist, tol):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(32, 1000, generator=g) * 4
    y, tau = O.rowwise_entmax_v2(x, alpha, n_iter, hist, return_tau=True)
    p, te = O.entmax_bisect_exact(x, alpha)
    assert (tau.double() - te).abs().max() < tol
    assert (y.double() - p).abs().max() < tol
    dy = torch.randn(32, 1000, generator=g)
    dx = O.rowwise_entmax_backward(y, dy, alpha)
    dxe = O.entmax_backward_exact(p, dy, alpha)
    assert (dx.double() - dxe).abs().max() < 2e-3


def test_v2_trajectory_matches_exact_fp32():
    g = torch.Generator().manual_seed(7)
    q, k, v, do = (torch.randn(s, generator=g) for s in
                   [(1, 4, 192, 32), (1, 2, 192, 32), (1, 2, 192, 32), (1, 4, 192, 32)])
    vl = torch.tensor([150])
    tr = O.v2_attention(q, k, v, 1, vl, do)
    ex = O.dense_entmax_attention(q, k, v, 1.5, True, vl, do)
    assert (tr["tau"][:, :, :150].double() - ex["tau"][:, :, :150]).abs().max() < 1e-5
    for key in ("out", "dq", "dk", "dv"):
        assert (tr[key].double() - ex[key]).abs().max() < 1e-4, key
    assert tr["out"][:, :, 150:].abs().max() == 0


def test_bitmap_pack_transpose_roundtrip():
    g = torch.Generator().manual_seed(3)
    bits = torch.rand(70, 70, generator=g) > 0.6
    words = O.pack_bitmap(bits)
    assert words.shape == (96, 3)
    assert (O.unpack_bitmap(words, 70) == bits).all()
    t = O.transpose_bitmap(words)
    assert (O.unpack_bitmap(t, 70) == bits.T).all()
    assert (O.transpose_bitmap(t) == words).all()


def test_select_bins():
    # adasplash_v2.py:273-289
    assert O.select_bins(64) == 8 and O.select_bins(16320) == 8
    assert O.select_bins(16384) == 4 and O.select_bins(65536) == 4


# ---- pins against outputs of the reference itself (generated on a B200) ----

def test_rowwise_oracle_vs_reference_golden():
    fx = _load("rowwise")
    x, dy = fx["x"], fx["dy"]
    for tag in ("a15_hist", "a2_default", "a1333", "a15_nohist_it10"):
        kw = fx[tag]["kwargs"]
        y = O.rowwise_entmax_v2(x, kw.get("alpha", 1.5), kw.get("n_iter", 2), kw.get("use_histogram", True))
        assert (y - fx[tag]["y"]).abs().max() < 2e-6, tag
        dx = O.rowwise_entmax_backward(fx[tag]["y"], dy, kw.get("alpha", 1.5))
        assert (dx - fx[tag]["dx"]).abs().max() < 1e-4, tag
    xs, dys = fx["x_small_f16"], fx["dy_small_f16"]
    for tag in ("small_a15", "small_a2", "small_a1333"):
        kw = fx[tag]["kwargs"]
        y = O.rowwise_entmax_v2(xs, kw["alpha"], 2, True)
        assert (y - fx[tag]["y"].float()).abs().max() < 1e-2, tag   # reference fp16 tolerance


@pytest.mark.parametrize("name,tol_out,tol_grad", [
    ("v2_fp32_smoke", 1e-5, 5e-5), ("v2_fp32_gqa_varlen", 1e-5, 5e-5), ("v2_fp32_niter1", 1e-5, 5e-5),
    ("v2_bf16_d128", 2e-2, 2e-2), ("v2_bf16_varlen", 2e-2, 2e-2), ("v2_fp16_d64", 5e-3, 5e-3),
])
def test_v2_oracle_vs_reference_golden(name, tol_out, tol_grad):
    fx = _load(name)
    vl = fx["varlen"]
    tr = O.v2_attention(fx["q"], fx["k"], fx["v"], fx["niter"], vl, fx["dout"])
    N = fx["q"].shape[2]
    for b in range(fx["q"].shape[0]):
        L = N if vl is None else int(vl[b])
        assert (tr["tau"][b, :, :L] - fx["taus"][b, :, :L]).abs().max() < 1e-5, "tau"
    assert (tr["bmask"] == fx["bmask"]).all(), "bitmap"
    assert (tr["out"] - fx["out"].float()).abs().max() < tol_out
    for key in (("dq", "dk", "dv") if fx["dq"] is not None else ()):
        # 16-bit: the reference forms delta in the input dtype (adasplash_v2.py:891),
        # the oracle in fp32, so gradients agree to the tolerance times their scale
        scale = 1.0 if fx["q"].dtype == torch.float32 else max(1.0, fx[key].float().abs().max().item())
        assert (tr[key] - fx[key].float()).abs().max() < tol_grad * scale, key
    # and the exact definition, at the reference's own test tolerance for fp32
    if fx["q"].dtype == torch.float32 and fx["niter"] == 10:
        ex = O.dense_entmax_attention(fx["q"], fx["k"], fx["v"], 1.5, True, vl, fx["dout"])
        for key in ("out", "dq", "dk", "dv"):
            assert (ex[key] - fx[key].double()).abs().max() < 1e-4, key


def test_v2_solver_oracle_four_bin_histogram_vs_reference():
    """N >= 16384 selects the 4-bin histogram (adasplash_v2.py:273-289).  The short sequence of
    the 16384-long fixture (5000 valid rows) pins that route of the oracle on the CPU: thresholds
    and block mask of one head against what the reference stored."""
    import sys
    fx = _load("v2_bf16_c4_slice")
    sys.path.insert(0, GOLD)
    import make_reference_fixtures as mk
    q, k, v, do, varlen, niter, _ = mk.big_case_inputs("v2_bf16_c4_slice")
    b, h, L, N = 1, 2, int(varlen[1]), q.shape[2]
    assert O.select_bins(N) == 4
    nbL = (L + 63) // 64
    z = O.v2_scaled_scores(q[b, h, :nbL * 64], k[b, 0, :nbL * 64], L, q.dtype)
    sol = O.v2_solve_head(z, L, N, niter)
    assert (sol["tau"][:L] - fx["taus"][b, h, :L]).abs().max() < 1e-5
    words = O.pack_bitmap(sol["bits"])
    ref = fx["bmask"][b, h]
    assert (words[:nbL, :words.shape[1]] == ref[:nbL, :words.shape[1]]).all()
    assert (ref[nbL:] == 0).all() and (ref[:, words.shape[1]:] == 0).all()


@pytest.mark.parametrize("name", ["v1_a1333_causal", "v1_a1333_full", "v1_a15_full", "v1_a2_causal", "v1_a2_full"])
def test_exact_oracle_vs_reference_v1_golden(name):
    # generic alpha / full attention: the reference's first-generation kernels at niter = 10
    fx = _load(name)
    ex = O.dense_entmax_attention(fx["q"], fx["k"], fx["v"], fx["alpha"], fx["is_causal"], None, fx["dout"])
    for key in ("out", "dq", "dk", "dv"):
        assert (ex[key].float() - fx[key]).abs().max() < 2e-5, key


def test_key_side_pairs_from_the_forward_support_differ_by_rounding_only():
    # The gather kernels take the key side's pairs from the forward's supports; the reference's
    # dK/dV kernel decides them from its own product.  On the reference's fixture the two
    # definitions of dK / dV agree to a fraction of the fixture tolerance (and everything else is
    # identical by construction).
    fx = torch.load(os.path.join(GOLD, "v2_bf16_d128.pt"), weights_only=False)
    a = O.v2_attention(fx["q"], fx["k"], fx["v"], fx["niter"], fx["varlen"], fx["dout"])
    b = O.v2_attention(fx["q"], fx["k"], fx["v"], fx["niter"], fx["varlen"], fx["dout"], key_side_pairs="query")
    for key in ("out", "out2", "dq"):
        assert torch.equal(a[key], b[key])
    for key in ("dk", "dv"):
        scale = max(1.0, a[key].abs().max().item())
        assert (a[key] - b[key]).abs().max().item() < 5e-3 * scale, key   # a quarter of the 2e-2 tolerance
