"""CPU restatement of the reference's entmax attention path (TEST INFRASTRUCTURE).

This file is the checker, never the product.  It restates, on the CPU with
torch/numpy, the algorithms of deep-spin/adasplash that the CUDA library
replaces.  Every function cites the reference file:line it follows.

Two kinds of oracle live here:

* *exact* oracles -- the mathematical definition (tau by fp64 bisection), which
  is what the reference's own tests compare against (they call the third-party
  ``entmax.entmax_bisect``, PyPI package ``entmax``, unpinned in
  requirements-dev.txt:5; not vendored in the reference and not installed, so
  its published algorithm -- plain bisection on ``sum_j p_j(tau) = 1`` -- is
  restated here);
* *trajectory* oracles -- an operation-for-operation restatement of what the
  reference kernels compute (histogram initialisation, Halley steps, bitmap at
  the penultimate tau, input-dtype rounding of q, p, u and dS).

Parity pin: the trajectory oracles are checked against outputs of the reference
itself (its Triton kernels executed on a B200) stored under tests/golden/ by
tests/golden/make_reference_fixtures.py; the exact oracles are checked against
the trajectory oracles and the reference outputs at the reference's own test
tolerances.
"""
from __future__ import annotations

import math

import numpy as np
import torch

F32 = torch.float32
F64 = torch.float64
MASKED_SCORE = -10000.0  # adasplash_v2.py:104 (SMALL_NUMBER)


# --------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------

def _rn(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round an fp32 tensor to `dtype` and return it as fp32 (Triton's `.to(dtype)`)."""
    if dtype == F32:
        return x.to(F32)
    return x.to(dtype).to(F32)


def select_bins(n_ctx: int, block_n: int = 64) -> int:
    """Histogram bin count of the v2 attention solver (adasplash_v2.py:273-289)."""
    max_count = (n_ctx + block_n - 1) // block_n
    for bins in (8, 4, 2):
        if max_count <= (1 << (64 // bins)) - 1:
            return bins
    raise ValueError("N_CTX too large")


# --------------------------------------------------------------------------
# exact oracles (definition of entmax; what the reference's tests compare to)
# --------------------------------------------------------------------------

def entmax_bisect_exact(x: torch.Tensor, alpha: float = 1.5, n_iter: int = 64):
    """Exact alpha-entmax over the last dim in fp64; returns (p, tau).

    tau solves sum_j [(alpha-1) x_j - tau]_+^(1/(alpha-1)) = 1 on the bracket
    [max-1, max] (the bracket of triton_entmax_v2.py:449-453).  Entries equal to
    -inf get probability 0.  This is the role `entmax_bisect` plays in
    tests/test_triton_entmax.py:37 and tests/test_adasplash_v2.py:63.
    """
    xs = x.to(F64) * (alpha - 1.0)
    mx = xs.max(dim=-1, keepdim=True).values
    lo = mx - 1.0
    hi = mx.clone()
    expo = 1.0 / (alpha - 1.0)

    def total(t):
        return torch.clamp(xs - t, min=0.0).pow(expo).sum(dim=-1, keepdim=True)

    for _ in range(n_iter):
        mid = 0.5 * (lo + hi)
        f = total(mid) - 1.0
        lo = torch.where(f >= 0, mid, lo)
        hi = torch.where(f >= 0, hi, mid)
    tau = 0.5 * (lo + hi)
    p = torch.clamp(xs - tau, min=0.0).pow(expo)
    return p, tau.squeeze(-1)


def entmax_backward_exact(p: torch.Tensor, dy: torch.Tensor, alpha: float = 1.5):
    """Exact entmax vector-Jacobian product in fp64 (triton_entmax_v2.py:539-617):
    u = p^(2-alpha) on the support, dx = u * (dy - sum(u dy) / sum(u))."""
    p = p.to(F64)
    dy = dy.to(F64)
    supp = p > 0
    u = torch.where(supp, p.clamp_min(1e-300).pow(2.0 - alpha), torch.zeros_like(p))
    usum = u.sum(-1, keepdim=True)
    s = (u * dy).sum(-1, keepdim=True) / torch.where(usum > 0, usum, torch.ones_like(usum))
    return u * dy - s * u


def _valid_masks(B, N, varlen, is_causal, device="cpu"):
    """key-valid mask (B,1,N,N) and query-valid mask (B,N) for right padding
    (examples/attention.py:66-83)."""
    cols = torch.arange(N)
    mask = torch.ones(B, 1, N, N, dtype=torch.bool)
    if is_causal:
        mask &= (cols[:, None] >= cols[None, :])[None, None]
    qvalid = torch.ones(B, N, dtype=torch.bool)
    if varlen is not None:
        vl = varlen.to(torch.int64).cpu()
        kvalid = cols[None, :] < vl[:, None]
        mask = mask & kvalid[:, None, None, :]
        qvalid = kvalid
    return mask, qvalid


def dense_entmax_attention(q, k, v, alpha=1.5, is_causal=True, varlen=None, dout=None,
                           work_dtype=F64):
    """Dense entmax attention, the semantics of `slow_entmax_attention`
    (examples/attention.py:34-91) with `triton_entmax` replaced by exact
    bisection, plus analytic gradients.

    q (B,Hq,N,D); k,v (B,Hkv,N,D) with Hq % Hkv == 0 (each kv head serves
    Hq/Hkv consecutive q heads, adasplash_v2.py:193-195).  Scores are scaled by
    1/sqrt(D) (examples/attention.py:61); causal and varlen-invalid keys get
    probability 0; padded query rows produce 0 (examples/attention.py:89-90).

    Returns dict(out, tau, p[, dq, dk, dv]).  tau is in the units of
    (alpha-1)*score, i.e. for alpha=1.5 the units of z = 0.5*score used by
    adasplash_v2.py.  Gradients of padded rows are zero.
    """
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    qd, kd, vd = q.to(work_dtype), k.to(work_dtype), v.to(work_dtype)
    kd_e = kd.repeat_interleave(G, dim=1)
    vd_e = vd.repeat_interleave(G, dim=1)
    scale = 1.0 / math.sqrt(D)
    scores = torch.matmul(qd, kd_e.transpose(-1, -2)) * scale
    mask, qvalid = _valid_masks(B, N, varlen, is_causal)
    scores = scores.masked_fill(~mask, float("-inf"))
    # padded query rows: give them a harmless finite row (result is zeroed below)
    row_ok = qvalid[:, None, :, None]
    scores = torch.where(row_ok, scores, torch.zeros_like(scores))
    p, tau = entmax_bisect_exact(scores, alpha)
    p = p.to(work_dtype) * row_ok
    out = torch.matmul(p, vd_e)
    res = {"out": out, "tau": tau, "p": p}
    if dout is not None:
        do = dout.to(work_dtype) * row_ok
        dp = torch.matmul(do, vd_e.transpose(-1, -2))
        dscores = entmax_backward_exact(p, dp, alpha).to(work_dtype) * row_ok
        dq = torch.matmul(dscores, kd_e) * scale
        dk_e = torch.matmul(dscores.transpose(-1, -2), qd) * scale
        dv_e = torch.matmul(p.transpose(-1, -2), do)
        res["dq"] = dq
        res["dk"] = dk_e.view(B, Hkv, G, N, D).sum(2)
        res["dv"] = dv_e.view(B, Hkv, G, N, D).sum(2)
    return res


# --------------------------------------------------------------------------
# row-wise entmax: trajectory restatement of triton_entmax_v2._fwd_entmax
# --------------------------------------------------------------------------

def _hist_tau_alpha15(counts, t_init, bins):
    """Closed-form lower bound from bin lower edges, alpha = 1.5
    (triton_entmax_v2.py:134-155; adasplash_v2.py:434-461).  counts: (rows,bins)
    fp32 with the top bin already decremented."""
    one = torch.ones_like(t_init)
    s_z, s_k, s_zz = one.clone(), one.clone(), one.clone()
    for sj in range(bins - 1, -1, -1):
        c = counts[:, sj]
        e = np.float32(sj / bins)
        n_z = s_z + c * e
        n_k = s_k + c
        n_zz = s_zz + c * np.float32(e * e)
        good = (n_k * e * e - 2 * n_z * e + n_zz) < 1.0
        s_zz = torch.where(good, n_zz, s_zz)
        s_z = torch.where(good, n_z, s_z)
        s_k = torch.where(good, n_k, s_k)
    return t_init + (s_z - torch.sqrt(s_z * s_z - s_k * (s_zz - 1.0))) / s_k


def _hist_tau_alpha2(counts, t_init, bins):
    """Closed-form lower bound, alpha = 2 (triton_entmax_v2.py:113-131)."""
    one = torch.ones_like(t_init)
    s_z, s_k = one.clone(), one.clone()
    for sj in range(bins - 1, -1, -1):
        c = counts[:, sj]
        e = np.float32(sj / bins)
        n_z = s_z + c * e
        n_k = s_k + c
        good = (n_z - n_k * e) < 1.0
        s_z = torch.where(good, n_z, s_z)
        s_k = torch.where(good, n_k, s_k)
    return t_init + (s_z - 1.0) / s_k


def _f_hist(tau, t_shift, raw_counts, bins):
    """Bin-centre model sum_b c_b [centre_b - tau]_+^2 - 1 (triton_entmax_v2.py:164-204)."""
    acc = torch.zeros_like(tau)
    for b in range(bins):
        centre = t_shift + np.float32((b + 0.5) / bins)
        d = centre - tau
        dpos = torch.where(d > 0, d, torch.zeros_like(d))
        acc = acc + raw_counts[:, b] * dpos * dpos
    return acc - 1.0


def _muller_init(t_lo, t_hi, t_shift, raw_counts, bins):
    """Quadratic (Lagrange) root on the histogram model (triton_entmax_v2.py:207-322)."""
    eps = 1e-10
    a, c = t_lo, t_hi
    b = 0.5 * (a + c)
    fa = _f_hist(a, t_shift, raw_counts, bins)
    fb = _f_hist(b, t_shift, raw_counts, bins)
    fc = _f_hist(c, t_shift, raw_counts, bins)
    denom = (a - b) * (a - c) * (b - c)
    degenerate = denom.abs() < eps
    A = (fa * (b - c) + fb * (c - a) + fc * (a - b)) / denom
    Bc = (fa * (c * c - b * b) + fb * (a * a - c * c) + fc * (b * b - a * a)) / denom
    C = (fa * b * c * (b - c) + fb * a * c * (c - a) + fc * a * b * (a - b)) / denom
    mid = 0.5 * (a + c)
    is_linear = A.abs() < eps
    x_lin = torch.where(Bc.abs() > eps, -C / Bc, mid)
    disc = Bc * Bc - 4 * A * C
    real = disc >= 0
    sq = torch.sqrt(torch.clamp(disc, min=0.0))
    r1 = (-Bc + sq) / (2 * A)
    r2 = (-Bc - sq) / (2 * A)
    v1 = (r1 >= a) & (r1 <= c)
    v2 = (r2 >= a) & (r2 <= c)
    d1 = (c - r1).abs()
    d2 = (c - r2).abs()
    x_quad = torch.where(v1 & v2, torch.where(d1 <= d2, r1, r2),
                         torch.where(v1, r1, torch.where(v2, r2, mid)))
    sden = fc - fa
    x_sec = torch.where(sden.abs() > eps, c - fc * (c - a) / sden, mid)
    x_quad = torch.where(real, x_quad, x_sec)
    x = torch.where(is_linear, x_lin, x_quad)
    x = torch.where(degenerate, mid, x)
    return torch.minimum(torch.maximum(x, a), c)


def _pow_masked(x_act, mask, coeff):
    """exp2(log2(max(x,1e-6))*c) on the mask (triton_entmax_v2.py:22-39, precise branch)."""
    val = torch.exp2(torch.log2(torch.clamp(x_act, min=1e-6)) * np.float32(coeff))
    return torch.where(mask, val, torch.zeros_like(val))


def _hybrid_update(t, t_lo, t_hi, t_prev, f_prev, a0, a1, a2, c0, c1, alpha, allow_secant):
    """Halley -> Newton -> secant -> bisection (triton_entmax_v2.py:42-110)."""
    eps, eps_den = 1e-6, 1e-12
    ff = a0 - 1.0
    df = -np.float32(c0) * a1
    ddf = np.float32(c0 * c1) * a2
    t_lo = torch.where(ff > 0, t, t_lo)
    t_hi = torch.where(ff < 0, t, t_hi)
    hden = 2 * df * df - ff * ddf
    th = t - (2 * ff * df) / hden
    hval = (th > t_lo - eps) & (th < t_hi + eps) & ~torch.isinf(th) & (hden.abs() > eps_den)
    if not alpha <= 1.5:
        hval = torch.zeros_like(hval)
    cand = torch.where(hval, th, torch.zeros_like(th))
    has = hval
    tn = t - ff / df
    nval = (tn > t_lo - eps) & (tn < t_hi + eps) & ~torch.isinf(tn) & (df.abs() > eps_den)
    if not alpha <= 2.0:
        nval = torch.zeros_like(nval)
    take = nval & ~has
    cand = torch.where(take, tn, cand)
    has = has | take
    if allow_secant:
        sden = ff - f_prev
        ts = t - ff * (t - t_prev) / sden
        sval = (ts > t_lo - eps) & (ts < t_hi + eps) & ~torch.isinf(ts) & (sden.abs() > eps_den)
        take = sval & ~has
        cand = torch.where(take, ts, cand)
        has = has | take
    return torch.where(has, cand, 0.5 * (t_lo + t_hi)), t_lo, t_hi


def rowwise_entmax_v2(x: torch.Tensor, alpha=1.5, n_iter=2, use_histogram=True,
                      return_tau=False):
    """Trajectory restatement (fp32) of the reference's row-wise entmax forward.

    Follows `triton_entmax` (triton_entmax_v2.py:690-716: alpha not in {1.5, 2}
    turns the histogram off and forces n_iter >= 10) and `_fwd_entmax`
    (triton_entmax_v2.py:361-536): scale by (alpha-1), row max, optional 4-bin
    histogram lower bound + quadratic start, n_iter hybrid updates, output
    [x(alpha-1) - tau]_+^(1/(alpha-1)) without renormalisation.
    Arithmetic is fp32 whatever x's dtype (the reference keeps fp16 products in
    fp16; that difference is inside its own fp16 tolerance of 1e-2).
    """
    if alpha not in (1.5, 2.0):
        use_histogram = False
        n_iter = max(n_iter, 10)
    shape = x.shape
    X = x.reshape(-1, shape[-1]).to(F32)
    sc = np.float32(alpha - 1)
    c0 = 1.0 / (alpha - 1)
    c1 = c0 - 1
    c2 = c1 - 1
    xs = X * sc
    mx = X.max(dim=-1).values * sc
    bins = 4
    if use_histogram and alpha <= 2.0:
        t_init = mx - 1.0
        proj = xs - t_init[:, None]
        b = torch.floor(proj * bins)
        b = torch.clamp(b, 0, bins - 1).to(torch.int64)
        inc = (proj >= 0)
        raw = torch.zeros(X.shape[0], bins, dtype=F32)
        for j in range(bins):
            raw[:, j] = ((b == j) & inc).sum(-1).to(F32)
        dec = raw.clone()
        dec[:, bins - 1] -= 1
        t_shift = t_init
        if alpha == 1.5:
            t0 = _hist_tau_alpha15(dec, t_init, bins)
        else:
            t0 = _hist_tau_alpha2(dec, t_init, bins)
        t_lo = t0
        t_hi = t0 + np.float32(1.0 / bins)
        t = _muller_init(t_lo, t_hi, t_shift, raw, bins)
    else:
        t_hi = mx
        t_lo = mx - 1.0
        t = 0.5 * (t_lo + t_hi)
    t_prev = t
    f_prev = torch.zeros_like(t)
    for it in range(n_iter):
        m = xs > t[:, None]
        act = torch.clamp(xs - t[:, None], min=0.0)
        zero = torch.zeros_like(act)
        if alpha == 2.0:
            a0 = torch.where(m, act, zero).sum(-1)
            a1 = m.to(F32).sum(-1)
            a2 = torch.zeros_like(a0)
        elif alpha == 1.5:
            a0 = torch.where(m, act * act, zero).sum(-1)
            a1 = torch.where(m, act, zero).sum(-1)
            a2 = m.to(F32).sum(-1)
        else:
            a0 = _pow_masked(act, m, c0).sum(-1)
            a1 = _pow_masked(act, m, c1).sum(-1)
            a2 = _pow_masked(act, m, c2).sum(-1)
        t_new, t_lo, t_hi = _hybrid_update(t, t_lo, t_hi, t_prev, f_prev, a0, a1, a2,
                                           c0, c1, alpha, it > 0)
        t_prev, f_prev, t = t, a0 - 1.0, t_new
    m = xs > t[:, None]
    act = torch.clamp(xs - t[:, None], min=0.0)
    if alpha == 2.0:
        y = torch.where(m, act, torch.zeros_like(act))
    elif alpha == 1.5:
        y = torch.where(m, act * act, torch.zeros_like(act))
    else:
        y = _pow_masked(act, m, c0)
    y = y.reshape(shape)
    if return_tau:
        return y, t.reshape(shape[:-1])
    return y


def rowwise_entmax_backward(y: torch.Tensor, dy: torch.Tensor, alpha=1.5):
    """fp32 restatement of `_bwd_entmax` (triton_entmax_v2.py:539-617)."""
    y = y.to(F32)
    dy = dy.to(F32)
    m = y > 0
    if alpha == 2.0:
        u = m.to(F32)
    elif alpha == 1.5:
        u = torch.where(m, torch.sqrt(y), torch.zeros_like(y))
    else:
        u = _pow_masked(y, m, 2.0 - alpha)
    s = (u * dy).sum(-1, keepdim=True) / u.sum(-1, keepdim=True)
    return u * dy - s * u


# --------------------------------------------------------------------------
# AdaSplash-2 attention: trajectory restatement of adasplash_v2.py
# --------------------------------------------------------------------------

def halley_bisect_update(t, t_lo, t_hi, a0, a1, a2):
    """adasplash_v2.py:68-90."""
    eps = 1e-5
    ff = a0 - 1.0
    df = -2 * a1
    ddf = 2 * a2
    t_lo = torch.where(ff > 0, t, t_lo)
    t_hi = torch.where(ff < 0, t, t_hi)
    new_t = t - (ff * df) / (df * df - 0.5 * ff * ddf)
    good = (new_t > t_lo - eps) & (new_t < t_hi + eps)
    t = torch.where(good, new_t, 0.5 * (t_lo + t_hi))
    return t, t_lo, t_hi


def v2_scaled_scores(q_h, k_h, length, dtype, scale_on="q"):
    """Masked score matrix z (N,N) fp32 of one head as every v2 kernel forms it
    (adasplash_v2.py:93-119, :184, :222-225): the operand named by `scale_on`
    is multiplied by fp32(0.5/sqrt(D)) and rounded to the input dtype, the dot
    product accumulates in fp32, causal / varlen-invalid entries become -10000.
    Rows >= length use q = 0 (masked loads, :220-222)."""
    N, D = q_h.shape
    sm = np.float32(1.0 / math.sqrt(D))
    sc = np.float32(0.5) * sm
    qf, kf = q_h.to(F32), k_h.to(F32)
    if scale_on == "q":
        qf = _rn(qf * sc, dtype)
    else:
        kf = _rn(kf * sc, dtype)
    rows = torch.arange(N)
    qf = torch.where((rows < length)[:, None], qf, torch.zeros_like(qf))
    z = qf @ kf.T
    ok = (rows[:, None] >= rows[None, :]) & (rows[None, :] < length)
    return torch.where(ok, z, torch.full_like(z, MASKED_SCORE))


def v2_solve_head(z, length, n_ctx, niter):
    """tau0 -> tau1 -> Halley refinements -> bitmap for one head.

    z: masked scores (N,N) of `v2_scaled_scores`.  Restates `_get_tau`
    (adasplash_v2.py:151-270: tau0 = max(-1000, rowmax) - 1), `_get_tau_v2`
    (:292-467: BINS-bin histogram of z - tau0 on [0,1], closed form from bin
    lower edges) and `_get_tau_v3` (:470-681: niter Halley/bisection updates,
    then a final sweep that records bit(m,n) = any(z > t) on each 64x64 tile
    for the tau *entering* that sweep and applies one more update).

    Returns dict(tau0, tau1, tau_pen, tau, bits) with bits a bool (nb, nb)
    array over 64x64 tiles (only valid causal tiles can be set).
    """
    N = z.shape[0]
    nb = (N + 63) // 64
    bins = select_bins(n_ctx, 64)
    mx = torch.clamp(z.max(dim=-1).values, min=-1.0e3)
    tau0 = mx - 1.0
    proj = z - tau0[:, None]
    b = torch.floor(proj * bins)
    b = torch.clamp(b, max=bins - 1)
    counts = torch.zeros(N, bins, dtype=F32)
    for j in range(bins):
        counts[:, j] = (b == j).sum(-1).to(F32)
    counts[:, bins - 1] -= 1
    tau1 = _hist_tau_alpha15(counts, tau0, bins)
    t_lo = tau1
    t_hi = tau1 + np.float32(1.0 / bins)
    t = 0.5 * (t_lo + t_hi)

    def sums(tt):
        m = (z > tt[:, None]).to(F32)
        pr = (z - tt[:, None]) * m
        return (pr * pr).sum(-1), pr.sum(-1), m.sum(-1)

    for _ in range(niter):
        a0, a1, a2 = sums(t)
        t, t_lo, t_hi = halley_bisect_update(t, t_lo, t_hi, a0, a1, a2)
    tau_pen = t
    a0, a1, a2 = sums(t)
    hit = torch.zeros(nb * 64, nb * 64, dtype=torch.bool)
    hit[:N, :N] = z > t[:, None]
    hit[length:, :] = False            # rows >= length have q = 0, t = 0-ish: never hit
    bits = hit.view(nb, 64, nb, 64).any(3).any(1)
    # tiles that the reference never visits (beyond the diagonal or beyond length) stay 0
    mi = torch.arange(nb)
    last = (torch.clamp((mi + 1) * 64, max=length) + 63) // 64 - 1
    visit = (mi[None, :] <= last[:, None]) & ((mi * 64) < length)[:, None]
    bits = bits & visit
    t, t_lo, t_hi = halley_bisect_update(t, t_lo, t_hi, a0, a1, a2)
    return {"tau0": tau0, "tau1": tau1, "tau_pen": tau_pen, "tau": t, "bits": bits}


def pack_bitmap(bits: torch.Tensor) -> torch.Tensor:
    """(nb,nb) bool -> int32 (max(32,ceil32(nb)), ceil(nb/32)): row = q-tile,
    word w bit j <=> k-tile 32w+j (adasplash_v2.py:643-647, :1345-1350)."""
    nb = bits.shape[0]
    nw = (nb + 31) // 32
    rows = max(32, ((nb + 31) // 32) * 32)
    out = np.zeros((rows, nw), dtype=np.uint32)
    bn = bits.numpy()
    for j in range(nb):
        out[:nb, j // 32] |= (bn[:, j].astype(np.uint32) << np.uint32(j % 32))
    return torch.from_numpy(out.view(np.int32).copy())


def unpack_bitmap(words: torch.Tensor, nb: int) -> torch.Tensor:
    w = words.cpu().numpy().view(np.uint32)
    out = np.zeros((nb, nb), dtype=bool)
    for j in range(nb):
        out[:, j] = (w[:nb, j // 32] >> np.uint32(j % 32)) & 1
    return torch.from_numpy(out)


def transpose_bitmap(words: torch.Tensor) -> torch.Tensor:
    """Bit-matrix transpose in the reference layout (adasplash_v2.py:901-940):
    out[n, w] bit j = in[32w + j, n // 32] bit (n % 32)."""
    rows, nw = words.shape
    w = words.numpy().view(np.uint32)
    out = np.zeros((rows, nw), dtype=np.uint32)
    for n in range(min(rows, nw * 32)):
        for r in range(rows):
            bit = (w[r, n // 32] >> np.uint32(n % 32)) & np.uint32(1)
            out[n, r // 32] |= bit << np.uint32(r % 32)
    return torch.from_numpy(out.view(np.int32).copy())


def v2_attention(q, k, v, niter=1, varlen=None, dout=None, tau_override=None,
                 bits_override=None, key_side_pairs="own"):
    """Operation-level restatement of `adasplash_v2` forward (+ backward).

    Forward: `_sparse_attention.forward` (adasplash_v2.py:1243-1438) =
    solver (see `v2_solve_head`) + `_get_output` (:696-835): on the tiles whose
    bit is set, u = max(z - tau, 0), out += rn(u*u) @ V, out2 += rn(u) @ V,
    s += sum(u); out2 /= s; both stored in q's dtype; rows >= varlen[b] are 0.

    Backward: `_bwd_preprocess` (:838-898, delta = rowsum(out2*dO); computed
    here in fp32, the reference forms it in the input dtype), `_bwd_q_kernel`
    (:943-1079) and `_bwd_kv_kernel` (:1082-1234; K is the pre-scaled, rounded
    operand there, Q is unscaled), dS and P rounded to the input dtype before
    their products, dq/dk scaled by fp32(1/sqrt(D)) and rounded on store.

    `key_side_pairs`: "own" = the reference's `_bwd_kv_kernel`, whose pairs are those with a
    positive score minus tau under ITS product (K scaled and rounded); "query" = only pairs that
    are also in the forward's support (Q scaled and rounded) -- what a backward that works from
    the forward's list of pairs computes.  The two differ in pairs within an operand rounding of
    the threshold, whose weights are of the size of that rounding.

    Returns dict(out, out2, tau, tau_pen, tau0, tau1, bmask[, delta, dq, dk, dv]).
    """
    B, Hq, N, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    dtype = q.dtype
    sm = np.float32(1.0 / math.sqrt(D))
    nb = (N + 63) // 64
    nw = (nb + 31) // 32
    rows_p = max(32, ((nb + 31) // 32) * 32)
    out = torch.zeros(B, Hq, N, D, dtype=F32)
    out2 = torch.zeros(B, Hq, N, D, dtype=F32)
    keys = ("tau", "tau_pen", "tau0", "tau1")
    taus = {kk: torch.zeros(B, Hq, N, dtype=F32) for kk in keys}
    bmask = torch.zeros(B, Hq, rows_p, nw, dtype=torch.int32)
    if dout is not None:
        dq = torch.zeros(B, Hq, N, D, dtype=F32)
        dk = torch.zeros(B, Hkv, N, D, dtype=F32)
        dv = torch.zeros(B, Hkv, N, D, dtype=F32)
        delta_all = torch.zeros(B, Hq, N, dtype=F32)
    for b in range(B):
        L = int(varlen[b]) if varlen is not None else N
        for h in range(Hq):
            kvh = h // G
            kf = k[b, kvh].to(F32)
            vf = v[b, kvh].to(F32)
            z = v2_scaled_scores(q[b, h], k[b, kvh], L, dtype, "q")
            sol = v2_solve_head(z, L, N, niter)
            if tau_override is not None:
                sol["tau"] = tau_override[b, h].to(F32)
            if bits_override is not None:
                sol["bits"] = bits_override[b, h]
            for kk in keys:
                taus[kk][b, h] = sol[kk]
            bmask[b, h] = pack_bitmap(sol["bits"])
            t = sol["tau"]
            el = torch.zeros(nb * 64, nb * 64, dtype=torch.bool)
            el[:] = sol["bits"].repeat_interleave(64, 0).repeat_interleave(64, 1)
            el = el[:N, :N]
            u = torch.clamp(z - t[:, None], min=0.0) * el
            s = u.sum(-1)
            o = _rn(u * u, dtype) @ vf
            o2 = (_rn(u, dtype) @ vf) / torch.where(s > 0, s, torch.ones_like(s))[:, None]
            rv = (torch.arange(N) < L)[:, None]
            o = _rn(o, dtype) * rv
            o2 = _rn(o2, dtype) * rv
            out[b, h] = o
            out2[b, h] = o2
            if dout is not None:
                do = dout[b, h].to(F32) * rv
                delta = (o2 * do).sum(-1)
                delta_all[b, h] = delta
                dp = do @ vf.T
                ds = _rn(u * (dp - delta[:, None]), dtype)
                dq[b, h] = _rn((ds @ kf) * sm, dtype) * rv
                zt = v2_scaled_scores(q[b, h], k[b, kvh], L, dtype, "k")
                ut = torch.clamp(zt - t[:, None], min=0.0) * el * rv
                if key_side_pairs == "query":
                    ut = ut * (u > 0)
                qf = q[b, h].to(F32) * rv
                dv[b, kvh] += _rn(ut * ut, dtype).T @ do
                dst = _rn(ut * (dp - delta[:, None]), dtype)
                dk[b, kvh] += (dst.T @ qf)
    res = {"out": out, "out2": out2, "bmask": bmask}
    res.update(taus)
    if dout is not None:
        kv_valid = torch.ones(B, 1, N, 1)
        if varlen is not None:
            kv_valid = (torch.arange(N)[None, :] < varlen.cpu()[:, None]).to(F32)[:, None, :, None]
        res["delta"] = delta_all
        res["dq"] = dq
        res["dk"] = _rn(dk * sm, dtype) * kv_valid
        res["dv"] = _rn(dv, dtype) * kv_valid
    return res


# --------------------------------------------------------------------------
# timed CPU baseline (benchmark's cpu_baseline / --impl reference leg)
# --------------------------------------------------------------------------

def cpu_dense_entmax15_attention(q, k, v, dout=None, n_bisect=30):
    """Multi-threaded fp32 CPU dense causal entmax-1.5 attention, forward and
    (if dout is given) backward: `slow_entmax_attention` semantics
    (examples/attention.py:34-91) with tau by vectorised fp32 bisection (the
    reference helper itself calls a Triton kernel and cannot run on a CPU).
    Same maths as `dense_entmax_attention`, in fp32 with in-place ops for speed."""
    B, Hq, N, D = q.shape
    G = Hq // k.shape[1]
    qf = q.to(F32)
    kf = k.to(F32).repeat_interleave(G, dim=1)
    vf = v.to(F32).repeat_interleave(G, dim=1)
    z = torch.matmul(qf, kf.transpose(-1, -2)).mul_(0.5 / math.sqrt(D))
    causal = torch.ones(N, N, dtype=torch.bool).tril_()
    z.masked_fill_(~causal, float("-inf"))
    mx = z.max(dim=-1, keepdim=True).values
    lo, hi = mx - 1.0, mx.clone()
    for _ in range(n_bisect):
        mid = (lo + hi).mul_(0.5)
        f = (z - mid).clamp_(min=0).square_().sum(-1, keepdim=True)
        ge = f >= 1.0
        lo = torch.where(ge, mid, lo)
        hi = torch.where(ge, hi, mid)
    tau = (lo + hi).mul_(0.5)
    u = (z - tau).clamp_(min=0)
    p = u * u
    out = torch.matmul(p, vf)
    if dout is None:
        return out, tau.squeeze(-1)
    do = dout.to(F32)
    dp = torch.matmul(do, vf.transpose(-1, -2))
    delta = (u * dp).sum(-1, keepdim=True) / u.sum(-1, keepdim=True)
    ds = u * (dp - delta)
    sc = 1.0 / math.sqrt(D)
    dq = torch.matmul(ds, kf).mul_(sc)
    dk = torch.matmul(ds.transpose(-1, -2), qf).mul_(sc)
    dv = torch.matmul(p.transpose(-1, -2), do)
    Hkv = k.shape[1]
    return out, tau.squeeze(-1), dq, dk.view(B, Hkv, G, N, D).sum(2), dv.view(B, Hkv, G, N, D).sum(2)
