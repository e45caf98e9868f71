"""GPU parity of the AdaSplash-2 attention path (through the C ABI) against
the CPU oracle, the exact dense definition and the reference's golden outputs.

Tolerances: fp32 1e-4 on out/dq/dk/dv and tau (the reference's own test
tolerance, tests/test_adasplash_v2.py:94-97); bf16/fp16 max-abs 2e-2 on outputs
and gradients against the reference; bitmaps bit-exact for identical fp32 tau.
"""
import json
import os
import sys

import pytest
import torch

import adasplash_b200 as adasplash
from adasplash_b200 import _lib, attention as att
from oracle import entmax_oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
# "tcgen05": the tensor-core solver with row supports (sparse heads run as gathers, the others on
# the tile kernels); "tiles": the tile kernels for every head; "simt": the CUDA-core kernels
PATHS = ["simt", "tcgen05", "tiles"]


def _randn(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.fixture(autouse=True)
def _reset_path():
    att.DEBUG_STATUS = True   # every call also checks the kernels' bounded-wait status word
    yield
    att.DEBUG_STATUS = False
    att.ROW_SUPPORTS = True
    _lib.set_kernel_path(None)


def _use(path, q):
    """Select a kernel family; skip if it does not cover this dtype / head dim."""
    att.ROW_SUPPORTS = path != "tiles"
    if path == "tiles":
        path = "tcgen05"
    _lib.set_kernel_path(path)
    if path == "tcgen05":
        import ctypes
        sh = att.make_shape(q, q, 1, None)
        if _lib.load().adasplash2_resolved_path(ctypes.byref(sh)) != _lib.PATH_TCGEN05:
            pytest.skip("tensor-core kernels do not cover this dtype/head dim")


def _run(q, k, v, do, niter, varlen):
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    vl = None if varlen is None else varlen.cuda()
    out = adasplash.adasplash_v2(qc, kc, vc, niter=niter, varlen=vl)
    saved = out.grad_fn.saved_tensors
    dq, dk, dv = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
    return {"out": out.detach().float().cpu(), "out2": saved[3].float().cpu(), "tau": saved[4].cpu(),
            "bmask": saved[5].cpu(), "dq": dq.float().cpu(), "dk": dk.float().cpu(),
            "dv": dv.float().cpu()}


def _mask_rows(do, varlen):
    if varlen is None:
        return do
    N = do.shape[2]
    return do * (torch.arange(N)[None, None, :, None] < varlen[:, None, None, None])


CASES_FP32 = [
    # B, Hq, Hkv, N, D, varlen
    (1, 1, 1, 256, 32, None), (2, 2, 2, 128, 64, None), (1, 2, 1, 256, 32, [160]),
    (2, 4, 2, 192, 16, [65, 130]), (1, 2, 2, 64, 128, None), (1, 1, 1, 128, 256, None),
    (2, 2, 1, 200, 64, [200, 64]), (1, 8, 2, 1024, 64, None),
]


@pytest.mark.parametrize("path", ["simt"])
@pytest.mark.parametrize("case", CASES_FP32)
def test_fp32_matches_exact_definition(path, case):
    B, Hq, Hkv, N, D, vl = case
    q, k, v = _randn((B, Hq, N, D), 1), _randn((B, Hkv, N, D), 2), _randn((B, Hkv, N, D), 3)
    varlen = None if vl is None else torch.tensor(vl, dtype=torch.int32)
    do = _mask_rows(_randn((B, Hq, N, D), 4), varlen)
    _use(path, q)
    got = _run(q, k, v, do, 10, varlen)
    ex = O.dense_entmax_attention(q, k, v, 1.5, True, varlen, do)
    for b in range(B):
        L = N if vl is None else vl[b]
        assert (got["tau"][b, :, :L].double() - ex["tau"][b, :, :L]).abs().max() < 1e-4
    for key in ("out", "dq", "dk", "dv"):
        assert (got[key].double() - ex[key]).abs().max() < 1e-4, key
    if vl is not None:
        for b in range(B):
            if vl[b] < N:
                assert got["out"][b, :, vl[b]:].abs().max() == 0
                assert got["dq"][b, :, vl[b]:].abs().max() == 0
                assert got["dk"][b, :, vl[b]:].abs().max() == 0


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [(1, 2, 1, 256, 64, None, 1.0), (1, 2, 2, 512, 128, None, 1.5),
                                  (2, 4, 1, 320, 128, [300, 129], 1.0), (1, 1, 1, 192, 64, [191], 1.0),
                                  (1, 2, 2, 128, 32, None, 1.0), (2, 4, 2, 200, 16, [200, 77], 1.0),
                                  (1, 2, 1, 384, 32, [300], 1.5)])
def test_16bit_matches_trajectory_oracle(path, dtype, case):
    B, Hq, Hkv, N, D, vl, sc = case
    q, k, v = (_randn(s, i, sc, dtype) for i, s in
               enumerate([(B, Hq, N, D), (B, Hkv, N, D), (B, Hkv, N, D)], 10))
    varlen = None if vl is None else torch.tensor(vl, dtype=torch.int64)
    do = _mask_rows(_randn((B, Hq, N, D), 14, 1.0, dtype), varlen)
    _use(path, q)
    got = _run(q, k, v, do, 1, varlen)
    tr = O.v2_attention(q, k, v, 1, varlen, do)
    for b in range(B):
        L = N if vl is None else vl[b]
        assert (got["tau"][b, :, :L] - tr["tau"][b, :, :L]).abs().max() < 1e-4
    assert (got["bmask"] == tr["bmask"]).all()
    for key in ("out", "out2", "dq", "dk", "dv"):
        scale = max(1.0, tr[key].abs().max().item())
        assert (got[key] - tr[key]).abs().max() < 2e-2 * scale, key


@pytest.mark.parametrize("path", PATHS)
def test_bitmap_bit_exact_for_given_tau(path):
    # thresholds chosen so that many tiles are empty; identical fp32 tau in, bitmap out
    B, Hq, Hkv, N, D = 1, 2, 1, 512, 128
    q, k = _randn((B, Hq, N, D), 20, 1.5, torch.bfloat16), _randn((B, Hkv, N, D), 21, 1.5, torch.bfloat16)
    _use(path, q)
    for shift in (0.0, 0.8, 2.5):
        taus = torch.full((B, Hq, N), 1.0 + shift) + _randn((B, Hq, N), 22) * 0.3
        bm = att.mask_from_tau(q.cuda(), k.cuda(), taus.cuda())
        ref = torch.zeros_like(bm.cpu())
        for h in range(Hq):
            z = O.v2_scaled_scores(q[0, h], k[0, 0], N, torch.bfloat16)
            hit = (z > taus[0, h][:, None]).view(N // 64, 64, N // 64, 64).any(3).any(1)
            ref[0, h] = O.pack_bitmap(hit)
        assert (bm.cpu() == ref).all(), shift


@pytest.mark.parametrize("path", PATHS)
def test_zero_scores_give_running_mean_of_v(path):
    # all-zero q/k: uniform attention over the causal prefix (tests/test_adasplash.py:173-184)
    B, H, N, D = 1, 2, 128, 64
    q = torch.zeros(B, H, N, D, dtype=torch.bfloat16)
    v = _randn((B, H, N, D), 30, 1.0, torch.bfloat16)
    _use(path, q)
    out = adasplash.adasplash_v2(q.cuda(), q.cuda(), v.cuda(), niter=4)
    ref = v.float().cumsum(2) / torch.arange(1, N + 1)[None, None, :, None]
    assert (out.float().cpu() - ref).abs().max() < 2e-2


@pytest.mark.parametrize("path", PATHS)
def test_deterministic(path):
    q, k, v, do = (_randn((1, 2, 256, 64), 40 + i, 1.0, torch.bfloat16) for i in range(4))
    _use(path, q)
    a = _run(q, k, v, do, 1, None)
    b = _run(q, k, v, do, 1, None)
    for key in a:
        assert torch.equal(a[key], b[key]), key


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("name,tol", [
    ("v2_fp32_smoke", 1e-4), ("v2_fp32_gqa_varlen", 1e-4), ("v2_fp32_niter1", 1e-4),
    ("v2_bf16_d128", 2e-2), ("v2_bf16_varlen", 2e-2), ("v2_fp16_d64", 2e-2),
])
def test_reference_golden(path, name, tol):
    fpath = os.path.join(GOLD, name + ".pt")
    if not os.path.exists(fpath):
        pytest.fail(f"tests/golden/{name}.pt missing")
    fx = torch.load(fpath, weights_only=False)
    _use(path, fx["q"])
    got = _run(fx["q"], fx["k"], fx["v"], fx["dout"], fx["niter"], fx["varlen"])
    N = fx["q"].shape[2]
    keys = ("out", "dq", "dk", "dv") if fx["dq"] is not None else ("out",)
    for b in range(fx["q"].shape[0]):
        L = N if fx["varlen"] is None else int(fx["varlen"][b])
        assert (got["tau"][b, :, :L] - fx["taus"][b, :, :L]).abs().max() < 1e-4
    assert (got["bmask"] == fx["bmask"]).all()
    assert (got["out"] - fx["out"].float()).abs().max() < tol
    if len(keys) > 1:
        _check_grads_vs_reference(got, fx, tol)


def _check_grads_vs_reference(got, fx, tol):
    """Gradients against the reference's own.  In 16-bit the reference forms
    delta = rowsum(out2*dO) in the input dtype (adasplash_v2.py:891), which costs it
    about two digits; this library accumulates delta in fp32.  So the 16-bit check is
    (i) agreement within `tol` relative to the gradient's scale and (ii) being at
    least as close to the exact fp64 gradients as the reference is."""
    exact = None
    if fx["q"].dtype != torch.float32:
        exact = O.dense_entmax_attention(fx["q"], fx["k"], fx["v"], 1.5, True, fx["varlen"], fx["dout"])
    for key in ("dq", "dk", "dv"):
        ref = fx[key].float()
        scale = max(1.0, ref.abs().max().item()) if exact is not None else 1.0
        assert (got[key] - ref).abs().max() < tol * scale, key
        if exact is not None:
            mine = (got[key].double() - exact[key]).abs().max().item()
            theirs = (ref.double() - exact[key]).abs().max().item()
            assert mine <= 1.25 * theirs + 1e-3, (key, mine, theirs)


def _popcount(t):
    return sum(bin(int(x) & 0xFFFFFFFF).count("1") for x in t.flatten().tolist())


def _log_parity(record):
    """Append the achieved errors of a fixture comparison to the file named by
    ADASPLASH_PARITY_LOG (one JSON object per line), if that variable is set."""
    path = os.environ.get("ADASPLASH_PARITY_LOG")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(record) + "\n")


def _strided_fixture(name):
    """A fixture whose inputs are regenerated from seeds and whose outputs are kept for every
    `row_stride`-th row (thresholds and block mask in full)."""
    fpath = os.path.join(GOLD, name + ".pt")
    if not os.path.exists(fpath):
        pytest.fail(f"tests/golden/{name}.pt missing (tests/golden/make_reference_fixtures.py --big-slices)")
    fx = torch.load(fpath, weights_only=False)
    if "case" in fx:
        sys.path.insert(0, GOLD)
        import make_reference_fixtures as mk
        q, k, v, do, varlen, niter, stride = mk.big_case_inputs(fx["case"])
    else:  # v2_bf16_d128_n2048: B = Hq = Hkv = 1, seeds seed + 0/100/200/300
        N, D = fx["taus"].shape[2], fx["out"].shape[3]
        q, k, v = (_randn((1, 1, N, D), fx["seed"] + 100 * i, fx["scale"], torch.bfloat16) for i in range(3))
        do = _randn((1, 1, N, D), fx["seed"] + 300, 1.0, torch.bfloat16)
        varlen, niter = None, fx["niter"]
    return fx, q, k, v, do, varlen, niter


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("name", ["v2_bf16_d128_n2048", "v2_bf16_c3_slice", "v2_bf16_c4_slice",
                                  "v2_bf16_c5_slice"])
def test_reference_golden_at_benchmark_lengths(path, name):
    """Against the reference's own outputs at the sequence lengths of the benchmark
    configurations (8192; 16384 with grouped heads, a short sequence and the 4-bin histogram;
    65536).  tau <= 1e-4; block mask equal to the reference's up to bits that a score within
    rounding of its threshold decides; out, out2, dq, dk, dv within 2e-2 of the tensor's scale."""
    fx, q, k, v, do, varlen, niter = _strided_fixture(name)
    _use(path, q)
    got = _run(q, k, v, do, niter, varlen)
    B, Hq, N, D = q.shape
    rec = {"fixture": name, "path": path}
    tau_err = 0.0
    for b in range(B):
        L = N if varlen is None else int(varlen[b])
        tau_err = max(tau_err, (got["tau"][b, :, :L] - fx["taus"][b, :, :L]).abs().max().item())
    rec["tau"] = tau_err
    assert tau_err < 1e-4
    flips = _popcount(got["bmask"] ^ fx["bmask"])
    rec["bitmap_flips"] = flips
    rec["bitmap_bits_set"] = _popcount(fx["bmask"])
    nb = (N + 63) // 64
    # a different summation order inside a score may move it across its threshold by an ulp
    assert flips <= 2 + 1e-5 * B * Hq * nb * nb, flips
    rows = slice(fx.get("row_offset", 0), None, fx["row_stride"])
    for key in ("out", "out2", "dq", "dk", "dv"):
        ref = fx[key].float()
        scale = max(1.0, fx.get(key + "_absmax", ref.abs().max().item()))
        err = (got[key][:, :, rows] - ref).abs().max().item()
        rec[key] = err
        rec[key + "_scale"] = scale
        assert err < 2e-2 * scale, (key, err, scale)
    _log_parity(rec)


@pytest.mark.parametrize("path", ["tcgen05"])
@pytest.mark.parametrize("shape", [(2, 4, 2, 2048, 128, [2048, 1500]),
                                   (1, 2, 1, 16384, 128, [16384]),      # 4-bin histogram (N >= 16384)
                                   (1, 2, 1, 16500, 64, [16500]),       # N not a multiple of 128
                                   (1, 1, 1, 65536, 128, [65536])])     # long-context tile counts
def test_tensor_core_path_matches_cuda_core_path(path, shape):
    # larger cases than the CPU oracle handles comfortably: the two kernel
    # families must agree (same rounding points, different summation order)
    B, Hq, Hkv, N, D, vl = shape
    q, k, v, do = (_randn(s, 50 + i, 1.5 if i < 3 else 1.0, torch.bfloat16) for i, s in
                   enumerate([(B, Hq, N, D), (B, Hkv, N, D), (B, Hkv, N, D), (B, Hq, N, D)]))
    varlen = torch.tensor(vl, dtype=torch.int32)
    do = _mask_rows(do, varlen)
    _use(path, q)
    a = _run(q, k, v, do, 1, varlen)
    _lib.set_kernel_path("simt")
    b = _run(q, k, v, do, 1, varlen)
    for bi in range(B):
        assert (a["tau"][bi, :, :vl[bi]] - b["tau"][bi, :, :vl[bi]]).abs().max() < 1e-5
    # the two families sum the 128 products of a score in different orders, so a
    # score within an ulp of its threshold may flip a bit: allow a handful per million tiles
    diff_bits = sum(bin(int(x) & 0xFFFFFFFF).count("1") for x in (a["bmask"] ^ b["bmask"]).flatten().tolist())
    nb = (N + 63) // 64
    assert diff_bits <= 2 + 1e-5 * B * Hq * nb * nb
    for key in ("out", "out2", "dq", "dk", "dv"):
        scale = max(1.0, b[key].abs().max().item())
        assert (a[key] - b[key]).abs().max() < 2e-2 * scale, key


@pytest.mark.parametrize("case", [
    # B, Hq, Hkv, N, D, varlen, scales of (q, k), dtype, kv heads expected on the gather kernels
    (1, 2, 2, 256, 64, None, (1.0, 1.0), torch.bfloat16, 2),
    (2, 4, 2, 1024, 128, [1024, 700], (1.5, 1.5), torch.bfloat16, 4),
    (1, 4, 1, 2048, 64, None, (1.5, 1.5), torch.float16, 1),
    (1, 2, 1, 1000, 128, [1000], (1.5, 1.5), torch.bfloat16, 1),      # N not a multiple of 32
    (3, 2, 2, 320, 64, [1, 70, 257], (1.5, 1.5), torch.bfloat16, 6),  # sequences of one row, of a tile and a bit
    (1, 2, 2, 2048, 128, None, (0.05, 1.0), torch.bfloat16, 0),       # flat rows: the pool overflows
    # unit-variance scores: the candidate pool overflows, the supports come from the final sweep
    (2, 4, 1, 16384, 128, [16384, 5000], (1.0, 1.0), torch.bfloat16, 2),
    (1, 2, 2, 512, 32, None, (1.5, 1.5), torch.bfloat16, 0),          # head dim without a gather route
])
def test_row_supports_match_tile_kernels(case):
    # Heads whose supports the solver could export run as gathers over K / V / Q / dO rows; the
    # result must be what the tile kernels give for the same thresholds (same rounding points,
    # another summation order), head by head, and two runs must agree bit for bit.
    B, Hq, Hkv, N, D, vl, (sq, sk), dtype, n_sparse = case
    q, k, v, do = (_randn(s, 80 + i, sc, dtype).cuda() for i, (s, sc) in
                   enumerate([((B, Hq, N, D), sq), ((B, Hkv, N, D), sk), ((B, Hkv, N, D), 1.5), ((B, Hq, N, D), 1.0)]))
    varlen = None if vl is None else torch.tensor(vl, dtype=torch.int32).cuda()
    _lib.set_kernel_path("tcgen05")
    shape = att.make_shape(q, k, 1, varlen)
    sup = att.support_buffer(shape, q.device)
    if n_sparse == 0 and D < 64:
        assert sup is None
        return
    sup.fill_(0x5A)   # whatever an allocator may hand out
    taus, bm = att.solve(q, k, 1, varlen, support=sup)
    taus0, bm0 = att.solve(q, k, 1, varlen)
    L = [N] * B if vl is None else vl
    # the same thresholds and block mask with and without the export -- bit for bit while the
    # solver's steps run on the same lists; a CTA whose pool overflows takes its steps on the
    # lists of a third sweep when supports are wanted and on sweeps of S otherwise, which sum the
    # same terms in another order
    for b in range(B):
        assert (taus[b, :, :L[b]] - taus0[b, :, :L[b]]).abs().max() < 2e-6
    assert _popcount(bm ^ bm0) <= 2
    dense = sup[256:256 + 4 * B * Hkv].view(torch.int32)
    assert int((dense == 0).sum()) == n_sparse
    out, out2 = att.forward_raw(q, k, v, taus, bm, varlen, support=sup)
    ref, ref2 = att.forward_raw(q, k, v, taus, bm, varlen)
    a = att.backward_raw(q, k, v, do, out2, taus, bm, varlen, 1, support=sup)
    a2 = att.backward_raw(q, k, v, do, out2, taus, bm, varlen, 1, support=sup)
    r = att.backward_raw(q, k, v, do, ref2, taus, bm, varlen, 1)
    for name, x, y in (("out", out, ref), ("out2", out2, ref2), ("dq", a[0], r[0]), ("dk", a[1], r[1]), ("dv", a[2], r[2])):
        scale = max(1.0, y.float().abs().max().item())
        assert (x.float() - y.float()).abs().max().item() < 1e-2 * scale, name
    for x, y in zip(a[:3], a2[:3]):
        assert torch.equal(x, y)
    if vl is not None:
        for b in range(B):
            if vl[b] < N:
                assert out[b, :, vl[b]:].abs().max() == 0 and a[0][b, :, vl[b]:].abs().max() == 0
                assert a[1][b, :, vl[b]:].abs().max() == 0 and a[2][b, :, vl[b]:].abs().max() == 0


@pytest.mark.parametrize("seed", range(12))
def test_row_supports_on_random_shapes(seed):
    # Seeded random problems (grouped heads, ragged lengths, odd sequence lengths, both head dims
    # and 16-bit dtypes, scales from flat to peaked, several refinement counts): whatever route
    # the device picks per kv head, the result with a support buffer must be what the tile
    # kernels alone give.
    import random
    rnd = random.Random(1000 + seed)
    D = rnd.choice([64, 128])
    Hkv = rnd.choice([1, 2, 3])
    Hq = Hkv * rnd.choice([1, 2, 4])
    B = rnd.choice([1, 2, 3])
    N = rnd.choice([64, 200, 333, 1024, 1500, 2048, 4097])
    vl = [rnd.randint(1, N) for _ in range(B)] if rnd.random() < 0.7 else None
    scale = rnd.choice([0.3, 1.0, 1.5, 2.0])
    niter = rnd.choice([0, 1, 3])
    dtype = rnd.choice([torch.bfloat16, torch.float16])
    q, k, v, do = (_randn(s, 7000 + 10 * seed + i, scale if i < 2 else 1.0, dtype).cuda() for i, s in
                   enumerate([(B, Hq, N, D), (B, Hkv, N, D), (B, Hkv, N, D), (B, Hq, N, D)]))
    varlen = None if vl is None else torch.tensor(vl, dtype=torch.int32).cuda()
    _lib.set_kernel_path("tcgen05")
    shape = att.make_shape(q, k, niter, varlen)
    sup = att.support_buffer(shape, q.device)
    assert sup is not None
    sup.fill_(0xC3)
    taus, bm = att.solve(q, k, niter, varlen, support=sup)
    out, out2 = att.forward_raw(q, k, v, taus, bm, varlen, support=sup)
    ref, ref2 = att.forward_raw(q, k, v, taus, bm, varlen)
    a = att.backward_raw(q, k, v, do, out2, taus, bm, varlen, niter, support=sup)
    r = att.backward_raw(q, k, v, do, ref2, taus, bm, varlen, niter)
    what = f"B={B} Hq={Hq} Hkv={Hkv} N={N} D={D} lens={vl} scale={scale} niter={niter} {dtype}"
    for name, x, y in (("out", out, ref), ("out2", out2, ref2), ("dq", a[0], r[0]), ("dk", a[1], r[1]), ("dv", a[2], r[2])):
        assert torch.isfinite(x.float()).all(), (name, what)
        tol = 1e-2 * max(1.0, y.float().abs().max().item())
        assert (x.float() - y.float()).abs().max().item() < tol, (name, what)


@pytest.mark.parametrize("scale, niter", [(0.05, 1), (0.05, 3), (0.4, 0), (1.5, 10), (1.5, 0)])
def test_solver_with_nearly_flat_rows(scale, niter):
    # Scores that are nearly flat put most of a row within 1 of its maximum: the solver's
    # candidate pool overflows and the CTA sweeps S for every step instead.  Peaked rows
    # (scale 1.5) stay on the candidate lists for all of their steps.  Both routes must give
    # what the CUDA-core kernels give.
    B, Hq, Hkv, N, D = 1, 2, 1, 2048, 128
    q = _randn((B, Hq, N, D), 70, scale, torch.bfloat16)
    k = _randn((B, Hkv, N, D), 71, 1.0, torch.bfloat16)
    _use("tcgen05", q)
    ta, ma = att.solve(q.cuda(), k.cuda(), niter)
    _lib.set_kernel_path("simt")
    tb, mb = att.solve(q.cuda(), k.cuda(), niter)
    torch.cuda.synchronize()
    # the two families sum the products of a score in different orders; with few refinements
    # tau is more sensitive to that than after niter >= 1 (bound: the library's 1e-4 on tau)
    err = (ta - tb).abs().max().item()
    assert err < (1e-4 if niter == 0 else 1e-5), err
    diff_bits = sum(bin(int(x) & 0xFFFFFFFF).count("1") for x in (ma ^ mb).flatten().tolist())
    assert diff_bits <= 2, diff_bits
    # nearly flat rows keep (almost) every causal 64x64 block
    nb = N // 64
    kept = sum(bin(int(x) & 0xFFFFFFFF).count("1") for x in ma.flatten().tolist())
    if scale < 0.1:
        assert kept > 0.9 * B * Hq * nb * (nb + 1) / 2


def test_c_abi_error_codes_on_device():
    import ctypes
    lib = _lib.load()
    q = torch.zeros(1, 2, 64, 64, device="cuda", dtype=torch.bfloat16)
    sh = _lib.AttnShape(B=1, Hq=2, Hkv=2, N=64, D=64, dtype=_lib.BF16, niter=1, varlen_is_i64=0,
                        path=_lib.PATH_SIMT)
    rc = lib.adasplash2_solve(q.data_ptr(), None, None, None, None, ctypes.byref(sh), None, 0, None, 0, None)
    assert rc == 1 and b"null pointer" in lib.adasplash_last_error_string()
    sh.path = 9
    rc = lib.adasplash2_fwd(*([q.data_ptr()] * 8), ctypes.byref(sh), None, 0, None, 0, None)
    assert rc == 1 and b"unknown path" in lib.adasplash_last_error_string()
