"""Generate the golden fixtures in this folder by running the reference itself.

The reference (deep-spin/adasplash) is Triton code and needs a GPU, so this
script is run once on a B200 box with the unmodified reference installed under
baseline/_ref (``python -m pip install --no-index --no-build-isolation --no-deps
--target baseline/_ref <reference checkout>``; that folder is git-ignored):

    python tests/golden/make_reference_fixtures.py --out tests/golden [--time] [--big-slices]

Inputs are drawn from seeded CPU generators and stored with the outputs, so the
tests never need the reference.  ``--big-slices`` writes the fixtures at the
sequence lengths of the benchmark configurations (inputs are regenerated from the
stored seed, outputs are kept for every ``row_stride``-th row, thresholds and
block masks in full).  ``--time`` additionally times the reference's kernels
(CUDA events, median after warm-up) and merges the result into
``reference_timings.json``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _gen(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


ATTN_CASES = {
    # name: (B, Hq, Hkv, N, D, dtype, input scale, niter, varlen)
    "v2_fp32_smoke": (1, 2, 2, 256, 32, torch.float32, 1.0, 10, None),
    "v2_fp32_gqa_varlen": (1, 2, 1, 256, 64, torch.float32, 1.0, 10, [160]),
    "v2_fp32_niter1": (1, 2, 2, 512, 64, torch.float32, 1.0, 1, None),
    "v2_bf16_d128": (1, 2, 1, 512, 128, torch.bfloat16, 1.5, 1, None),
    "v2_bf16_varlen": (2, 2, 2, 256, 64, torch.bfloat16, 1.0, 1, [200, 256]),
    "v2_fp16_d64": (1, 1, 1, 256, 64, torch.float16, 1.0, 1, None),
    "v2_bf16_d128_n2048": (1, 1, 1, 2048, 128, torch.bfloat16, 1.5, 1, None),
}

# Slices of the benchmark configurations: same sequence length, head dim, dtype, input scale
# and niter, few heads.  name: (B, Hq, Hkv, N, D, input scale, niter, varlen, row_stride)
BIG_CASES = {
    "v2_bf16_c3_slice": (1, 2, 2, 8192, 128, 1.5, 1, None, 32),
    # 4-bin histogram (N >= 16384), grouped-query heads, one full and one short sequence
    "v2_bf16_c4_slice": (2, 4, 1, 16384, 128, 1.0, 1, [16384, 5000], 128),
    "v2_bf16_c5_slice": (1, 1, 1, 65536, 128, 1.5, 1, None, 128),
}
BIG_ROW_OFFSET = 5
BIG_SEED0 = 5000

V1_CASES = {
    # name: (alpha, is_causal)
    "v1_a1333_causal": (1.333, True), "v1_a1333_full": (1.333, False),
    "v1_a15_full": (1.5, False), "v1_a2_causal": (2.0, True), "v1_a2_full": (2.0, False),
}


def make_attention(adasplash, out_dir):
    for idx, (name, (B, Hq, Hkv, N, D, dt, sc, niter, vl)) in enumerate(ATTN_CASES.items()):
        seed = 1000 + idx
        q = _gen((B, Hq, N, D), seed, sc, dt)
        k = _gen((B, Hkv, N, D), seed + 100, sc, dt)
        v = _gen((B, Hkv, N, D), seed + 200, sc, dt)
        do = _gen((B, Hq, N, D), seed + 300, 1.0, dt)
        varlen = None if vl is None else torch.tensor(vl, dtype=torch.int32)
        if varlen is not None:
            rows = torch.arange(N)[None, None, :, None] < varlen[:, None, None, None]
            do = do * rows
        qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
        out = adasplash.adasplash_v2(qc, kc, vc, niter=niter,
                                     varlen=None if varlen is None else varlen.cuda())
        saved = out.grad_fn.saved_tensors
        out2, taus, bmask = saved[3], saved[4], saved[5]
        if dt == torch.float16:
            # the reference's fp16 backward does not compile under Triton 3.6
            # (tl.sqrt / bf16-style promotion on fp16 operands): forward only
            dq = dk = dv = None
        else:
            dq, dk, dv = (g.cpu() for g in torch.autograd.grad(out, (qc, kc, vc), do.cuda()))
        fx = {"q": q, "k": k, "v": v, "dout": do, "varlen": varlen, "niter": niter,
              "out": out.detach().cpu(), "out2": out2.cpu(), "taus": taus.cpu(),
              "bmask": bmask.cpu(), "dq": dq, "dk": dk, "dv": dv}
        if name.endswith("n2048"):  # keep the file small: inputs are regenerated from the seed
            for key in ("q", "k", "v", "dout"):
                fx[key] = None
            fx["seed"] = seed
            fx["scale"] = sc
            for key in ("out", "out2", "dq", "dk", "dv"):
                fx[key] = fx[key][:, :, ::8].contiguous()
            fx["row_stride"] = 8
        torch.save(fx, os.path.join(out_dir, name + ".pt"))
        print("wrote", name, flush=True)


def big_case_inputs(name):
    """q, k, v, dO, varlen of a BIG_CASES entry (CPU tensors); the tests call this too."""
    idx = list(BIG_CASES).index(name)
    B, Hq, Hkv, N, D, sc, niter, vl, stride = BIG_CASES[name]
    seed = BIG_SEED0 + 10 * idx
    dt = torch.bfloat16
    q = _gen((B, Hq, N, D), seed, sc, dt)
    k = _gen((B, Hkv, N, D), seed + 1, sc, dt)
    v = _gen((B, Hkv, N, D), seed + 2, sc, dt)
    do = _gen((B, Hq, N, D), seed + 3, 1.0, dt)
    varlen = None if vl is None else torch.tensor(vl, dtype=torch.int32)
    if varlen is not None:
        do = do * (torch.arange(N)[None, None, :, None] < varlen[:, None, None, None])
    return q, k, v, do, varlen, niter, stride


def make_big_slices(adasplash, out_dir, only=None):
    for name in BIG_CASES:
        if only and name not in only:
            continue
        q, k, v, do, varlen, niter, stride = big_case_inputs(name)
        qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
        out = adasplash.adasplash_v2(qc, kc, vc, niter=niter,
                                     varlen=None if varlen is None else varlen.cuda())
        saved = out.grad_fn.saved_tensors
        out2, taus, bmask = saved[3], saved[4], saved[5]
        dq, dk, dv = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
        rows = slice(BIG_ROW_OFFSET, None, stride)
        fx = {"case": name, "row_stride": stride, "row_offset": BIG_ROW_OFFSET, "niter": niter,
              "varlen": varlen, "taus": taus.cpu(), "bmask": bmask.cpu()}
        for key, t in (("out", out.detach()), ("out2", out2), ("dq", dq), ("dk", dk), ("dv", dv)):
            fx[key] = t[:, :, rows].contiguous().cpu()
            fx[key + "_absmax"] = float(t.float().abs().max())
        torch.save(fx, os.path.join(out_dir, name + ".pt"))
        print("wrote", name, flush=True)
        del qc, kc, vc, out, dq, dk, dv
        torch.cuda.empty_cache()


def make_v1(adasplash, out_dir):
    B, H, N, D = 1, 2, 128, 32
    for idx, (name, (alpha, causal)) in enumerate(V1_CASES.items()):
        seed = 2000 + idx
        q, k, v = (_gen((B, H, N, D), seed + 100 * i) for i in range(3))
        do = _gen((B, H, N, D), seed + 300)
        qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
        out = adasplash.adasplash(qc, kc, vc, alpha=alpha, is_causal=causal, niter=10)
        dq, dk, dv = torch.autograd.grad(out, (qc, kc, vc), do.cuda())
        torch.save({"q": q, "k": k, "v": v, "dout": do, "alpha": alpha, "is_causal": causal,
                    "out": out.detach().cpu(), "dq": dq.cpu(), "dk": dk.cpu(), "dv": dv.cpu()},
                   os.path.join(out_dir, name + ".pt"))
        print("wrote", name, flush=True)


V1_BF16_CASES = {
    # name: (alpha, is_causal) -- bf16 inputs: the cases the tensor-core kernels serve
    "v1_bf16_a2_full": (2.0, False), "v1_bf16_a2_causal": (2.0, True), "v1_bf16_a15_full": (1.5, False),
}


def make_v1_bf16(adasplash, out_dir):
    B, H, N, D = 1, 2, 256, 64
    for idx, (name, (alpha, causal)) in enumerate(V1_BF16_CASES.items()):
        seed = 2500 + idx
        q, k, v = (_gen((B, H, N, D), seed + 100 * i, 1.0, torch.bfloat16) for i in range(3))
        do = _gen((B, H, N, D), seed + 300, 1.0, torch.bfloat16)
        qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
        out = adasplash.adasplash(qc, kc, vc, alpha=alpha, is_causal=causal, niter=10)
        try:
            dq, dk, dv = (g.cpu() for g in torch.autograd.grad(out, (qc, kc, vc), do.cuda()))
        except Exception as e:  # noqa: BLE001  (a backward that does not compile for this dtype)
            print(name, "backward failed:", type(e).__name__, str(e)[:200], flush=True)
            dq = dk = dv = None
        torch.save({"q": q, "k": k, "v": v, "dout": do, "alpha": alpha, "is_causal": causal,
                    "out": out.detach().cpu(), "dq": dq, "dk": dk, "dv": dv},
                   os.path.join(out_dir, name + ".pt"))
        print("wrote", name, flush=True)


def time_v1(adasplash, out_dir):
    """alpha = 2, full attention, B=4 H=32 N=8192 D=64 bf16: the first-generation kernels."""
    path = os.path.join(out_dir, "reference_timings.json")
    res = json.load(open(path)) if os.path.exists(path) else {}
    g = torch.Generator(device="cuda").manual_seed(77)
    q, k, v, do = (torch.randn(4, 32, 8192, 64, device="cuda", generator=g).bfloat16() for _ in range(4))
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))

    def fb():
        o = adasplash.adasplash(q, k, v, alpha=2.0, is_causal=False)
        torch.autograd.grad(o, (q, k, v), do)
    t0 = time.time()
    fb()
    torch.cuda.synchronize()
    res["V1_a2_full_B4_H32_N8192_D64_first_call_s"] = time.time() - t0
    res["V1_a2_full_B4_H32_N8192_D64_fwd_ms"] = _time(lambda: adasplash.adasplash(q, k, v, alpha=2.0, is_causal=False), 5)
    res["V1_a2_full_B4_H32_N8192_D64_fwdbwd_ms"] = _time(fb, 5)
    print("v1", res["V1_a2_full_B4_H32_N8192_D64_fwd_ms"], res["V1_a2_full_B4_H32_N8192_D64_fwdbwd_ms"], flush=True)
    with open(path, "w") as f:
        json.dump(res, f, indent=1)


def make_rowwise(adasplash, out_dir):
    fx = {}
    x = _gen((16, 4096), 3000, 4.0)
    dy = _gen((16, 4096), 3001)
    fx["x"], fx["dy"] = x, dy
    for tag, kw in (("a15_hist", dict(alpha=1.5, n_iter=2, use_histogram=True)),
                    ("a2_default", dict(alpha=2.0)),
                    ("a1333", dict(alpha=1.333, use_histogram=False)),
                    ("a15_nohist_it10", dict(alpha=1.5, n_iter=10, use_histogram=False))):
        xc = x.cuda().requires_grad_(True)
        y = adasplash.triton_entmax(xc, **kw)
        (dx,) = torch.autograd.grad(y, xc, dy.cuda())
        fx[tag] = {"kwargs": kw, "y": y.detach().cpu(), "dx": dx.cpu()}
    xs = _gen((4, 8, 100), 3002, 2.0, torch.float16)
    dys = _gen((4, 8, 100), 3003, 1.0, torch.float16)
    fx["x_small_f16"], fx["dy_small_f16"] = xs, dys
    for tag, kw in (("small_a15", dict(alpha=1.5)), ("small_a2", dict(alpha=2.0)),
                    ("small_a1333", dict(alpha=1.333))):
        # forward only: the reference's fp16 backward (tl.sqrt on fp16) does not
        # compile under Triton 3.6
        y = adasplash.triton_entmax(xs.cuda(), **kw)
        fx[tag] = {"kwargs": kw, "y": y.detach().cpu(), "dx": None}
    torch.save(fx, os.path.join(out_dir, "rowwise.pt"))
    print("wrote rowwise", flush=True)


def _time(fn, reps=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def _time_attention_case(adasplash, res, tag, B, Hq, Hkv, N, D, sc, reps, varlen_seed=None):
    g = torch.Generator(device="cuda").manual_seed(1234)

    def rn(shape, s):
        return (torch.randn(shape, device="cuda", generator=g) * s).bfloat16()
    q, k, v = (rn((B, h, N, D), sc).requires_grad_(True) for h in (Hq, Hkv, Hkv))
    do = rn((B, Hq, N, D), 1.0)
    varlen = None
    if varlen_seed is not None:
        gc = torch.Generator().manual_seed(varlen_seed)
        varlen = torch.randint(N // 4, N + 1, (B,), generator=gc, dtype=torch.int32)
        res[tag + "_varlen"] = [int(x) for x in varlen]
        do = do * (torch.arange(N, device="cuda")[None, None, :, None] < varlen.cuda()[:, None, None, None])
        varlen = varlen.cuda()
    t0 = time.time()
    out = adasplash.adasplash_v2(q, k, v, niter=1, varlen=varlen)
    bm = out.grad_fn.saved_tensors[5][0, 0].clone()
    torch.autograd.grad(out, (q, k, v), do)
    torch.cuda.synchronize()
    res[tag + "_first_call_s"] = time.time() - t0
    res[tag + "_fwd_ms"] = _time(lambda: adasplash.adasplash_v2(q, k, v, niter=1, varlen=varlen), reps)

    def fb():
        o = adasplash.adasplash_v2(q, k, v, niter=1, varlen=varlen)
        torch.autograd.grad(o, (q, k, v), do)
    res[tag + "_fwdbwd_ms"] = _time(fb, reps)
    L = N if varlen is None else int(varlen[0])
    nb = (L + 63) // 64
    active = sum(bin(int(w) & 0xFFFFFFFF).count("1") for w in bm.flatten().tolist())
    res[tag + "_block_sparsity_head0"] = 1.0 - active / (nb * (nb + 1) / 2)
    print(tag, res[tag + "_fwd_ms"], res[tag + "_fwdbwd_ms"], flush=True)


TIME_CASES = {
    # tag: (B, Hq, Hkv, N, D, input scale, reps, varlen seed)
    "small": ("B1_H2_N256_D64", (1, 2, 2, 256, 64, 1.0, 50, None)),
    "n4096": ("B1_H8_N4096_D128", (1, 8, 8, 4096, 128, 1.5, 10, None)),
    "c3": ("C3_B4_H32_N8192_D128", (4, 32, 32, 8192, 128, 1.5, 5, None)),
    "c4": ("C4_B8_Hq32_Hkv8_N16384_D128_varlen", (8, 32, 8, 16384, 128, 1.0, 3, 20263)),
    # one (batch, kv-head) shard of the long-context configuration: 1/16 of its work
    "c5shard": ("C5shard_B1_Hq8_Hkv1_N65536_D128", (1, 8, 1, 65536, 128, 1.5, 3, None)),
}


def time_reference(adasplash, out_dir, cases, suffix=""):
    path = os.path.join(out_dir, "reference_timings.json")
    res = json.load(open(path)) if os.path.exists(path) else {}
    res.update({"device": torch.cuda.get_device_name(0), "torch": torch.__version__})
    import triton
    res["triton"] = triton.__version__

    def flush():
        with open(path, "w") as f:
            json.dump(res, f, indent=1)
    if "rowwise" in cases:
        # row-wise, 16384 x 4096 fp32
        x = (torch.randn(16384, 4096, device="cuda") * 4).requires_grad_(True)
        dy = torch.randn(16384, 4096, device="cuda")
        for tag, kw in (("a15_hist", dict(alpha=1.5, n_iter=2, use_histogram=True)),
                        ("a2_default", dict(alpha=2.0)), ("a1333", dict(alpha=1.333, use_histogram=False))):
            y = adasplash.triton_entmax(x, **kw)
            res["rowwise_fwd_ms_" + tag] = _time(lambda: adasplash.triton_entmax(x, **kw))
            res["rowwise_bwd_ms_" + tag] = _time(lambda: torch.autograd.grad(y, x, dy, retain_graph=True))
            print(tag, res["rowwise_fwd_ms_" + tag], res["rowwise_bwd_ms_" + tag], flush=True)
        del x, dy
        flush()
    for name, (tag, cfg) in TIME_CASES.items():
        if name in cases:
            _time_attention_case(adasplash, res, tag + suffix, *cfg)
            torch.cuda.empty_cache()
            flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden"))
    ap.add_argument("--ref", default=os.path.join(ROOT, "baseline", "_ref"))
    ap.add_argument("--time", default="", help="comma list of: rowwise," + ",".join(TIME_CASES) + " (or 'all')")
    ap.add_argument("--skip-fixtures", action="store_true", help="do not rewrite the small fixtures")
    ap.add_argument("--big-slices", default=None, nargs="?", const="all",
                    help="write the benchmark-length slice fixtures (all, or a comma list of names)")
    ap.add_argument("--v1-bf16", action="store_true", help="write the bf16 first-generation fixtures and time that path")
    ap.add_argument("--single-config", action="store_true",
                    help="set the reference's ADASPLASH_TEST_FAST_AUTOTUNE=1 (one tuning candidate per kernel, "
                         "as its own test suite does): at 65536 positions the full autotune compiles for more "
                         "than 16 minutes.  Timings taken this way get the suffix _single_config.")
    a = ap.parse_args()
    if a.single_config:
        os.environ["ADASPLASH_TEST_FAST_AUTOTUNE"] = "1"
    sys.path.insert(0, a.ref)
    import adasplash
    assert os.path.abspath(adasplash.__file__).startswith(os.path.abspath(a.ref)), adasplash.__file__
    os.makedirs(a.out, exist_ok=True)
    if not a.skip_fixtures:
        make_rowwise(adasplash, a.out)
        make_attention(adasplash, a.out)
        make_v1(adasplash, a.out)
    # Slices first: the reference's autotuner is keyed on (sequence length, head dim) only, so the
    # few-head slice tunes in a minute or two and a timing case of the same length that follows in
    # this process reuses the choice.  (Tuning on a full-size batch runs every candidate on it:
    # the 16384-long configuration took 560 s that way.)
    if a.v1_bf16:
        make_v1_bf16(adasplash, a.out)
        time_v1(adasplash, a.out)
    if a.big_slices:
        make_big_slices(adasplash, a.out, None if a.big_slices == "all" else a.big_slices.split(","))
    if a.time:
        cases = ["rowwise"] + list(TIME_CASES) if a.time == "all" else a.time.split(",")
        time_reference(adasplash, a.out, cases, "_single_config" if a.single_config else "")


if __name__ == "__main__":
    main()
