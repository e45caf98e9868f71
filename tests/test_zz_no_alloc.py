"""The allocation-free backward entry point against the ordinary one.

`adasplash2_bwd_static` serves callers that cannot obtain device memory at call
time (plugins that only receive pointers, code inside allocation-free regions):
its scratch is a fixed array inside the library.  The test calls it through the
C ABI twice in a row -- the second call starts from whatever the first left in
the shared array -- and requires the same dq, dk, dv as `adasplash2_bwd` with
caller-owned scratch.  The file sorts last so that a stop-at-first-failure run
has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _randn(shape, seed, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("case", [
    # B, Hq, Hkv, N, D, dtype, varlen
    (2, 4, 2, 384, 128, torch.bfloat16, [384, 200]),
    (1, 2, 2, 256, 32, torch.float32, None),
])
def test_static_backward_matches_ordinary_backward_twice(case):
    from adasplash_b200 import _lib, attention as att
    B, Hq, Hkv, N, D, dtype, vl = case
    lib = _lib.load()
    q, k, v = _randn((B, Hq, N, D), 1, 1.5, dtype), _randn((B, Hkv, N, D), 2, 1.5, dtype), _randn((B, Hkv, N, D), 3, 1.0, dtype)
    varlen = None if vl is None else torch.tensor(vl, dtype=torch.int32, device="cuda")
    taus, bmask = att.solve(q, k, 1, varlen)
    out, out2 = att.forward_raw(q, k, v, taus, bmask, varlen)
    shape = att.make_shape(q, k, 1, varlen)
    st = torch.cuda.current_stream().cuda_stream
    ptr = lambda t: None if t is None else t.data_ptr()
    for trial in range(2):
        do = _randn((B, Hq, N, D), 10 + trial, 1.0, dtype)
        ref_dq, ref_dk, ref_dv, _, _ = att.backward_raw(q, k, v, do, out2, taus, bmask, varlen, 1)
        dq, dk, dv = torch.full_like(q, 7), torch.full_like(k, 7), torch.full_like(v, 7)
        rc = lib.adasplash2_bwd_static(ptr(q), ptr(k), ptr(v), ptr(do), ptr(out2), ptr(varlen), ptr(taus),
                                       ptr(bmask), ptr(dq), ptr(dk), ptr(dv), ctypes.byref(shape), st)
        assert rc == 0, lib.adasplash_last_error_string()
        # the caller owns no workspace: a NULL workspace reads the status word of the built-in array
        assert lib.adasplash2_check_status(None, st) == 0, lib.adasplash_last_error_string()
        torch.cuda.synchronize()
        # same kernels, same inputs, deterministic: the results must be identical
        tol = 0.0
        for name, a, b in (("dq", dq, ref_dq), ("dk", dk, ref_dk), ("dv", dv, ref_dv)):
            assert (a.float() - b.float()).abs().max().item() <= tol, (trial, name)


def test_static_backward_allocates_nothing():
    """The property the entry point exists for: once its address is cached, a call leaves both
    torch's allocator counters and the device's free memory untouched."""
    from adasplash_b200 import _lib, attention as att
    lib = _lib.load()
    B, Hq, Hkv, N, D = 1, 2, 1, 256, 64
    q, k, v, do = (_randn((B, h, N, D), 20 + i) for i, h in enumerate((Hq, Hkv, Hkv, Hq)))
    taus, bmask = att.solve(q, k, 1, None)
    out, out2 = att.forward_raw(q, k, v, taus, bmask, None)
    shape = att.make_shape(q, k, 1, None)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    st = torch.cuda.current_stream().cuda_stream
    args = [t.data_ptr() for t in (q, k, v, do, out2)] + [None] + [t.data_ptr() for t in (taus, bmask, dq, dk, dv)]

    def call():
        assert lib.adasplash2_bwd_static(*args, ctypes.byref(shape), st) == 0, lib.adasplash_last_error_string()
        torch.cuda.synchronize()
    call()  # first call on the device: looks up and caches the array's address
    stats0 = torch.cuda.memory_stats()
    free0, _ = torch.cuda.mem_get_info()
    call()
    free1, _ = torch.cuda.mem_get_info()
    stats1 = torch.cuda.memory_stats()
    assert free1 == free0
    for key in ("allocation.all.allocated", "segment.all.allocated", "allocated_bytes.all.current",
                "reserved_bytes.all.current"):
        assert stats1[key] == stats0[key], key


def test_static_backward_rejects_partial_backward():
    from adasplash_b200 import _lib
    lib = _lib.load()
    sh = _lib.AttnShape(B=1, Hq=2, Hkv=2, N=128, D=64, dtype=_lib.BF16, niter=1, varlen_is_i64=0, path=0)
    sh.bwd_stages = 4   # dQ alone would read delta left behind by an earlier call
    one = torch.zeros(1, device="cuda")
    p = one.data_ptr()
    rc = lib.adasplash2_bwd_static(p, p, p, p, p, None, p, p, p, p, p, ctypes.byref(sh), None)
    assert rc == 1 and b"bwd_stages" in lib.adasplash_last_error_string()


def test_static_backward_rejects_oversized_problems():
    from adasplash_b200 import _lib
    lib = _lib.load()
    # 4 * B*Hq*N alone exceeds the 8 MiB built-in buffer
    sh = _lib.AttnShape(B=8, Hq=32, Hkv=8, N=16384, D=128, dtype=_lib.BF16, niter=1, varlen_is_i64=0, path=0)
    one = torch.zeros(1, device="cuda")
    p = one.data_ptr()
    rc = lib.adasplash2_bwd_static(p, p, p, p, p, None, p, p, p, p, p, ctypes.byref(sh), None)
    assert rc == 3
    msg = lib.adasplash_last_error_string().decode()
    assert "built-in buffer" in msg and "adasplash2_bwd" in msg
