"""The give-up path of the bounded device-side waits, exercised without hanging anything.

Every mbarrier wait of the tensor-core kernels gives up after a fixed number of SM clocks,
records a code in the status word, lets the CTA drain and free its TMEM, and returns.  Here the
limit is shortened to 2^16 clocks and the producer warp is told to issue no streamed loads, on a
problem of one CTA: the first wait for a K tile runs out, `adasplash2_check_status` reports
ADS_ERR_TIMEOUT, and the next ordinary call on the same GPU gives the right answer.
"""
import pytest
import torch

from adasplash_b200 import _lib, attention as att

pytestmark = pytest.mark.gpu


def _randn(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()


@pytest.fixture
def short_waits():
    lib = _lib.load()
    torch.cuda.synchronize()
    yield lib
    torch.cuda.synchronize()
    assert lib.adasplash2_debug_waits(0, 0) == 0   # default limit, loads on


@pytest.mark.parametrize("kernel", ["solve", "fwd", "bwd"])
def test_wait_gives_up_and_the_gpu_stays_usable(short_waits, kernel):
    lib = short_waits
    _lib.set_kernel_path("tcgen05")
    try:
        B, H, N, D = 1, 1, 128, 128   # one CTA in every kernel
        q, k, v, do = (_randn((B, H, N, D), 80 + i, 1.5 if i < 2 else 1.0) for i in range(4))
        taus, bmask = att.solve(q, k, 1)
        out, out2 = att.forward_raw(q, k, v, taus, bmask)
        ref = att.backward_raw(q, k, v, do, out2, taus, bmask)
        torch.cuda.synchronize()
        shape = att.make_shape(q, k, 1, None)
        ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
        st = torch.cuda.current_stream().cuda_stream
        import ctypes
        sp = ctypes.byref(shape)
        P = lambda t: t.data_ptr()
        assert lib.adasplash2_debug_waits(1 << 16, 1) == 0
        if kernel == "solve":
            t2, m2 = torch.empty_like(taus), torch.empty_like(bmask)
            rc = lib.adasplash2_solve(P(q), P(k), None, P(t2), P(m2), sp, P(ws), 256, None, 0, st)
        elif kernel == "fwd":
            o, o2 = torch.empty_like(q), torch.empty_like(q)
            rc = lib.adasplash2_fwd(P(q), P(k), P(v), None, P(taus), P(bmask), P(o), P(o2), sp, P(ws), 256, None, 0, st)
        else:
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            delta, bmt = torch.empty_like(taus), torch.empty_like(bmask)
            rc = lib.adasplash2_bwd(P(q), P(k), P(v), P(do), P(out2), None, P(taus), P(bmask), P(bmt), P(delta),
                                    P(dq), P(dk), P(dv), sp, P(ws), 256, None, 0, st)
        assert rc == 0, lib.adasplash_last_error_string()   # the launch itself succeeds
        rc = lib.adasplash2_check_status(P(ws), st)
        msg = lib.adasplash_last_error_string().decode()
        assert rc == 5, (rc, msg)                            # ADS_ERR_TIMEOUT
        assert any(code in msg for code in ("code 102", "code 103")), msg
        assert lib.adasplash2_debug_waits(0, 0) == 0
        # the same GPU, the same context: an ordinary call is correct again
        t3, m3 = att.solve(q, k, 1)
        o3, o23 = att.forward_raw(q, k, v, t3, m3)
        again = att.backward_raw(q, k, v, do, o23, t3, m3)
        torch.cuda.synchronize()
        assert torch.equal(t3, taus) and torch.equal(m3, bmask) and torch.equal(o3, out)
        for a, b in zip(again[:3], ref[:3]):
            assert torch.equal(a, b)
    finally:
        _lib.set_kernel_path(None)
