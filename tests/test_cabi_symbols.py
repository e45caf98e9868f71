"""The shared library loads without a GPU and exports every symbol that
include/adasplash_b200.h declares (no compute calls here)."""
import ctypes
import os
import re

from adasplash_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "adasplash_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(adasplash2?_[a-z0-9_]+)\s*\(", text)))


def test_header_matches_binding_table():
    assert _declared() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in _declared():
        assert hasattr(lib, name), name


def test_error_reporting_without_gpu():
    lib = _lib.load()
    before = lib.adasplash_launch_count()
    # negative sizes are rejected before any CUDA call
    rc = lib.adasplash_entmax_fwd(None, None, None, -1, 4, 1.5, 2, 1, 0, 0, None)
    assert rc == 1
    assert b"bad argument" in lib.adasplash_last_error_string()
    sh = _lib.AttnShape(B=1, Hq=3, Hkv=2, N=64, D=64, dtype=0, niter=1, varlen_is_i64=0, path=0)
    assert lib.adasplash2_resolved_path(ctypes.byref(sh)) == -1
    assert b"not a multiple" in lib.adasplash_last_error_string()
    sh = _lib.AttnShape(B=1, Hq=2, Hkv=2, N=64, D=48, dtype=0, niter=1, varlen_is_i64=0, path=0)
    assert lib.adasplash2_workspace_bytes(ctypes.byref(sh)) == 0
    sh = _lib.AttnShape(B=1, Hq=2, Hkv=2, N=32, D=64, dtype=0, niter=1, varlen_is_i64=0, path=0)
    assert lib.adasplash2_resolved_path(ctypes.byref(sh)) == -1
    assert lib.adasplash_launch_count() == before


def test_backward_rejects_misaligned_rows_without_gpu():
    # dout / out2 are read 16 bytes at a time; a misaligned base is refused before any launch
    lib = _lib.load()
    before = lib.adasplash_launch_count()
    sh = _lib.AttnShape(B=1, Hq=2, Hkv=2, N=64, D=64, dtype=2, niter=1, varlen_is_i64=0, path=0)
    a = 0x1000  # stands for a device address; never dereferenced by the argument checks
    args = [a, a, a, a + 8, a, None, a, a, a, a, a, a, a]   # dout = a + 8
    rc = lib.adasplash2_bwd(*args, ctypes.byref(sh), a, 256, None, 0, None)
    assert rc == 1
    assert b"16-byte aligned" in lib.adasplash_last_error_string()
    assert lib.adasplash_launch_count() == before


def test_bitmap_extent_matches_reference_layout():
    # rows_padded = max(32, ceil32(nb)), n_words = ceil(nb/32) (adasplash_v2.py:1345-1350)
    lib = _lib.load()
    for n, rows, words in ((64, 32, 1), (2048, 32, 1), (2112, 64, 2), (8192, 128, 4), (65536, 1024, 32)):
        sh = _lib.AttnShape(B=2, Hq=3, Hkv=3, N=n, D=64, dtype=2, niter=1, varlen_is_i64=0, path=0)
        r, w = ctypes.c_int32(), ctypes.c_int32()
        total = lib.adasplash2_bitmap_words(ctypes.byref(sh), ctypes.byref(r), ctypes.byref(w))
        assert (r.value, w.value, total) == (rows, words, 6 * rows * words)


def test_support_and_workspace_sizes_without_gpu():
    # The gather route exists for 16-bit inputs, head dim 64 / 128 and up to 65536 keys; elsewhere no support buffer is asked for and the workspace is the status word.
    lib = _lib.load()

    def sizes(**kw):
        base = dict(B=2, Hq=4, Hkv=2, N=4096, D=128, dtype=2, niter=1, varlen_is_i64=0, path=0)
        base.update(kw)
        sh = _lib.AttnShape(**base)
        return lib.adasplash2_support_bytes(ctypes.byref(sh)), lib.adasplash2_workspace_bytes(ctypes.byref(sh))

    rows = 2 * 4 * 4096
    sup, ws = sizes()
    # cursor + route counters + key norms, (first, count) per row, 32 entries of 8 bytes per row
    assert sup == 256 + 256 + 256 + rows * 8 + rows * 32 * 8
    # status word + the backward's sorted copy, run table (16 blocks of 256 rows per head) and key-block table
    blocks = 2 * 4 * 16
    assert ws == 256 + rows * 32 * 8 + blocks * 8 + ((blocks * 129 * 2 + 255) // 256) * 256   # 4096 / 32 + 1 table entries per block
    assert sizes(dtype=0) == (0, 256)            # fp32: CUDA-core kernels
    assert sizes(D=32) == (0, 256)               # head dim without a gather route
    assert sizes(N=131072) == (0, 256)           # key indices would not fit 16 bits
    assert sizes(alpha=2.0, non_causal=1)[0] == sup     # first-generation semantics: any alpha, causal or full
    assert sizes(path=1) == (0, 256)             # CUDA-core kernels asked for explicitly
    # a support buffer that is too small is refused before any launch
    sh = _lib.AttnShape(B=2, Hq=4, Hkv=2, N=4096, D=128, dtype=2, niter=1, varlen_is_i64=0, path=0)
    a = 0x1000
    before = lib.adasplash_launch_count()
    rc = lib.adasplash2_solve(a, a, None, a, a, ctypes.byref(sh), a, 256, a, 1024, None)
    assert rc == 3 and b"support buffer too small" in lib.adasplash_last_error_string()
    args = [a] * 5 + [None] + [a] * 7
    rc = lib.adasplash2_bwd(*args, ctypes.byref(sh), a, 256, a, sup, None)
    assert rc == 3 and b"workspace" in lib.adasplash_last_error_string()
    assert lib.adasplash_launch_count() == before
