"""ctypes binding of the C ABI declared in include/adasplash_b200.h.

The shared library is built in-tree by `python -m adasplash_b200.build`.  There
is no fallback: if the library is missing, or a call returns a non-zero status,
an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_C" / "libadasplash_b200.so"

F32, F16, BF16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TCGEN05 = 0, 1, 2
_PATH_NAMES = {"auto": PATH_AUTO, "simt": PATH_SIMT, "tcgen05": PATH_TCGEN05}


class AttnShape(Structure):
    _fields_ = [(n, c_int32) for n in
                ("B", "Hq", "Hkv", "N", "D", "dtype", "niter", "varlen_is_i64", "path", "bwd_stages")] + [
                    ("alpha", c_float), ("non_causal", c_int32)]


# name -> (restype, argtypes); every symbol include/adasplash_b200.h declares
SIGNATURES = {
    "adasplash_entmax_fwd": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float,
                                       c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "adasplash_entmax_bwd": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float,
                                       c_int32, c_int32, c_void_p]),
    "adasplash2_workspace_bytes": (c_size_t, [POINTER(AttnShape)]),
    "adasplash2_bitmap_words": (c_int64, [POINTER(AttnShape), POINTER(c_int32), POINTER(c_int32)]),
    "adasplash2_support_bytes": (c_size_t, [POINTER(AttnShape)]),
    "adasplash2_solve": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   POINTER(AttnShape), c_void_p, c_size_t, c_void_p, c_size_t, c_void_p]),
    "adasplash2_mask_from_tau": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           POINTER(AttnShape), c_void_p, c_size_t, c_void_p]),
    "adasplash2_fwd": (c_int32, [c_void_p] * 8 + [POINTER(AttnShape), c_void_p, c_size_t, c_void_p, c_size_t,
                                 c_void_p]),
    "adasplash2_bwd": (c_int32, [c_void_p] * 13 + [POINTER(AttnShape), c_void_p, c_size_t, c_void_p, c_size_t,
                                 c_void_p]),
    "adasplash2_bwd_static": (c_int32, [c_void_p] * 11 + [POINTER(AttnShape), c_void_p]),
    "adasplash2_check_status": (c_int32, [c_void_p, c_void_p]),
    "adasplash2_debug_waits": (c_int32, [c_int64, c_int32]),
    "adasplash2_resolved_path": (c_int32, [POINTER(AttnShape)]),
    "adasplash_launch_count": (c_int64, []),
    "adasplash_last_error_string": (c_char_p, []),
}

_lib = None
_lock = threading.Lock()
_forced_path = None


class AdasplashError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the CUDA library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise AdasplashError(
                    f"{LIB_PATH} not found: build it with `python -m adasplash_b200.build` "
                    "(there is no CPU or PyTorch fallback)")
            lib = ctypes.CDLL(str(LIB_PATH))
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(status: int) -> None:
    if status != 0:
        msg = load().adasplash_last_error_string()
        raise AdasplashError(f"adasplash_b200 status {status}: {msg.decode() if msg else '?'}")


def set_kernel_path(name) -> None:
    """Force the attention kernel family: 'auto', 'simt' or 'tcgen05' (None = env/default)."""
    global _forced_path
    if name is not None and name not in _PATH_NAMES:
        raise ValueError(f"unknown kernel path {name!r}")
    _forced_path = name


def kernel_path() -> int:
    name = _forced_path or os.environ.get("ADASPLASH_B200_PATH", "auto")
    if name not in _PATH_NAMES:
        raise ValueError(f"ADASPLASH_B200_PATH={name!r} is not one of {sorted(_PATH_NAMES)}")
    return _PATH_NAMES[name]


def dtype_code(dtype) -> int:
    import torch
    try:
        return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[dtype]
    except KeyError:
        raise AssertionError(f"unsupported dtype {dtype}; expected float32, float16 or bfloat16")


def launch_count() -> int:
    return int(load().adasplash_launch_count())
