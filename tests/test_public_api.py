"""Drop-in boundary: names, parameter lists and lazy loading match the
reference's adasplash/__init__.py (pinned there by tests/test_public_api.py:7-51)."""
import inspect
import subprocess
import sys

import adasplash_b200 as adasplash

EXPECTED = {
    "adasplash": ["q", "k", "v", "alpha", "is_causal", "varlen", "niter"],
    "adasplash2": ["q", "k", "v", "niter", "varlen"],
    "adasplash_v1": ["q", "k", "v", "alpha", "is_causal", "varlen", "niter"],
    "adasplash_v2": ["q", "k", "v", "niter", "varlen"],
    "adasplash_no_block_mask": ["q", "k", "v", "alpha", "is_causal", "varlen", "niter"],
    "triton_entmax": ["x", "alpha", "n_iter", "use_histogram", "fast_math"],
    "triton_entmax_v1": ["x", "alpha", "n_iter", "fast_math"],
    "triton_entmax_v2": ["x", "alpha", "n_iter", "use_histogram", "fast_math"],
    "triton_sparsemax": ["x", "kwargs"],
    "triton_entmax15": ["x", "kwargs"],
}

DEFAULTS = {
    "adasplash": dict(alpha=1.5, is_causal=True, varlen=None, niter=None),
    "adasplash_v2": dict(niter=1, varlen=None),
    "adasplash_v1": dict(alpha=1.5, is_causal=False, varlen=None, niter=10),
    "triton_entmax": dict(alpha=1.5, n_iter=2, use_histogram=True, fast_math=False),
    "triton_entmax_v1": dict(alpha=1.5, n_iter=10, fast_math=True),
}


def test_names_and_version():
    assert adasplash.__version__ == "0.2.0"
    assert set(adasplash.__all__) == set(EXPECTED) | {"__version__"}


def test_signatures():
    for name, params in EXPECTED.items():
        sig = inspect.signature(getattr(adasplash, name))
        assert list(sig.parameters) == params, name
    for name, dflt in DEFAULTS.items():
        sig = inspect.signature(getattr(adasplash, name))
        for k, v in dflt.items():
            assert sig.parameters[k].default == v, (name, k)


def test_import_is_lazy():
    code = ("import sys, adasplash_b200; "
            "assert 'adasplash_b200._lib' not in sys.modules; "
            "assert 'adasplash_b200.attention' not in sys.modules; "
            "import torch; assert not torch.cuda.is_initialized()")
    subprocess.run([sys.executable, "-c", code], check=True)


def test_v1_semantics_route_to_the_cuda_library_only():
    # alpha != 1.5 or full attention go to the v1 entry point, which has no CPU path either
    import pytest
    import torch
    q = torch.zeros(1, 1, 64, 16)
    with pytest.raises(AssertionError, match="CUDA"):
        adasplash.adasplash(q, q, q, alpha=2.0)
    with pytest.raises(AssertionError, match="CUDA"):
        adasplash.adasplash(q, q, q, is_causal=False)
