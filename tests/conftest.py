"""pytest configuration: the `gpu` marker and shared fixtures.

`-m "not gpu"` covers the oracle against the golden vectors, the host logic and the
C-ABI symbol table; `-m gpu` holds the parity tests proper, which call the CUDA
library through its C ABI and compare with the oracle on the same seeded inputs.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# tolerances of the parity gate for floating-point outputs (bf16 operands, fp32 accumulate)
MAX_ABS_TOL = 2e-2
MEAN_REL_TOL = 5e-3


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device")


def _cuda_ok():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _cuda_ok():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "attn_golden.npz"))


@pytest.fixture(scope="session")
def lib_built():
    from mx230_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def handle(lib_built):
    """One library handle on cuda:0 with a workspace large enough for every test."""
    import torch
    from mx230_b200.common import Handle
    torch.cuda.set_device(0)
    h = Handle(0, 256 << 20)
    yield h
    h.check_status()
    h.close()


def assert_close(got, want, what, max_abs=MAX_ABS_TOL, mean_rel=MEAN_REL_TOL):
    """Parity gate: max-abs error and norm-wise mean relative error sum|g-w|/sum|w|."""
    import oracle
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values in the result"
    ma, mr = oracle.max_abs_err(got, want), oracle.mean_rel_err(got, want)
    assert ma <= max_abs and mr <= mean_rel, \
        f"{what}: max-abs {ma:.3e} (tol {max_abs:g}), mean-rel {mr:.3e} (tol {mean_rel:g})"
    return ma, mr
