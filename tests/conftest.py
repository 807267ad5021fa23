import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def out_tolerance(dtype, want):
    """Absolute tolerance for attention outputs: 1e-4 in float32; in 16-bit types
    2e-2 plus half a unit in the last place of the stored value (bfloat16 keeps 8
    significant bits, float16 11: an output of magnitude 12 cannot be stored in
    bfloat16 more finely than +-0.03, whatever computed it)."""
    import torch
    if dtype == torch.float32:
        return 1e-4 + 0.0 * want.abs()
    rel = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    return 2e-2 + rel * want.abs()


def assert_out_close(got, want, dtype, tag=""):
    tol = out_tolerance(dtype, want)
    err = (got.double() - want.double()).abs()
    assert bool((err <= tol).all()), (tag, float(err.max()), float((err - tol).max()))
