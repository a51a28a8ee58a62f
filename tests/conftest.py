import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.pyoracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU code, when oracle/_ref/libref.so has been built."""
    from oracle import pyoracle
    if not os.path.exists(pyoracle.REF_SO):
        pytest.skip("oracle/_ref/libref.so not built on this machine")
    return pyoracle.Ref()


@pytest.fixture(scope="session")
def tb():
    """The product library on cuda:0 (no fallback: a missing library is an error, not a skip)."""
    import torch
    assert torch.cuda.is_available(), "a test marked gpu ran without a CUDA device"
    from turkce_llm_b200 import lib
    lib.init(0)
    return lib


def golden_path(name):
    return os.path.join(GOLDEN, name)


def rel_to_maxabs(got, want):
    """The reference's compare_tensor metric (tests/test_gpu_train.c:53-66): max |got-want| / max |want|."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(got - want).max() / (np.abs(want).max() + 1e-30))


def compare_tensor_bad(got, want, rel_tol):
    """Count of elements outside the reference's per-element tolerance (tests/test_gpu_train.c:53-66)."""
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    maxabs = np.abs(want).max() if want.size else 0.0
    floor = maxabs * rel_tol + 1e-12
    tol = floor + rel_tol * np.abs(want)
    return int((np.abs(got - want) > tol).sum())
