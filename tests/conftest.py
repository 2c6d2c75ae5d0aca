import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device; run with -m gpu")


@pytest.fixture(scope="session")
def reference_fixtures():
    """The reference's own torch fixtures for this path (tests/golden/make_golden.py)."""
    return json.load(open(os.path.join(GOLDEN, "reference_fixtures.json")))


@pytest.fixture(scope="session")
def seeded_cases():
    idx = json.load(open(os.path.join(GOLDEN, "seeded_cases.json")))
    arrays = np.load(os.path.join(GOLDEN, "seeded_cases.npz"))
    return idx, arrays


@pytest.fixture(scope="session")
def gemm_lib():
    """Builds (if stale) and loads the CUDA library; never substitutes anything for it."""
    from tensotron_b200 import build, runtime
    build.build()
    return runtime.load_library()


@pytest.fixture(scope="session")
def rt(gemm_lib):
    import torch
    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    from tensotron_b200 import ops
    return ops.runtime(0)


def fixture_close(got, exp, atol=2e-4, rtol=2e-4):
    """The reference's fixture tolerance (tests/Tensotron.Tests/Fixtures.cs:65-79)."""
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    exp = np.asarray(exp, dtype=np.float64).reshape(-1)
    assert got.shape == exp.shape, (got.shape, exp.shape)
    bad = np.abs(got - exp) > atol + rtol * np.abs(exp)
    assert not bad.any(), "max err %g at %d" % (np.abs(got - exp).max(), int(np.argmax(np.abs(got - exp))))


def fp32_bound(K, a, b):
    """Strict-FP32 acceptance bound: 1e-5 * sqrt(K) * max|A| * max|B|."""
    amax = float(np.abs(a).max()) if np.size(a) else 0.0
    bmax = float(np.abs(b).max()) if np.size(b) else 0.0
    return 1e-5 * np.sqrt(max(K, 1)) * amax * bmax
