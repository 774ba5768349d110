import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (runs the CUDA kernels through the C ABI)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure), built on demand from oracle/Makefile."""
    import oracle as O

    O.build()
    return O


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "golden_small.npz"))


@pytest.fixture(scope="session")
def dev():
    """One CudaDevice (galois_b200 context on cuda:0) for the whole session."""
    import galois_b200 as gb

    d = gb.CudaDevice(0)
    yield d
    d.close()


# tolerances stated by the task for float outputs (order of block-scale accumulation differs)
REL_L2_TOL = 1e-4
MAX_ABS_TOL = 1e-3


def assert_close(got, want, rel_l2=REL_L2_TOL, max_abs=MAX_ABS_TOL):
    import numpy as np

    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.all(np.isfinite(got) == np.isfinite(want))
    fin = np.isfinite(want)
    diff = np.abs(got[fin] - want[fin])
    denom = np.linalg.norm(want[fin])
    rel = np.linalg.norm(got[fin] - want[fin]) / denom if denom > 0 else np.linalg.norm(got[fin])
    assert rel <= rel_l2, f"relative L2 {rel:.3e} > {rel_l2:.1e}"
    if diff.size:
        assert diff.max() <= max_abs, f"max abs {diff.max():.3e} > {max_abs:.1e}"
