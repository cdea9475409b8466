"""pytest configuration: the `gpu` marker and the shared fixtures.

`-m "not gpu"` runs the oracle pins, the host logic and the ABI checks on CPU;
`-m gpu` runs the parity tests proper through the C ABI on a B200.
"""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    import checkers
    return checkers.Oracle()


@pytest.fixture(scope="session")
def ref():
    import checkers
    r = checkers.Reference.try_load()
    if r is None:
        pytest.skip("oracle/_ref/libthvm_cpu_ref.so not built (no reference checkout)")
    return r


@pytest.fixture(scope="session")
def _cuda_session():
    import torch  # noqa: F401  (device discovery only)
    import tinyhvm_b200
    be = tinyhvm_b200.CudaBackend()      # raises without a GPU or without the built library
    yield be
    err = be.last_error()
    be.shutdown()
    assert err == "", f"sticky backend error at teardown: {err}"


@pytest.fixture
def cuda(_cuda_session):
    """The process-wide backend.  The library's state is global, and the drop-in tests drive it through the
    reference's own thvm_init / thvm_free, which shut it down when they finish: bring it back up if so."""
    be = _cuda_session
    if not be.lib.thvm_cuda_stream():
        assert be.lib.thvm_cuda_init() == 0, be.last_error()
    return be
