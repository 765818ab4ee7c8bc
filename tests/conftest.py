import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure), built on demand with gcc."""
    from oracle import binding
    binding.build()
    return binding


@pytest.fixture(scope="session")
def nbo_lib():
    """The product library; built on demand when absent (nvcc cross-compiles without a GPU)."""
    import subprocess
    from nabla_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        subprocess.run(["make", "-C", os.path.join(ROOT, "nabla_b200", "csrc")], check=True,
                       capture_output=True)
    return _lib.load()
