import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def nv():
    """The product package; importing it loads libnova_b200.so (built on demand where nvcc exists)."""
    import __graft_entry__ as g
    lib = os.path.join(g.PKG_DIR, "libnova_b200.so")
    if not os.path.exists(lib):
        g.build()
    return g.load_package()


@pytest.fixture(scope="session")
def ob():
    """The checker (CPU oracle + reference-derived libraries): test infrastructure only."""
    from oracle import binding
    binding.oracle()
    return binding
