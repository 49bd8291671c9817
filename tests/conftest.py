import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure), built on demand with gcc."""
    from oracle import binding
    binding.build()
    return binding


@pytest.fixture(scope="session")
def L():
    """The product package; importing it loads liblumen_b200.so and fails loudly if it is missing."""
    import lumen_b200
    return lumen_b200


@pytest.fixture(scope="session")
def ctx(L):
    return L.default_context()
