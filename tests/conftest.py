import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def flint():
    """The C-ABI library through its Python mirror. Builds it if the source is newer."""
    from libwaifu_b200 import build as B
    if B.needs_build():
        B.build()
    from libwaifu_b200 import flint as F
    F.lib()
    return F
