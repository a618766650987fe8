import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "onemodel-csharp_b200"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def ctx():
    """One device context for the whole GPU session (fp32 FMA products; tests switch flags as they need)."""
    import om_binding as omb
    c = omb.Context(0, 0)
    yield c
    c.close()


@pytest.fixture(scope="session")
def oracle_built():
    from oracle import oracle
    oracle.build()
    return oracle
