import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as ge
    return ge.load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own compiled code, where oracle/_ref was built or carried along."""
    from oracle.binding import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/libsdref.so not present")
    return Reference()


@pytest.fixture(scope="session")
def sdq(pkg):
    """The C-ABI library bound to GPU 0.  Fails (does not skip) when the library is missing."""
    return pkg.Sdq(int(os.environ.get("LOCAL_RANK", "0")))


GOLDEN = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
