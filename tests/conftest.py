import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "tests", ROOT / "oracle"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden():
    import json

    return json.loads((ROOT / "tests" / "golden" / "reference_vectors.json").read_text())


@pytest.fixture(scope="session")
def oracle():
    import support

    return support.Oracle()


@pytest.fixture(scope="session")
def reflib():
    """The reference's own compiled host scheduler, if it has been built."""
    import support

    lib = support.RefLib.try_load()
    if lib is None:
        pytest.skip("oracle/_ref/libref_sched.so not built (no reference checkout)")
    return lib


@pytest.fixture(scope="session")
def engine():
    """The product package; building the library is the caller's job."""
    import bmoe_b200

    bmoe_b200._capi.load()
    return bmoe_b200
