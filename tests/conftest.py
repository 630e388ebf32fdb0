"""Test configuration: markers and import paths."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for entry in (str(ROOT), str(ROOT / "tests")):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "expects_wait_timeout: the test makes a bounded wait run out on purpose")


@pytest.fixture(scope="session")
def golden():
    from helpers import Golden

    return Golden()


@pytest.fixture(autouse=True)
def device_status_stays_clean(request):
    """After every GPU test the status word of the pipelined kernels must be zero: a bounded wait that gave up
    leaves garbage in the outputs of that launch, and nothing else would notice."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch

    if not torch.cuda.is_available():
        return
    from white_matter_b200 import _native

    status = _native.device_status(True)
    if request.node.get_closest_marker("expects_wait_timeout") is None:
        assert status == 0, f"wait {status & 255} gave up in block {status >> 8}"
