import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def ref():
    """The CPU oracle (test infrastructure; the product never imports it)."""
    from oracle import ref as r

    r.build()
    r.lib()
    return r


@pytest.fixture(scope="session")
def gpu():
    """A context on cuda:0 through the C ABI. Fails (does not skip) without the
    built library or a device: the GPU tier must never pass on a fallback."""
    from zllm_b200 import abi

    ctx = abi.Context(0)
    yield ctx
    ctx.close()


@pytest.fixture()
def launcher(gpu):
    from zllm_b200 import kernels

    return kernels.Launcher(gpu)
