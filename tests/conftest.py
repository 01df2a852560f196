import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselected on CPU-only machines")


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return ROOT / "tests" / "golden"


@pytest.fixture(scope="session")
def built_lib():
    """libmgr_b200.so, brought up to date with its sources (nvcc cross-compiles without a GPU). The build is
    incremental: with unchanged sources it only compares fingerprints, so a stale library is never tested."""
    from mgrrmsnorm_b200 import _capi, build

    build.build()
    return _capi.lib()


@pytest.fixture
def mgr_env():
    """Setter for the library's MGR_* overrides: `mgr_env("MGR_RMSNORM_PATH", "ring")`. The library reads its
    environment once, so every change is followed by mgr_reload_env(); the old values come back (and are
    re-read) when the test ends."""
    import os

    from mgrrmsnorm_b200 import _capi

    saved = {}

    def set_(name: str, value: str) -> None:
        saved.setdefault(name, os.environ.get(name))
        os.environ[name] = value
        _capi.reload_env()

    yield set_
    for name, old in saved.items():
        if old is None:
            os.environ.pop(name, None)
        else:
            os.environ[name] = old
    if saved:
        _capi.reload_env()


@pytest.fixture(scope="session", autouse=True)
def no_kernel_gave_up_a_wait():
    """After the last test on a GPU machine: no kernel of the session may have left the timeout status behind
    (tests that write the status word on purpose clear it themselves)."""
    yield
    if not _has_gpu():
        return
    from mgrrmsnorm_b200 import _capi

    if _capi.LIB_PATH.exists():
        assert _capi.lib().mgr_device_status(1) == _capi.MGR_OK, "a kernel's bounded wait ran out during the test session"
