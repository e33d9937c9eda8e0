import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped (not failed) when no device is visible and -m gpu was not asked for."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device visible")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _restore_launch_knobs():
    """The library caches its FMS_TUNE_* environment; a test that changed it (monkeypatch, then
    ``gpu_util.reload_tune()``) must not leak its launch shapes into the next test.  Set up before
    and therefore torn down after ``monkeypatch``, so the reload sees the restored environment."""
    yield
    from fm_b200 import capi
    if capi._lib is not None:
        capi._lib.fms_tune_reload()
