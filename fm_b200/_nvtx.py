"""Optional NVTX ranges around the scan's forward, backward and carry exchange.

Off by default (a range costs a few microseconds per call, which is visible next to 30-60 us
kernels); ``FMS_NVTX=1`` in the environment switches them on for a profiler timeline.  The
reference has no tracing of its own beyond compile-time ``--ptxas-options=-v``
(fm/scan/fm_scan.py:27-28).
"""
from __future__ import annotations

import contextlib
import os

_ON = os.environ.get("FMS_NVTX", "0") not in ("", "0")


@contextlib.contextmanager
def _range(name: str):
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def nvtx_range(name: str):
    """Context manager: an NVTX range when FMS_NVTX=1, otherwise nothing."""
    return _range(name) if _ON else contextlib.nullcontext()
