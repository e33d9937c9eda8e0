"""fm_b200 -- the scan path of lexionbear/fm, rebuilt for NVIDIA B200 (sm_100a).

Public surface (mirrors fm/scan/fm_scan.py of the reference):

* ``fm_scan(gates, tokens, initial_state=None)`` -- differentiable scan
  ``h_t = a_t * h_{t-1} + x_t`` along the last axis of ``(B, D, T)`` tensors.
* ``FM_Scan`` -- the ``torch.autograd.Function`` behind it.
* ``fm_scan_forward`` / ``fm_scan_backward`` -- the C++ entry points (same names and argument
  order as the reference's pybind module), thin shims over the C ABI of
  ``include/fm_scan_b200.h``.
* ``fm_scan(..., mode="fm")`` / ``FM_Scan_Outer`` -- the reference's own layout
  (B,M,L) x (B,D,L) -> (B,M,D,L) with the ``1 - gate`` token weight, gradient reductions fused.
* ``fm_memory`` -- the layer around the scan (fm/scan/fm_scan.py:102-133).
* ``fm_b200.capi`` -- ctypes binding of that C ABI (raw device pointers).

There is no CPU fallback: importing works anywhere, but calling an op without the compiled
CUDA library or without a CUDA device raises.
"""
from .fm_scan import (FM_Scan, FM_Scan_Outer, fm_scan, fm_scan_backward, fm_scan_backward_ex,  # noqa: F401
                      fm_scan_backward_fm, fm_scan_forward)

from .fm_memory import fm_memory  # noqa: F401,E402

__version__ = "0.1.0"
