"""fm_b200 -- the scan path of lexionbear/fm, rebuilt for NVIDIA B200 (sm_100a).

Public surface (mirrors fm/scan/fm_scan.py of the reference):

* ``fm_scan(gates, tokens, initial_state=None)`` -- differentiable scan
  ``h_t = a_t * h_{t-1} + x_t`` along the last axis of ``(B, D, T)`` tensors.
* ``FM_Scan`` -- the ``torch.autograd.Function`` behind it.
* ``fm_scan_forward`` / ``fm_scan_backward`` -- the C++ entry points (same names and argument
  order as the reference's pybind module), thin shims over the C ABI of
  ``include/fm_scan_b200.h``.
* ``fm_b200.capi`` -- ctypes binding of that C ABI (raw device pointers).

There is no CPU fallback: importing works anywhere, but calling an op without the compiled
CUDA library or without a CUDA device raises.
"""
from .fm_scan import FM_Scan, fm_scan, fm_scan_backward, fm_scan_backward_ex, fm_scan_forward  # noqa: F401

__version__ = "0.1.0"
