"""Forward + backward for tensors that live in HOST memory (ctypes over the C ABI).

``HostPipeline`` owns a device staging area (a torch allocation handed to
``fms_pipeline_create``, which itself allocates no device memory) and streams blocks of rows
host -> device -> kernels -> host on three internal streams, so both PCIe directions and the
kernels overlap.  This is the entry a host-resident caller would use where the reference offers
only its CPU loop (fm/scan/fm_pytorch.py:3-42).
"""
from __future__ import annotations

import ctypes

import torch

from . import capi

_P, _I64, _I, _SZ = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t


def _bind():
    L = capi.lib()
    if not getattr(L, "_fms_pipeline_bound", False):
        L.fms_pipeline_workspace_bytes.restype = _SZ
        L.fms_pipeline_workspace_bytes.argtypes = [_I64, _I64, _I]
        L.fms_pipeline_create.restype = _I
        L.fms_pipeline_create.argtypes = [ctypes.POINTER(_P), _P, _SZ]
        L.fms_pipeline_destroy.restype = _I
        L.fms_pipeline_destroy.argtypes = [_P]
        L.fms_plain_forward_backward_host.restype = _I
        L.fms_plain_forward_backward_host.argtypes = [_P] * 7 + [_I64, _I64, _I, _P]
        L.fms_pipeline_copy_probe.restype = _I
        L.fms_pipeline_copy_probe.argtypes = [_P] * 7 + [_I64, _I64, _I, _P]
        L._fms_pipeline_bound = True
    return L


def workspace_bytes(rows_per_block: int, T: int, dtype: torch.dtype) -> int:
    return int(_bind().fms_pipeline_workspace_bytes(rows_per_block, T, capi.dtype_tag(dtype)))


class HostPipeline:
    """Staging area + streams for ``forward_backward`` on host tensors; one call at a time."""

    def __init__(self, rows_per_block: int, T: int, dtype: torch.dtype, device=None):
        self._L = _bind()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        nbytes = workspace_bytes(rows_per_block, T, dtype)
        if nbytes == 0:
            raise ValueError("rows_per_block and T must be positive and dtype fp32/fp16/bf16")
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        handle = _P()
        with torch.cuda.device(self.device):
            rc = self._L.fms_pipeline_create(ctypes.byref(handle), self.workspace.data_ptr(), nbytes)
        if rc != capi.FMS_OK:
            raise capi.FmsError("fms_pipeline_create", rc, capi.status_string(rc),
                                int(self._L.fms_last_cuda_error()))
        self._handle = handle

    def forward_backward(self, gates, tokens, grad_states, states, grad_gates, grad_tokens):
        """All six are contiguous CPU tensors (ideally pinned) of one shape (..., T) and dtype.

        Asynchronous with respect to the host: the work is ordered on the current stream of the
        pipeline's device; synchronise that stream before reading the outputs.
        """
        self._run("fms_plain_forward_backward_host", gates, tokens, grad_states, states, grad_gates, grad_tokens)

    def copy_only(self, gates, tokens, grad_states, states, grad_gates, grad_tokens):
        """The same copies in the same order with the kernels skipped (``fms_pipeline_copy_probe``):
        what the host links alone allow.  The outputs receive stale staging data."""
        self._run("fms_pipeline_copy_probe", gates, tokens, grad_states, states, grad_gates, grad_tokens)

    def _run(self, entry, gates, tokens, grad_states, states, grad_gates, grad_tokens):
        ts = (gates, tokens, grad_states, states, grad_gates, grad_tokens)
        for t in ts:
            if t.is_cuda or not t.is_contiguous() or t.shape != gates.shape or t.dtype != gates.dtype:
                raise RuntimeError("host pipeline expects contiguous CPU tensors of one shape and dtype")
        T = gates.shape[-1]
        rows = gates.numel() // T if T else 0
        with torch.cuda.device(self.device):
            rc = getattr(self._L, entry)(
                self._handle, *(t.data_ptr() for t in ts), rows, T, capi.dtype_tag(gates.dtype),
                torch.cuda.current_stream(self.device).cuda_stream)
        if rc != capi.FMS_OK:
            raise capi.FmsError(entry, rc, capi.status_string(rc),
                                int(self._L.fms_last_cuda_error()))

    def close(self):
        if getattr(self, "_handle", None):
            torch.cuda.synchronize(self.device)
            self._L.fms_pipeline_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
