"""ctypes binding of the C ABI declared in ``include/fm_scan_b200.h``.

This is the binding a host program without torch would write; the tests call the kernels
through it so that parity is established at the C boundary, not only through the torch shim.
Pointers are plain integers (``tensor.data_ptr()``), the stream is a ``cudaStream_t`` value.
The library is loaded lazily and loading fails loudly when it has not been built: there is no
fallback implementation.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfm_scan_b200.so"

FMS_F32, FMS_F16, FMS_BF16 = 0, 1, 2
FMS_OK = 0
FMS_ERR_BAD_SHAPE, FMS_ERR_BAD_DTYPE, FMS_ERR_NULL_POINTER, FMS_ERR_MISALIGNED = 1, 2, 3, 4
FMS_ERR_LAUNCH, FMS_ERR_WORKSPACE, FMS_ERR_TOO_LARGE, FMS_ERR_NO_DEVICE = 5, 6, 7, 8

_P, _I64, _I = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int

# name -> argument types; every function returns int.  Kept in one table so the export test can
# compare it with the header.
SIGNATURES = {
    "fms_plain_forward": [_P, _P, _P, _P, _P, _I64, _I64, _I, _P],
    "fms_plain_backward": [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I, _P],
    "fms_plain_reduce": [_P, _P, _P, _P, _I64, _I64, _I, _P],
    "fms_plain_reduce_reverse": [_P, _P, _P, _P, _I64, _I64, _I, _P],
    "fms_combine_carries": [_P, _P, _P, _P, _P, _I64, _I64, _I, _P],
    "fms_plain_forward_split": [_P, _P, _P, _P, _P, _I64, _I64, _I, _P, ctypes.c_size_t, _P],
    "fms_fm_forward": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I, _P],
    "fms_fm_backward": [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I, _P, ctypes.c_size_t, _P],
    "fms_plain_forward_split_static": [_P, _P, _P, _P, _P, _I64, _I64, _I, _P],
    "fms_plain_backward_split": [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I, _P, ctypes.c_size_t, _P],
}

_lib = None


class FmsError(RuntimeError):
    def __init__(self, fn: str, status: int, text: str, cuda_error: int):
        super().__init__(f"{fn} failed: {text} (status {status}, cuda error {cuda_error})")
        self.status = status
        self.cuda_error = cuda_error


def lib() -> ctypes.CDLL:
    """Load ``libfm_scan_b200.so`` (raises if it was not built)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m fm_b200.build` "
                "(there is no fallback implementation)")
        L = ctypes.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = _I
        L.fms_version.restype = _I
        L.fms_status_string.restype = ctypes.c_char_p
        L.fms_status_string.argtypes = [_I]
        L.fms_last_cuda_error.restype = _I
        L.fms_tune_reload.restype = None
        L.fms_tune_reload.argtypes = []
        L.fms_plain_split_segments.restype = _I64
        L.fms_plain_split_segments.argtypes = [_I64, _I64, _I]
        L.fms_plain_split_workspace_bytes.restype = ctypes.c_size_t
        L.fms_plain_split_workspace_bytes.argtypes = [_I64, _I64, _I]
        L.fms_fm_backward_workspace_bytes.restype = ctypes.c_size_t
        L.fms_fm_backward_workspace_bytes.argtypes = [_I64, _I64, _I64, _I64, _I]
        _lib = L
    return _lib


def status_string(status: int) -> str:
    return lib().fms_status_string(int(status)).decode()


def call(name: str, *args, check: bool = True) -> int:
    """Call an entry point; raise ``FmsError`` on a non-zero status unless ``check`` is False."""
    L = lib()
    rc = int(getattr(L, name)(*args))
    if rc != FMS_OK and check:
        raise FmsError(name, rc, status_string(rc), int(L.fms_last_cuda_error()))
    return rc


def dtype_tag(torch_dtype) -> int:
    import torch
    try:
        return {torch.float32: FMS_F32, torch.float16: FMS_F16, torch.bfloat16: FMS_BF16}[torch_dtype]
    except KeyError:
        raise TypeError("Unsupported tensor dtype: expecting bfloat16, float16 or float32") from None


def ptr(t) -> int | None:
    """Device address of a tensor, or None (NULL) for None."""
    return None if t is None else t.data_ptr()
