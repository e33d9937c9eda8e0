"""The C-ABI library without a GPU: it loads, exports what the header declares, and its argument
checks answer before any CUDA call."""
import ctypes
import re
from pathlib import Path

import pytest

from fm_b200 import capi

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "fm_scan_b200.h").read_text()


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(fms_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("fms_plain_forward", "fms_plain_backward", "fms_plain_reduce", "fms_plain_reduce_reverse",
                 "fms_combine_carries", "fms_plain_forward_backward_host", "fms_version"):
        assert must in names


def test_library_exports_every_declared_symbol():
    L = capi.lib()
    for name in declared_functions():
        assert hasattr(L, name), f"{name} is declared in the header but not exported"


def test_ctypes_table_covers_the_compute_entry_points():
    for name in capi.SIGNATURES:
        assert name in declared_functions()


def test_version_and_status_strings():
    assert capi.lib().fms_version() >= 100
    assert capi.status_string(capi.FMS_OK) == "ok"
    assert "dtype" in capi.status_string(capi.FMS_ERR_BAD_DTYPE)
    assert "unknown" in capi.status_string(12345)


def test_argument_checks_need_no_device():
    buf = (ctypes.c_char * 256)()
    p = ctypes.addressof(buf)
    p = (p + 15) // 16 * 16
    call = lambda *a: capi.call("fms_plain_forward", *a, check=False)
    assert call(p, p, None, p, None, 4, 8, 99, None) == capi.FMS_ERR_BAD_DTYPE
    assert call(p, p, None, p, None, -1, 8, capi.FMS_F32, None) == capi.FMS_ERR_BAD_SHAPE
    assert call(p, p, None, p, None, 4, -8, capi.FMS_F32, None) == capi.FMS_ERR_BAD_SHAPE
    assert call(p, p, None, p, None, 2 ** 40, 2 ** 40, capi.FMS_F32, None) == capi.FMS_ERR_BAD_SHAPE
    assert call(p, None, None, p, None, 4, 8, capi.FMS_F32, None) == capi.FMS_ERR_NULL_POINTER
    assert call(p + 2, p, None, p, None, 4, 8, capi.FMS_F32, None) == capi.FMS_ERR_MISALIGNED
    assert call(p + 1, p, None, p, None, 4, 8, capi.FMS_BF16, None) == capi.FMS_ERR_MISALIGNED
    # empty problems are accepted without touching the device
    assert call(None, None, None, None, None, 0, 8, capi.FMS_F32, None) == capi.FMS_OK
    assert capi.call("fms_plain_backward", p, p, p, None, None, p, None, None, 4, 8, capi.FMS_F16, None,
                     check=False) == capi.FMS_ERR_NULL_POINTER
    assert capi.call("fms_combine_carries", None, None, None, None, None, -1, 4, 0, None,
                     check=False) == capi.FMS_ERR_BAD_SHAPE
    with pytest.raises(capi.FmsError) as e:
        capi.call("fms_plain_reduce", p, p, p, p, 4, 8, 7, None)
    assert e.value.status == capi.FMS_ERR_BAD_DTYPE


def test_pipeline_rejects_a_missing_workspace_without_a_device():
    from fm_b200 import host_pipeline as hp
    L = hp._bind()
    handle = ctypes.c_void_p()
    assert L.fms_pipeline_create(ctypes.byref(handle), None, 1 << 20) == capi.FMS_ERR_WORKSPACE
    assert L.fms_pipeline_create(None, None, 0) == capi.FMS_ERR_NULL_POINTER
    import torch
    assert hp.workspace_bytes(4096, 8192, torch.bfloat16) == 12 * 4096 * 8192 * 2
    assert hp.workspace_bytes(1, 3, torch.float16) == 12 * 256


def test_ops_refuse_cpu_tensors():
    import torch
    from fm_b200.ops import CudaScanOps
    with pytest.raises(RuntimeError, match="CUDA"):
        CudaScanOps.forward(torch.zeros(2, 8), torch.zeros(2, 8))


def test_fm_mode_argument_checks_need_no_device():
    L = capi.lib()
    buf = (ctypes.c_char * 256)()
    p = (ctypes.addressof(buf) + 15) // 16 * 16
    fwd = lambda *a: capi.call("fms_fm_forward", *a, check=False)
    assert fwd(p, p, None, p, 1, 2, 3, 8, 42, None) == capi.FMS_ERR_BAD_DTYPE
    assert fwd(p, p, None, p, 1, -2, 3, 8, capi.FMS_F32, None) == capi.FMS_ERR_BAD_SHAPE
    assert fwd(p, p, None, p, 2 ** 31, 2 ** 31, 2 ** 31, 8, capi.FMS_F32, None) == capi.FMS_ERR_BAD_SHAPE
    assert fwd(p, None, None, p, 1, 2, 3, 8, capi.FMS_F32, None) == capi.FMS_ERR_NULL_POINTER
    assert fwd(p + 2, p, None, p, 1, 2, 3, 8, capi.FMS_F32, None) == capi.FMS_ERR_MISALIGNED
    assert fwd(None, None, None, None, 0, 2, 3, 8, capi.FMS_F32, None) == capi.FMS_OK  # empty batch
    # fp32 gradients accumulate in place; 16-bit ones need fp32 accumulators for both outputs
    assert L.fms_fm_backward_workspace_bytes(1, 32, 2048, 8192, capi.FMS_F32) == 0
    assert L.fms_fm_backward_workspace_bytes(1, 32, 2048, 8192, capi.FMS_BF16) == (32 + 2048) * 8192 * 4
    assert L.fms_fm_backward_workspace_bytes(1, 32, 2048, 8192, 9) == 0
    rc = capi.call("fms_fm_backward", p, p, p, p, None, p, p, None, 1, 2, 3, 8, capi.FMS_BF16, None, 0, None,
                   check=False)
    assert rc == capi.FMS_ERR_WORKSPACE


def test_split_plan_is_pure_arithmetic():
    L = capi.lib()
    assert L.fms_plain_split_segments(32768, 8192, capi.FMS_BF16) == 1      # plenty of rows
    assert L.fms_plain_split_segments(4, 8191, capi.FMS_F32) == 1           # too short to split
    nseg = L.fms_plain_split_segments(4, 1 << 20, capi.FMS_F32)
    assert nseg > 1 and 4 * nseg >= 148 * 8 and (1 << 20) // nseg >= 2048
    assert L.fms_plain_split_workspace_bytes(4, 1 << 20, capi.FMS_F32) >= 4 * nseg * 12
    assert L.fms_plain_split_workspace_bytes(32768, 8192, capi.FMS_BF16) == 0
    # the built-in scratch refuses more units than it holds, before touching the device
    buf = (ctypes.c_char * 64)()
    p = (ctypes.addressof(buf) + 15) // 16 * 16
    rc = capi.call("fms_plain_forward_split_static", p, p, None, p, None, 2100, 16384, capi.FMS_F32, None,
                   check=False)
    assert rc == capi.FMS_ERR_TOO_LARGE   # not even two segments for each of 2100 rows fit 4096 units
