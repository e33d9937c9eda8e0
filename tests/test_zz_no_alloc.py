"""The entry point for callers that may not allocate device memory.

`fms_plain_forward_split_static` is for hosts that cannot give the library scratch: a plugin in
a framework that owns all device memory and bars its plugins from the CUDA allocator, a loop
that cannot tolerate the device-wide synchronisation an allocation implies, a process whose
pool already holds the whole GPU.  It keeps the split path's per-segment carries in a fixed
48 KiB array inside the library instead of a caller workspace.

Collected last (file name) so that a run stopping at the first failure has already run
everything else.  It must pass alone in a fresh process and after the other tests: it relies on
nothing but the library, and the shared array needs no clearing between calls.
"""
import numpy as np
import pytest
import torch

from fm_b200 import capi
from oracle import c_oracle as oc
from tests import gpu_util as G
from tests import helpers as H

pytestmark = pytest.mark.gpu


def forward_static(a, x, h0=None, want_last=False, check=True):
    T = a.shape[-1]
    rows = a.numel() // T
    h = torch.empty_like(a)
    h_last = torch.empty(a.shape[:-1], device=a.device, dtype=torch.float32) if want_last else None
    rc = capi.call("fms_plain_forward_split_static", capi.ptr(a), capi.ptr(x), capi.ptr(h0), capi.ptr(h),
                   capi.ptr(h_last), rows, T, capi.dtype_tag(a.dtype), G.stream_ptr(), check=check)
    return rc, h, h_last


@pytest.mark.parametrize("storage,R,T", [("f32", 5, 150_000), ("bf16", 2, 400_003)])
def test_static_scratch_matches_workspace_entry_twice_in_a_row(storage, R, T):
    a, x, _, h0 = H.make_inputs(R, T, 91, "sigmoid+3", storage, with_h0=True)
    ad, xd, h0d = G.dev(a, storage), G.dev(x, storage), G.dev(h0)
    nseg, nbytes = G.split_plan(R, T, ad.dtype)
    assert nseg > 1 and R * nseg <= 4096, "the case must exercise the scratch"
    want, want_last = G.forward_split(ad, xd, h0d, want_last=True)   # existing entry point
    torch.cuda.synchronize()
    rtol, atol = (H.FP32_RTOL, H.FP32_ATOL) if storage == "f32" else (H.LOWP_RTOL, H.lowp_atol(G.host(want)))
    # the CPU oracle in double on the same rounded inputs (a handful of rows: cheap)
    f64 = np.float64
    h_ref, last_ref = oc.plain_forward(a.astype(f64), x.astype(f64), h0.astype(f64), dtype=f64, return_last=True)
    o_atol = (H.FP32_ATOL * max(1.0, float(np.abs(h_ref).max()))) if storage == "f32" else H.lowp_atol(h_ref)
    for call in range(2):                                            # second call reuses the array as left
        rc, got, got_last = forward_static(ad, xd, h0d, want_last=True)
        torch.cuda.synchronize()
        assert rc == capi.FMS_OK
        H.assert_close(G.host(got), G.host(want), rtol, atol, f"call {call}: states")
        H.assert_close(G.host(got_last), G.host(want_last), 1e-5, 1e-5, f"call {call}: h_last")
        H.assert_close(G.host(got), h_ref, rtol, o_atol, f"call {call}: states vs oracle")
        H.assert_close(G.host(got_last), last_ref, 1e-4, 1e-4, f"call {call}: h_last vs oracle")
    # a different problem in between must not disturb the next call either
    b, y, _ = H.make_inputs(3, 70_000, 92, "sigmoid", storage)
    forward_static(G.dev(b, storage), G.dev(y, storage))
    rc, got, _ = forward_static(ad, xd, h0d)
    torch.cuda.synchronize()
    H.assert_close(G.host(got), G.host(want), rtol, atol, "after another problem: states")


@pytest.mark.parametrize("storage,R,T", [("bf16", 8, 4_194_304), ("f32", 64, 1_048_576), ("f32", 2000, 16384)])
def test_static_scratch_replans_inside_its_capacity(storage, R, T):
    """Shapes for which the library's usual plan needs more than 4096 units (4688, 4736 and 6000
    here): the static entry uses fewer, longer segments instead of refusing."""
    a, x, _, h0 = H.make_inputs(R, T, 93, "sigmoid+3", storage, with_h0=True)
    ad, xd, h0d = G.dev(a, storage), G.dev(x, storage), G.dev(h0)
    nseg, _ = G.split_plan(R, T, ad.dtype)
    assert R * nseg > 4096 and R * 2 <= 4096
    want, want_last = G.forward_split(ad, xd, h0d, want_last=True)
    f64 = np.float64
    h_ref = oc.plain_forward(a.astype(f64), x.astype(f64), h0.astype(f64), dtype=f64)
    for call in range(2):
        rc, got, got_last = forward_static(ad, xd, h0d, want_last=True)
        torch.cuda.synchronize()
        assert rc == capi.FMS_OK
        if storage == "f32":
            tol = (H.FP32_RTOL, H.FP32_ATOL * max(1.0, float(np.abs(h_ref).max())))
        else:
            tol = (H.LOWP_RTOL, H.lowp_atol(h_ref))
        H.assert_close(G.host(got), h_ref, *tol, f"call {call}: states vs oracle")
        H.assert_close(G.host(got), G.host(want), tol[0], tol[1] * 2, f"call {call}: states vs workspace entry")
        H.assert_close(G.host(got_last), G.host(want_last), 1e-4, 1e-4, f"call {call}: h_last")


def test_static_scratch_limit_and_fallthrough():
    # 2100 rows: the plan wants 3 segments (6300 units) and not even 2 per row fit 4096:
    # refused, nothing launched, output untouched
    R, T = 2100, 16384
    a = torch.full((R, T), 0.5, device="cuda")
    nseg, _ = G.split_plan(R, T, a.dtype)
    assert R * nseg > 4096 and R * 2 > 4096
    h_before = torch.full((R, T), -7.0, device="cuda")
    rc = capi.call("fms_plain_forward_split_static", capi.ptr(a), capi.ptr(a), None, capi.ptr(h_before), None,
                   R, T, capi.FMS_F32, G.stream_ptr(), check=False)
    torch.cuda.synchronize()
    assert rc == capi.FMS_ERR_TOO_LARGE and "capacity" in capi.status_string(rc)
    assert bool((h_before == -7.0).all())
    # shapes that need no split use no scratch and go straight to the ordinary kernel
    a2, x2, _ = H.make_inputs(64, 512, 3, "sigmoid", "f32")
    rc, got, _ = forward_static(G.dev(a2), G.dev(x2))
    want = G.forward(G.dev(a2), G.dev(x2))
    torch.cuda.synchronize()
    assert rc == capi.FMS_OK and torch.equal(got, want)
