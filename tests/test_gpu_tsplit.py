"""The fused split-along-T kernels on ONE GPU: the ranks are emulated one after the other in
dependency order (forward: block 0 first; backward: last block first), so every carry a kernel
waits for has been published before that kernel is launched and nothing can hang.  Also the
bounded waits running out."""
import ctypes

import numpy as np
import pytest
import torch

from fm_b200 import capi
from fm_b200.peer_exchange import _bind_fused
from oracle import c_oracle as oc
from tests import gpu_util as G
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _buffers(rows, world):
    L = _bind_fused()
    nbytes = int(L.fms_tsplit_exchange_bytes(rows, world))
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    return L, bufs, ptrs, int(L.fms_tsplit_exchange_status_offset(rows, world))


def _status(buf, off):
    return int(buf[off:off + 4].view(torch.int32).item())


def _run_step(L, ptrs, world, blocks, h0, number, wait=0.5):
    """blocks[k] = (a, x, G) device tensors of block k.  Returns per-block (h, ga, gx), grad_h0."""
    st = torch.cuda.current_stream().cuda_stream
    rows = blocks[0][0].shape[0]
    tag = capi.dtype_tag(blocks[0][0].dtype)
    hs, hins = [], []
    for k in range(world):                                   # forward: earlier blocks first
        a, x, _ = blocks[k]
        h = torch.empty_like(a)
        hin = torch.empty(rows, device="cuda", dtype=torch.float32)
        rc = L.fms_tsplit_forward(a.data_ptr(), x.data_ptr(), capi.ptr(h0) if k == 0 else None, h.data_ptr(),
                                  hin.data_ptr(), rows, a.shape[1], tag, ptrs, world, k, number, wait, st)
        assert rc == capi.FMS_OK, capi.status_string(rc)
        hs.append(h)
        hins.append(hin)
    grads = [None] * world
    gh0 = torch.empty(rows, device="cuda", dtype=torch.float32)
    for k in range(world - 1, -1, -1):                       # backward: later blocks first
        a, _, Gd = blocks[k]
        ga, gx = torch.empty_like(a), torch.empty_like(a)
        rc = L.fms_tsplit_backward(a.data_ptr(), hs[k].data_ptr(), Gd.data_ptr(), hins[k].data_ptr(), ga.data_ptr(),
                                   gx.data_ptr(), gh0.data_ptr() if k == 0 else None, rows, a.shape[1], tag, ptrs,
                                   world, k, number, wait, st)
        assert rc == capi.FMS_OK, capi.status_string(rc)
        grads[k] = (ga, gx)
    torch.cuda.synchronize()
    return hs, grads, gh0


LAUNCHES = [{},                                                      # staged ring, 16 warps per row, no look-ahead
            {"FMS_TUNE_TSPLIT_K": "8", "FMS_TUNE_TSPLIT_LOOK": "1"},     # staged ring, 8 warps, look-ahead 1
            {"FMS_TUNE_TSPLIT_K": "24", "FMS_TUNE_TSPLIT_L2_HINT": "1", "FMS_TUNE_TSPLIT_LOOK": "3"},
            {"FMS_TUNE_TSPLIT_LOOK": "1000"},                            # whole next row before a row's second pass
            {"FMS_TUNE_TSPLIT_STAGED": "0"},                             # register prefetch, 8 warps
            {"FMS_TUNE_TSPLIT_STAGED": "0", "FMS_TUNE_TSPLIT_K": "16", "FMS_TUNE_TSPLIT_U": "2",
             "FMS_TUNE_TSPLIT_BWD_U": "4"}]
SHAPES = [("f32", 2, 37, 4096 + 512), ("bf16", 3, 300, 8192), ("f16", 8, 5, 1024), ("f32", 4, 700, 2052),
          ("f32", 2, 450, 40000),                                        # several rows per CTA, 5 super-tiles, ragged
          ("bf16", 2, 2, 1 << 21)]                                       # too long for the staged kernels' table


@pytest.mark.parametrize("launch", range(len(LAUNCHES)))
@pytest.mark.parametrize("storage,world,R,Tk", SHAPES)
def test_fused_split_matches_the_oracle_over_three_steps(storage, world, R, Tk, launch):
    import os
    import subprocess
    import sys
    child = os.environ.get("FMS_TSPLIT_CHILD")
    if child is None and launch:
        # the launch shape of these kernels is read once per process: each non-default shape runs ALL
        # its cases in one child process (started from the first case)
        if (storage, world, R, Tk) != SHAPES[0]:
            pytest.skip("runs in the child process started by the first case")
        env = dict(os.environ, **LAUNCHES[launch], FMS_TSPLIT_CHILD=str(launch))
        res = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu",
                              f"{__file__}::test_fused_split_matches_the_oracle_over_three_steps"],
                             env=env, capture_output=True, text=True)
        assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
        return
    if child is not None and int(child) != launch:
        pytest.skip("another launch shape")
    L, bufs, ptrs, status_off = _buffers(R, world)
    T = world * Tk
    f64 = np.float64
    for number in (1, 2, 3):                                 # both slot generations and a reuse
        a, x, Gd, h0 = H.make_inputs(R, T, 700 + number, "sigmoid+3" if storage == "f32" else "sigmoid01", storage,
                                     with_h0=True)
        blocks = [tuple(G.dev(np.ascontiguousarray(v[:, k * Tk:(k + 1) * Tk]), storage) for v in (a, x, Gd))
                  for k in range(world)]
        hs, grads, gh0 = _run_step(L, ptrs, world, blocks, G.dev(h0), number)
        h = np.concatenate([G.host(t) for t in hs], 1)
        ga = np.concatenate([G.host(g[0]) for g in grads], 1)
        gx = np.concatenate([G.host(g[1]) for g in grads], 1)
        h_ref = oc.plain_forward(a.astype(f64), x.astype(f64), h0.astype(f64), dtype=f64)
        ga_ref, gx_ref, gh0_ref = oc.plain_backward(a.astype(f64), h.astype(f64), Gd.astype(f64), h0.astype(f64),
                                                    dtype=f64)
        if storage == "f32":
            tol = lambda r: (H.FP32_RTOL, H.FP32_ATOL * max(1.0, float(np.abs(r).max())))
        else:
            tol = lambda r: (H.LOWP_RTOL, H.lowp_atol(r) + 1e-3)
        H.assert_close(h, h_ref, *tol(h_ref), f"step {number}: states")
        H.assert_close(gx, gx_ref, *tol(gx_ref), f"step {number}: grad_tokens")
        H.assert_close(ga, ga_ref, *tol(ga_ref), f"step {number}: grad_gates")
        H.assert_close(G.host(gh0), gh0_ref, 1e-3, 1e-3 * max(1.0, float(np.abs(gh0_ref).max())), f"step {number}: grad_h0")
    for b in bufs:
        assert _status(b, status_off) == 0


def test_fused_split_waits_run_out_and_are_reported():
    """Block 1 runs although block 0 never published: every CTA gives up after the bound, the fault
    is recorded, the kernel ends and the device still answers."""
    R, Tk, world = 64, 2048, 2
    L, bufs, ptrs, status_off = _buffers(R, world)
    a = torch.full((R, Tk), 0.5, device="cuda")
    h, hin = torch.empty_like(a), torch.empty(R, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = L.fms_tsplit_forward(a.data_ptr(), a.data_ptr(), None, h.data_ptr(), hin.data_ptr(), R, Tk, capi.FMS_F32, ptrs,
                              world, 1, 1, 0.05, st)
    t1.record()
    torch.cuda.synchronize()
    assert rc == capi.FMS_OK
    assert 20.0 < t0.elapsed_time(t1) < 2000.0
    assert _status(bufs[1], status_off) == 1
    assert bool((hin == 0).all())                            # carries that did not arrive count as zero
    # reverse direction: block 0 waits for block 1
    ga, gx = torch.empty_like(a), torch.empty_like(a)
    rc = L.fms_tsplit_backward(a.data_ptr(), h.data_ptr(), a.data_ptr(), hin.data_ptr(), ga.data_ptr(), gx.data_ptr(),
                               None, R, Tk, capi.FMS_F32, ptrs, world, 0, 1, 0.05, st)
    torch.cuda.synchronize()
    assert rc == capi.FMS_OK and _status(bufs[0], status_off) == 2
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


def test_fused_split_back_pressure():
    """Forward-only: block 0 runs exchanges 1, 2 and 3 while block 1 has not run at all.  Exchange
    3 would reuse the slots of exchange 1: its kernel records the missing acknowledgement and
    publishes nothing, so block 1 still gets exchange 1's carries."""
    R, Tk, world = 50, 1024, 2
    L, bufs, ptrs, status_off = _buffers(R, world)
    st = torch.cuda.current_stream().cuda_stream
    a = torch.full((R, Tk), 1.0, device="cuda")              # P = 1, S = sum of the tokens
    hin = torch.empty(R, device="cuda")
    for e in (1, 2, 3):
        x = torch.full((R, Tk), float(e), device="cuda")
        rc = L.fms_tsplit_forward(a.data_ptr(), x.data_ptr(), None, torch.empty_like(a).data_ptr(), hin.data_ptr(), R,
                                  Tk, capi.FMS_F32, ptrs, world, 0, e, 0.05, st)
        assert rc == capi.FMS_OK
        torch.cuda.synchronize()
        assert _status(bufs[0], status_off) == (4 if e == 3 else 0)
    h = torch.empty_like(a)
    rc = L.fms_tsplit_forward(a.data_ptr(), torch.zeros_like(a).data_ptr(), None, h.data_ptr(), hin.data_ptr(), R, Tk,
                              capi.FMS_F32, ptrs, world, 1, 1, 0.05, st)
    torch.cuda.synchronize()
    assert rc == capi.FMS_OK and _status(bufs[1], status_off) == 0
    assert torch.equal(hin, torch.full((R,), float(Tk), device="cuda"))   # exchange 1: Tk tokens of 1.0


def test_fused_split_argument_checks():
    L = _bind_fused()
    assert L.fms_tsplit_exchange_bytes(100, 9) == 0 and L.fms_tsplit_exchange_bytes(100, 8) > 0
    buf = torch.zeros(int(L.fms_tsplit_exchange_bytes(4, 2)), dtype=torch.uint8, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
    a = torch.zeros(4, 1001, device="cuda", dtype=torch.bfloat16)       # rows not 16-byte aligned
    hin = torch.empty(4, device="cuda")
    rc = L.fms_tsplit_forward(a.data_ptr(), a.data_ptr(), None, a.data_ptr(), hin.data_ptr(), 4, 1001, capi.FMS_BF16,
                              ptrs, 2, 0, 1, 0.1, None)
    assert rc == capi.FMS_ERR_MISALIGNED
    rc = L.fms_tsplit_forward(a.data_ptr(), a.data_ptr(), None, a.data_ptr(), hin.data_ptr(), 4, 1000, capi.FMS_BF16,
                              ptrs, 2, 0, 0, 0.1, None)
    assert rc == capi.FMS_ERR_BAD_SHAPE                      # exchange numbers start at 1
