"""The peer-memory carry exchange on ONE GPU: ranks emulated one after the other (every flag is
raised before the kernel that waits for it is launched), the bounded waits running out, and the
back-pressure that keeps a fast rank from overwriting carries a slow rank has not folded."""
import ctypes

import numpy as np
import pytest
import torch

from fm_b200 import capi
from fm_b200.peer_exchange import _bind

pytestmark = pytest.mark.gpu


def _buffers(rows, world):
    L = _bind()
    nbytes = int(L.fms_peer_exchange_bytes(rows, world))
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    return L, bufs, ptrs, int(L.fms_peer_exchange_status_offset(rows, world))


@pytest.mark.parametrize("world", [2, 3, 8])
def test_publish_then_fold_reproduces_the_serial_fold(world):
    rows = 1000
    L, bufs, ptrs, status_off = _buffers(rows, world)
    rng = np.random.default_rng(world)
    P = rng.uniform(0.2, 1.0, (world, rows)).astype(np.float32)
    S = rng.standard_normal((world, rows)).astype(np.float32)
    c0 = rng.standard_normal(rows).astype(np.float32)
    st = torch.cuda.current_stream().cuda_stream
    for number in (1, 2, 3):  # three exchanges: both slot generations and reuse of the first
        Pd = torch.from_numpy(P * number / 3).cuda()
        Sd = torch.from_numpy(S + number).cuda()
        for reverse in (0, 1):
            for r in range(world):
                assert L.fms_peer_publish(Pd[r].data_ptr(), Sd[r].data_ptr(), rows, ptrs, world, r, reverse,
                                          number, 0.5, st) == capi.FMS_OK
            c0d = torch.from_numpy(c0).cuda()
            for r in range(world):
                out = torch.empty(rows, device="cuda")
                assert L.fms_peer_wait_fold(ptrs, c0d.data_ptr(), out.data_ptr(), rows, world, r,
                                            reverse, number, 0.5, st) == capi.FMS_OK
                c = c0.astype(np.float64).copy()
                order = range(r) if not reverse else range(world - 1, r, -1)
                for src in order:
                    c = (P[src] * number / 3).astype(np.float32) * c + (S[src] + number).astype(np.float32)
                np.testing.assert_allclose(out.cpu().numpy(), c, rtol=1e-5, atol=1e-5)
    torch.cuda.synchronize()
    for b in bufs:
        assert int(b[status_off:status_off + 4].view(torch.int32).item()) == 0


def test_wait_runs_out_and_reports_it():
    """Nothing raises the flag: the kernel gives up after its bound, records it and ends normally;
    the context stays usable."""
    rows, world = 64, 2
    L, bufs, ptrs, status_off = _buffers(rows, world)
    c0 = torch.arange(rows, device="cuda", dtype=torch.float32)
    out = torch.full((rows,), -1.0, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    assert L.fms_peer_wait_fold(ptrs, c0.data_ptr(), out.data_ptr(), rows, world, 1, 0, 1, 0.05,
                                st) == capi.FMS_OK
    t1.record()
    torch.cuda.synchronize()
    assert 20.0 < t0.elapsed_time(t1) < 1000.0          # about the 50 ms bound, not forever
    assert int(bufs[1][status_off:status_off + 4].view(torch.int32).item()) == 1
    assert torch.equal(out, c0)                          # the carry-in is passed through
    # reverse direction reports code 2; rank world-1 depends on nobody in reverse and does not wait
    assert L.fms_peer_wait_fold(ptrs, None, out.data_ptr(), rows, world, 0, 1, 1, 0.05, st) == capi.FMS_OK
    torch.cuda.synchronize()
    assert int(bufs[0][status_off:status_off + 4].view(torch.int32).item()) == 2
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0   # device still answers


def _status(buf, off):
    return int(buf[off:off + 4].view(torch.int32).item())


def test_a_fast_publisher_cannot_overwrite_what_a_slow_reader_still_needs():
    """Forward-only sequence, rank 0 far ahead of rank 1: exchanges 1 and 2 go out (two slot
    generations), exchange 3 would reuse the slots of 1, which rank 1 has not folded yet.  The
    publisher's bounded wait for the acknowledgement runs out, it records that and publishes
    nothing, so rank 1 still folds exchange 1's carries -- not exchange 3's."""
    rows, world = 300, 2
    L, bufs, ptrs, status_off = _buffers(rows, world)
    st = torch.cuda.current_stream().cuda_stream
    P = [torch.full((rows,), 0.5, device="cuda") for _ in range(4)]
    S = [torch.full((rows,), float(e), device="cuda") for e in range(4)]   # S of exchange e is e
    for e in (1, 2):
        assert L.fms_peer_publish(P[e].data_ptr(), S[e].data_ptr(), rows, ptrs, world, 0, 0, e, 0.05, st) == capi.FMS_OK
    torch.cuda.synchronize()
    assert _status(bufs[0], status_off) == 0
    assert L.fms_peer_publish(P[3].data_ptr(), S[3].data_ptr(), rows, ptrs, world, 0, 0, 3, 0.05, st) == capi.FMS_OK
    torch.cuda.synchronize()
    assert _status(bufs[0], status_off) == 4           # FMS_PEER_ERR_ACK_TIMEOUT on the publisher
    out = torch.empty(rows, device="cuda")
    assert L.fms_peer_wait_fold(ptrs, None, out.data_ptr(), rows, world, 1, 0, 1, 0.05, st) == capi.FMS_OK
    torch.cuda.synchronize()
    assert _status(bufs[1], status_off) == 0
    assert torch.equal(out, torch.full((rows,), 1.0, device="cuda"))       # exchange 1: 0.5 * 0 + 1


def test_a_later_exchange_in_the_slot_is_reported_not_folded():
    """If the numbering is broken anyway (here: rank 1 asks for exchange 1 after exchange 3 went
    into the same slot generation of a fresh buffer pair), the fold refuses the newer data."""
    rows, world = 64, 2
    L, bufs, ptrs, status_off = _buffers(rows, world)
    st = torch.cuda.current_stream().cuda_stream
    P = torch.full((rows,), 0.5, device="cuda")
    S = torch.full((rows,), 3.0, device="cuda")
    # pretend rank 1 acknowledged exchange 1 so that exchange 3 is let through
    ack_off = status_off - 8 - 2 * world * 4
    bufs[0][ack_off:ack_off + 2 * world * 4].view(torch.int32)[1] = 1
    assert L.fms_peer_publish(P.data_ptr(), S.data_ptr(), rows, ptrs, world, 0, 0, 3, 0.05, st) == capi.FMS_OK
    c0 = torch.arange(rows, device="cuda", dtype=torch.float32)
    out = torch.empty(rows, device="cuda")
    assert L.fms_peer_wait_fold(ptrs, c0.data_ptr(), out.data_ptr(), rows, world, 1, 0, 1, 0.05, st) == capi.FMS_OK
    torch.cuda.synchronize()
    assert _status(bufs[0], status_off) == 0
    assert _status(bufs[1], status_off) == 3           # FMS_PEER_ERR_OVERRUN
    assert torch.equal(out, c0)


def test_forward_only_loop_with_every_rank_one_exchange_ahead():
    """Six forward exchanges in a row, no reverse exchange between them, each rank publishing
    exchange e+1 before the others fold e (the furthest the protocol allows)."""
    rows, world = 500, 3
    L, bufs, ptrs, status_off = _buffers(rows, world)
    st = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(5)
    P = rng.uniform(0.2, 1.0, (8, world, rows)).astype(np.float32)
    S = rng.standard_normal((8, world, rows)).astype(np.float32)
    Pd, Sd = torch.from_numpy(P).cuda(), torch.from_numpy(S).cuda()

    def publish(e):
        for r in range(world):
            assert L.fms_peer_publish(Pd[e, r].data_ptr(), Sd[e, r].data_ptr(), rows, ptrs, world, r, 0, e, 0.5,
                                      st) == capi.FMS_OK

    publish(1)
    for e in range(1, 7):
        publish(e + 1)                                  # one ahead
        for r in range(world):
            out = torch.empty(rows, device="cuda")
            assert L.fms_peer_wait_fold(ptrs, None, out.data_ptr(), rows, world, r, 0, e, 0.5, st) == capi.FMS_OK
            c = np.zeros(rows, np.float32)
            for src in range(r):
                c = P[e, src] * c + S[e, src]
            np.testing.assert_allclose(out.cpu().numpy(), c, rtol=1e-5, atol=1e-5)
    torch.cuda.synchronize()
    for b in bufs:
        assert _status(b, status_off) == 0


def test_argument_checks():
    L = _bind()
    assert L.fms_peer_exchange_bytes(100, 9) == 0 and L.fms_peer_exchange_bytes(100, 8) > 0
    buf = (ctypes.c_void_p * 2)(None, None)
    assert L.fms_peer_publish(None, None, 10, buf, 2, 0, 0, 1, 1.0, None) == capi.FMS_ERR_NULL_POINTER
    assert L.fms_peer_publish(None, None, 10, buf, 2, 5, 0, 1, 1.0, None) == capi.FMS_ERR_BAD_SHAPE
    assert L.fms_peer_publish(None, None, 10, buf, 2, 0, 0, 0, 1.0, None) == capi.FMS_ERR_BAD_SHAPE  # numbers start at 1
