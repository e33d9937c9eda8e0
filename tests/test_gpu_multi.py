"""Two-or-more-GPU paths: row sharding (no collective) and the split-along-T scan over NCCL.

Needs >= 2 visible GPUs; skipped otherwise.  NVLS is switched off for these short-lived child
processes.
"""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import c_oracle as oc
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _length(mode):
    """Total sequence length: blocks of the fused kernels must be 16-byte aligned for every world size."""
    return 8 * 1032 if mode == "time_fused" else 8 * 1031


def _worker(rank, world, port, mode, storage, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from fm_b200 import fm_scan, sharding
        from fm_b200.time_split import fm_scan_time_split
        from tests import gpu_util as G

        B, D, T = 2, 24, _length(mode)
        a, x, Gd, h0 = H.make_inputs(B * D, T, 123, "sigmoid+3", storage, with_h0=True)
        if mode == "time_peer_forward_only":
            # inference-style loop: forward exchanges only, one rank lagging behind the others
            import time
            from fm_b200.peer_exchange import PeerCarryExchange
            tb = sharding.time_blocks(T, world)[rank]
            ad, xd = (G.dev(np.ascontiguousarray(v[:, tb[0]:tb[1]]), storage, dev).view(B, D, -1) for v in (a, x))
            exchange = PeerCarryExchange(B * D)
            outs = []
            with torch.no_grad():
                for it in range(6):
                    if rank == world - 1 and it % 2 == 1:
                        torch.cuda.synchronize()
                        time.sleep(0.05)            # the last block falls behind
                    outs.append(G.host(fm_scan_time_split(ad, xd * float(it + 1), exchange=exchange)))
            exchange.check()
            torch.cuda.synchronize()
            np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **{f"h{i}": o.reshape(B * D, -1) for i, o in enumerate(outs)})
            dist.barrier()
            return
        if mode == "rows":
            blk = sharding.row_blocks(B * D, world)[rank]
            ad, xd, gd = (G.dev(v[blk[0]:blk[1]], storage, dev).requires_grad_(v is not Gd)
                          for v in (a, x, Gd))
            h = fm_scan(ad, xd)
            h.backward(gd)
        else:
            tb = sharding.time_blocks(T, world)[rank]
            ad, xd, gd = (G.dev(np.ascontiguousarray(v[:, tb[0]:tb[1]]), storage, dev)
                          .view(B, D, -1).requires_grad_(v is not Gd) for v in (a, x, Gd))
            h0d = G.dev(h0, storage, dev).view(B, D).requires_grad_(True)
            exchange = None
            if mode == "time_peer":
                from fm_b200.peer_exchange import PeerCarryExchange
                exchange = PeerCarryExchange(B * D)
            if mode == "time_fused":
                from fm_b200.peer_exchange import FusedTimeSplit
                exchange = FusedTimeSplit(B * D)
            h = fm_scan_time_split(ad, xd, h0d, exchange=exchange)
            h.backward(gd)
            if exchange is not None:
                # a second round on the same buffers (next exchange numbers, other parity)
                ad.grad = xd.grad = h0d.grad = None
                h = fm_scan_time_split(ad, xd, h0d, exchange=exchange)
                h.backward(gd)
                exchange.check()
        torch.cuda.synchronize()
        out = dict(h=G.host(h).reshape(-1, h.shape[-1]), ga=G.host(ad.grad).reshape(-1, h.shape[-1]),
                   gx=G.host(xd.grad).reshape(-1, h.shape[-1]))
        if mode != "rows":
            out["gh0"] = G.host(h0d.grad).reshape(-1)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **out)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _run(world, mode, storage, tmp_path):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), mode, storage, str(tmp_path)), nprocs=world, join=True)
    return [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("storage", ["f32", "bf16"])
def test_row_sharding_is_bit_identical_to_one_gpu(tmp_path, storage):
    from fm_b200 import fm_scan
    from tests import gpu_util as G
    world = min(_ngpu(), 4)
    parts = _run(world, "rows", storage, tmp_path)
    B, D, T = 2, 24, 8 * 1031
    a, x, Gd, _ = H.make_inputs(B * D, T, 123, "sigmoid+3", storage, with_h0=True)
    ad, xd = (G.dev(v, storage).requires_grad_(True) for v in (a, x))
    h = fm_scan(ad, xd)
    h.backward(G.dev(Gd, storage))
    torch.cuda.synchronize()
    assert np.array_equal(np.concatenate([p["h"] for p in parts]), G.host(h))
    assert np.array_equal(np.concatenate([p["ga"] for p in parts]), G.host(ad.grad))
    assert np.array_equal(np.concatenate([p["gx"] for p in parts]), G.host(xd.grad))


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("transport", ["time", "time_peer", "time_fused"])
@pytest.mark.parametrize("storage", ["f32", "bf16"])
def test_time_split_over_nccl_matches_oracle(tmp_path, storage, transport):
    """transport "time": NCCL all-gather; "time_peer": peer stores + flags in symmetric memory;
    "time_fused": one kernel per direction with the exchange inside it."""
    world = min(_ngpu(), 8)
    parts = _run(world, transport, storage, tmp_path)
    B, D, T = 2, 24, _length(transport)
    a, x, Gd, h0 = H.make_inputs(B * D, T, 123, "sigmoid+3", storage, with_h0=True)
    f64 = np.float64
    h = np.concatenate([p["h"] for p in parts], 1)
    h_ref = oc.plain_forward(a.astype(f64), x.astype(f64), h0.astype(f64), dtype=f64)
    ga_ref, gx_ref, gh0_ref = oc.plain_backward(a.astype(f64), h.astype(f64), Gd.astype(f64),
                                                h0.astype(f64), dtype=f64)
    if storage == "f32":
        tol = lambda ref: (H.FP32_RTOL, H.FP32_ATOL * max(1.0, float(np.abs(ref).max())))
    else:
        tol = lambda ref: (H.LOWP_RTOL, H.lowp_atol(ref))
    H.assert_close(h, h_ref, *tol(h_ref), "time-split states")
    H.assert_close(np.concatenate([p["gx"] for p in parts], 1), gx_ref, *tol(gx_ref), "time-split grad_tokens")
    H.assert_close(np.concatenate([p["ga"] for p in parts], 1), ga_ref, *tol(ga_ref), "time-split grad_gates")
    H.assert_close(parts[0]["gh0"], gh0_ref, 1e-2 if storage != "f32" else 1e-4, 1e-2 if storage != "f32" else 1e-5,
                   "time-split grad_h0")


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_forward_only_loop_over_peer_exchange_with_a_lagging_rank(tmp_path):
    """No backward pass orders the ranks here: only the acknowledgements keep a fast rank from
    reusing a slot generation that the lagging rank has not folded yet."""
    world = min(_ngpu(), 4)
    parts = _run(world, "time_peer_forward_only", "f32", tmp_path)
    B, D, T = 2, 24, 8 * 1031
    a, x, _, _ = H.make_inputs(B * D, T, 123, "sigmoid+3", "f32", with_h0=True)
    f64 = np.float64
    for it in range(6):
        h = np.concatenate([p[f"h{it}"] for p in parts], 1)
        h_ref = oc.plain_forward(a.astype(f64), (x * np.float32(it + 1)).astype(f64), dtype=f64)
        H.assert_close(h, h_ref, H.FP32_RTOL, H.FP32_ATOL * max(1.0, float(np.abs(h_ref).max())),
                       f"forward-only iteration {it}")
