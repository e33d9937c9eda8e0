"""Host logic of the split-along-T scan on CPU ranks (gloo, world_size 2 and 3)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fm_b200 import sharding
from oracle import c_oracle as oc
from tests import helpers as H


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T_blocks, with_h0, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fm_b200.time_split import fm_scan_time_split
        from tests.cpu_ops import OracleScanOps

        R, T = 6, sum(T_blocks)
        a, x, G, h0 = H.make_inputs(R, T, 77, "sigmoid+3", "f32", with_h0=True)
        b = sum(T_blocks[:rank])
        e = b + T_blocks[rank]
        at = torch.from_numpy(a[:, b:e].copy()).double().view(2, 3, -1).requires_grad_(True)
        xt = torch.from_numpy(x[:, b:e].copy()).double().view(2, 3, -1).requires_grad_(True)
        h0t = None
        if with_h0 == "rank0" and rank != 0:
            pass  # only the first block passes an initial state at all: nothing may hang on that
        elif with_h0:
            # ranks other than 0 pass garbage on purpose: only rank 0's initial state counts
            h0t = torch.from_numpy(h0 if rank == 0 else h0 * 0 + 123).double().view(2, 3).requires_grad_(True)
        h = fm_scan_time_split(at, xt, h0t, ops=OracleScanOps)
        h.backward(torch.from_numpy(G[:, b:e].copy()).double().view(2, 3, -1))
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), h=h.detach().numpy().reshape(R, -1),
                 ga=at.grad.numpy().reshape(R, -1), gx=xt.grad.numpy().reshape(R, -1),
                 gh0=(h0t.grad.numpy().reshape(R) if h0t is not None else np.zeros(R)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T_blocks,with_h0", [((40, 40), False), ((37, 64), True), ((5, 1, 90), True),
                                              ((33, 20, 11), "rank0")])
def test_time_split_matches_unsplit_scan(tmp_path, T_blocks, with_h0):
    world = len(T_blocks)
    mp.spawn(_worker, args=(world, _free_port(), T_blocks, with_h0, str(tmp_path)), nprocs=world, join=True)
    R, T = 6, sum(T_blocks)
    a, x, G, h0 = H.make_inputs(R, T, 77, "sigmoid+3", "f32", with_h0=True)
    f64 = np.float64
    h0_used = h0.astype(f64) if with_h0 else None
    h_ref = oc.plain_forward(a.astype(f64), x.astype(f64), h0_used, dtype=f64)
    ga_ref, gx_ref, gh0_ref = oc.plain_backward(a.astype(f64), h_ref, G.astype(f64), h0_used, dtype=f64)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    # carries travel as fp32, everything else is double in this test
    np.testing.assert_allclose(np.concatenate([p["h"] for p in parts], 1), h_ref, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(np.concatenate([p["gx"] for p in parts], 1), gx_ref, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(np.concatenate([p["ga"] for p in parts], 1), ga_ref, rtol=1e-5, atol=2e-5)
    if with_h0:
        np.testing.assert_allclose(parts[0]["gh0"], gh0_ref, rtol=1e-5, atol=1e-5)
        for p in parts[1:]:
            assert not p["gh0"].any()


def test_row_blocks_cover_rows_exactly():
    for rows in (0, 1, 7, 8, 32768, 2304):
        for world in (1, 2, 3, 4, 8):
            blocks = sharding.row_blocks(rows, world)
            assert len(blocks) == world and blocks[0][0] == 0 and blocks[-1][1] == rows
            assert all(b[1] == n[0] for b, n in zip(blocks, blocks[1:]))
            sizes = [e - b for b, e in blocks]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.row_blocks(4, 0)


def test_shard_rows_returns_contiguous_views():
    t = torch.arange(2 * 6 * 5).view(2, 6, 5)
    parts = [sharding.shard_rows(t, r, 4) for r in range(4)]
    assert torch.equal(torch.cat(parts), t.view(12, 5))
    assert all(p.is_contiguous() for p in parts)


def _mismatch_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fm_b200.time_split import fm_scan_time_split
        from tests.cpu_ops import OracleScanOps
        rows = 6 if rank == 0 else 5          # rank 1 holds a different number of rows
        a = torch.rand(1, rows, 16, dtype=torch.float64)
        try:
            fm_scan_time_split(a, a.clone(), ops=OracleScanOps, validate=True)
            outcome = "no error"
        except RuntimeError as e:
            outcome = "raised" if "disagree" in str(e) else f"other: {e}"
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write(outcome)
    finally:
        dist.destroy_process_group()


def test_time_split_reports_mismatched_rows_on_every_rank(tmp_path):
    mp.spawn(_mismatch_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert [(tmp_path / f"rank{r}.txt").read_text() for r in range(2)] == ["raised", "raised"]
