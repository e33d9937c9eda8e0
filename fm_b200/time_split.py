"""Scan of sequences split along T across the ranks of a process group.

Rank k of the group owns the contiguous time block k of every row (``gates``/``tokens`` of shape
(B, D, T_k); blocks may differ in length).  The reference cannot do this at all: its longest
sequence is what one CTA walks serially (fm/scan/fm_scan.cuh:84,211-216, at most 131072 steps).

Forward, per rank:
    1. carry-only pass        (P_k, S_k) = (prod a, h_last from a zero start)        reads a, x
    2. one all-gather of (P, S) -- 2 x rows fp32 per rank
    3. fold the carries of the ranks before k  ->  h_in,k   (h_in,0 = initial_state or 0; rank 0
       folds the initial state into the S it publishes, the other ranks ignore theirs)
    4. the ordinary forward scan of the block with h0 = h_in,k                        reads a, x; writes h
Backward mirrors it in reverse time order with c_t = a_t * delta_t as the carried quantity:
    1. carry-only reverse pass S'_k = c at the block start from a zero carry-in       reads a, G
       (the gate product P_k is reused from forward)
    2. all-gather of S'
    3. fold the carries of the ranks after k   ->  c_in,k
    4. the ordinary backward of the block with carry_in = c_in,k and h0 = h_in,k      reads a, h, G; writes 2
Rank 0's dL/dh0 output is the gradient of ``initial_state``.

The collective is whatever the group's backend provides (NCCL over NVLink on GPUs); with a
``PeerCarryExchange`` the all-gather and the fold are replaced by peer stores + flags in
symmetric memory and a fold-on-arrival kernel; with a ``FusedTimeSplit`` steps 1-4 of each
direction are one kernel (the second pass re-reads the row from L2).  The local
passes come from an ops object: ``CudaScanOps`` (the CUDA kernels) by default.  Tests on CPU
ranks inject another ops object to exercise the exchange logic over gloo; the package itself
ships no CPU scan.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ._nvtx import nvtx_range
from .ops import CudaScanOps
from .peer_exchange import FusedTimeSplit


def _gather(t: torch.Tensor, group) -> torch.Tensor:
    """all-gather equal-shaped per-rank tensors -> (world, *t.shape), rank-major."""
    world = dist.get_world_size(group)
    flat = t.contiguous().view(-1)
    out = torch.empty(world * flat.numel(), device=t.device, dtype=t.dtype)
    dist.all_gather_into_tensor(out, flat, group=group)
    return out.view((world,) + tuple(t.shape))


class _TimeSplitScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gates, tokens, initial_state, group, ops, exchange):
        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        rows_shape = gates.shape[:-1]
        ctx.fused = False
        if isinstance(exchange, FusedTimeSplit) and FusedTimeSplit.applies(gates):
            # one kernel: carry pass, peer exchange and scan pass fused row by row
            h0 = None
            if rank == 0 and initial_state is not None:
                h0 = initial_state.to(torch.float32).reshape(-1).contiguous()
            with nvtx_range("fm_scan.time_split.forward(fused: carry pass + exchange + scan pass)"):
                states, h_in = exchange.forward(gates, tokens, h0)
            ctx.save_for_backward(gates, states, h_in)
            ctx.group, ctx.ops, ctx.rank, ctx.world, ctx.exchange = group, ops, rank, world, exchange
            ctx.fused = True
            ctx.h0_dtype = None if initial_state is None else initial_state.dtype
            ctx.h0_needs_grad = initial_state is not None and ctx.needs_input_grad[2]
            ctx.h0_shape = None if initial_state is None else initial_state.shape
            return states
        if isinstance(exchange, FusedTimeSplit):
            raise RuntimeError("FusedTimeSplit needs 16-byte aligned rows (T_k * element size % 16 == 0); "
                               "use PeerCarryExchange or the default all-gather for this shape")
        with nvtx_range("fm_scan.time_split.carry_pass"):
            P, S = ops.reduce(gates, tokens)
        # The initial state belongs to the first block only.  Rank 0 folds it into the carry it
        # publishes (S_0 <- P_0*h0 + S_0) and scans from it; the other ranks never look at their
        # `initial_state` argument, so no collective depends on who passed one.
        carry0 = None
        if rank == 0 and initial_state is not None:
            carry0 = initial_state.to(torch.float32).reshape(-1).contiguous()
            S = torch.addcmul(S.reshape(-1), P.reshape(-1), carry0)
        if exchange is not None:
            # peer stores + flags over NVLink, fold on arrival (fm_b200.peer_exchange)
            P_keep = P.reshape(-1).contiguous()
            h_in = exchange.exchange(P_keep, S.reshape(-1).contiguous(), carry0, reverse=False)
            h_in = h_in.reshape(rows_shape)
        else:
            PS = _gather(torch.stack([P.reshape(-1), S.reshape(-1)]), group)  # (world, 2, rows)
            P_keep = PS[:, 0].contiguous()
            if rank == 0:
                h_in = (carry0 if carry0 is not None else torch.zeros_like(P_keep[0])).reshape(rows_shape)
            else:
                h_in_all, _ = ops.combine(P_keep, PS[:, 1].contiguous(), None, reverse=False)
                h_in = h_in_all[rank].reshape(rows_shape).contiguous()
        with nvtx_range("fm_scan.time_split.scan_pass"):
            states = ops.forward(gates, tokens, h_in)
        ctx.save_for_backward(gates, states, h_in, P_keep)
        ctx.group, ctx.ops, ctx.rank, ctx.world, ctx.exchange = group, ops, rank, world, exchange
        ctx.h0_dtype = None if initial_state is None else initial_state.dtype
        ctx.h0_needs_grad = initial_state is not None and ctx.needs_input_grad[2]
        return states

    @staticmethod
    def backward(ctx, grad_states):
        if ctx.fused:
            gates, states, h_in = ctx.saved_tensors
            with nvtx_range("fm_scan.time_split.backward(fused)"):
                grad_gates, grad_tokens, grad_h0 = ctx.exchange.backward(
                    gates, states, grad_states.contiguous(), h_in, want_grad_h0=ctx.h0_needs_grad)
            d_h0 = None
            if ctx.h0_needs_grad:
                d_h0 = grad_h0 if ctx.rank == 0 else torch.zeros_like(grad_h0)
                d_h0 = d_h0.reshape(ctx.h0_shape).to(ctx.h0_dtype)
            return grad_gates, grad_tokens, d_h0, None, None, None
        gates, states, h_in, P_keep = ctx.saved_tensors
        group, ops, rank = ctx.group, ctx.ops, ctx.rank
        grad_states = grad_states.contiguous()
        S_rev = ops.reduce_reverse(gates, grad_states)
        if ctx.exchange is not None:
            c_in = ctx.exchange.exchange(P_keep, S_rev.reshape(-1).contiguous(), None, reverse=True)
            c_in = c_in.reshape(h_in.shape)
        else:
            S_all = _gather(S_rev.reshape(-1), group)  # (world, rows)
            c_in_all, _ = ops.combine(P_keep, S_all, None, reverse=True)
            c_in = c_in_all[rank].reshape(h_in.shape).contiguous()
        grad_gates, grad_tokens, grad_h0 = ops.backward(gates, states, grad_states, h_in, c_in,
                                                        want_grad_h0=ctx.h0_needs_grad)
        d_h0 = None
        if ctx.h0_needs_grad:
            # dL/d(initial_state) is rank 0's carry-out; other ranks contribute nothing
            d_h0 = grad_h0 if rank == 0 else torch.zeros_like(grad_h0)
            d_h0 = d_h0.to(ctx.h0_dtype)
        return grad_gates, grad_tokens, d_h0, None, None, None


def _validate_layout(gates, group):
    """Every rank must hold the same rows (B, D) in the same dtype; a mismatch would otherwise
    surface as a hang or as garbage carries.  One small all-gather of a descriptor."""
    rows = 1
    for s in gates.shape[:-1]:
        rows *= s
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.float64: 3}.get(gates.dtype, -1)
    mine = torch.tensor([rows, gates.dim(), code], device=gates.device, dtype=torch.int64)
    everyone = _gather(mine, group)
    if not bool((everyone == mine).all()):
        raise RuntimeError(
            "fm_scan_time_split: ranks disagree on (rows, rank of tensor, dtype): "
            f"{everyone.tolist()} -- every rank must hold the same (B, D) rows of one dtype")


def fm_scan_time_split(gates, tokens, initial_state=None, group=None, ops=None, validate=False,
                       exchange=None):
    """Differentiable scan of this rank's time block; ranks are ordered along T by group rank.

    Arguments:
        gates, tokens: (B, D, T_k) contiguous tensors of this rank's block (same dtype).
        initial_state: (B, D) state before the first block.  Only rank 0's argument is read; the
            other ranks may pass anything, None included (no collective depends on it).
        group: process group spanning the time blocks (default: the world group).
        ops: local scan passes (default ``CudaScanOps``).
        exchange: a ``fm_b200.peer_exchange.PeerCarryExchange`` built for these rows: the carries
            then travel as peer stores over NVLink with flags instead of an all-gather.  A
            ``fm_b200.peer_exchange.FusedTimeSplit`` goes further: each direction is ONE kernel in
            which the carry pass, the exchange and the scan pass are fused row by row, so the block
            moves the HBM bytes of an unsplit scan (needs 16-byte aligned rows).
        validate: exchange a shape/dtype descriptor first and raise on every rank if the ranks
            disagree (one extra small all-gather; off by default).
    Returns:
        states of this rank's block, (B, D, T_k).
    """
    if not dist.is_initialized():
        raise RuntimeError("fm_scan_time_split needs an initialised torch.distributed process group")
    if gates.shape != tokens.shape:
        raise RuntimeError("gates and tokens must have the same shape")
    if validate:
        _validate_layout(gates, group)
    return _TimeSplitScan.apply(gates, tokens, initial_state, group, ops or CudaScanOps, exchange)
