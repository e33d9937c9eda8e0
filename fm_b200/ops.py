"""Tensor-level calls into the C ABI (``include/fm_scan_b200.h``) on the current CUDA stream.

These are the building blocks of the split-along-T scan (``fm_b200.time_split``): forward and
backward with explicit per-row carries, the carry-only passes, and the carry fold.  Every
function takes CUDA tensors, launches on ``torch.cuda.current_stream()`` of the tensors' device
and returns without synchronising.  There is no CPU implementation behind them.
"""
from __future__ import annotations

import torch

from . import capi


def _rows_T(t: torch.Tensor):
    T = t.shape[-1]
    rows = 1
    for s in t.shape[:-1]:
        rows *= s
    return rows, T


def _check(t: torch.Tensor, name: str, like: torch.Tensor | None = None):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (the scan has no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if like is not None and (t.shape != like.shape or t.dtype != like.dtype or t.device != like.device):
        raise RuntimeError(f"{name} must match gates in shape, dtype and device")


def _carry(t, rows: int, name: str, device):
    if t is None:
        return None
    if t.device != device or t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != rows:
        raise RuntimeError(f"{name} must be a contiguous fp32 CUDA tensor with one element per row")
    return t


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


class CudaScanOps:
    """Local (one GPU) passes of the scan, fp32 carries."""

    @staticmethod
    def forward(gates, tokens, h0=None, want_last=False):
        _check(gates, "gates")
        _check(tokens, "tokens", gates)
        rows, T = _rows_T(gates)
        h0 = _carry(h0, rows, "h0", gates.device)
        states = torch.empty_like(gates)
        h_last = torch.empty(gates.shape[:-1], device=gates.device, dtype=torch.float32) if want_last else None
        with torch.cuda.device(gates.device):
            capi.call("fms_plain_forward", capi.ptr(gates), capi.ptr(tokens), capi.ptr(h0),
                      capi.ptr(states), capi.ptr(h_last), rows, T, capi.dtype_tag(gates.dtype),
                      _stream(gates))
        return (states, h_last) if want_last else states

    @staticmethod
    def backward(gates, states, grad_states, h0=None, carry_in=None, want_grad_h0=False):
        _check(gates, "gates")
        _check(states, "states", gates)
        _check(grad_states, "grad_states", gates)
        rows, T = _rows_T(gates)
        h0 = _carry(h0, rows, "h0", gates.device)
        carry_in = _carry(carry_in, rows, "carry_in", gates.device)
        grad_gates = torch.empty_like(gates)
        grad_tokens = torch.empty_like(gates)
        grad_h0 = (torch.empty(gates.shape[:-1], device=gates.device, dtype=torch.float32)
                   if want_grad_h0 else None)
        with torch.cuda.device(gates.device):
            capi.call("fms_plain_backward", capi.ptr(gates), capi.ptr(states), capi.ptr(grad_states),
                      capi.ptr(h0), capi.ptr(carry_in), capi.ptr(grad_gates), capi.ptr(grad_tokens),
                      capi.ptr(grad_h0), rows, T, capi.dtype_tag(gates.dtype), _stream(gates))
        return grad_gates, grad_tokens, grad_h0

    @staticmethod
    def reduce(gates, tokens):
        """(P, S): product of the gates and last state from a zero start, per row."""
        _check(gates, "gates")
        _check(tokens, "tokens", gates)
        rows, T = _rows_T(gates)
        P = torch.empty(gates.shape[:-1], device=gates.device, dtype=torch.float32)
        S = torch.empty_like(P)
        with torch.cuda.device(gates.device):
            capi.call("fms_plain_reduce", capi.ptr(gates), capi.ptr(tokens), capi.ptr(P), capi.ptr(S),
                      rows, T, capi.dtype_tag(gates.dtype), _stream(gates))
        return P, S

    @staticmethod
    def reduce_reverse(gates, grad_states):
        """S_rev = a_0 * delta_0 from a zero carry-in, per row."""
        _check(gates, "gates")
        _check(grad_states, "grad_states", gates)
        rows, T = _rows_T(gates)
        S = torch.empty(gates.shape[:-1], device=gates.device, dtype=torch.float32)
        with torch.cuda.device(gates.device):
            capi.call("fms_plain_reduce_reverse", capi.ptr(gates), capi.ptr(grad_states), None,
                      capi.ptr(S), rows, T, capi.dtype_tag(gates.dtype), _stream(gates))
        return S

    @staticmethod
    def combine(P, S, carry0=None, reverse=False):
        """Fold (nchunks, rows) carries: returns (carry entering each chunk, carry leaving the last)."""
        if not (P.is_cuda and P.dtype == torch.float32 and P.is_contiguous() and P.dim() == 2
                and S.shape == P.shape and S.dtype == P.dtype and S.is_contiguous()):
            raise RuntimeError("P and S must be contiguous fp32 CUDA tensors of shape (nchunks, rows)")
        nchunks, rows = P.shape
        carry0 = _carry(carry0, rows, "carry0", P.device)
        out = torch.empty_like(P)
        total = torch.empty(rows, device=P.device, dtype=torch.float32)
        with torch.cuda.device(P.device):
            capi.call("fms_combine_carries", capi.ptr(P), capi.ptr(S), capi.ptr(carry0), capi.ptr(out),
                      capi.ptr(total), nchunks, rows, int(bool(reverse)), _stream(P))
        return out, total
