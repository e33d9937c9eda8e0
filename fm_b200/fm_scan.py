"""Python op API of the scan, mirroring fm/scan/fm_scan.py of the reference.

``fm_scan(gates, tokens, initial_state=None)`` keeps the reference's call surface
(fm/scan/fm_scan.py:84-99) on the plain recurrence and layout

    gates a, tokens x, states h : (B, D, T)        h[b,d,t] = a[b,d,t] * h[b,d,t-1] + x[b,d,t]

``FM_Scan`` is the autograd function (fm/scan/fm_scan.py:37-81): forward allocates the output
and saves ``(gates, states)``; backward runs one fused reverse kernel that writes ``grad_gates``
and ``grad_tokens`` directly in the inputs' shape (no full-size temporaries, no reductions) and
returns ``(d_gates, d_tokens, d_initial_state)``.  Unlike the reference, a non-zero
``initial_state`` is honoured in backward and receives its gradient.

The compiled extension is loaded lazily on first use; if it is missing the call raises --
nothing here computes on the CPU.
"""
from __future__ import annotations

import importlib

import torch

from ._nvtx import nvtx_range

_ext = None


def _load_ext():
    global _ext
    if _ext is None:
        try:
            _ext = importlib.import_module("fm_b200._fm_scan_ext")
        except ImportError as e:
            raise RuntimeError(
                "fm_b200._fm_scan_ext is not built or cannot be loaded "
                "(run `python -m fm_b200.build`); there is no fallback implementation") from e
    return _ext


def fm_scan_forward(gates, tokens, initial_state, out):
    """C++ entry point, reference signature (fm/scan/fm_scan.cuh:344-345): writes and returns ``out``."""
    return _load_ext().fm_scan_forward(gates, tokens, initial_state, out)


def fm_scan_backward(gates, outGrad, firstPropGrad, tokenGradOut, cached_output, input_tokens, gateGradOut):
    """C++ entry point, reference signature (fm/scan/fm_scan.cuh:361-366)."""
    return _load_ext().fm_scan_backward(gates, outGrad, firstPropGrad, tokenGradOut, cached_output,
                                        input_tokens, gateGradOut)


def fm_scan_backward_ex(gates, outGrad, carry_in, tokenGradOut, cached_output, gateGradOut,
                        initial_state=None, grad_initial_state=None):
    """Backward with the forward initial state and its gradient (fp32, one value per row)."""
    return _load_ext().fm_scan_backward_ex(gates, outGrad, carry_in, tokenGradOut, cached_output,
                                           gateGradOut, initial_state, grad_initial_state)


def fm_scan_backward_fm(gates, outGrad, tokenGradOut, cached_output, input_tokens, gateGradOut,
                        initial_state=None, grad_initial_state=None):
    """FM-mode backward with the reductions over D and M fused into the kernel."""
    return _load_ext().fm_scan_backward_fm(gates, outGrad, tokenGradOut, cached_output, input_tokens,
                                           gateGradOut, initial_state, grad_initial_state)


class FM_Scan_Outer(torch.autograd.Function):
    """The reference's operator in its own layout (fm/scan/fm_scan.py:37-81):
    gates (B,M,L), tokens (B,D,L), initial_state (B,M,D) -> states (B,M,D,L) with
    ``h = g*h + (1-g)*x``.  Backward returns ``d_gates (B,M,L)``, ``d_tokens (B,D,L)`` and
    ``d_initial_state`` straight from one kernel: the two (B,M,D,L) temporaries and the two sums
    of the reference's backward (fm/scan/fm_scan.py:70-78) are fused away."""

    @staticmethod
    def forward(ctx, gates, tokens, initial_state=None):
        B1, M, L1 = gates.shape
        B, D, L = tokens.shape
        assert L1 == L
        assert B == B1
        assert gates.is_contiguous()
        assert tokens.is_contiguous()
        if initial_state is not None:
            assert initial_state.shape == (B, M, D)
            assert initial_state.is_contiguous()
        output = torch.empty([B, M, D, L], device=gates.device, dtype=gates.dtype)
        states = fm_scan_forward(gates, tokens, initial_state, output)
        ctx.save_for_backward(tokens, gates, states, initial_state)
        ctx.h0_needs_grad = initial_state is not None and ctx.needs_input_grad[2]
        return states

    @staticmethod
    def backward(ctx, grad_output):
        tokens, gates, states, initial_state = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        d_gates = torch.empty_like(gates)
        d_tokens = torch.empty_like(tokens)
        d_h0 = None
        if ctx.h0_needs_grad:
            d_h0 = torch.empty(initial_state.shape, device=gates.device, dtype=torch.float32)
        fm_scan_backward_fm(gates, grad_output, d_tokens, states, tokens, d_gates, initial_state, d_h0)
        if d_h0 is not None:
            d_h0 = d_h0.to(initial_state.dtype)
        return d_gates, d_tokens, d_h0


class FM_Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gates, tokens, initial_state=None):
        assert gates.dim() >= 1 and gates.shape == tokens.shape, \
            f"gates {tuple(gates.shape)} and tokens {tuple(tokens.shape)} must have the same shape"
        assert gates.is_contiguous()
        assert tokens.is_contiguous()
        if initial_state is not None:
            assert initial_state.shape == gates.shape[:-1]
            assert initial_state.is_contiguous()
        output = torch.empty_like(gates)
        with nvtx_range("fm_scan.forward"):
            states = fm_scan_forward(gates, tokens, initial_state, output)
        ctx.save_for_backward(gates, states, initial_state)
        ctx.h0_needs_grad = initial_state is not None and ctx.needs_input_grad[2]
        return states

    @staticmethod
    def backward(ctx, grad_output):
        gates, states, initial_state = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        d_gates = torch.empty_like(gates)
        d_tokens = torch.empty_like(gates)
        d_h0 = None
        if ctx.h0_needs_grad:
            d_h0 = torch.empty(initial_state.shape, device=gates.device, dtype=torch.float32)
        with nvtx_range("fm_scan.backward"):
            fm_scan_backward_ex(gates, grad_output, None, d_tokens, states, d_gates, initial_state, d_h0)
        if d_h0 is not None:
            d_h0 = d_h0.to(initial_state.dtype)
        return d_gates, d_tokens, d_h0


class FM_Scan_BTD(torch.autograd.Function):
    """The plain scan on channel-last tensors: gates, tokens, states (B, T, D), recurrence along T,
    initial_state (B, D).  This is the layout the reference's layer holds before it transposes
    for every call (fm/scan/fm_scan.py:118-119)."""

    @staticmethod
    def forward(ctx, gates, tokens, initial_state=None):
        assert gates.dim() == 3 and gates.shape == tokens.shape
        assert gates.is_contiguous()
        assert tokens.is_contiguous()
        if initial_state is not None:
            assert initial_state.shape == (gates.shape[0], gates.shape[2])
            assert initial_state.is_contiguous()
        states = _load_ext().fm_scan_btd_forward(gates, tokens, initial_state, torch.empty_like(gates))
        ctx.save_for_backward(gates, states, initial_state)
        ctx.h0_needs_grad = initial_state is not None and ctx.needs_input_grad[2]
        return states

    @staticmethod
    def backward(ctx, grad_output):
        gates, states, initial_state = ctx.saved_tensors
        d_gates, d_tokens = torch.empty_like(gates), torch.empty_like(gates)
        d_h0 = None
        if ctx.h0_needs_grad:
            d_h0 = torch.empty(initial_state.shape, device=gates.device, dtype=torch.float32)
        _load_ext().fm_scan_btd_backward(gates, grad_output.contiguous(), d_tokens, states, d_gates,
                                         initial_state, d_h0)
        if d_h0 is not None:
            d_h0 = d_h0.to(initial_state.dtype)
        return d_gates, d_tokens, d_h0


def fm_scan(gates, tokens, initial_state=None, mode="plain"):
    """Solve the first-order recurrence along the last axis.

    ``mode="plain"`` (default): ``h_t = a_t * h_{t-1} + x_t`` on independent rows.
        gates (torch.Tensor): a, shape (B, D, T), contiguous CUDA tensor, fp32 / fp16 / bf16.
            Any T >= 1 (the reference required a power of two in [32, 131072]).
        tokens (torch.Tensor): x, same shape, dtype and device.
        initial_state (torch.Tensor, optional): h_{-1}, shape (B, D); zeros when omitted.
        Returns states h, shape (B, D, T), dtype of ``gates``.

    ``mode="fm"``: the reference's operator in its own layout (fm/scan/fm_scan.py:84-99),
        ``h[b,m,d,t] = g[b,m,t] * h[b,m,d,t-1] + (1 - g[b,m,t]) * x[b,d,t]``
        gates (B, M, L), tokens (B, D, L), initial_state (B, M, D) -> states (B, M, D, L).

    ``mode="btd"``: the plain recurrence on channel-last tensors, gates, tokens (B, T, D),
        initial_state (B, D) -> states (B, T, D); D * element size must be a multiple of 16 bytes.

    Arithmetic is fp32 in all modes.
    """
    if mode == "btd":
        return FM_Scan_BTD.apply(gates, tokens, initial_state)
    if mode == "fm":
        return FM_Scan_Outer.apply(gates, tokens, initial_state)
    if mode != "plain":
        raise ValueError("mode must be 'plain', 'fm' or 'btd'")
    return FM_Scan.apply(gates, tokens, initial_state)
