"""The Factorization-Memory layer around the scan, mirroring ``fm_memory`` of the reference
(fm/scan/fm_scan.py:102-133): same arguments, same returns.

Everything except the scan is stock torch, as in the reference; the scan is this package's
FM-mode op (one fused backward kernel instead of two (B,M,D,L) temporaries and two sums).
"""
from __future__ import annotations

import torch

from .fm_scan import _load_ext, fm_scan


class _FusedLayer(torch.autograd.Function):
    """Scan + RMS norm over D + read-out over M as one differentiable op on (B,.,L) tensors.

    forward(decay (B,M,L), tokens (B,D,L), out_weight (B,M,L), initial_state (B,M,D) | None)
        -> out (B,D,L), normalised states (B,M,D,L)
    Saved for backward: the inputs, the normalised states and the fp32 norm factor (B,M,L); the
    raw states are recovered from them inside the backward kernel.
    """

    @staticmethod
    def forward(ctx, decay, tokens, out_weight, initial_state, mem_norm, eps):
        B, M, L = decay.shape
        D = tokens.shape[1]
        out = torch.empty_like(tokens)
        states = torch.empty((B, M, D, L), device=decay.device, dtype=decay.dtype)
        rnorm = torch.empty((B, M, L), device=decay.device, dtype=torch.float32)
        _load_ext().fm_memory_forward_train(decay, tokens, out_weight, initial_state, out, states, rnorm,
                                            bool(mem_norm), float(eps))
        ctx.save_for_backward(decay, tokens, out_weight, states, rnorm, initial_state)
        ctx.mem_norm = bool(mem_norm)
        ctx.h0_needs_grad = initial_state is not None and ctx.needs_input_grad[3]
        ctx.set_materialize_grads(False)
        return out, states

    @staticmethod
    def backward(ctx, g_out, g_states):
        decay, tokens, out_weight, states, rnorm, initial_state = ctx.saved_tensors
        if g_out is None:
            g_out = torch.zeros_like(tokens)
        d_decay, d_tokens, d_weight = torch.empty_like(decay), torch.empty_like(tokens), torch.empty_like(out_weight)
        d_h0 = None
        if ctx.h0_needs_grad:
            d_h0 = torch.empty(initial_state.shape, device=decay.device, dtype=torch.float32)
        _load_ext().fm_memory_backward(decay, tokens, out_weight, states, rnorm, ctx.mem_norm, g_out.contiguous(),
                                       None if g_states is None else g_states.contiguous(), initial_state,
                                       d_decay, d_tokens, d_weight, d_h0)
        if d_h0 is not None:
            d_h0 = d_h0.to(initial_state.dtype)
        return d_decay, d_tokens, d_weight, d_h0, None, None


def _rows_aligned(t, L):
    return t.is_cuda and (L * t.element_size()) % 16 == 0 and (L * 4) % 16 == 0


def _fused_readout_applies(need_states, tensors, L):
    """The no-states path: nothing needs a gradient, the caller does not want the states, and rows
    are 16-byte aligned."""
    if need_states:
        return False
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        return False
    return _rows_aligned(tensors[0], L)


def fm_memory(alpha, update_scale, output_scale, inputs, initial_state=None, mem_norm=True, norm_eps=1e-6,
              need_states=True, fused=True):
    """
    alpha: (B, L, M)   update_scale: (B, L, 1)   output_scale: (B, L, 1)   inputs: (B, L, D)
    initial_state: (B, M, D)   mem_norm: bool   norm_eps: float

    return: output (B, L, D), memory_states (B, M, D, L)

    ``need_states=False`` (inference): when no argument requires a gradient the layer output is
    computed by recomputing the scan inside two read-out kernels and the (B, M, D, L) states are
    never written; ``memory_states`` is then returned as None.  The norm is evaluated in fp32
    there, where the reference evaluates it in the storage dtype.

    ``fused=True`` (default): with 16-byte aligned rows the scan, the norm and the read-out run as
    one differentiable op (two forward kernels, two backward kernels; the gradient of the raw
    states is generated inside the reverse scan).  ``fused=False`` keeps the reference's
    composition: FM-mode scan, then stock torch norm and einsum.
    """
    update_weight = alpha * update_scale                                 # fm_scan.py:117
    tokens = inputs.transpose(1, 2).contiguous()                         # (B, D, L)  fm_scan.py:118
    update_weight = update_weight.transpose(1, 2).contiguous()           # (B, M, L)  fm_scan.py:119
    decay_weight = 1.0 - update_weight                                   # fm_scan.py:120

    if _fused_readout_applies(need_states, (alpha, update_scale, output_scale, inputs, initial_state),
                              tokens.shape[-1]):
        out_weight = (alpha * output_scale).transpose(1, 2).contiguous()  # (B, M, L)
        out = torch.empty_like(tokens)                                    # (B, D, L)
        _load_ext().fm_memory_readout(decay_weight, tokens, out_weight, initial_state, out, bool(mem_norm),
                                      float(norm_eps))
        return out.transpose(1, 2).contiguous(), None

    if fused and _rows_aligned(tokens, tokens.shape[-1]):
        out_weight = (alpha * output_scale).transpose(1, 2).contiguous()  # (B, M, L)
        out, states = _FusedLayer.apply(decay_weight, tokens, out_weight, initial_state, bool(mem_norm),
                                        float(norm_eps))
        return out.transpose(1, 2).contiguous(), states

    memory_states = fm_scan(decay_weight, tokens, initial_state, mode="fm")  # (B, M, D, L)  fm_scan.py:122

    if mem_norm:                                                         # RMS norm over D, fm_scan.py:125-127
        memory_rms = torch.rsqrt(torch.mean(memory_states ** 2, dim=2, keepdim=True) + norm_eps)
        memory_states = memory_states * memory_rms

    output_weight = alpha * output_scale                                 # fm_scan.py:130
    output = torch.einsum('blm,bmdl->bld', output_weight, memory_states).contiguous()  # fm_scan.py:131
    return output, memory_states
