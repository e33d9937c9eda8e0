"""The reference's CPU scan restated with torch ops -- TEST/BASELINE INFRASTRUCTURE ONLY.

``fm_scan_loop`` follows ``fm_scan_pytorch`` (fm/scan/fm_pytorch.py:19-42) step for
step: one Python iteration per time step, each a broadcast multiply-add over all
rows, results stacked along a new last axis; backward is ordinary autograd
through the T-step graph, as in the reference.  ``plain_scan_loop`` is the same
loop with the update weight ``1 - gates`` dropped (fm_pytorch.py:22,37), i.e. the
recurrence h_t = a_t * h_{t-1} + x_t on (B, D, T) tensors.

This is the implementation ``bench.py --impl reference`` times on the host
cores: the reference's own CPU code cannot be shipped, so its loop structure
(T dispatch-bound steps) is reproduced here and checked against the golden
vectors the real function produced.
"""
from __future__ import annotations

import torch


def fm_scan_loop(gates: torch.Tensor, tokens: torch.Tensor, initial_state=None) -> torch.Tensor:
    """gates (B,M,L), tokens (B,D,L), initial_state (B,M,D) -> states (B,M,D,L)."""
    B, M, L = gates.shape
    B1, D, L1 = tokens.shape
    assert B == B1 and L == L1
    updates = 1 - gates
    if initial_state is None:
        state = torch.zeros([B, M, D], device=gates.device, dtype=gates.dtype)
    else:
        assert initial_state.shape == (B, M, D)
        state = initial_state
    steps = []
    for t in range(L):
        state = (gates[:, :, t].unsqueeze(-1) * state
                 + updates[:, :, t].unsqueeze(-1) * tokens[:, :, t].unsqueeze(1))
        steps.append(state)
    return torch.stack(steps, dim=3)


def plain_scan_loop(gates: torch.Tensor, tokens: torch.Tensor, initial_state=None) -> torch.Tensor:
    """gates, tokens (B,D,T), initial_state (B,D) -> states (B,D,T)."""
    assert gates.shape == tokens.shape
    B, D, T = gates.shape
    if initial_state is None:
        state = torch.zeros([B, D], device=gates.device, dtype=gates.dtype)
    else:
        assert initial_state.shape == (B, D)
        state = initial_state
    steps = []
    for t in range(T):
        state = gates[:, :, t] * state + tokens[:, :, t]
        steps.append(state)
    return torch.stack(steps, dim=2)


def plain_fwd_bwd(gates, tokens, grad_states, initial_state=None):
    """Forward + autograd backward of the PLAIN loop; returns (h, grad_a, grad_x)."""
    a = gates.detach().clone().requires_grad_(True)
    x = tokens.detach().clone().requires_grad_(True)
    h = plain_scan_loop(a, x, initial_state)
    (h * grad_states).sum().backward()
    return h.detach(), a.grad, x.grad


def fm_memory_loop(alpha, update_scale, output_scale, inputs, initial_state=None, mem_norm=True, norm_eps=1e-6):
    """The layer around the scan (fm/scan/fm_scan.py:102-133) on top of ``fm_scan_loop``; same
    arguments and returns as the reference's ``fm_memory``."""
    update_weight = alpha * update_scale
    tokens = inputs.transpose(1, 2).contiguous()
    update_weight = update_weight.transpose(1, 2).contiguous()
    decay_weight = 1.0 - update_weight
    memory_states = fm_scan_loop(decay_weight, tokens, initial_state)
    if mem_norm:
        memory_rms = torch.rsqrt(torch.mean(memory_states ** 2, dim=2, keepdim=True) + norm_eps)
        memory_states = memory_states * memory_rms
    output_weight = alpha * output_scale
    output = torch.einsum('blm,bmdl->bld', output_weight, memory_states).contiguous()
    return output, memory_states
