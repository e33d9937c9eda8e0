"""Oracle-backed stand-in for ``fm_b200.ops.CudaScanOps`` so that the exchange logic of the
split-along-T scan can run on CPU ranks (gloo).  Test infrastructure only."""
import numpy as np
import torch

from oracle import c_oracle as oc


def _np(t, dtype=np.float64):
    return None if t is None else t.detach().cpu().numpy().astype(dtype)


class OracleScanOps:
    dtype = np.float64

    @classmethod
    def forward(cls, gates, tokens, h0=None, want_last=False):
        h, last = oc.plain_forward(_np(gates), _np(tokens), _np(h0), dtype=cls.dtype, return_last=True)
        h = torch.from_numpy(h).to(gates.dtype)
        return (h, torch.from_numpy(last).float()) if want_last else h

    @classmethod
    def backward(cls, gates, states, grad_states, h0=None, carry_in=None, want_grad_h0=False):
        ga, gx, gh0 = oc.plain_backward(_np(gates), _np(states), _np(grad_states), _np(h0),
                                        _np(carry_in), dtype=cls.dtype)
        return (torch.from_numpy(ga).to(gates.dtype), torch.from_numpy(gx).to(gates.dtype),
                torch.from_numpy(gh0).float() if want_grad_h0 else None)

    @classmethod
    def reduce(cls, gates, tokens):
        P, S = oc.plain_reduce(_np(gates), _np(tokens), dtype=cls.dtype)
        return torch.from_numpy(P).float(), torch.from_numpy(S).float()

    @classmethod
    def reduce_reverse(cls, gates, grad_states):
        a, G = _np(gates), _np(grad_states)
        h = np.zeros_like(a)
        _, _, gh0 = oc.plain_backward(a, h, G, dtype=cls.dtype)
        return torch.from_numpy(gh0).float()

    @staticmethod
    def combine(P, S, carry0=None, reverse=False):
        n, rows = P.shape
        out = torch.empty_like(P)
        c = torch.zeros(rows) if carry0 is None else carry0.clone().float()
        order = range(n - 1, -1, -1) if reverse else range(n)
        for k in order:
            out[k] = c
            c = P[k] * c + S[k]
        return out, c
