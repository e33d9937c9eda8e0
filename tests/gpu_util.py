"""Helpers for the GPU parity tests: run the scan through the C ABI on torch-owned device buffers."""
from __future__ import annotations

import numpy as np
import torch

from fm_b200 import capi

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def dev(arr, storage="f32", device="cuda"):
    """fp32 numpy array (already rounded to `storage`) -> device tensor of that storage type."""
    if arr is None:
        return None
    return torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)).to(device).to(TORCH_DT[storage])


def host(t):
    return None if t is None else t.detach().to(torch.float32).cpu().numpy()


def reload_tune():
    """Make the library read its FMS_TUNE_* environment again (it reads it once per process)."""
    capi.lib().fms_tune_reload()


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def forward(a, x, h0=None, want_last=False, out=None):
    """a, x: device tensors (..., T); h0: fp32 device tensor (...) or None."""
    T = a.shape[-1]
    rows = a.numel() // T if T else int(np.prod(a.shape[:-1]))
    h = torch.empty_like(a) if out is None else out
    h_last = torch.empty(a.shape[:-1], device=a.device, dtype=torch.float32) if want_last else None
    capi.call("fms_plain_forward", capi.ptr(a), capi.ptr(x), capi.ptr(h0), capi.ptr(h),
              capi.ptr(h_last), rows, T, capi.dtype_tag(a.dtype), stream_ptr())
    return (h, h_last) if want_last else h


def backward(a, h, G, h0=None, carry_in=None, want_gh0=False, outs=None):
    T = a.shape[-1]
    rows = a.numel() // T if T else int(np.prod(a.shape[:-1]))
    ga, gx = (torch.empty_like(a), torch.empty_like(a)) if outs is None else outs
    gh0 = torch.empty(a.shape[:-1], device=a.device, dtype=torch.float32) if want_gh0 else None
    capi.call("fms_plain_backward", capi.ptr(a), capi.ptr(h), capi.ptr(G), capi.ptr(h0),
              capi.ptr(carry_in), capi.ptr(ga), capi.ptr(gx), capi.ptr(gh0), rows, T,
              capi.dtype_tag(a.dtype), stream_ptr())
    return (ga, gx, gh0) if want_gh0 else (ga, gx)


def reduce(a, x):
    T = a.shape[-1]
    rows = a.numel() // T if T else int(np.prod(a.shape[:-1]))
    P = torch.empty(a.shape[:-1], device=a.device, dtype=torch.float32)
    S = torch.empty_like(P)
    capi.call("fms_plain_reduce", capi.ptr(a), capi.ptr(x), capi.ptr(P), capi.ptr(S), rows, T,
              capi.dtype_tag(a.dtype), stream_ptr())
    return P, S


def reduce_reverse(a, G, want_P=True):
    T = a.shape[-1]
    rows = a.numel() // T if T else int(np.prod(a.shape[:-1]))
    P = torch.empty(a.shape[:-1], device=a.device, dtype=torch.float32) if want_P else None
    S = torch.empty(a.shape[:-1], device=a.device, dtype=torch.float32)
    capi.call("fms_plain_reduce_reverse", capi.ptr(a), capi.ptr(G), capi.ptr(P), capi.ptr(S), rows, T,
              capi.dtype_tag(a.dtype), stream_ptr())
    return P, S


def combine(P, S, carry0=None, reverse=False):
    """P, S: (nchunks, rows) fp32 device tensors."""
    nchunks, rows = P.shape
    out = torch.empty_like(P)
    total = torch.empty(rows, device=P.device, dtype=torch.float32)
    capi.call("fms_combine_carries", capi.ptr(P), capi.ptr(S), capi.ptr(carry0), capi.ptr(out),
              capi.ptr(total), nchunks, rows, int(reverse), stream_ptr())
    return out, total


def split_plan(rows, T, dtype):
    L = capi.lib()
    tag = capi.dtype_tag(dtype)
    return int(L.fms_plain_split_segments(rows, T, tag)), int(L.fms_plain_split_workspace_bytes(rows, T, tag))


def forward_split(a, x, h0=None, want_last=False):
    T = a.shape[-1]
    rows = a.numel() // T
    nseg, nbytes = split_plan(rows, T, a.dtype)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=a.device)
    h = torch.empty_like(a)
    h_last = torch.empty(a.shape[:-1], device=a.device, dtype=torch.float32) if want_last else None
    capi.call("fms_plain_forward_split", capi.ptr(a), capi.ptr(x), capi.ptr(h0), capi.ptr(h),
              capi.ptr(h_last), rows, T, capi.dtype_tag(a.dtype), ws.data_ptr(), nbytes, stream_ptr())
    return (h, h_last) if want_last else h


def backward_split(a, h, G, h0=None, carry_in=None, want_gh0=False):
    T = a.shape[-1]
    rows = a.numel() // T
    nseg, nbytes = split_plan(rows, T, a.dtype)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=a.device)
    ga, gx = torch.empty_like(a), torch.empty_like(a)
    gh0 = torch.empty(a.shape[:-1], device=a.device, dtype=torch.float32) if want_gh0 else None
    capi.call("fms_plain_backward_split", capi.ptr(a), capi.ptr(h), capi.ptr(G), capi.ptr(h0),
              capi.ptr(carry_in), capi.ptr(ga), capi.ptr(gx), capi.ptr(gh0), rows, T,
              capi.dtype_tag(a.dtype), ws.data_ptr(), nbytes, stream_ptr())
    return (ga, gx, gh0) if want_gh0 else (ga, gx)


def fm_forward(g, x, h0=None):
    """g (B,M,L), x (B,D,L) device tensors; h0 (B,M,D) fp32 or None -> h (B,M,D,L)."""
    B, M, L = g.shape
    D = x.shape[1]
    h = torch.empty((B, M, D, L), device=g.device, dtype=g.dtype)
    capi.call("fms_fm_forward", capi.ptr(g), capi.ptr(x), capi.ptr(h0), capi.ptr(h), B, M, D, L,
              capi.dtype_tag(g.dtype), stream_ptr())
    return h


def fm_backward(g, x, h, G, h0=None, want_gh0=False):
    B, M, L = g.shape
    D = x.shape[1]
    dg, dx = torch.empty_like(g), torch.empty_like(x)
    gh0 = torch.empty((B, M, D), device=g.device, dtype=torch.float32) if want_gh0 else None
    tag = capi.dtype_tag(g.dtype)
    nbytes = int(capi.lib().fms_fm_backward_workspace_bytes(B, M, D, L, tag))
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=g.device)
    capi.call("fms_fm_backward", capi.ptr(g), capi.ptr(x), capi.ptr(h), capi.ptr(G), capi.ptr(h0),
              capi.ptr(dg), capi.ptr(dx), capi.ptr(gh0), B, M, D, L, tag, ws.data_ptr() if nbytes else None,
              nbytes, stream_ptr())
    return (dg, dx, gh0) if want_gh0 else (dg, dx)
