"""ctypes/numpy wrapper over the C oracle (``fm_scan_oracle.c``).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA path, never the product.
Each function follows the reference loop ``fm_scan_pytorch``
(fm/scan/fm_pytorch.py:19-42) or the backward autograd derives from it
(the quantities of fm/scan/fm_scan.cuh:184-207 + fm/scan/fm_scan.py:75-78).
Parity is pinned by ``tests/test_oracle.py`` against ``tests/golden/*.npz``,
which hold outputs of the unmodified reference function.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile ``liboracle.so`` next to its source with gcc (via the Makefile)."""
    src = _HERE / "fm_scan_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-s", "-C", str(_HERE), "-B", "liboracle.so"], check=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(ctypes.c_int(int(n)))


def _sfx(dtype) -> str:
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError(f"oracle computes in float32 or float64, not {dtype}")


def _c(arr, dtype):
    return np.ascontiguousarray(arr, dtype=dtype)


def _p(arr):
    return None if arr is None else arr.ctypes.data_as(ctypes.c_void_p)


def plain_forward(a, x, h0=None, dtype=np.float32, return_last=False):
    """h[..., t] = a[..., t] * h[..., t-1] + x[..., t] along the last axis.

    ``a`` and ``x`` have the same shape ``(..., T)``; ``h0`` has shape ``(...)``.
    """
    a = _c(a, dtype)
    x = _c(x, dtype)
    assert a.shape == x.shape
    T = a.shape[-1] if a.ndim else 1
    R = a.size // T if T else 0
    h = np.empty_like(a)
    h_last = np.empty(a.shape[:-1], dtype=dtype)
    h0c = None if h0 is None else _c(h0, dtype)
    if h0c is not None:
        assert h0c.size == R
    fn = getattr(lib(), f"oracle_plain_forward_{_sfx(dtype)}")
    fn(_p(a), _p(x), _p(h0c), _p(h), _p(h_last), ctypes.c_int64(R), ctypes.c_int64(T))
    if T == 0:
        h_last[...] = 0 if h0c is None else h0c.reshape(h_last.shape)
    return (h, h_last) if return_last else h


def plain_backward(a, h, G, h0=None, carry_in=None, dtype=np.float32):
    """Returns (grad_a, grad_x, grad_h0) for the PLAIN scan given saved states ``h``."""
    a = _c(a, dtype)
    h = _c(h, dtype)
    G = _c(G, dtype)
    assert a.shape == h.shape == G.shape
    T = a.shape[-1]
    R = a.size // T if T else 0
    ga = np.empty_like(a)
    gx = np.empty_like(a)
    gh0 = np.empty(a.shape[:-1], dtype=dtype)
    h0c = None if h0 is None else _c(h0, dtype)
    cin = None if carry_in is None else _c(carry_in, dtype)
    fn = getattr(lib(), f"oracle_plain_backward_{_sfx(dtype)}")
    fn(_p(a), _p(h), _p(G), _p(h0c), _p(cin), _p(ga), _p(gx), _p(gh0),
       ctypes.c_int64(R), ctypes.c_int64(T))
    return ga, gx, gh0


def plain_reduce(a, x, dtype=np.float32):
    """Per-row carries (P = prod a, S = last state from a zero start)."""
    a = _c(a, dtype)
    x = _c(x, dtype)
    T = a.shape[-1]
    R = a.size // T if T else 0
    P = np.empty(a.shape[:-1], dtype=dtype)
    S = np.empty(a.shape[:-1], dtype=dtype)
    fn = getattr(lib(), f"oracle_plain_reduce_{_sfx(dtype)}")
    fn(_p(a), _p(x), _p(P), _p(S), ctypes.c_int64(R), ctypes.c_int64(T))
    return P, S


def fm_forward(g, x, h0=None, dtype=np.float32):
    """Reference operator: g (B,M,L), x (B,D,L), h0 (B,M,D) -> h (B,M,D,L)."""
    g = _c(g, dtype)
    x = _c(x, dtype)
    B, M, L = g.shape
    B1, D, L1 = x.shape
    assert B == B1 and L == L1
    h0c = None if h0 is None else _c(h0, dtype)
    if h0c is not None:
        assert h0c.shape == (B, M, D)
    h = np.empty((B, M, D, L), dtype=dtype)
    fn = getattr(lib(), f"oracle_fm_forward_{_sfx(dtype)}")
    fn(_p(g), _p(x), _p(h0c), _p(h), *(ctypes.c_int64(v) for v in (B, M, D, L)))
    return h


def fm_backward(g, x, h, G, h0=None, dtype=np.float32):
    """Returns (d_gates (B,M,L), d_tokens (B,D,L), d_h0 (B,M,D))."""
    g = _c(g, dtype)
    x = _c(x, dtype)
    h = _c(h, dtype)
    G = _c(G, dtype)
    B, M, L = g.shape
    D = x.shape[1]
    assert h.shape == (B, M, D, L) and G.shape == h.shape
    h0c = None if h0 is None else _c(h0, dtype)
    dg = np.empty((B, M, L), dtype=dtype)
    dx = np.empty((B, D, L), dtype=dtype)
    dh0 = np.empty((B, M, D), dtype=dtype)
    fn = getattr(lib(), f"oracle_fm_backward_{_sfx(dtype)}")
    fn(_p(g), _p(x), _p(h), _p(G), _p(h0c), _p(dg), _p(dx), _p(dh0),
       *(ctypes.c_int64(v) for v in (B, M, D, L)))
    return dg, dx, dh0
