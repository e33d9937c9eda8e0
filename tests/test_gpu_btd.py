"""The plain scan on channel-last (B, T, D) tensors against the oracle (rows = (b, d), time axis
moved last) and against the (B, D, T) kernels."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as oc
from tests import gpu_util as G
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("storage,B,T,D", [("f32", 2, 300, 8), ("bf16", 3, 1000, 40), ("f16", 1, 17, 264),
                                            ("f32", 1, 1, 4), ("bf16", 2, 4096, 256), ("f32", 4, 77, 132)])
def test_channel_last_scan_matches_oracle(storage, B, T, D):
    from fm_b200 import fm_scan
    a, x, Gd, h0 = H.make_inputs(B * D, T, 300 + T, "sigmoid01", storage, with_h0=True)   # rows = (b, d)
    to_btd = lambda v: np.ascontiguousarray(v.reshape(B, D, T).transpose(0, 2, 1))
    ad = G.dev(to_btd(a), storage).requires_grad_(True)
    xd = G.dev(to_btd(x), storage).requires_grad_(True)
    h0d = G.dev(h0.reshape(B, D), storage).requires_grad_(True)
    h = fm_scan(ad, xd, h0d, mode="btd")
    h.backward(G.dev(to_btd(Gd), storage))
    torch.cuda.synchronize()
    back = lambda t: G.host(t).transpose(0, 2, 1).reshape(B * D, T)
    f64 = np.float64
    hs = back(h)
    h_ref = oc.plain_forward(a.astype(f64), x.astype(f64), h0.astype(f64), dtype=f64)
    ga_ref, gx_ref, gh0_ref = oc.plain_backward(a.astype(f64), hs.astype(f64), Gd.astype(f64), h0.astype(f64), dtype=f64)
    if storage == "f32":
        tol = lambda r: (H.FP32_RTOL, H.FP32_ATOL * max(1.0, float(np.abs(r).max())))
    else:
        tol = lambda r: (H.LOWP_RTOL, H.lowp_atol(r) + 1e-3)
    H.assert_close(hs, h_ref, *tol(h_ref), "states")
    H.assert_close(back(xd.grad), gx_ref, *tol(gx_ref), "grad_tokens")
    H.assert_close(back(ad.grad), ga_ref, *tol(ga_ref), "grad_gates")
    H.assert_close(G.host(h0d.grad).reshape(-1), gh0_ref, 2e-2 if storage != "f32" else 1e-4,
                   (2e-2 if storage != "f32" else 1e-5) * max(1.0, float(np.abs(gh0_ref).max())), "grad_h0")


def test_channel_last_rejects_unaligned_channels():
    from fm_b200 import fm_scan
    a = torch.rand(1, 8, 3, device="cuda")       # 3 fp32 channels = 12 bytes per step
    with pytest.raises(RuntimeError, match="aligned"):
        fm_scan(a, a.clone(), mode="btd")
