"""The CPU oracle against the golden outputs of the unmodified reference function."""
import numpy as np
import pytest

from oracle import c_oracle as oc
from tests import helpers as H


def _sampled(arr, g):
    return arr[:, g["sample_idx"]] if "sample_idx" in g else arr


@pytest.mark.parametrize("name", H.golden_names("plain_via_fold"))
def test_plain_forward_matches_reference_bit_for_bit(name):
    g = H.load_golden(name)
    a, x = g["a"], g["x"]
    xp = ((np.float32(1) - a) * x).astype(np.float32)  # update weight folded into the tokens
    h = oc.plain_forward(a, xp, g.get("h0"))
    assert np.array_equal(_sampled(h, g), g["ref32_h"]), name


@pytest.mark.parametrize("name", H.golden_names("plain_via_fold"))
def test_plain_backward_matches_reference(name):
    g = H.load_golden(name)
    a, x, G = g["a"], g["x"], g["G"]
    xp = ((np.float32(1) - a) * x).astype(np.float32)
    h = oc.plain_forward(a, xp, g.get("h0"))
    ga, gx, gh0 = oc.plain_backward(a, h, G, g.get("h0"))
    d_tokens = (np.float32(1) - a) * gx
    d_gates = ga - x * gx
    H.assert_close(_sampled(d_tokens, g), g["ref32_d_tokens"], H.FP32_RTOL, H.FP32_ATOL, "d_tokens")
    # d_gates is a difference of two products of comparable size; its rounding scales with them
    scale = float(np.max(np.abs(ga)) + np.max(np.abs(x * gx)))
    H.assert_close(_sampled(d_gates, g), g["ref32_d_gates"], H.FP32_RTOL, 2e-7 * scale + H.FP32_ATOL,
                   "d_gates")
    if "ref32_d_h0" in g:
        H.assert_close(gh0, g["ref32_d_h0"], H.FP32_RTOL, H.FP32_ATOL, "d_h0")


@pytest.mark.parametrize("name", [n for n in H.golden_names("plain_via_fold")
                                  if "ref64_h" in H.manifest()[n]["arrays"]])
def test_plain_double_precision_matches_reference(name):
    g = H.load_golden(name)
    a, x, G = (g[k].astype(np.float64) for k in ("a", "x", "G"))
    h0 = g["h0"].astype(np.float64) if "h0" in g else None
    xp = (1.0 - a) * x
    h = oc.plain_forward(a, xp, h0, dtype=np.float64)
    ga, gx, gh0 = oc.plain_backward(a, h, G, h0, dtype=np.float64)
    H.assert_close(_sampled(h, g), g["ref64_h"], 1e-13, 1e-13, "h64")
    H.assert_close(_sampled((1.0 - a) * gx, g), g["ref64_d_tokens"], 1e-12, 1e-12, "d_tokens64")
    H.assert_close(_sampled(ga - x * gx, g), g["ref64_d_gates"], 1e-11, 1e-11, "d_gates64")
    if "ref64_d_h0" in g:
        H.assert_close(gh0, g["ref64_d_h0"], 1e-12, 1e-12, "d_h0_64")


@pytest.mark.parametrize("name", H.golden_names("fm"))
def test_fm_mode_matches_reference(name):
    g = H.load_golden(name)
    h = oc.fm_forward(g["g"], g["x"], g.get("h0"))
    assert np.array_equal(h, g["ref32_h"]), name
    dg, dx, dh0 = oc.fm_backward(g["g"], g["x"], h, g["G"], g.get("h0"))
    H.assert_close(dx, g["ref32_d_tokens"], 1e-5, 2e-6, "fm d_tokens")
    H.assert_close(dg, g["ref32_d_gates"], 1e-5, 5e-6, "fm d_gates")
    if "ref32_d_h0" in g:
        H.assert_close(dh0, g["ref32_d_h0"], 1e-5, 1e-6, "fm d_h0")
    h64 = oc.fm_forward(g["g"], g["x"], g.get("h0"), dtype=np.float64)
    H.assert_close(h64, g["ref64_h"], 1e-13, 1e-13, "fm h64")
    dg, dx, dh0 = oc.fm_backward(g["g"], g["x"], h64, g["G"], g.get("h0"), dtype=np.float64)
    H.assert_close(dx, g["ref64_d_tokens"], 1e-12, 1e-12, "fm d_tokens64")
    H.assert_close(dg, g["ref64_d_gates"], 1e-12, 1e-12, "fm d_gates64")


def test_fold_identity_plain_rows_equal_fm_with_unit_dims():
    """FM mode with M = D = 1 is the plain scan of (a, (1-a) x) row for row."""
    a, x, G = H.make_inputs(7, 130, 5, "sigmoid01")
    h_fm = oc.fm_forward(a.reshape(7, 1, 130), x.reshape(7, 1, 130)).reshape(7, 130)
    h_pl = oc.plain_forward(a, ((np.float32(1) - a) * x).astype(np.float32))
    assert np.array_equal(h_fm, h_pl)


def test_reduce_composes_across_chunks():
    """(P, S) of consecutive chunks chain to the unsplit scan: h_last = P h_in + S."""
    a, x, _ = H.make_inputs(5, 4 * 97, 6, "sigmoid+3")
    a64, x64 = a.astype(np.float64), x.astype(np.float64)
    h, h_last = oc.plain_forward(a64, x64, dtype=np.float64, return_last=True)
    carry = np.zeros(5)
    for k in range(4):
        sl = slice(k * 97, (k + 1) * 97)
        P, S = oc.plain_reduce(a64[:, sl], x64[:, sl], dtype=np.float64)
        hk = oc.plain_forward(a64[:, sl], x64[:, sl], carry, dtype=np.float64)
        np.testing.assert_allclose(hk, h[:, sl], rtol=1e-12, atol=1e-12)
        carry = P * carry + S
    np.testing.assert_allclose(carry, h_last, rtol=1e-12, atol=1e-12)


def test_backward_is_gradient_of_forward_fd():
    """Finite differences in double precision on a tiny case, including h0 and carry terms."""
    rng = np.random.default_rng(3)
    R, T = 3, 9
    a = rng.uniform(0.2, 0.99, (R, T))
    x = rng.standard_normal((R, T))
    G = rng.standard_normal((R, T))
    h0 = rng.standard_normal(R)

    def loss(a_, x_, h0_):
        return float((oc.plain_forward(a_, x_, h0_, dtype=np.float64) * G).sum())

    h = oc.plain_forward(a, x, h0, dtype=np.float64)
    ga, gx, gh0 = oc.plain_backward(a, h, G, h0, dtype=np.float64)
    eps = 1e-6
    for (r, t) in [(0, 0), (1, 4), (2, 8)]:
        da = a.copy(); da[r, t] += eps
        dx = x.copy(); dx[r, t] += eps
        assert abs((loss(da, x, h0) - loss(a, x, h0)) / eps - ga[r, t]) < 1e-4
        assert abs((loss(a, dx, h0) - loss(a, x, h0)) / eps - gx[r, t]) < 1e-4
    dh = h0.copy(); dh[1] += eps
    assert abs((loss(a, x, dh) - loss(a, x, h0)) / eps - gh0[1]) < 1e-4


@pytest.mark.parametrize("name", H.golden_names("layer"))
def test_layer_restatement_matches_the_reference_layer(name):
    """``oracle.torch_loop.fm_memory_loop`` against outputs of the reference's own ``fm_memory``
    (compiled from the reference file's syntax tree and run over its CPU scan): output, returned
    states and the gradients of every input, fp32 and fp64."""
    import torch
    from oracle.torch_loop import fm_memory_loop
    g = H.load_golden(name)
    mem_norm = H.manifest()[name]["mem_norm"]
    for tag, dt, rtol, atol in (("ref32_", torch.float32, 1e-5, 2e-6), ("ref64_", torch.float64, 1e-12, 1e-12)):
        args = [torch.from_numpy(g[k]).to(dt).requires_grad_(True)
                for k in ("alpha", "update_scale", "output_scale", "inputs")]
        h0 = torch.from_numpy(g["h0"]).to(dt).requires_grad_(True) if "h0" in g else None
        out, states = fm_memory_loop(*args, initial_state=h0, mem_norm=mem_norm)
        ((out * torch.from_numpy(g["W"]).to(dt)).sum() + (states * torch.from_numpy(g["Gs"]).to(dt)).sum()).backward()
        if dt == torch.float32:
            # same torch ops in the same order as the reference: forward is bit-identical
            assert np.array_equal(out.detach().numpy(), g[tag + "out"]), name
            assert np.array_equal(states.detach().numpy(), g[tag + "states"]), name
        got = {"out": out.detach(), "states": states.detach(), "d_alpha": args[0].grad,
               "d_update_scale": args[1].grad, "d_output_scale": args[2].grad, "d_inputs": args[3].grad}
        if h0 is not None:
            got["d_h0"] = h0.grad
        for k, v in got.items():
            ref = g[tag + k]
            H.assert_close(v.numpy(), ref, rtol, atol * max(1.0, float(np.abs(ref).max())), f"{name} {tag}{k}")
