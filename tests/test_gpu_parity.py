"""Parity of the CUDA path (through the C ABI) with the pinned CPU oracle and the golden fixtures."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as oc
from tests import gpu_util as G
from tests import helpers as H

pytestmark = pytest.mark.gpu


def tol(storage, ref):
    if storage == "f32":
        return H.FP32_RTOL, H.FP32_ATOL
    return H.LOWP_RTOL, H.lowp_atol(ref)


def close_to_reference(got, ref32, ref64, storage, what, scaled=False):
    """The stated tolerance, with the reference's own fp32 rounding not charged to the kernel.

    fp32 storage: |got - ref64| <= atol + rtol |ref64| against the oracle run in double precision
    (the reference loop takes its dtype from the gates, fm/scan/fm_pytorch.py:28), and against the
    fp32 run with that run's own distance to the double-precision result added to the bound --
    two fp32 evaluations in different association orders can each sit one rounding away from the
    truth on opposite sides.  16-bit storage: rtol 2e-2 plus 1e-2 of the tensor's RMS, against
    the fp32 run directly.

    `scaled` is for long-memory fp32 data (a ~ 0.95, |h| up to ~14, |grad_gates| up to ~100): one
    fp32 rounding of such a value already exceeds 1e-6, and the next element can be near zero, so
    the absolute term is taken relative to the tensor's largest magnitude:
    atol = 1e-6 * max(1, max|ref|).  The benchmark's fp32 configurations with sigmoid gates are
    checked with the unscaled tolerance.
    """
    if storage != "f32":
        H.assert_close(got, ref32, H.LOWP_RTOL, H.lowp_atol(ref32), what)
        return
    atol = H.FP32_ATOL * (max(1.0, float(np.abs(ref64).max(initial=0))) if scaled else 1.0)
    H.assert_close(got, ref64, H.FP32_RTOL, atol, what + " (vs double)")
    got = np.asarray(got, np.float64)
    slack = np.abs(ref32.astype(np.float64) - ref64)
    bad = np.abs(got - ref32) > atol + H.FP32_RTOL * np.abs(ref32) + slack
    assert not bad.any(), f"{what}: {int(bad.sum())} elements beyond tolerance + reference rounding"


def check_fwd_bwd(a, x, Gd, storage, h0=None, carry_in=None, what="", scaled=False):
    """Kernel vs oracle on fp32 arrays already rounded to `storage`."""
    ad, xd, gd = (G.dev(v, storage) for v in (a, x, Gd))
    h0d = None if h0 is None else G.dev(h0)
    cind = None if carry_in is None else G.dev(carry_in)
    h, h_last = G.forward(ad, xd, h0d, want_last=True)
    ga, gx, gh0 = G.backward(ad, h, gd, h0d, cind, want_gh0=True)
    torch.cuda.synchronize()

    f64 = np.float64
    opt64 = lambda v: None if v is None else v.astype(f64)
    h_ref, hl_ref = oc.plain_forward(a, x, h0, return_last=True)
    h_ref64, hl_ref64 = oc.plain_forward(a.astype(f64), x.astype(f64), opt64(h0), dtype=f64,
                                         return_last=True)
    close_to_reference(G.host(h), h_ref, h_ref64, storage, what + " states", scaled)
    H.assert_close(G.host(h_last), hl_ref64, 1e-5 if storage == "f32" else 1e-4,
                   (1e-6 if storage == "f32" else 1e-4) * (1 + float(np.abs(hl_ref).max(initial=0))),
                   what + " h_last")
    # backward is checked against the oracle fed with the states the kernel itself saved
    # (rounded to storage), which is what both the reference's CUDA path and this one read back
    h_saved = G.host(h)
    ga_ref, gx_ref, gh0_ref = oc.plain_backward(a, h_saved, Gd, h0, carry_in)
    ga_ref64, gx_ref64, gh0_ref64 = oc.plain_backward(a.astype(f64), h_saved.astype(f64), Gd.astype(f64),
                                                      opt64(h0), opt64(carry_in), dtype=f64)
    close_to_reference(G.host(gx), gx_ref, gx_ref64, storage, what + " grad_tokens", scaled)
    close_to_reference(G.host(ga), ga_ref, ga_ref64, storage, what + " grad_gates", scaled)
    H.assert_close(G.host(gh0), gh0_ref64, 1e-4, 1e-5 * (1 + float(np.abs(gh0_ref).max(initial=0))),
                   what + " grad_h0")


# ------------------------------------------------------------------ golden fixtures ----------
@pytest.mark.parametrize("name", H.golden_names("plain_via_fold"))
def test_golden_through_fold(name):
    """Outputs of the unmodified reference: reference(a, x) == plain(a, (1-a)x), gradients by chain rule."""
    g = H.load_golden(name)
    storage = H.manifest()[name]["storage"]
    a, x, Gd = g["a"], g["x"], g["G"]
    h0 = g.get("h0")
    xp = H.round_storage(((np.float32(1) - a) * x).astype(np.float32), storage)
    ad, xd, gd = (G.dev(v, storage) for v in (a, xp, Gd))
    h0d = None if h0 is None else G.dev(h0)
    h = G.forward(ad, xd, h0d)
    ga, gx, gh0 = G.backward(ad, h, gd, h0d, None, want_gh0=True)
    torch.cuda.synchronize()
    sel = (lambda v: v[:, g["sample_idx"]]) if "sample_idx" in g else (lambda v: v)
    r, at = tol(storage, g["ref32_h"])
    H.assert_close(sel(G.host(h)), g["ref32_h"], r, at, name + " states")
    gxh, gah = G.host(gx), G.host(ga)
    d_tokens = (np.float32(1) - a) * gxh
    d_gates = gah - x * gxh
    r, at = tol(storage, g["ref32_d_tokens"])
    H.assert_close(sel(d_tokens), g["ref32_d_tokens"], r, at, name + " d_tokens")
    # d_gates = grad_a' - x*grad_x' cancels; its error scales with the two terms
    scale = float(np.abs(gah).max() + np.abs(x * gxh).max())
    if storage == "f32":
        r, at = H.FP32_RTOL, 2e-7 * scale + H.FP32_ATOL
    else:
        r, at = H.LOWP_RTOL, 1e-2 * scale
    H.assert_close(sel(d_gates), g["ref32_d_gates"], r, at, name + " d_gates")
    if "ref32_d_h0" in g:
        H.assert_close(G.host(gh0), g["ref32_d_h0"], 1e-5, 1e-6, name + " d_h0")


# ------------------------------------------------------------------ seeded inputs vs oracle --
@pytest.mark.parametrize("storage", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("T", list(range(1, 20)) + [31, 32, 33, 63, 64, 65, 127, 128, 129, 130,
                                                     255, 256, 257, 511, 512, 513, 1000, 1024, 2047,
                                                     2048, 2049, 3073, 4096])
def test_every_tail_residue(storage, T):
    a, x, Gd, h0 = H.make_inputs(5, T, 100 + T, "sigmoid01", storage, with_h0=True)
    cin = np.linspace(-1, 1, 5).astype(np.float32)
    check_fwd_bwd(a, x, Gd, storage, h0, cin, f"{storage} T={T}")


@pytest.mark.parametrize("storage,R,T,gates", [
    ("f32", 128, 1024, "sigmoid"),      # configuration 1, full
    ("f32", 64, 4096, "sigmoid"),       # configuration 2, rows subset
    ("bf16", 64, 8192, "long"),         # configuration 3, rows subset
    ("f32", 8, 32768, "sigmoid+3"),     # configuration 4, one chunk length
    ("f16", 3 * 16, 16385, "sigmoid01"),  # configuration 5, longest ragged length
    ("f16", 3 * 768, 31, "sigmoid01"),  # configuration 5, full row count, short rows
    ("f16", 3 * 768, 1, "sigmoid01"),
    ("bf16", 5, 8192, "uniform09"),     # the reference notebook's usage cell: a = 0.9 + 0.1 U
])
def test_benchmark_configurations(storage, R, T, gates):
    if gates == "uniform09":
        rng = np.random.Generator(np.random.PCG64(77))
        a = H.round_storage((0.9 + 0.1 * rng.random((R, T), dtype=np.float32)), storage)
        x = H.round_storage(rng.standard_normal((R, T), dtype=np.float32), storage)
        Gd = H.round_storage(rng.standard_normal((R, T), dtype=np.float32), storage)
    else:
        a, x, Gd = H.make_inputs(R, T, 2000 + T, gates, storage)
    check_fwd_bwd(a, x, Gd, storage, what=f"{storage} {R}x{T} {gates}", scaled=(gates == "sigmoid+3"))


@pytest.mark.parametrize("storage", ["f32", "f16"])
@pytest.mark.parametrize("offsets", [(1, 1, 1), (0, 1, 2), (3, 0, 5)])
def test_views_with_odd_element_offsets(storage, offsets):
    """Tensors whose base is not 16-byte aligned, with equal and with different phases."""
    R, T = 7, 1003
    a, x, Gd = H.make_inputs(R, T, 31, "sigmoid", storage)
    dt = G.TORCH_DT[storage]

    def shifted(arr, off):
        buf = torch.zeros(R * T + 16, device="cuda", dtype=dt)
        view = buf[off:off + R * T].view(R, T)
        view.copy_(G.dev(arr, storage))
        return view

    ad, xd, gd = shifted(a, offsets[0]), shifted(x, offsets[1]), shifted(Gd, offsets[2])
    hbuf = torch.zeros(R * T + 16, device="cuda", dtype=dt)
    hout = hbuf[offsets[2]:offsets[2] + R * T].view(R, T)
    h = G.forward(ad, xd, out=hout)
    ga, gx = G.backward(ad, h, gd)
    torch.cuda.synchronize()
    h_ref = oc.plain_forward(a, x)
    r, at = tol(storage, h_ref)
    H.assert_close(G.host(h), h_ref, r, at, "states")
    ga_ref, gx_ref, _ = oc.plain_backward(a, G.host(h), Gd)
    r, at = tol(storage, gx_ref)
    H.assert_close(G.host(gx), gx_ref, r, at, "grad_tokens")
    H.assert_close(G.host(ga), ga_ref, *tol(storage, ga_ref), "grad_gates")
    # nothing outside the view was written
    assert float(hbuf[:offsets[2]].abs().sum()) == 0.0 and float(hbuf[offsets[2] + R * T:].abs().sum()) == 0.0


@pytest.mark.parametrize("storage", ["f32", "bf16"])
@pytest.mark.parametrize("T", [1, 31, 1000, 3073])
def test_outputs_stay_inside_their_buffers(storage, T):
    """Guard bytes before and after every output survive (stand-in for a memory checker)."""
    R = 9
    a, x, Gd = H.make_inputs(R, T, 5, "sigmoid", storage)
    dt = G.TORCH_DT[storage]
    pad = 64
    bufs = [torch.full((R * T + 2 * pad,), 7.0, device="cuda", dtype=dt) for _ in range(3)]
    outs = [b[pad:pad + R * T].view(R, T) for b in bufs]
    ad, xd, gd = (G.dev(v, storage) for v in (a, x, Gd))
    G.forward(ad, xd, out=outs[0])
    G.backward(ad, outs[0], gd, outs=(outs[1], outs[2]))
    torch.cuda.synchronize()
    for b in bufs:
        assert bool((b[:pad] == 7.0).all()) and bool((b[pad + R * T:] == 7.0).all())
    H.assert_close(G.host(outs[0]), oc.plain_forward(a, x), *tol(storage, oc.plain_forward(a, x)), "states")


@pytest.mark.parametrize("storage", ["f32", "bf16"])
def test_reduce_and_split_along_time(storage):
    """Carries of chunks + combine + scan-with-carry reproduce the unsplit scan, both directions."""
    R, T, K = 33, 8 * 517, 8
    a, x, Gd = H.make_inputs(R, T, 9, "sigmoid+3", storage)
    ad, xd, gd = (G.dev(v, storage) for v in (a, x, Gd))
    L = T // K
    chunks = [slice(k * L, (k + 1) * L) for k in range(K)]
    # forward: reduce each chunk, combine, scan each chunk with its carry-in
    PS = [G.reduce(ad[:, c].contiguous(), xd[:, c].contiguous()) for c in chunks]
    P = torch.stack([p for p, _ in PS]); S = torch.stack([s for _, s in PS])
    P_ref, S_ref = zip(*[oc.plain_reduce(a[:, c], x[:, c]) for c in chunks])
    H.assert_close(G.host(P), np.stack(P_ref), 1e-4, 1e-30, "P")
    H.assert_close(G.host(S), np.stack(S_ref), 1e-4, 1e-5, "S")
    h_in, total = G.combine(P, S)
    h_parts = [G.forward(ad[:, c].contiguous(), xd[:, c].contiguous(), h_in[k].contiguous())
               for k, c in enumerate(chunks)]
    h = torch.cat(h_parts, dim=1)
    h_whole, h_last = G.forward(ad, xd, want_last=True)
    torch.cuda.synchronize()
    h_ref = oc.plain_forward(a, x)
    h_ref64 = oc.plain_forward(a.astype(np.float64), x.astype(np.float64), dtype=np.float64)
    close_to_reference(G.host(h), h_ref, h_ref64, storage, "split states", scaled=True)
    H.assert_close(G.host(total), G.host(h_last), 1e-4, 1e-5, "total carry")
    if storage == "f32":
        H.assert_close(G.host(h), G.host(h_whole), 1e-5, 2e-5, "split vs whole")
    # backward: reverse carries, combine in reverse, scan each chunk with carry_in and h0
    Srev = torch.stack([G.reduce_reverse(ad[:, c].contiguous(), gd[:, c].contiguous())[1] for c in chunks])
    c_in, gh0_total = G.combine(P, Srev, reverse=True)
    parts = [G.backward(ad[:, c].contiguous(), h_parts[k], gd[:, c].contiguous(), h_in[k].contiguous(),
                        c_in[k].contiguous()) for k, c in enumerate(chunks)]
    ga = torch.cat([p[0] for p in parts], dim=1); gx = torch.cat([p[1] for p in parts], dim=1)
    ga_w, gx_w, gh0_w = G.backward(ad, h_whole, gd, want_gh0=True)
    torch.cuda.synchronize()
    ga_ref, gx_ref, gh0_ref = oc.plain_backward(a, G.host(h), Gd)
    ga_ref64, gx_ref64, _ = oc.plain_backward(a.astype(np.float64), G.host(h).astype(np.float64),
                                              Gd.astype(np.float64), dtype=np.float64)
    close_to_reference(G.host(gx), gx_ref, gx_ref64, storage, "split grad_tokens", scaled=True)
    close_to_reference(G.host(ga), ga_ref, ga_ref64, storage, "split grad_gates", scaled=True)
    H.assert_close(G.host(gh0_total), gh0_ref, 1e-4, 1e-5, "split grad_h0")
    H.assert_close(G.host(gh0_w), gh0_ref, 1e-4, 1e-5, "whole grad_h0")


def test_gates_exactly_zero_and_one():
    """a = 0 resets the state, a = 1 accumulates: rows of pure resets / pure cumulative sums."""
    R, T = 4, 777
    rng = np.random.default_rng(0)
    x = rng.standard_normal((R, T)).astype(np.float32)
    Gd = rng.standard_normal((R, T)).astype(np.float32)
    a = np.ones((R, T), np.float32)
    a[1] = 0.0
    a[2, ::7] = 0.0
    a[3, 100:] = 0.0
    check_fwd_bwd(a, x, Gd, "f32", what="0/1 gates", scaled=True)  # a = 1 rows are 777-term sums
    h = G.host(G.forward(G.dev(a), G.dev(x)))
    np.testing.assert_allclose(h[0], np.cumsum(x[0].astype(np.float64)), rtol=1e-5, atol=1e-4)
    assert np.array_equal(h[1], x[1])


def test_zero_rows_and_zero_length_are_no_ops():
    e = torch.empty((0, 16), device="cuda")
    G.forward(e, e)
    e2 = torch.empty((3, 0), device="cuda")
    h0 = torch.arange(3, device="cuda", dtype=torch.float32)
    _, last = G.forward(e2, e2, h0, want_last=True)
    torch.cuda.synchronize()
    assert torch.equal(last, h0)


def test_full_size_configuration_3_properties():
    """(16,2048,8192) bf16: oracle on a row subset, plus linearity in the tokens on all rows."""
    R, T = 16 * 2048, 8192
    gen = torch.Generator(device="cuda").manual_seed(3)
    u = torch.rand(R, T, device="cuda", generator=gen)
    a = (1.0 - torch.pow(10.0, -4.0 + 3.0 * u)).to(torch.bfloat16)
    del u
    x = torch.randn(R, T, device="cuda", generator=gen).to(torch.bfloat16)
    Gd = torch.randn(R, T, device="cuda", generator=gen).to(torch.bfloat16)
    h = G.forward(a, x)
    ga, gx = G.backward(a, h, Gd)
    rows = torch.arange(0, R, 257, device="cuda")
    rows = torch.cat([rows, torch.tensor([R - 1], device="cuda")])
    an, xn, gn = (G.host(t[rows]) for t in (a, x, Gd))
    h_ref = oc.plain_forward(an, xn)
    H.assert_close(G.host(h[rows]), h_ref, *tol("bf16", h_ref), "c3 states")
    ga_ref, gx_ref, _ = oc.plain_backward(an, G.host(h[rows]), gn)
    H.assert_close(G.host(gx[rows]), gx_ref, *tol("bf16", gx_ref), "c3 grad_tokens")
    H.assert_close(G.host(ga[rows]), ga_ref, *tol("bf16", ga_ref), "c3 grad_gates")
    # size-independent property: scan(a, 2x) == 2 scan(a, x) exactly (power-of-two scaling)
    h2 = G.forward(a, (x.float() * 2).to(torch.bfloat16))
    assert torch.equal(h2.float(), h.float() * 2)
    # grad_tokens of the backward is the same operator run in reverse on G with shifted gates:
    # reversing time turns it into a forward scan
    a_shift = torch.cat([a[:, 1:], torch.ones(R, 1, device="cuda", dtype=a.dtype)], dim=1)
    gx_alt = G.forward(a_shift.flip(1).contiguous(), Gd.flip(1).contiguous()).flip(1)
    err = (gx_alt.float() - gx.float()).abs()
    bound = 2e-2 * gx.float().abs() + 1e-2 * gx.float().pow(2).mean().sqrt()
    assert bool((err <= bound).all())


def test_full_size_configuration_2_against_oracle():
    """(8,1024,4096) fp32 on all rows against the C oracle."""
    a, x, Gd = H.make_inputs(8 * 1024, 4096, 42, "sigmoid", "f32")
    check_fwd_bwd(a, x, Gd, "f32", what="c2 full")


@pytest.mark.parametrize("storage,pinned", [("bf16", True), ("f32", True), ("f16", False)])
def test_host_buffer_pipeline_equals_device_path(storage, pinned):
    """fms_plain_forward_backward_host (blocks of rows on three streams) is bit-identical to the
    device entry points, for pinned and for pageable host memory, with a ragged last block."""
    from fm_b200.host_pipeline import HostPipeline
    R, T = 203, 1000
    a, x, Gd = H.make_inputs(R, T, 8, "sigmoid", storage)
    dt = G.TORCH_DT[storage]
    mk = lambda v: (torch.from_numpy(v).to(dt).pin_memory() if pinned else torch.from_numpy(v).to(dt))
    ah, xh, gh = mk(a), mk(x), mk(Gd)
    outs = [torch.empty_like(ah).pin_memory() if pinned else torch.empty_like(ah) for _ in range(3)]
    pipe = HostPipeline(16, T, dt)   # 16-row blocks: 13 blocks, the last one ragged
    pipe.forward_backward(ah, xh, gh, *outs)
    pipe.forward_backward(ah, xh, gh, *outs)  # a second call reuses the staging area
    torch.cuda.synchronize()
    pipe.close()
    ad, xd, gd = ah.cuda(), xh.cuda(), gh.cuda()
    h = G.forward(ad, xd)
    ga, gx = G.backward(ad, h, gd)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], h.cpu()) and torch.equal(outs[1], ga.cpu()) and torch.equal(outs[2], gx.cpu())


def test_torch_op_autograd_and_errors():
    """The public op: autograd with initial_state, and the reference's error conventions."""
    from fm_b200 import fm_scan, fm_scan_forward
    a, x, Gd, h0 = H.make_inputs(6, 300, 12, "sigmoid", "f32", with_h0=True)
    ad, xd, h0d = (G.dev(v).requires_grad_(True) for v in (a.reshape(2, 3, 300), x.reshape(2, 3, 300),
                                                           h0.reshape(2, 3)))
    h = fm_scan(ad, xd, h0d)
    h.backward(G.dev(Gd.reshape(2, 3, 300)))
    torch.cuda.synchronize()
    h_ref = oc.plain_forward(a, x, h0)
    ga_ref, gx_ref, gh0_ref = oc.plain_backward(a, h_ref, Gd, h0)
    H.assert_close(G.host(h).reshape(6, 300), h_ref, 1e-5, 1e-6, "op states")
    H.assert_close(G.host(ad.grad).reshape(6, 300), ga_ref, 1e-5, 2e-6, "op grad_gates")
    H.assert_close(G.host(xd.grad).reshape(6, 300), gx_ref, 1e-5, 2e-6, "op grad_tokens")
    H.assert_close(G.host(h0d.grad).reshape(6), gh0_ref, 1e-5, 2e-6, "op grad_h0")
    with pytest.raises(RuntimeError):      # dtype mismatch, as TORCH_CHECK in the reference
        fm_scan_forward(ad.detach(), xd.detach().half(), None, torch.empty_like(ad))
    with pytest.raises(RuntimeError):      # unsupported dtype
        fm_scan_forward(ad.detach().double(), xd.detach().double(), None, torch.empty_like(ad).double())
    with pytest.raises(RuntimeError):      # CPU tensor
        fm_scan_forward(ad.detach().cpu(), xd.detach().cpu(), None, torch.empty_like(ad).cpu())
    with pytest.raises(AssertionError):    # non-contiguous input, as the reference's Python asserts
        fm_scan(ad.detach().transpose(0, 1), xd.detach().transpose(0, 1))


@pytest.mark.parametrize("storage,R,T", [("f32", 3, 200_000), ("bf16", 1, 1_000_003), ("f16", 16, 65_536),
                                         ("f32", 1, 8191)])
def test_split_inside_one_gpu_for_few_long_rows(storage, R, T):
    """Rows cut into segments (carries, fold, scan): same results as the oracle and as the
    unsplit entry points; the last shape is too short to split and must fall through."""
    a, x, Gd, h0 = H.make_inputs(R, T, 55, "sigmoid+3", storage, with_h0=True)
    cin = np.linspace(-0.5, 0.5, R).astype(np.float32)
    ad, xd, gd = (G.dev(v, storage) for v in (a, x, Gd))
    h0d, cind = G.dev(h0), G.dev(cin)
    nseg, nbytes = G.split_plan(R, T, ad.dtype)
    assert (nseg > 1) == (T >= 8192) and (nbytes > 0) == (nseg > 1)
    h, h_last = G.forward_split(ad, xd, h0d, want_last=True)
    ga, gx, gh0 = G.backward_split(ad, h, gd, h0d, cind, want_gh0=True)
    h_u, h_last_u = G.forward(ad, xd, h0d, want_last=True)
    ga_u, gx_u, gh0_u = G.backward(ad, h, gd, h0d, cind, want_gh0=True)
    torch.cuda.synchronize()
    f64 = np.float64
    h_ref = oc.plain_forward(a, x, h0)
    h_ref64 = oc.plain_forward(a.astype(f64), x.astype(f64), h0.astype(f64), dtype=f64)
    close_to_reference(G.host(h), h_ref, h_ref64, storage, "split states", scaled=True)
    hs = G.host(h)
    ga_ref, gx_ref, gh0_ref = oc.plain_backward(a, hs, Gd, h0, cin)
    ga_ref64, gx_ref64, gh0_ref64 = oc.plain_backward(a.astype(f64), hs.astype(f64), Gd.astype(f64),
                                                      h0.astype(f64), cin.astype(f64), dtype=f64)
    close_to_reference(G.host(gx), gx_ref, gx_ref64, storage, "split grad_tokens", scaled=True)
    close_to_reference(G.host(ga), ga_ref, ga_ref64, storage, "split grad_gates", scaled=True)
    H.assert_close(G.host(gh0), gh0_ref64, 1e-4, 1e-4, "split grad_h0")
    H.assert_close(G.host(h_last), h_ref64[:, -1], 1e-4, 1e-4, "split h_last")
    # against the unsplit kernels: same values up to the re-association of the carries
    r, at = (1e-5, 2e-5) if storage == "f32" else (H.LOWP_RTOL, H.lowp_atol(h_ref))
    H.assert_close(G.host(h), G.host(h_u), r, at, "split vs unsplit states")
    H.assert_close(G.host(gx), G.host(gx_u), r, at * 4, "split vs unsplit grad_tokens")
    H.assert_close(G.host(gh0), G.host(gh0_u), 1e-4, 1e-4, "split vs unsplit grad_h0")


@pytest.mark.parametrize("K", [1, 2, 4, 8])
@pytest.mark.parametrize("storage,T", [("f32", 5000), ("bf16", 8192), ("f16", 3073), ("bf16", 100)])
def test_warps_per_row_variants_agree(monkeypatch, K, storage, T):
    """K warps cooperating on a row (shared-memory carry exchange) against the oracle."""
    monkeypatch.setenv("FMS_TUNE_FWD_K", str(K))
    monkeypatch.setenv("FMS_TUNE_BWD_K", str(K))
    G.reload_tune()
    a, x, Gd, h0 = H.make_inputs(7, T, 400 + T, "sigmoid01", storage, with_h0=True)
    cin = np.linspace(-1, 1, 7).astype(np.float32)
    check_fwd_bwd(a, x, Gd, storage, h0, cin, f"K={K} {storage} T={T}")
    ad, xd = G.dev(a, storage), G.dev(x, storage)
    P, S = G.reduce(ad, xd)
    P_ref, S_ref = oc.plain_reduce(a.astype(np.float64), x.astype(np.float64), dtype=np.float64)
    H.assert_close(G.host(P), P_ref, 1e-4, 1e-30, "P")
    H.assert_close(G.host(S), S_ref, 1e-4, 1e-5, "S")


@pytest.mark.parametrize("U", [1, 2, 4])
def test_unroll_variants_agree(monkeypatch, U):
    monkeypatch.setenv("FMS_TUNE_FWD_U", str(U))
    monkeypatch.setenv("FMS_TUNE_BWD_U", str(U))
    G.reload_tune()
    a, x, Gd = H.make_inputs(9, 4096 + 512, 17, "sigmoid", "bf16")
    check_fwd_bwd(a, x, Gd, "bf16", what=f"U={U}")


@pytest.mark.parametrize("K", [1, 2, 8])
@pytest.mark.parametrize("storage,R,T,ctas", [("f32", 37, 1024, 2), ("bf16", 53, 2048 + 256, 3),
                                              ("f16", 19, 8, 1), ("f32", 4, 4096, 1)])
def test_persistent_walk_over_several_rows(monkeypatch, K, storage, R, T, ctas):
    """A grid smaller than the number of rows: every warp/CTA walks several rows, prefetching the
    next row while it finishes the current one; carries must reset at every row boundary."""
    monkeypatch.setenv("FMS_TUNE_MAX_CTAS", str(ctas))
    monkeypatch.setenv("FMS_TUNE_FWD_K", str(K))
    monkeypatch.setenv("FMS_TUNE_BWD_K", str(K))
    G.reload_tune()
    a, x, Gd, h0 = H.make_inputs(R, T, 600 + R, "sigmoid01", storage, with_h0=True)
    cin = np.linspace(-1, 1, R).astype(np.float32)
    check_fwd_bwd(a, x, Gd, storage, h0, cin, f"persistent K={K} {storage} {R}x{T}")
    ad, xd, gd = (G.dev(v, storage) for v in (a, x, Gd))
    P, S = G.reduce(ad, xd)
    P2, S2 = G.reduce_reverse(ad, gd)
    torch.cuda.synchronize()
    f64 = np.float64
    P_ref, S_ref = oc.plain_reduce(a.astype(f64), x.astype(f64), dtype=f64)
    H.assert_close(G.host(P), P_ref, 1e-4, 1e-30, "P")
    H.assert_close(G.host(S), S_ref, 1e-4, 1e-5, "S")
    _, _, Srev_ref = oc.plain_backward(a.astype(f64), np.zeros_like(a, dtype=f64), Gd.astype(f64), dtype=f64)
    H.assert_close(G.host(P2), P_ref, 1e-4, 1e-30, "P (reverse)")
    H.assert_close(G.host(S2), Srev_ref, 1e-4, 1e-5, "S_rev")


def test_randomised_shapes_and_launch_shapes(monkeypatch):
    """Seeded sweep over dtype, rows, length, alignment offset and every launch-shape knob
    (warps per row, tiles per step, persistent walk, grid cap) against the oracle in double."""
    import random
    rnd = random.Random(20261125)
    done = 0
    while done < 80:
        storage = rnd.choice(["f32", "f16", "bf16"])
        R = rnd.choice([1, 2, 3, 5, 17, 64, 257, 1000])
        T = rnd.choice([1, 2, 7, 8, 15, 16, 31, 33, 100, 255, 256, 512, 777, 1024, 2048, 3000, 4097, 8192, 20000])
        if R * T > 2_000_000:
            continue
        for name, choices in (("FMS_TUNE_FWD_K", [0, 1, 2, 4, 8]), ("FMS_TUNE_BWD_K", [0, 1, 2, 4, 8]),
                              ("FMS_TUNE_FWD_U", [0, 1, 2, 4]), ("FMS_TUNE_BWD_U", [0, 1, 2, 4]),
                              ("FMS_TUNE_PERSIST", [0, 1]), ("FMS_TUNE_MAX_CTAS", [0, 1, 3, 50])):
            v = rnd.choice(choices)
            if v:
                monkeypatch.setenv(name, str(v))
            else:
                monkeypatch.delenv(name, raising=False)
        G.reload_tune()
        gates = rnd.choice(["sigmoid", "sigmoid01", "sigmoid+3"])
        off = rnd.choice([0, 0, 1, 3])
        a, x, Gd, h0 = H.make_inputs(R, T, 9000 + done, gates, storage, with_h0=True)
        cin = np.linspace(-1, 1, R).astype(np.float32)
        dt = G.TORCH_DT[storage]

        def place(arr):
            buf = torch.zeros(R * T + 8, device="cuda", dtype=dt)
            view = buf[off:off + R * T].view(R, T)
            view.copy_(G.dev(arr, storage))
            return view

        ad, xd, gd = place(a), place(x), place(Gd)
        h, hl = G.forward(ad, xd, G.dev(h0), want_last=True)
        ga, gx, gh0 = G.backward(ad, h, gd, G.dev(h0), G.dev(cin), want_gh0=True)
        torch.cuda.synchronize()
        f64 = np.float64
        hs = G.host(h)
        h_ref = oc.plain_forward(a.astype(f64), x.astype(f64), h0.astype(f64), dtype=f64)
        ga_ref, gx_ref, gh0_ref = oc.plain_backward(a.astype(f64), hs.astype(f64), Gd.astype(f64), h0.astype(f64),
                                                    cin.astype(f64), dtype=f64)
        what = f"case {done}: {storage} {R}x{T} {gates} offset {off}"
        if storage == "f32":
            tol = lambda r: (H.FP32_RTOL, H.FP32_ATOL * max(1.0, float(np.abs(r).max(initial=0))))
        else:
            tol = lambda r: (H.LOWP_RTOL, H.lowp_atol(r) + 1e-3)
        H.assert_close(hs, h_ref, *tol(h_ref), what + " states")
        H.assert_close(G.host(gx), gx_ref, *tol(gx_ref), what + " grad_tokens")
        H.assert_close(G.host(ga), ga_ref, *tol(ga_ref), what + " grad_gates")
        H.assert_close(G.host(gh0), gh0_ref, 1e-3, 1e-3 * max(1.0, float(np.abs(gh0_ref).max())), what + " grad_h0")
        done += 1
