"""FM mode -- the reference's literal operator (B,M,L) x (B,D,L) -> (B,M,D,L) -- on the GPU."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as oc
from tests import gpu_util as G
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", H.golden_names("fm"))
def test_fm_goldens_from_the_reference(name):
    g = H.load_golden(name)
    gd, xd, Gd = G.dev(g["g"]), G.dev(g["x"]), G.dev(g["G"])
    h0d = G.dev(g["h0"]) if "h0" in g else None
    h = G.fm_forward(gd, xd, h0d)
    dg, dx, dh0 = G.fm_backward(gd, xd, h, Gd, h0d, want_gh0=True)
    torch.cuda.synchronize()
    H.assert_close(G.host(h), g["ref32_h"], 1e-5, 1e-6, name + " states")
    H.assert_close(G.host(h), g["ref64_h"], 1e-5, 1e-6, name + " states vs double")
    scale_x = float(np.abs(g["ref64_d_tokens"]).max())
    scale_g = float(np.abs(g["ref64_d_gates"]).max())
    H.assert_close(G.host(dx), g["ref64_d_tokens"], 1e-5, 1e-6 * max(1, scale_x), name + " d_tokens")
    H.assert_close(G.host(dg), g["ref64_d_gates"], 1e-5, 1e-6 * max(1, scale_g), name + " d_gates")
    if "ref64_d_h0" in g:
        H.assert_close(G.host(dh0), g["ref64_d_h0"], 1e-5, 1e-6, name + " d_h0")


@pytest.mark.parametrize("storage,B,M,D,L", [
    ("f32", 2, 3, 5, 257), ("bf16", 1, 4, 16, 2048), ("f16", 2, 2, 7, 1000), ("f16", 1, 3, 4, 31),
    ("bf16", 1, 32, 64, 8192),   # the notebook's usage shape with D cut from 2048 to 64
    ("f32", 1, 1, 5, 32),        # the notebook's correctness cell
    ("bf16", 2, 9, 17, 520),     # M, D not multiples of the CTA block, ragged last tile
])
@pytest.mark.parametrize("blocked", [1, 0])
def test_fm_against_oracle(monkeypatch, blocked, storage, B, M, D, L):
    # blocked = 1: CTA-blocked reductions (aligned shapes); 0: one output row per CTA
    monkeypatch.setenv("FMS_TUNE_FM_BLOCKED", str(blocked))
    G.reload_tune()
    rng = np.random.Generator(np.random.PCG64(B * 1000 + M * 100 + D * 10 + L))
    g = H.round_storage((0.5 + 0.5 * rng.random((B, M, L), dtype=np.float32)), storage)
    x = H.round_storage(rng.standard_normal((B, D, L), dtype=np.float32), storage)
    Gr = H.round_storage(rng.standard_normal((B, M, D, L), dtype=np.float32), storage)
    h0 = H.round_storage(rng.standard_normal((B, M, D), dtype=np.float32), storage)
    gd, xd, Gd, h0d = G.dev(g, storage), G.dev(x, storage), G.dev(Gr, storage), G.dev(h0)
    h = G.fm_forward(gd, xd, h0d)
    dg, dx, dh0 = G.fm_backward(gd, xd, h, Gd, h0d, want_gh0=True)
    torch.cuda.synchronize()
    f64 = np.float64
    h_ref = oc.fm_forward(g.astype(f64), x.astype(f64), h0.astype(f64), dtype=f64)
    hs = G.host(h)
    dg_ref, dx_ref, dh0_ref = oc.fm_backward(g.astype(f64), x.astype(f64), hs.astype(f64), Gr.astype(f64),
                                             h0.astype(f64), dtype=f64)
    if storage == "f32":
        tol = lambda ref: (H.FP32_RTOL, H.FP32_ATOL * max(1.0, float(np.abs(ref).max())))
    else:
        tol = lambda ref: (H.LOWP_RTOL, H.lowp_atol(ref))
    H.assert_close(hs, h_ref, *tol(h_ref), "fm states")
    H.assert_close(G.host(dx), dx_ref, *tol(dx_ref), "fm d_tokens")
    H.assert_close(G.host(dg), dg_ref, *tol(dg_ref), "fm d_gates")
    H.assert_close(G.host(dh0), dh0_ref, 1e-4, 1e-4 * max(1.0, float(np.abs(dh0_ref).max())), "fm d_h0")


@pytest.mark.parametrize("rows_per_cta", [7, 8])
@pytest.mark.parametrize("storage,B,M,D,L", [("bf16", 2, 9, 17, 520), ("f32", 1, 5, 23, 1028)])
def test_fm_backward_rows_per_cta(monkeypatch, rows_per_cta, storage, B, M, D, L):
    """The blocked backward takes 7 or 8 token rows per CTA from the shape; both instantiations
    against the oracle on shapes with several tiles, a ragged last tile, M and D that are no
    multiples of the block, and an initial state (FMS_TUNE_FM_DC forces the choice)."""
    monkeypatch.setenv("FMS_TUNE_FM_DC", str(rows_per_cta))
    G.reload_tune()
    rng = np.random.Generator(np.random.PCG64(rows_per_cta * 7 + L))
    g = H.round_storage((0.5 + 0.5 * rng.random((B, M, L), dtype=np.float32)), storage)
    x = H.round_storage(rng.standard_normal((B, D, L), dtype=np.float32), storage)
    Gr = H.round_storage(rng.standard_normal((B, M, D, L), dtype=np.float32), storage)
    h0 = H.round_storage(rng.standard_normal((B, M, D), dtype=np.float32), storage)
    gd, xd, Gd, h0d = G.dev(g, storage), G.dev(x, storage), G.dev(Gr, storage), G.dev(h0)
    h = G.fm_forward(gd, xd, h0d)
    dg, dx, dh0 = G.fm_backward(gd, xd, h, Gd, h0d, want_gh0=True)
    torch.cuda.synchronize()
    f64 = np.float64
    hs = G.host(h)
    dg_ref, dx_ref, dh0_ref = oc.fm_backward(g.astype(f64), x.astype(f64), hs.astype(f64), Gr.astype(f64),
                                             h0.astype(f64), dtype=f64)
    if storage == "f32":
        tol = lambda ref: (H.FP32_RTOL, H.FP32_ATOL * max(1.0, float(np.abs(ref).max())))
    else:
        tol = lambda ref: (H.LOWP_RTOL, H.lowp_atol(ref))
    H.assert_close(G.host(dx), dx_ref, *tol(dx_ref), "fm d_tokens")
    H.assert_close(G.host(dg), dg_ref, *tol(dg_ref), "fm d_gates")
    H.assert_close(G.host(dh0), dh0_ref, 1e-4, 1e-4 * max(1.0, float(np.abs(dh0_ref).max())), "fm d_h0")


def test_fm_mode_through_the_torch_op():
    from fm_b200 import fm_scan
    g = H.load_golden("fm_2x3x5x64_h0")
    gd = G.dev(g["g"]).requires_grad_(True)
    xd = G.dev(g["x"]).requires_grad_(True)
    h0d = G.dev(g["h0"]).requires_grad_(True)
    h = fm_scan(gd, xd, h0d, mode="fm")
    assert h.shape == (2, 3, 5, 64)
    h.backward(G.dev(g["G"]))
    torch.cuda.synchronize()
    H.assert_close(G.host(h), g["ref32_h"], 1e-5, 1e-6, "op states")
    H.assert_close(G.host(gd.grad), g["ref32_d_gates"], 1e-5, 1e-5, "op d_gates")
    H.assert_close(G.host(xd.grad), g["ref32_d_tokens"], 1e-5, 1e-5, "op d_tokens")
    H.assert_close(G.host(h0d.grad), g["ref32_d_h0"], 1e-5, 1e-5, "op d_h0")
    with pytest.raises(ValueError):
        fm_scan(gd, xd, mode="outer")


def test_fm_equals_plain_on_broadcast_rows(monkeypatch):
    """FM(g, x) is the plain scan of (g, (1-g) x) on the B*M*D broadcast rows -- bit for bit
    (row-per-CTA forward; the blocked forward associates the tile scan differently and is
    covered by the oracle cases)."""
    monkeypatch.setenv("FMS_TUNE_FM_BLOCKED", "0")
    G.reload_tune()
    rng = np.random.Generator(np.random.PCG64(5))
    B, M, D, L = 2, 3, 4, 512
    g = rng.random((B, M, L), dtype=np.float32)
    x = rng.standard_normal((B, D, L), dtype=np.float32)
    gd, xd = G.dev(g), G.dev(x)
    h_fm = G.fm_forward(gd, xd)
    a_rows = gd[:, :, None, :].expand(B, M, D, L).contiguous()
    x_rows = ((1.0 - gd)[:, :, None, :] * xd[:, None, :, :]).contiguous()
    h_plain = G.forward(a_rows.view(-1, L), x_rows.view(-1, L)).view(B, M, D, L)
    torch.cuda.synchronize()
    assert torch.equal(h_fm, h_plain)


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("use_states", [False, True])
@pytest.mark.parametrize("mem_norm", [True, False])
def test_fm_memory_layer_matches_loop_restatement(mem_norm, use_states, fused):
    """The layer around the scan, forward and gradients, against the torch-loop restatement:
    the fused op (state gradient generated in-kernel) and the reference's composition; with and
    without a loss term on the returned states."""
    from fm_b200 import fm_memory
    from oracle.torch_loop import fm_memory_loop
    gen = torch.Generator().manual_seed(11)
    B, L, M, D = 2, 96, 3, 8
    alpha = torch.softmax(torch.randn(B, L, M, generator=gen), dim=-1)
    upd = torch.sigmoid(torch.randn(B, L, 1, generator=gen))
    outs = torch.sigmoid(torch.randn(B, L, 1, generator=gen))
    inp = torch.randn(B, L, D, generator=gen)
    h0 = torch.randn(B, M, D, generator=gen)
    W = torch.randn(B, L, D, generator=gen)

    Wm = torch.randn(B, M, D, L, generator=gen)

    def run(fn, dev, dtype):
        args = [t.to(dev, dtype).requires_grad_(True) for t in (alpha, upd, outs, inp, h0)]
        kw = {"fused": fused} if fn is fm_memory else {}
        out, mem = fn(args[0], args[1], args[2], args[3], args[4], mem_norm=mem_norm, **kw)
        loss = (out * W.to(dev, dtype)).sum()
        if use_states:
            loss = loss + (mem * Wm.to(dev, dtype)).sum()
        loss.backward()
        return [out.detach().cpu().double(), mem.detach().cpu().double()] + [a.grad.cpu().double() for a in args]

    got = run(fm_memory, "cuda", torch.float32)
    ref = run(fm_memory_loop, "cpu", torch.float64)
    names = ["output", "memory_states", "d_alpha", "d_update_scale", "d_output_scale", "d_inputs", "d_h0"]
    for n, a, b in zip(names, got, ref):
        scale = max(1.0, float(b.abs().max()))
        H.assert_close(a.numpy(), b.numpy(), 1e-4, 2e-5 * scale, n)


@pytest.mark.parametrize("mem_norm", [True, False])
@pytest.mark.parametrize("dtype,B,L,M,D", [(torch.float32, 2, 96, 3, 8), (torch.bfloat16, 1, 1024, 12, 37),
                                            (torch.float32, 1, 520, 9, 17)])
def test_fm_memory_readout_without_states(mem_norm, dtype, B, L, M, D):
    """need_states=False: the layer output from the two read-out kernels (states never written)
    against the torch-loop restatement of the layer in double precision."""
    from fm_b200 import fm_memory
    from oracle.torch_loop import fm_memory_loop
    gen = torch.Generator().manual_seed(21)
    alpha = torch.softmax(torch.randn(B, L, M, generator=gen), dim=-1)
    upd = torch.sigmoid(torch.randn(B, L, 1, generator=gen))
    outs = torch.sigmoid(torch.randn(B, L, 1, generator=gen))
    inp = torch.randn(B, L, D, generator=gen)
    h0 = torch.randn(B, M, D, generator=gen)
    args = [t.to(dtype) for t in (alpha, upd, outs, inp, h0)]
    with torch.no_grad():
        out, mem = fm_memory(*(a.cuda() for a in args), mem_norm=mem_norm, need_states=False)
        out_full, mem_full = fm_memory(*(a.cuda() for a in args), mem_norm=mem_norm)
    assert mem is None and mem_full is not None and out.shape == (B, L, D)
    ref, _ = fm_memory_loop(*(a.double() for a in args), mem_norm=mem_norm)
    scale = max(1.0, float(ref.abs().max()))
    if dtype == torch.float32:
        H.assert_close(out.cpu().double().numpy(), ref.numpy(), 1e-4, 2e-5 * scale, "fused read-out")
    else:
        H.assert_close(out.float().cpu().numpy(), ref.numpy(), 2e-2, 2e-2 * scale, "fused read-out bf16")
        H.assert_close(out_full.float().cpu().numpy(), ref.numpy(), 3e-2, 5e-2 * scale, "unfused bf16")
    # with a gradient requested the layer must keep the differentiable path
    a0 = args[0].cuda().requires_grad_(True)
    out2, mem2 = fm_memory(a0, *(a.cuda() for a in args[1:]), mem_norm=mem_norm, need_states=False)
    assert mem2 is not None and out2.requires_grad


@pytest.mark.parametrize("mem_norm", [True, False])
def test_fused_layer_bf16_against_double(mem_norm):
    """The fused op itself on bf16 tensors at a ragged shape (M, D not multiples of the CTA block,
    several tiles), against a double-precision evaluation of the same rounded inputs."""
    from fm_b200.fm_memory import _FusedLayer
    from oracle.torch_loop import fm_scan_loop
    gen = torch.Generator().manual_seed(31)
    B, L, M, D = 1, 776, 11, 19
    decay = (0.7 + 0.3 * torch.rand(B, M, L, generator=gen)).to(torch.bfloat16)
    tokens = torch.randn(B, D, L, generator=gen).to(torch.bfloat16)
    weight = torch.rand(B, M, L, generator=gen).to(torch.bfloat16)
    Wt = torch.randn(B, D, L, generator=gen)

    args = [t.cuda().requires_grad_(True) for t in (decay, tokens, weight)]
    out, states = _FusedLayer.apply(args[0], args[1], args[2], None, mem_norm, 1e-6)
    (out.double() * Wt.cuda().double()).sum().backward()
    got = [out.detach().double().cpu(), states.detach().double().cpu()] + [a.grad.double().cpu() for a in args]

    ref_args = [t.double().requires_grad_(True) for t in (decay, tokens, weight)]
    h = fm_scan_loop(ref_args[0], ref_args[1])
    if mem_norm:
        h = h * torch.rsqrt(torch.mean(h ** 2, dim=2, keepdim=True) + 1e-6)
    ref_out = torch.einsum('bml,bmdl->bdl', ref_args[2], h)
    (ref_out * Wt.double()).sum().backward()
    ref = [ref_out.detach(), h.detach()] + [a.grad for a in ref_args]
    for n, a, b in zip(["output", "states", "d_decay", "d_tokens", "d_weight"], got, ref):
        H.assert_close(a.numpy(), b.numpy(), 2e-2, 2e-2 * float(b.abs().pow(2).mean().sqrt()), n)


def test_fm_randomised_shapes(monkeypatch):
    """Seeded sweep over dtype, (B, M, D, L) with ragged blocks and tiles, exact 0/1 gates, with and
    without an initial state, blocked and row-per-CTA kernels, against the oracle in double."""
    import random
    rnd = random.Random(1125)
    done = 0
    while done < 40:
        storage = rnd.choice(["f32", "f16", "bf16"])
        B, M, D = rnd.choice([1, 2, 3]), rnd.choice([1, 2, 7, 8, 9, 16, 33]), rnd.choice([1, 3, 8, 15, 16, 40, 65])
        L = rnd.choice([8, 16, 24, 64, 128, 256, 264, 512, 1000, 1024, 2056])
        if B * M * D * L > 1_500_000:
            continue
        monkeypatch.setenv("FMS_TUNE_FM_BLOCKED", str(rnd.choice([0, 1])))
        G.reload_tune()
        rng = np.random.Generator(np.random.PCG64(7000 + done))
        g = 0.3 + 0.7 * rng.random((B, M, L), dtype=np.float32)
        if rnd.random() < 0.3:
            mask = rng.random((B, M, L))
            g = np.where(mask < 0.05, 0.0, np.where(mask > 0.95, 1.0, g)).astype(np.float32)
        g = H.round_storage(g, storage)
        x = H.round_storage(rng.standard_normal((B, D, L), dtype=np.float32), storage)
        Gr = H.round_storage(rng.standard_normal((B, M, D, L), dtype=np.float32), storage)
        h0 = H.round_storage(rng.standard_normal((B, M, D), dtype=np.float32), storage) if rnd.random() < 0.5 else None
        gd, xd, Gd = G.dev(g, storage), G.dev(x, storage), G.dev(Gr, storage)
        h0d = None if h0 is None else G.dev(h0)
        h = G.fm_forward(gd, xd, h0d)
        dg, dx, dh0 = G.fm_backward(gd, xd, h, Gd, h0d, want_gh0=True)
        torch.cuda.synchronize()
        f64 = np.float64
        h064 = None if h0 is None else h0.astype(f64)
        hs = G.host(h)
        h_ref = oc.fm_forward(g.astype(f64), x.astype(f64), h064, dtype=f64)
        dg_ref, dx_ref, dh0_ref = oc.fm_backward(g.astype(f64), x.astype(f64), hs.astype(f64), Gr.astype(f64), h064,
                                                 dtype=f64)
        if storage == "f32":
            tol = lambda r: (1e-5, 2e-6 * max(1.0, float(np.abs(r).max())))
        else:
            tol = lambda r: (H.LOWP_RTOL, H.lowp_atol(r) + 1e-3)
        what = f"case {done}: {storage} {(B, M, D, L)}"
        H.assert_close(hs, h_ref, *tol(h_ref), what + " states")
        H.assert_close(G.host(dx), dx_ref, *tol(dx_ref), what + " d_tokens")
        H.assert_close(G.host(dg), dg_ref, *tol(dg_ref), what + " d_gates")
        H.assert_close(G.host(dh0), dh0_ref, 1e-3, 1e-3 * max(1.0, float(np.abs(dh0_ref).max())), what + " d_h0")
        done += 1


@pytest.mark.parametrize("path", ["fused", "composed", "readout"])
@pytest.mark.parametrize("name", H.golden_names("layer"))
def test_layer_against_reference_goldens(name, path):
    """The layer on the GPU against outputs of the reference's own ``fm_memory`` (see
    tests/golden/make_golden.py): the fused training op, the reference's composition over the
    FM-mode scan, and the read-out that never writes the states.  Compared with the reference's
    double-precision run; fp32 tolerance scaled by each tensor's largest magnitude."""
    from fm_b200 import fm_memory
    g = H.load_golden(name)
    mem_norm = H.manifest()[name]["mem_norm"]
    dev = "cuda"
    args = [torch.from_numpy(g[k]).to(dev).requires_grad_(path != "readout")
            for k in ("alpha", "update_scale", "output_scale", "inputs")]
    h0 = torch.from_numpy(g["h0"]).to(dev).requires_grad_(path != "readout") if "h0" in g else None

    def close(got, key, rtol=1e-4, atol=2e-5):
        ref = g["ref64_" + key]
        H.assert_close(got.detach().double().cpu().numpy(), ref, rtol, atol * max(1.0, float(np.abs(ref).max())),
                       f"{name} {path} {key}")

    if path == "readout":
        with torch.no_grad():
            out, states = fm_memory(*args, initial_state=h0, mem_norm=mem_norm, need_states=False)
        assert states is None
        close(out, "out")
        return
    out, states = fm_memory(*args, initial_state=h0, mem_norm=mem_norm, fused=(path == "fused"))
    ((out * torch.from_numpy(g["W"]).to(dev)).sum() + (states * torch.from_numpy(g["Gs"]).to(dev)).sum()).backward()
    close(out, "out")
    close(states, "states")
    for k, t in zip(("d_alpha", "d_update_scale", "d_output_scale", "d_inputs"), args):
        close(t.grad, k)
    if h0 is not None:
        close(h0.grad, "d_h0")
