"""The reference's own ``FM_Scan`` autograd class, unmodified, running over this library's extension.

``fm/scan/fm_scan.py`` of the reference cannot be imported as a module for this purpose (its
import compiles and binds the reference's own kernel, fm_scan.py:18-35), so the class
``FM_Scan`` (fm_scan.py:37-81) is taken out of the file's syntax tree and executed with the names
``fm_scan_forward`` / ``fm_scan_backward`` bound to ``fm_b200._fm_scan_ext`` -- exactly the swap a
maintainer of the reference would make.  Its backward passes two (B, M, D, L) gradient buffers and
sums them itself (fm_scan.py:70-78), so this exercises the unreduced output contract.

The reference file is read from ``baseline/_ref`` (see baseline/make_ref.py), which is not part
of the repository; the tests skip when it is absent.
"""
import ast
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

REF_FILE = Path(__file__).resolve().parent.parent / "baseline" / "_ref" / "fm" / "scan" / "fm_scan.py"


def _reference_class():
    from fm_b200.fm_scan import _load_ext
    ext = _load_ext()
    tree = ast.parse(REF_FILE.read_text(), filename=str(REF_FILE))
    cls = [n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == "FM_Scan"]
    assert len(cls) == 1
    ns = {"torch": torch, "fm_scan_forward": ext.fm_scan_forward, "fm_scan_backward": ext.fm_scan_backward}
    exec(compile(ast.Module(body=cls, type_ignores=[]), str(REF_FILE), "exec"), ns)
    return ns["FM_Scan"]


@pytest.mark.skipif(not REF_FILE.exists(), reason="baseline/_ref is absent (python baseline/make_ref.py)")
@pytest.mark.parametrize("name", ["nb_fm_1x1x5x32", "fm_1x4x8x300", "fm_2x3x5x64_h0"])
def test_reference_autograd_class_over_this_extension(name):
    FM_Scan = _reference_class()
    g = H.load_golden(name)
    gates = torch.from_numpy(g["g"]).cuda().requires_grad_(True)
    tokens = torch.from_numpy(g["x"]).cuda().requires_grad_(True)
    if "h0" in g:
        # the reference's backward ignores the forward initial state (it passes zeros as h_{-1},
        # fm_scan.py:65,73): only the forward can be compared for this fixture
        h = FM_Scan.apply(gates, tokens, torch.from_numpy(g["h0"]).cuda())
        H.assert_close(h.detach().cpu().numpy(), g["ref64_h"], 1e-5, 2e-6, name + " states")
        return
    h = FM_Scan.apply(gates, tokens)
    (h * torch.from_numpy(g["G"]).cuda()).sum().backward()
    torch.cuda.synchronize()
    H.assert_close(h.detach().cpu().numpy(), g["ref64_h"], 1e-5, 2e-6, name + " states")
    for got, key in ((gates.grad, "d_gates"), (tokens.grad, "d_tokens")):
        ref = g["ref64_" + key]
        H.assert_close(got.cpu().numpy(), ref, 1e-5, 2e-6 * max(1.0, float(np.abs(ref).max())), f"{name} {key}")


@pytest.mark.skipif(not REF_FILE.exists(), reason="baseline/_ref is absent (python baseline/make_ref.py)")
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_reference_class_16bit_matches_fused_backward(dtype):
    """Same class on 16-bit tensors at a shape with several tiles per row: the per-row terms it
    sums must agree with this library's fused reductions (fp32 sums, rounded once)."""
    from fm_b200 import fm_scan
    FM_Scan = _reference_class()
    gen = torch.Generator().manual_seed(5)
    B, M, D, L = 2, 3, 9, 2048
    gates = torch.sigmoid(torch.randn(B, M, L, generator=gen) + 2).to(dtype).cuda()
    tokens = torch.randn(B, D, L, generator=gen).to(dtype).cuda()
    G = torch.randn(B, M, D, L, generator=gen).to(dtype).cuda()
    a1, x1 = gates.clone().requires_grad_(True), tokens.clone().requires_grad_(True)
    h1 = FM_Scan.apply(a1, x1)
    (h1.float() * G.float()).sum().backward()
    a2, x2 = gates.clone().requires_grad_(True), tokens.clone().requires_grad_(True)
    h2 = fm_scan(a2, x2, mode="fm")
    (h2.float() * G.float()).sum().backward()
    assert torch.equal(h1, h2)
    for got, ref, what in ((a1.grad, a2.grad, "d_gates"), (x1.grad, x2.grad, "d_tokens")):
        ref = ref.float().cpu().numpy()
        # the class sums 16-bit per-row terms in 16-bit precision; the fused path sums in fp32
        H.assert_close(got.float().cpu().numpy(), ref, 5e-2, 5e-2 * float(np.sqrt(np.mean(ref ** 2))), what)
