"""Generate the golden fixtures in this folder from the UNMODIFIED reference.

Run where the reference checkout is available (it is not needed to run the tests):

    FM_REFERENCE=/path/to/lexionbear-fm python tests/golden/make_golden.py

    FM_REFERENCE=... python tests/golden/make_golden.py layer_     # only cases whose name starts so

It imports ``fm_scan_pytorch`` from the reference's ``fm/scan/fm_pytorch.py``
(pure torch, CPU), runs it -- forward and autograd backward with the loss
``(states * G).sum()`` -- on seeded inputs shaped like the benchmark configurations,
and stores inputs and outputs as ``.npz``.  The reference op has the form
(gates (B,M,L), tokens (B,D,L)) -> states (B,M,D,L) with the update weight
``1 - gates`` applied to the tokens; the plain recurrence h_t = a_t h_{t-1} + x_t on
R rows is pinned through the fold  M = D = 1, B = R:

    reference(a[R,1,T], x[R,1,T])  ==  plain(a, (1 - a) * x)          (forward)
    grad_x_ref = (1 - a) * grad_x'          grad_a_ref = grad_a' - x * grad_x'

where primes are the plain scan's gradients.  Inputs of 16-bit cases are rounded
once to bf16/fp16 and stored as float32, so every consumer sees the same bits.

The ``layer_*`` cases pin the layer around the scan.  The reference's module
``fm/scan/fm_scan.py`` cannot be imported without a GPU (it JIT-compiles its CUDA at
import, fm_scan.py:18-33), so the FUNCTION ``fm_memory`` (fm_scan.py:102-133) is taken out
of the file's syntax tree, compiled unchanged, and run with the name ``fm_scan`` bound to
the reference's CPU scan ``fm_scan_pytorch`` -- the reference's own layer arithmetic over
the reference's own scan, in fp32 and fp64, with all five input gradients.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REF = os.environ.get("FM_REFERENCE")
if not REF:
    raise SystemExit("set FM_REFERENCE to a checkout of lexionbear/fm")
sys.path.insert(0, REF)
from fm.scan.fm_pytorch import fm_scan_pytorch  # noqa: E402  (the reference itself)


def run_reference(gates, tokens, G, h0=None, dtype=torch.float32):
    g = gates.to(dtype).clone().requires_grad_(True)
    x = tokens.to(dtype).clone().requires_grad_(True)
    h0t = None
    if h0 is not None:
        h0t = h0.to(dtype).clone().contiguous().requires_grad_(True)
    h = fm_scan_pytorch(g, x, h0t)
    (h * G.to(dtype)).sum().backward()
    out = {"h": h.detach(), "d_gates": g.grad, "d_tokens": x.grad}
    if h0t is not None:
        out["d_h0"] = h0t.grad
    return out


def rnd(t, storage):
    if storage == "f32":
        return t
    return t.to({"bf16": torch.bfloat16, "f16": torch.float16}[storage]).to(torch.float32)


def folded_case(name, R, T, seed, gate_kind, storage="f32", with_h0=False, want64=True,
                sample=None):
    """PLAIN-shaped case run through the M = D = 1 fold of the reference."""
    gen = torch.Generator().manual_seed(seed)
    if gate_kind == "sigmoid":
        a = torch.sigmoid(torch.randn(R, T, generator=gen))
    elif gate_kind == "sigmoid+3":
        a = torch.sigmoid(torch.randn(R, T, generator=gen) + 3.0)
    elif gate_kind == "long":
        a = 1.0 - torch.pow(10.0, -4.0 + 3.0 * torch.rand(R, T, generator=gen))
    elif gate_kind == "uniform_half":  # the reference notebook's correctness cell
        a = 0.5 + 0.5 * torch.rand(R, T, generator=gen)
    elif gate_kind == "sigmoid01":  # 5 % exact zeros, 5 % exact ones
        a = torch.sigmoid(torch.randn(R, T, generator=gen))
    else:
        raise ValueError(gate_kind)
    if gate_kind == "uniform_half":
        x = torch.rand(R, T, generator=gen)
    else:
        x = torch.randn(R, T, generator=gen)
    G = torch.randn(R, T, generator=gen)
    if gate_kind == "sigmoid01":
        u = torch.rand(R, T, generator=gen)
        a = torch.where(u < 0.05, torch.zeros_like(a), a)
        a = torch.where(u > 0.95, torch.ones_like(a), a)
    h0 = torch.randn(R, generator=gen) if with_h0 else None
    a, x, G = rnd(a, storage), rnd(x, storage), rnd(G, storage)
    if h0 is not None:
        h0 = rnd(h0, storage)

    g3, x3, G4 = a.reshape(R, 1, T), x.reshape(R, 1, T), G.reshape(R, 1, 1, T)
    h03 = None if h0 is None else h0.reshape(R, 1, 1)
    ref32 = run_reference(g3, x3, G4, h03, torch.float32)
    arrays = {"a": a.numpy(), "x": x.numpy(), "G": G.numpy()}
    if h0 is not None:
        arrays["h0"] = h0.numpy()
    def flat(k, v):
        return v.reshape(R).numpy() if k == "d_h0" else v.reshape(R, T).numpy()

    outs = {"ref32_" + k: flat(k, v) for k, v in ref32.items()}
    if want64:
        ref64 = run_reference(g3, x3, G4, h03, torch.float64)
        outs.update({"ref64_" + k: flat(k, v) for k, v in ref64.items()})
    if sample is not None:  # keep only every `sample`-th position of the outputs
        idx = np.arange(0, T, sample)
        arrays["sample_idx"] = idx
        outs = {k: (v if v.ndim == 1 else v[:, idx]) for k, v in outs.items()}
    arrays.update(outs)
    meta = dict(name=name, mode="plain_via_fold", R=R, T=T, seed=seed, gates=gate_kind,
                storage=storage)
    return name, arrays, meta


def fm_case(name, B, M, D, L, seed, gate_kind="sigmoid", with_h0=False):
    gen = torch.Generator().manual_seed(seed)
    if gate_kind == "uniform_half":
        g = 0.5 + 0.5 * torch.rand(B, M, L, generator=gen)
        x = torch.rand(B, D, L, generator=gen)
    else:
        g = torch.sigmoid(torch.randn(B, M, L, generator=gen))
        x = torch.randn(B, D, L, generator=gen)
    G = torch.randn(B, M, D, L, generator=gen)
    h0 = torch.randn(B, M, D, generator=gen) if with_h0 else None
    arrays = {"g": g.numpy(), "x": x.numpy(), "G": G.numpy()}
    if h0 is not None:
        arrays["h0"] = h0.numpy()
    for tag, dt in (("ref32_", torch.float32), ("ref64_", torch.float64)):
        for k, v in run_reference(g, x, G, h0, dt).items():
            arrays[tag + k] = v.numpy()
    meta = dict(name=name, mode="fm", B=B, M=M, D=D, L=L, seed=seed, gates=gate_kind)
    return name, arrays, meta


def reference_fm_memory():
    """The reference's ``fm_memory`` compiled from its source file without importing the module."""
    import ast
    path = Path(REF) / "fm" / "scan" / "fm_scan.py"
    tree = ast.parse(path.read_text(), filename=str(path))
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "fm_memory"]
    assert len(fn) == 1, "fm_memory not found in the reference"
    module = ast.Module(body=fn, type_ignores=[])
    ns = {"torch": torch, "fm_scan": fm_scan_pytorch}
    exec(compile(module, str(path), "exec"), ns)
    return ns["fm_memory"]


def layer_case(name, B, L, M, D, seed, mem_norm, with_h0):
    """fm_memory(alpha (B,L,M), update_scale (B,L,1), output_scale (B,L,1), inputs (B,L,D), h0)
    with the loss (output * W).sum() + (memory_states * Gs).sum()."""
    fm_memory = reference_fm_memory()
    gen = torch.Generator().manual_seed(seed)
    alpha = torch.softmax(torch.randn(B, L, M, generator=gen), dim=-1)
    upd = torch.sigmoid(torch.randn(B, L, 1, generator=gen))
    outs = torch.sigmoid(torch.randn(B, L, 1, generator=gen))
    inp = torch.randn(B, L, D, generator=gen)
    W = torch.randn(B, L, D, generator=gen)
    Gs = 0.1 * torch.randn(B, M, D, L, generator=gen)
    h0 = torch.randn(B, M, D, generator=gen) if with_h0 else None
    arrays = {"alpha": alpha.numpy(), "update_scale": upd.numpy(), "output_scale": outs.numpy(),
              "inputs": inp.numpy(), "W": W.numpy(), "Gs": Gs.numpy()}
    if h0 is not None:
        arrays["h0"] = h0.numpy()
    for tag, dt in (("ref32_", torch.float32), ("ref64_", torch.float64)):
        args = [t.to(dt).clone().requires_grad_(True) for t in (alpha, upd, outs, inp)]
        h0t = None if h0 is None else h0.to(dt).clone().requires_grad_(True)
        out, states = fm_memory(*args, initial_state=h0t, mem_norm=mem_norm)
        ((out * W.to(dt)).sum() + (states * Gs.to(dt)).sum()).backward()
        arrays[tag + "out"] = out.detach().numpy()
        arrays[tag + "states"] = states.detach().numpy()
        for k, t in zip(("d_alpha", "d_update_scale", "d_output_scale", "d_inputs"), args):
            arrays[tag + k] = t.grad.numpy()
        if h0t is not None:
            arrays[tag + "d_h0"] = h0t.grad.numpy()
    meta = dict(name=name, mode="layer", B=B, L=L, M=M, D=D, seed=seed, mem_norm=bool(mem_norm))
    return name, arrays, meta


def main():
    only = sys.argv[1] if len(sys.argv) > 1 else ""
    cases = [
        # configuration 1 of the benchmark: fp32 (2,64,1024), full shape
        folded_case("c1_fp32_2x64x1024", 128, 1024, 1001, "sigmoid", want64=False),
        # configuration 2 distribution, 4 rows of T = 4096
        folded_case("c2_fp32_rows4_T4096", 4, 4096, 1002, "sigmoid"),
        # configuration 3: bf16 storage, long-memory gates, 4 rows of T = 8192
        folded_case("c3_bf16_rows4_T8192", 4, 8192, 1003, "long", storage="bf16"),
        # configuration 4 distribution: one split-along-T chunk length, 2 rows
        folded_case("c4_fp32_rows2_T32768", 2, 32768, 1004, "sigmoid+3", sample=8),
        # configuration 5: fp16 storage, ragged lengths, exact 0/1 gates
        folded_case("c5_fp16_rows12_T1", 12, 1, 1051, "sigmoid01", storage="f16"),
        folded_case("c5_fp16_rows12_T31", 12, 31, 1052, "sigmoid01", storage="f16"),
        folded_case("c5_fp16_rows12_T1000", 12, 1000, 1053, "sigmoid01", storage="f16"),
        folded_case("c5_fp16_rows6_T3073", 6, 3073, 1054, "sigmoid01", storage="f16"),
        folded_case("c5_fp16_rows2_T16385", 2, 16385, 1055, "sigmoid01", storage="f16", sample=4),
        # initial state carried in (and its gradient)
        folded_case("h0_fp32_rows16_T257", 16, 257, 1060, "sigmoid", with_h0=True),
        # the reference notebook's correctness-cell shape (batch,dim,seqlen,mem = 1,5,32,1)
        fm_case("nb_fm_1x1x5x32", 1, 1, 5, 32, 1070, "uniform_half"),
        # general FM mode with broadcast over M and D, with initial state
        fm_case("fm_2x3x5x64_h0", 2, 3, 5, 64, 1071, "sigmoid", with_h0=True),
        fm_case("fm_1x4x8x300", 1, 4, 8, 300, 1072, "sigmoid"),
    ] if not only else []
    # the layer around the scan (fm_memory), with and without the RMS norm / initial state
    layer_specs = [("layer_norm_h0_2x64x3x8", 2, 64, 3, 8, 1080, True, True),
                   ("layer_nonorm_1x128x4x8", 1, 128, 4, 8, 1081, False, False),
                   ("layer_norm_1x40x8x16", 1, 40, 8, 16, 1082, True, False)]
    cases += [layer_case(*spec) for spec in layer_specs if spec[0].startswith(only)]
    manifest_path = HERE / "manifest.json"
    manifest = json.loads(manifest_path.read_text())["cases"] if only and manifest_path.exists() else {}
    for name, arrays, meta in cases:
        path = HERE / f"{name}.npz"
        np.savez_compressed(path, **arrays)
        digest = hashlib.sha256()
        for k in sorted(arrays):
            digest.update(k.encode())
            digest.update(np.ascontiguousarray(arrays[k]).tobytes())
        meta["sha256"] = digest.hexdigest()
        meta["arrays"] = {k: [str(v.dtype), list(v.shape)] for k, v in arrays.items()}
        manifest[name] = meta
        print(name, {k: v.shape for k, v in arrays.items()}, f"{path.stat().st_size/1e3:.0f} kB")
    meta_all = {"torch": torch.__version__, "reference_function": "fm/scan/fm_pytorch.py:fm_scan_pytorch",
                "reference_layer": "fm/scan/fm_scan.py:fm_memory (from the syntax tree) over fm_scan_pytorch",
                "cases": manifest}
    (HERE / "manifest.json").write_text(json.dumps(meta_all, indent=1) + "\n")


if __name__ == "__main__":
    main()
