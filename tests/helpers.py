"""Shared test helpers: golden fixtures, seeded inputs of the benchmark configurations, tolerances."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"

# Tolerances of the comparison with the reference scan.
# fp32 storage: the stated bar.  16-bit storage with fp32 accumulation: rtol 2e-2 as stated;
# the absolute term is 1e-2 of the tensor's RMS because gradients cross zero.
FP32_RTOL, FP32_ATOL = 1e-5, 1e-6
LOWP_RTOL = 2e-2


def lowp_atol(ref: np.ndarray) -> float:
    return 1e-2 * float(np.sqrt(np.mean(np.square(ref.astype(np.float64)))) + 1e-30)


def manifest() -> dict:
    return json.loads((GOLDEN / "manifest.json").read_text())["cases"]


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz") as z:
        return {k: z[k] for k in z.files}


def golden_names(mode: str):
    return [k for k, v in manifest().items() if v["mode"] == mode]


def round_storage(arr: np.ndarray, storage: str) -> np.ndarray:
    """Round an fp32 array once to the storage type and return it as fp32 again."""
    import torch
    if storage in ("f32", "fp32"):
        return np.ascontiguousarray(arr, dtype=np.float32)
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "fp16": torch.float16}[storage]
    return torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)).to(dt).to(torch.float32).numpy()


def make_inputs(R: int, T: int, seed: int, gates: str = "sigmoid", storage: str = "f32",
                with_h0: bool = False):
    """Seeded (a, x, G[, h0]) as fp32 arrays already rounded to `storage`.

    Distributions are those of the benchmark configurations: `sigmoid` a = sigmoid(N(0,1));
    `sigmoid+3` a = sigmoid(N(0,1)+3); `long` a = 1 - 10^U(-4,-1); `sigmoid01` sigmoid with 5 %
    of the entries exactly 0 and 5 % exactly 1.  x, G ~ N(0,1).
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    z = rng.standard_normal((R, T), dtype=np.float32)
    if gates == "sigmoid":
        a = 1.0 / (1.0 + np.exp(-z))
    elif gates == "sigmoid+3":
        a = 1.0 / (1.0 + np.exp(-(z + 3.0)))
    elif gates == "long":
        u = rng.random((R, T), dtype=np.float32)
        a = 1.0 - np.power(10.0, -4.0 + 3.0 * u)
    elif gates == "sigmoid01":
        a = 1.0 / (1.0 + np.exp(-z))
        u = rng.random((R, T), dtype=np.float32)
        a = np.where(u < 0.05, 0.0, a)
        a = np.where(u > 0.95, 1.0, a)
    else:
        raise ValueError(gates)
    x = rng.standard_normal((R, T), dtype=np.float32)
    G = rng.standard_normal((R, T), dtype=np.float32)
    out = [round_storage(a.astype(np.float32), storage), round_storage(x, storage),
           round_storage(G, storage)]
    if with_h0:
        out.append(round_storage(rng.standard_normal((R,), dtype=np.float32), storage))
    return tuple(out)


def assert_close(got, ref, rtol, atol, what=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    err = np.abs(got - ref)
    bound = atol + rtol * np.abs(ref)
    bad = err > bound
    if bad.any() or not np.isfinite(got).all():
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.size} out of tolerance (rtol={rtol}, atol={atol}); "
            f"worst at {i}: got {got[i]!r} ref {ref[i]!r} err {err[i]:.3e} bound {bound[i]:.3e}")
