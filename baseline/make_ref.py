"""Put the UNMODIFIED reference under ``baseline/_ref/`` so that it can run beside this library.

    python baseline/make_ref.py [/path/to/lexionbear-fm] [--prebuild]

The reference (lexionbear/fm, MIT) is not an installable package -- it has no ``setup.py`` or
``pyproject.toml`` -- so "installing" it means placing its ``fm/`` tree (5 files) and LICENSE in
``baseline/_ref/``, which is git-ignored: the files never enter this repository's history.
Its module ``fm/scan/fm_scan.py`` JIT-compiles its CUDA kernel at import with
``torch.utils.cpp_extension.load_inline`` (fm/scan/fm_scan.py:18-33); with ``--prebuild`` that
import is done here, without a GPU, for compute capability 10.0 and with
``TORCH_EXTENSIONS_DIR=baseline/_ref/torch_extensions`` so the built extension sits beside the
sources and a later import on a B200 box finds it instead of compiling for minutes.

Users of ``baseline/_ref``: ``bench.py`` (``reference_cuda`` figures: the reference's own CUDA op
timed on the same GPU, a stated comparison, never the target) and
``tests/test_gpu_reference_dropin.py`` (the reference's ``FM_Scan`` class run over this library's
extension).  Both skip or report ``unavailable`` when the folder is absent.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
EXT_DIR = DEST / "torch_extensions"


def reference_env() -> dict:
    """Environment under which the reference module must be imported to find the prebuilt op."""
    return {"TORCH_EXTENSIONS_DIR": str(EXT_DIR), "TORCH_CUDA_ARCH_LIST": "10.0"}


def install(src: Path) -> None:
    src = Path(src)
    if not (src / "fm" / "scan" / "fm_scan.cuh").exists():
        raise SystemExit(f"{src} does not look like a checkout of lexionbear/fm")
    (DEST / "fm" / "scan").mkdir(parents=True, exist_ok=True)
    for f in sorted((src / "fm" / "scan").iterdir()):
        if f.is_file():
            shutil.copy2(f, DEST / "fm" / "scan" / f.name)
    if (src / "LICENSE").exists():
        shutil.copy2(src / "LICENSE", DEST / "LICENSE")


def prebuild() -> None:
    """Import the reference module once so that load_inline compiles its extension in-tree."""
    os.environ.update(reference_env())
    EXT_DIR.mkdir(parents=True, exist_ok=True)
    sys.path.insert(0, str(DEST))
    import fm.scan.fm_scan  # noqa: F401  (compiles and loads the reference's extension)


def find_reference():
    """A checkout of the reference: ``$FM_REFERENCE``, else a folder ``reference`` beside this repository."""
    for cand in (os.environ.get("FM_REFERENCE"), HERE.parent.parent / "reference"):
        if cand and (Path(cand) / "fm" / "scan" / "fm_scan.cuh").exists():
            return Path(cand)
    return None


def ensure(prebuilt: bool = True) -> bool:
    """Place the reference if a checkout can be found and, unless it is there already, build its
    extension.  Returns False when no checkout is available (nothing is done then)."""
    src = find_reference()
    if src is None:
        return False
    install(src)
    if prebuilt and not (EXT_DIR / "fm_scan" / "fm_scan.so").exists():
        import subprocess
        subprocess.run([sys.executable, str(Path(__file__).resolve()), str(src), "--prebuild"], check=True,
                       env=dict(os.environ, **reference_env()), stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return True


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    src = Path(args[0]) if args else find_reference()
    if src is None:
        raise SystemExit("no checkout of lexionbear/fm found: pass its path or set FM_REFERENCE")
    install(src)
    if "--prebuild" in sys.argv:
        prebuild()
    print("reference placed in", DEST)
