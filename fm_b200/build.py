"""Ahead-of-time, in-tree build of the native pieces (sm_100a only).

The reference JIT-compiles its kernel at import with ``load_inline`` and no architecture flag
(fm/scan/fm_scan.py:18-33).  Here everything is compiled ahead of time into the package folder:

* ``fm_b200/lib/libfm_scan_b200.so`` -- CUDA kernels + the C ABI of ``include/fm_scan_b200.h``
  (nvcc, ``-gencode arch=compute_100a,code=sm_100a``); no torch dependency.
* ``fm_b200/_fm_scan_ext.so`` -- the thin torch C++ extension exporting ``fm_scan_forward`` /
  ``fm_scan_backward`` (g++), linked against the library above.

``python -m fm_b200.build`` builds both; ``ensure_built()`` rebuilds whatever is older than its
sources.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
LIB_DIR = PKG / "lib"
CAPI_LIB = LIB_DIR / "libfm_scan_b200.so"
EXT_LIB = PKG / "_fm_scan_ext.so"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _cuda_home() -> Path:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").exists():
            return Path(cand)
    nvcc = shutil.which("nvcc")
    if nvcc:
        return Path(nvcc).resolve().parent.parent
    raise RuntimeError("nvcc not found: set CUDA_HOME")


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed ({res.returncode}):\n{' '.join(map(str, cmd))}\n"
                           f"{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout, res.stderr, sep="\n", flush=True)
    return res


def capi_sources():
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))


def build_capi(force: bool = False, verbose: bool = False) -> Path:
    """nvcc -> libfm_scan_b200.so (kernels + C ABI)."""
    srcs = capi_sources()
    if not force and _newer(CAPI_LIB, srcs):
        return CAPI_LIB
    LIB_DIR.mkdir(exist_ok=True)
    nvcc = _cuda_home() / "bin" / "nvcc"
    cmd = [nvcc, *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "--threads", "0", "-Xptxas", "-v",
           "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared", f"-I{INCLUDE}", f"-I{CSRC}",
           "-o", CAPI_LIB, *sorted(CSRC.glob("*.cu"))]
    res = _run(cmd, verbose)
    (LIB_DIR / "ptxas.log").write_text(res.stderr)  # registers / spills of every kernel
    return CAPI_LIB


def build_ext(force: bool = False, verbose: bool = False) -> Path:
    """g++ -> _fm_scan_ext.so, the torch extension that forwards to the C ABI."""
    src = CSRC / "torch_ext.cpp"
    if not force and _newer(EXT_LIB, [src, CAPI_LIB, *INCLUDE.glob("*.h")]):
        return EXT_LIB
    import torch
    from torch.utils import cpp_extension as ce

    cuda = _cuda_home()
    incs = [f"-I{p}" for p in ce.include_paths()] + [f"-I{cuda / 'include'}", f"-I{INCLUDE}",
                                                     f"-I{sysconfig.get_paths()['include']}"]
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_fm_scan_ext",
           "-DTORCH_API_INCLUDE_EXTENSION_H", *incs, src, "-o", EXT_LIB,
           f"-L{LIB_DIR}", "-lfm_scan_b200", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu",
           "-ltorch_python", "-lc10", "-lc10_cuda", f"-L{cuda / 'lib64'}", "-lcudart",
           "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, verbose)
    return EXT_LIB


def ensure_built(verbose: bool = False) -> None:
    build_capi(verbose=verbose)
    build_ext(verbose=verbose)


def build_all(force: bool = True, verbose: bool = True) -> None:
    build_capi(force=force, verbose=verbose)
    build_ext(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv or True, verbose=True)
