"""In-tree builds of the two native libraries.

* ``_oracle``: the C++17 CPU oracle (pybind11 module, g++).
* ``libskml_cuda.so``: the sm_100a kernels behind a plain C ABI (nvcc), loaded with ctypes.

Both are rebuilt only when a source file is newer than the library.
Run ``python -m sketchml_b200.build`` to build both.
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
CSRC = ROOT / "csrc"

ORACLE_SO = PKG / ("_oracle" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
CUDA_SO = PKG / "libskml_cuda.so"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, log_name):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"{log_name} build failed:\n{' '.join(map(str, cmd))}\n{proc.stdout}")
    return proc.stdout


def oracle_sources():
    return [CSRC / "cpu" / "bindings.cpp", CSRC / "cpu" / "oracle.h", CSRC / "common" / "skml_common.h"]


def cuda_sources():
    cu = sorted((CSRC / "cuda").glob("*.cu"))
    hdr = sorted((CSRC / "cuda").glob("*.cuh")) + sorted((CSRC / "cuda").glob("*.h"))
    return cu, hdr + [CSRC / "common" / "skml_common.h"]


def build_oracle(force: bool = False) -> Path:
    if not force and not _newer(ORACLE_SO, oracle_sources()):
        return ORACLE_SO
    import pybind11

    tmp = ORACLE_SO.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [
        os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
        f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
        str(CSRC / "cpu" / "bindings.cpp"), "-o", str(tmp),
    ]
    _run(cmd, "oracle")
    os.replace(tmp, ORACLE_SO)
    return ORACLE_SO


def nvcc_path() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    cu, deps = cuda_sources()
    if not cu:
        raise RuntimeError("no CUDA sources found under csrc/cuda")
    if not force and not _newer(CUDA_SO, list(cu) + list(deps)):
        return CUDA_SO
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libskml_cuda.so")
    tmp = CUDA_SO.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc, *NVCC_ARCH, "-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "--expt-relaxed-constexpr", "-Xptxas", "-v" if verbose else "-O3",
           f"-I{CSRC / 'common'}", f"-I{CSRC / 'cuda'}", *map(str, cu), "-o", str(tmp), "-lcudart"]
    out = _run(cmd, "cuda")
    os.replace(tmp, CUDA_SO)
    if verbose:
        print(out)
    return CUDA_SO


def build_all(force: bool = False, verbose: bool = False):
    return build_oracle(force), build_cuda(force, verbose)


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "-v" in sys.argv
    for p in build_all(force, verbose):
        print("built", p)
