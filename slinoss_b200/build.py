"""Ahead-of-time build of the sm_100a kernels into ``slinoss_b200/_C``.

``python -m slinoss_b200.build`` (or ``build()``) compiles every ``csrc/*.cu``
with nvcc for ``sm_100a`` and links one C-ABI shared library,
``_C/libslinoss_b200.so``, whose exports are declared in
``include/slinoss_b200.h``.  There is no JIT and no fallback: importing the ops
without this library raises.  ``build_selftest()`` builds ``csrc/selftest/*.cu`` into a
second, test-only library (``include/slinoss_b200_selftest.h``) that the product never loads.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT_DIR = PKG / "_C"
LIB = OUT_DIR / "libslinoss_b200.so"
SELFTEST_LIB = OUT_DIR / "libslinoss_b200_selftest.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _headers():
    inc = PKG.parent / "include"
    return (list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc")) + list(inc.glob("*.h")))


def _compile_and_link(sources, lib: Path, force: bool, verbose: bool) -> Path:
    OUT_DIR.mkdir(exist_ok=True)
    newest = max(f.stat().st_mtime for f in list(sources) + _headers())
    diag = os.environ.get("SLX_DIAG") == "1"
    marker = OUT_DIR / (lib.stem + ".flags")
    flags = "diag" if diag else "release"
    same_flags = marker.exists() and marker.read_text().strip() == flags
    if not force and same_flags and lib.exists() and lib.stat().st_mtime >= newest:
        return lib

    def compile_one(src: Path) -> Path:
        obj = OUT_DIR / (src.stem + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if diag:  # SLX_DIAG=1: phase-clock stamps in the tensor-core kernels (never the shipped build)
            cmd.insert(1, "-DSLX_DIAG")
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    tmp = OUT_DIR / f"{lib.stem}.{os.getpid()}.tmp.so"
    cmd = [_nvcc(), "-shared", "-o", str(tmp), *map(str, objs), "-gencode",
           "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    marker.write_text(flags + "\n")
    return lib


def build(force: bool = False, verbose: bool = False) -> Path:
    """The product library: every ``csrc/*.cu``."""
    return _compile_and_link(sorted(CSRC.glob("*.cu")), LIB, force, verbose)


def build_selftest(force: bool = False, verbose: bool = False) -> Path:
    """The test-only library: every ``csrc/selftest/*.cu``."""
    return _compile_and_link(sorted((CSRC / "selftest").glob("*.cu")), SELFTEST_LIB, force, verbose)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_selftest(force="--force" in sys.argv, verbose="-v" in sys.argv))
