"""Ahead-of-time build of the sm_100a kernels into ``slinoss_b200/_C``.

``python -m slinoss_b200.build`` (or ``build()``) compiles every ``csrc/*.cu``
with nvcc for ``sm_100a`` and links one C-ABI shared library,
``_C/libslinoss_b200.so``, whose exports are declared in
``include/slinoss_b200.h``.  There is no JIT and no fallback: importing the ops
without this library raises.
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

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _newest_source_mtime() -> float:
    files = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc")) + [PKG.parent / "include" / "slinoss_b200.h"]
    return max(f.stat().st_mtime for f in files)


def build(force: bool = False, verbose: bool = False) -> Path:
    OUT_DIR.mkdir(exist_ok=True)
    if not force and LIB.exists() and LIB.stat().st_mtime >= _newest_source_mtime():
        return LIB
    sources = sorted(CSRC.glob("*.cu"))
    objs = []

    def compile_one(src: Path) -> Path:
        obj = OUT_DIR / (src.stem + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
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
    tmp = OUT_DIR / f"libslinoss_b200.{os.getpid()}.tmp.so"
    cmd = [_nvcc(), "-shared", "-o", str(tmp), *map(str, objs), "-gencode",
           "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
