"""Compile the C oracle (``scan_oracle.c``) into ``oracle/_build/liboracle.so``.

TEST INFRASTRUCTURE ONLY: the resulting library is the checker, never the
product.  ``python -m oracle.build`` or ``oracle.build.build()``.
"""

from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "scan_oracle.c"
OUT_DIR = HERE / "_build"
OUT = OUT_DIR / "liboracle.so"


def build(force: bool = False) -> Path:
    OUT_DIR.mkdir(exist_ok=True)
    if not force and OUT.exists() and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    tmp = OUT_DIR / f"liboracle.{os.getpid()}.tmp.so"
    cmd = [
        "gcc", "-O2", "-std=c99", "-fcx-limited-range", "-fPIC", "-shared", "-fopenmp",
        "-o", str(tmp), str(SRC), "-lm",
    ]
    subprocess.run(cmd, check=True)
    os.replace(tmp, OUT)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
