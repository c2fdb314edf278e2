"""Helpers shared by the test modules."""

from __future__ import annotations

from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"


def golden(name: str) -> dict:
    with np.load(GOLDEN / name) as z:
        return {k: z[k] for k in z.files}


def rel_err(got, ref) -> float:
    """||got - ref||_2 / ||ref||_2 (the parity metric of every scan test)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref.ravel())
    num = np.linalg.norm((got - ref).ravel())
    return float(num / den) if den > 0 else float(num)
