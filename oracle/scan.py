"""ctypes front end of the C scan oracle -- TEST INFRASTRUCTURE ONLY.

Every function takes/returns numpy float64 arrays in the reference's canonical
layouts with the leading ``(batch, heads)`` axes kept (they are flattened to
``BH`` for the C side).  See ``scan_oracle.c`` for the reference citations.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np

from . import build as _build

_LIB: Optional[ctypes.CDLL] = None
_dp = ctypes.POINTER(ctypes.c_double)


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(str(_build.build()))
        _LIB.slx_oracle_chunk_scan.restype = ctypes.c_int
        _LIB.slx_oracle_v2x2ssd_fwd.restype = ctypes.c_int
    return _LIB


def _c(x: Optional[np.ndarray]):
    if x is None:
        return None
    assert x.dtype == np.float64 and x.flags["C_CONTIGUOUS"]
    return x.ctypes.data_as(_dp)


def _f64(x) -> Optional[np.ndarray]:
    if x is None:
        return None
    return np.ascontiguousarray(np.asarray(x, dtype=np.float64))


def _dims(U: np.ndarray, B: np.ndarray):
    b, h, T, P = U.shape
    D = B.shape[-1]
    return b, h, T, P, D // 2


def v2x2ssm_fwd(U, M, K, B, C, *, initial_states=None, B_prev=None, U_prev=None):
    """Sequential oracle (reference.py:704). Returns (Y, final_state)."""
    U, M, K, B, C = map(_f64, (U, M, K, B, C))
    init, bp, up = map(_f64, (initial_states, B_prev, U_prev))
    b, h, T, P, N = _dims(U, B)
    Y = np.zeros((b, h, T, P))
    fin = np.zeros((b, h, P, 2 * N))
    lib().slx_oracle_v2x2ssm_fwd(b * h, T, P, N, _c(U), _c(M), _c(K), _c(B), _c(C),
                                 _c(init), _c(bp), _c(up), _c(Y), _c(fin))
    return Y, fin


def v2x2ssm_bwd(U, M, K, B, C, *, dY, d_final=None, initial_states=None,
                B_prev=None, U_prev=None):
    """Gradients of the scan (what autograd gives through reference.py:1195).

    Returns dict with dU,dM,dK,dB,dC,d_initial,dB_prev,dU_prev."""
    U, M, K, B, C = map(_f64, (U, M, K, B, C))
    init, bp, up = map(_f64, (initial_states, B_prev, U_prev))
    dY, d_final = _f64(dY), _f64(d_final)
    b, h, T, P, N = _dims(U, B)
    D = 2 * N
    out = dict(
        dU=np.zeros_like(U), dM=np.zeros_like(M), dK=np.zeros_like(K),
        dB=np.zeros_like(B), dC=np.zeros_like(C),
        d_initial=np.zeros((b, h, P, D)), dB_prev=np.zeros((b, h, D)),
        dU_prev=np.zeros((b, h, P)),
    )
    lib().slx_oracle_v2x2ssm_bwd(
        b * h, T, P, N, _c(U), _c(M), _c(K), _c(B), _c(C), _c(init), _c(bp), _c(up),
        _c(dY), _c(d_final), _c(out["dU"]), _c(out["dM"]), _c(out["dK"]),
        _c(out["dB"]), _c(out["dC"]), _c(out["d_initial"]), _c(out["dB_prev"]),
        _c(out["dU_prev"]))
    return out


def chunk_increment(U, M, K, B, *, B_prev=None, U_prev=None, chunk_size: int):
    """Stage 1 (reference.py:937). Returns (inc, m_chunk)."""
    U, M, K, B = map(_f64, (U, M, K, B))
    bp, up = _f64(B_prev), _f64(U_prev)
    b, h, T, P, N = _dims(U, B)
    NC = (T + chunk_size - 1) // chunk_size
    inc = np.zeros((b, h, NC, P, 2 * N))
    mch = np.zeros((b, h, NC, 2))
    lib().slx_oracle_chunk_increment(b * h, T, P, N, chunk_size, _c(U), _c(M), _c(K),
                                     _c(B), _c(bp), _c(up), _c(inc), _c(mch))
    return inc, mch


def state_passing(inc, m_chunk, *, initial_states=None):
    """Stage 2 (reference.py:1015). Returns (chunk_starts, final_state)."""
    inc, m_chunk, init = _f64(inc), _f64(m_chunk), _f64(initial_states)
    b, h, NC, P, D = inc.shape
    starts = np.zeros_like(inc)
    fin = np.zeros((b, h, P, D))
    lib().slx_oracle_state_passing(b * h, NC, P, D // 2, _c(inc), _c(m_chunk),
                                   _c(init), _c(starts), _c(fin))
    return starts, fin


def chunk_scan(U, M, K, B, C, chunk_starts, *, B_prev=None, U_prev=None,
               chunk_size: int):
    """Stage 3 (reference.py:1059). Raises ValueError on exact-zero M."""
    U, M, K, B, C, chunk_starts = map(_f64, (U, M, K, B, C, chunk_starts))
    bp, up = _f64(B_prev), _f64(U_prev)
    b, h, T, P, N = _dims(U, B)
    Y = np.zeros((b, h, T, P))
    bad = lib().slx_oracle_chunk_scan(b * h, T, P, N, chunk_size, _c(U), _c(M), _c(K),
                                      _c(B), _c(C), _c(chunk_starts), _c(bp), _c(up),
                                      _c(Y))
    if bad:
        raise ValueError("M must be strictly nonzero in chunked scan paths.")
    return Y


def v2x2ssd_fwd(U, M, K, B, C, *, chunk_size: int, initial_states=None,
                B_prev=None, U_prev=None):
    """Staged forward (reference.py:1195). Returns (Y, final, chunk_starts, m_chunk)."""
    U, M, K, B, C = map(_f64, (U, M, K, B, C))
    init, bp, up = map(_f64, (initial_states, B_prev, U_prev))
    b, h, T, P, N = _dims(U, B)
    NC = (T + chunk_size - 1) // chunk_size
    Y = np.zeros((b, h, T, P))
    fin = np.zeros((b, h, P, 2 * N))
    starts = np.zeros((b, h, NC, P, 2 * N))
    mch = np.zeros((b, h, NC, 2))
    bad = lib().slx_oracle_v2x2ssd_fwd(b * h, T, P, N, chunk_size, _c(U), _c(M), _c(K),
                                       _c(B), _c(C), _c(init), _c(bp), _c(up), _c(Y),
                                       _c(fin), _c(starts), _c(mch))
    if bad:
        raise ValueError("M must be strictly nonzero in chunked scan paths.")
    return Y, fin, starts, mch
