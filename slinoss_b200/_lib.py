"""ctypes binding of ``libslinoss_b200.so`` (the C ABI in ``include/slinoss_b200.h``).

The library is the only compute path of this package: if it is missing or a
symbol is absent, the import of any op fails loudly -- there is no CPU or
framework fallback.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path
from typing import Optional

import torch

LIB_PATH = Path(__file__).resolve().parent / "_C" / "libslinoss_b200.so"

SLX_F32, SLX_BF16, SLX_F16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: SLX_F32, torch.bfloat16: SLX_BF16, torch.float16: SLX_F16}


class ScanShape(Structure):
    _fields_ = [("batch_heads", c_int32), ("T", c_int32), ("P", c_int32), ("N", c_int32),
                ("chunk", c_int32), ("dtype", c_int32), ("starts_dtype", c_int32)]


class PrepShape(Structure):
    _fields_ = [("batch", c_int32), ("T", c_int32), ("heads", c_int32), ("P", c_int32),
                ("N", c_int32), ("dtype", c_int32), ("normalize_bc", c_int32),
                ("dt_min", c_float), ("dt_max", c_float), ("r_min", c_float), ("r_max", c_float),
                ("theta_bound", c_float), ("k_max", c_float), ("eps", c_float),
                ("value_stride", c_int64), ("params_stride", c_int64), ("bc_stride", c_int64)]


class DecodeShape(Structure):
    _fields_ = [("batch", c_int32), ("heads", c_int32), ("P", c_int32), ("N", c_int32),
                ("dtype", c_int32), ("normalize_bc", c_int32),
                ("dt_min", c_float), ("dt_max", c_float), ("r_min", c_float), ("r_max", c_float),
                ("theta_bound", c_float), ("k_max", c_float), ("eps", c_float)]


class GlueShape(Structure):
    _fields_ = [("batch", c_int32), ("T", c_int32), ("heads", c_int32), ("P", c_int32), ("dtype", c_int32),
                ("gate_stride", c_int64), ("gate_batch_stride", c_int64)]


class ConvShape(Structure):
    _fields_ = [("batch", c_int32), ("T", c_int32), ("channels", c_int32), ("width", c_int32),
                ("dtype", c_int32), ("silu", c_int32), ("x_stride", c_int64),
                ("x_batch_stride", c_int64)]


# name -> (restype, argtypes); mirrors include/slinoss_b200.h one to one
_P = c_void_p
SIGNATURES = {
    "slx_abi_version": (c_int32, []),
    "slx_scan_starts_dtype": (c_int32, [POINTER(ScanShape)]),
    "slx_last_error_string": (c_char_p, []),
    "slx_chunk_increment_fwd": (c_int32, [POINTER(ScanShape)] + [_P] * 7 + [c_int32] + [_P] * 2),
    "slx_state_passing_fwd": (c_int32, [c_int32] * 4 + [_P, c_int32] + [_P] * 3 + [c_int32] + [_P] * 2),
    "slx_chunk_scan_fwd": (c_int32, [POINTER(ScanShape)] + [_P] * 10),
    "slx_v2x2ssd_fwd": (c_int32, [POINTER(ScanShape)] + [_P] * 14),
    "slx_v2x2ssd_bwd_workspace_bytes": (c_size_t, [POINTER(ScanShape)]),
    "slx_chunk_scan_bwd_dz0": (c_int32, [POINTER(ScanShape)] + [_P] * 4 + [c_int32, _P]),
    "slx_state_passing_bwd_partials_bytes": (c_size_t, [c_int32] * 4),
    "slx_state_passing_bwd": (c_int32, [c_int32] * 4 + [_P, c_int32] + [_P] * 2 + [c_int32] + [_P] * 7),
    "slx_chunk_scan_bwd": (c_int32, [POINTER(ScanShape)] + [_P] * 19),
    "slx_v2x2ssd_bwd": (c_int32, [POINTER(ScanShape)] + [_P] * 21 + [c_size_t, _P]),
    "slx_v2x2ssd_bwd_begin": (c_int32, [POINTER(ScanShape)] + [_P] * 6 + [c_size_t, _P]),
    "slx_v2x2ssd_bwd_finish": (c_int32, [POINTER(ScanShape)] + [_P] * 21 + [c_size_t, _P]),
    "slx_scanprep_fwd": (c_int32, [POINTER(PrepShape)] + [_P] * 11),
    "slx_scanprep_bwd_workspace_bytes": (c_size_t, [POINTER(PrepShape)]),
    "slx_scanprep_bwd": (c_int32, [POINTER(PrepShape)] + [_P] * 15 + [c_size_t, _P]),
    "slx_cconv1d_bwd_noalloc": (c_int32, [POINTER(ConvShape)] + [_P] * 11),
    "slx_gate_skip_fwd": (c_int32, [POINTER(GlueShape)] + [_P] * 6),
    "slx_gate_skip_bwd_workspace_bytes": (c_size_t, [POINTER(GlueShape)]),
    "slx_gate_skip_bwd": (c_int32, [POINTER(GlueShape)] + [_P] * 10 + [c_size_t, _P]),
    "slx_set_tensor_path": (c_int32, [c_int32]),
    "slx_set_persistent_ctas": (c_int32, [c_int32]),
    "slx_read_tc_status": (c_int32, [POINTER(c_int32)]),
    "slx_read_scan_status": (c_int32, [POINTER(c_int32)]),
    "slx_decode_step": (c_int32, [POINTER(DecodeShape)] + [_P] * 15),
    "slx_cconv1d_fwd": (c_int32, [POINTER(ConvShape)] + [_P] * 7),
    "slx_cconv1d_update": (c_int32, [POINTER(ConvShape)] + [_P] * 7),
    "slx_segment_fold": (c_int32, [c_int32] * 4 + [_P, c_int64, _P, c_int64, c_int32, _P, _P]),
    "slx_segment_axpy": (c_int32, [c_int32] * 3 + [_P] * 3 + [c_int32, _P, _P]),
    "slx_segment_transition": (c_int32, [c_int32] * 2 + [_P] * 3),
    "slx_cconv1d_bwd_workspace_bytes": (c_size_t, [POINTER(ConvShape)]),
    "slx_cconv1d_bwd": (c_int32, [POINTER(ConvShape)] + [_P] * 11 + [c_size_t, _P]),
}

SELFTEST_LIB_PATH = LIB_PATH.with_name("libslinoss_b200_selftest.so")
SELFTEST_SIGNATURES = {
    "slx_umma_selftest": (c_int32, [c_int32] + [_P] * 5),
    "slx_selftest_last_error_string": (c_char_p, []),
}

_lib: Optional[ctypes.CDLL] = None
_selftest: Optional[ctypes.CDLL] = None


def selftest_lib() -> ctypes.CDLL:
    """The test-only library (tile-engine self-test); never loaded by the ops."""
    global _selftest
    if _selftest is None:
        if not SELFTEST_LIB_PATH.exists():
            raise RuntimeError(f"{SELFTEST_LIB_PATH} is missing: run slinoss_b200.build.build_selftest().")
        handle = ctypes.CDLL(str(SELFTEST_LIB_PATH))
        for name, (res, args) in SELFTEST_SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _selftest = handle
    return _selftest


def lib() -> ctypes.CDLL:
    """Load the shared library (once) and bind every declared symbol."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the sm_100a kernels first "
                "(python -m slinoss_b200.build). There is no fallback path.")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the export is absent
            fn.restype = res
            fn.argtypes = args
        _lib = handle
        # SLX_SCAN_KERNELS=0|1|2 picks the kernel family at load time (see set_tensor_path)
        env = os.environ.get("SLX_SCAN_KERNELS")
        if env is not None:
            handle.slx_set_tensor_path(int(env))
    return _lib


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}; expected float32, bfloat16 or float16") from None


_CODE_DTYPE = {v: k for k, v in _DTYPE_CODE.items()}


def scan_shape(batch_heads: int, T: int, P: int, N: int, chunk: int, dtype: torch.dtype,
               starts: Optional[torch.dtype] = None) -> "ScanShape":
    """Shape struct of the scan entry points.  ``starts`` is the dtype of ``chunk_starts`` /
    ``d_inc`` and with it the kernel family (activation dtype: tcgen05 kernels, fp32: exact
    kernels); ``None`` takes the library's recommendation for the shape."""
    s = ScanShape(batch_heads, T, P, N, chunk, dtype_code(dtype), SLX_F32)
    s.starts_dtype = (int(lib().slx_scan_starts_dtype(ctypes.byref(s))) if starts is None
                      else dtype_code(starts))
    return s


def starts_dtype(shape: "ScanShape") -> torch.dtype:
    """dtype in which the stages of this shape exchange chunk_starts."""
    return _CODE_DTYPE[int(shape.starts_dtype)]


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class guard:
    """Make ``device`` the current CUDA device around a library call.

    The library launches on the current device of the calling thread, so every call is wrapped
    in this guard with the device of the tensors it is given: a model that lives on ``cuda:1``
    while ``cuda:0`` is current still launches on ``cuda:1``.  A no-op when the device is
    already current."""

    __slots__ = ("device", "ctx")

    def __init__(self, device) -> None:
        self.device = torch.device(device)
        self.ctx = None

    def __enter__(self):
        d = self.device
        if d.type != "cuda":
            raise ValueError(f"slinoss_b200 kernels need CUDA tensors; got device {d}.")
        idx = d.index
        if idx is not None and idx != torch.cuda.current_device():
            self.ctx = torch.cuda.device(idx)
            self.ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self.ctx is not None:
            ctx, self.ctx = self.ctx, None
            return ctx.__exit__(*exc)
        return False


def same_device(*tensors) -> torch.device:
    """Device shared by every given tensor (``None`` entries are skipped); raises the reference's
    error when they differ (slinoss/ops/v2x2ssd/reference.py:133-137)."""
    devs = [t.device for t in tensors if t is not None]
    if not devs:
        raise ValueError("no tensor given")
    if any(d != devs[0] for d in devs):
        raise ValueError(f"All inputs must be on the same device. Got {devs}.")
    return devs[0]


def check(status: int, what: str) -> None:
    """Turn a non-zero C status into the exception the reference would raise."""
    if status == 0:
        return
    msg = lib().slx_last_error_string().decode("utf-8", "replace")
    if status < 0:
        if status == -5:
            raise TypeError(f"{what}: {msg}")
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: CUDA error {status}: {msg}")


def set_tensor_path(enable) -> int:
    """Process-wide choice of the kernel family for shapes the tcgen05 kernels cover:
    ``False``/0 = fp32-exact CUDA-core kernels, 1 = one-chunk-per-CTA tcgen05 kernels,
    ``True``/2 = persistent warp-specialised tcgen05 kernels (default).  Returns the previous
    value (0, 1 or 2)."""
    code = 2 if enable is True else (0 if enable is False else int(enable))
    return int(lib().slx_set_tensor_path(code))


def set_persistent_ctas(max_ctas: int) -> int:
    """Cap on the CTAs of the persistent tensor-core kernels (0 = one per SM, the default).
    Returns the previous cap."""
    return int(lib().slx_set_persistent_ctas(int(max_ctas)))


def _status_device(device) -> torch.device:
    return torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)


def read_scan_status(device=None) -> int:
    """Synchronising read-and-clear (one atomic exchange on the device) of the scan's input
    status word of ``device`` (default: the current device).  Non-zero: some launch on that
    device since the last read met a transition of magnitude exactly 0 and produced NaN.
    The word is one per device, shared by every stream and thread that uses the device."""
    out = c_int32(0)
    with guard(_status_device(device)):
        check(lib().slx_read_scan_status(ctypes.byref(out)), "read_scan_status")
    return int(out.value)


def read_tc_status(device=None) -> int:
    """Synchronising read-and-clear (one atomic exchange on the device) of the tensor-core
    kernels' status word of ``device`` (default: the current device).  Non-zero: a bounded
    completion wait ran out in some launch on that device since the last read; the outputs of
    the affected chunks were filled with NaN."""
    out = c_int32(0)
    with guard(_status_device(device)):
        check(lib().slx_read_tc_status(ctypes.byref(out)), "read_tc_status")
    return int(out.value)
