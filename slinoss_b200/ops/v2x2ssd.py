"""``v2x2ssd`` on B200: host side of the chunked scan.

``v2x2ssd_b200`` has the signature, return values and error behaviour of the
reference's ``slinoss.ops.v2x2ssd.v2x2ssd_cute`` (slinoss/ops/v2x2ssd/cute/
api.py:52-172); the stage functions mirror ``chunk_increment_cute`` /
``state_passing_cute`` / ``chunk_scan_cute`` (cute/kernels/fwd/__init__.py:740,
897,1125).  All arithmetic happens in the sm_100a kernels behind the C ABI;
this file validates, allocates outputs with torch and wires autograd.
"""

from __future__ import annotations

from ctypes import byref
from typing import Optional, Tuple

import torch

from .. import _lib

_ACT_DTYPES = (torch.float32, torch.bfloat16, torch.float16)
_CHUNKS = (16, 32, 64, 128)


def _check_contiguous(name: str, x: torch.Tensor) -> None:
    if not x.is_contiguous():
        raise ValueError(f"{name} must be contiguous; got strides {x.stride()}.")


def _validate_inputs(U, M, K, B, C, initial_states, B_prev, U_prev) -> Tuple[int, int, int, int, int]:
    """Same checks and messages as reference.py:124-204 (_validate_inputs)."""
    tensors = (U, M, K, B, C)
    if not all(torch.is_floating_point(t) for t in tensors):
        raise ValueError("U, M, K, B, and C must be floating-point tensors.")
    device = U.device
    if not all(t.device == device for t in tensors):
        raise ValueError(f"All inputs must be on the same device. Got {[t.device for t in tensors]}.")
    for name, t in (("U", U), ("M", M), ("K", K), ("B", B), ("C", C)):
        _check_contiguous(name, t)
    if U.ndim != 4:
        raise ValueError(f"U must be (batch,heads,T,P). Got {tuple(U.shape)}.")
    if M.ndim != 4 or M.shape[-1] != 2:
        raise ValueError(f"M must be (batch,heads,T,2). Got {tuple(M.shape)}.")
    if K.ndim != 5 or K.shape[-2:] != (2, 2):
        raise ValueError(f"K must be (batch,heads,T,2,2). Got {tuple(K.shape)}.")
    if B.ndim != 4:
        raise ValueError(f"B must be (batch,heads,T,2N). Got {tuple(B.shape)}.")
    if C.ndim != 4:
        raise ValueError(f"C must be (batch,heads,T,2N). Got {tuple(C.shape)}.")
    b, h, T, P = map(int, U.shape)
    for name, t in (("M", M), ("K", K), ("B", B), ("C", C)):
        if tuple(t.shape[:3]) != (b, h, T):
            raise ValueError(f"Leading (batch,heads,T) dims of {name} must match U.")
    D = int(B.shape[-1])
    if D % 2 != 0:
        raise ValueError(f"B/C 2N dim must be divisible by 2. Got {D}.")
    if tuple(C.shape) != (b, h, T, D):
        raise ValueError("C must match B exactly.")
    if (B_prev is None) ^ (U_prev is None):
        raise ValueError("B_prev and U_prev must be passed together (or both omitted).")
    if initial_states is not None:
        if tuple(initial_states.shape) != (b, h, P, D):
            raise ValueError("initial_states must be (batch,heads,P,2N) "
                             f"={(b, h, P, D)}. Got {tuple(initial_states.shape)}.")
        _check_contiguous("initial_states", initial_states)
        if initial_states.device != device:
            raise ValueError("initial_states must be on the same device as inputs.")
    if B_prev is not None:
        if tuple(B_prev.shape) != (b, h, D):
            raise ValueError(f"B_prev must be (batch,heads,2N)={(b, h, D)}. Got {tuple(B_prev.shape)}.")
        if tuple(U_prev.shape) != (b, h, P):
            raise ValueError(f"U_prev must be (batch,heads,P)={(b, h, P)}. Got {tuple(U_prev.shape)}.")
        _check_contiguous("B_prev", B_prev)
        _check_contiguous("U_prev", U_prev)
        if B_prev.device != device or U_prev.device != device:
            raise ValueError("B_prev and U_prev must be on the same device as inputs.")
    return b, h, T, D // 2, P


def _resolve_dtypes(input_dtypes, compute_dtype, output_dtype, default_output_dtype):
    """reference.py:59-80 (_resolve_dtypes)."""
    if compute_dtype is None:
        promoted = input_dtypes[0]
        for dt in input_dtypes[1:]:
            promoted = torch.promote_types(promoted, dt)
        rdtype = torch.float32 if promoted in (torch.float16, torch.bfloat16) else promoted
    else:
        rdtype = compute_dtype
    if rdtype not in (torch.float32, torch.float64):
        raise ValueError(f"compute_dtype must be float32 or float64, got {rdtype}.")
    odtype = default_output_dtype if output_dtype is None else output_dtype
    if odtype not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
        raise ValueError(f"output_dtype must be a real floating dtype, got {odtype}.")
    return rdtype, odtype


def _resolve_empty_outputs(b, h, P, D, device, odtype, initial_states, B_prev, U_prev):
    """T == 0 semantics of reference.py:670-701."""
    Y = torch.empty((b, h, 0, P), device=device, dtype=odtype)
    final = (torch.zeros((b, h, P, D), device=device, dtype=odtype) if initial_states is None
             else initial_states.to(dtype=odtype).contiguous())
    if B_prev is None:
        B_last = torch.zeros((b, h, D), device=device, dtype=odtype)
        U_last = torch.zeros((b, h, P), device=device, dtype=odtype)
    else:
        B_last = B_prev.to(dtype=odtype).contiguous()
        U_last = U_prev.to(dtype=odtype).contiguous()
    return Y, final, B_last, U_last


def _require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and t.device.type != "cuda":
            raise ValueError("slinoss_b200 v2x2ssd requires CUDA tensors.")


def _aligned(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """The kernels use 16-byte accesses: a view that starts at an odd offset of its storage is
    copied to a fresh (aligned) tensor."""
    if t is None or t.data_ptr() % 16 == 0:
        return t
    return t.clone(memory_format=torch.contiguous_format)


def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else _aligned(t.detach().to(torch.float32).contiguous())


def _shape(b, h, T, P, N, L, dtype) -> _lib.ScanShape:
    if L not in _CHUNKS:
        raise ValueError(f"chunk_size must be one of {_CHUNKS} for the sm_100a kernels. Got {L}.")
    return _lib.scan_shape(b * h, T, P, N, L, dtype)


# --------------------------------------------------------------------------- #
# stage-level entry points
# --------------------------------------------------------------------------- #

def _stage_inputs(U, M, K, B, C, B_prev, U_prev):
    """Validation and dtype handling shared by the stage-level entry points: the checks of
    ``_validate_inputs`` (same messages as the reference), then M and K as fp32, U/B/C in one
    activation dtype, everything 16-byte aligned -- what ``v2x2ssd_b200`` does for the fused op."""
    _validate_inputs(U, M, K, B, B if C is None else C, None, B_prev, U_prev)
    _require_cuda(U, M, K, B, C, B_prev, U_prev)
    act = torch.promote_types(U.dtype, B.dtype)
    if C is not None:
        act = torch.promote_types(act, C.dtype)
    if act not in _ACT_DTYPES:
        raise TypeError(f"U/B/C must be float32, bfloat16 or float16. Got {act}.")
    cast = lambda t: None if t is None else _aligned(t if t.dtype == act else t.to(act))
    f32 = lambda t: _aligned(t if t.dtype == torch.float32 else t.to(torch.float32))
    return cast(U), f32(M), f32(K), cast(B), cast(C)


def chunk_increment_b200(U, M, K, B, *, B_prev=None, U_prev=None, chunk_size: int,
                         inc_dtype: torch.dtype = torch.float32):
    """Stage 1 -> ``(inc (b,h,C,P,2N), m_chunk (b,h,C,2) fp32)``.  Inputs are checked as
    the reference checks them (contiguous, matching shapes, one device).  ``inc`` is fp32 like the
    reference's by default; ``inc_dtype`` = the activation dtype (tensor-core shapes only) stores
    it as the fused op does, halving the traffic of this stage's output and the next stage's input."""
    if inc_dtype not in _ACT_DTYPES:
        raise TypeError(f"inc_dtype must be float32, bfloat16 or float16. Got {inc_dtype}.")
    U, M, K, B, _ = _stage_inputs(U, M, K, B, None, B_prev, U_prev)
    b, h, T, P = map(int, U.shape)
    D = int(B.shape[-1])
    L = int(chunk_size)
    if L <= 0:
        raise ValueError(f"chunk_size must be positive. Got {chunk_size}.")
    NC = (T + L - 1) // L
    s = _shape(b, h, T, P, D // 2, L, U.dtype)
    inc = torch.empty((b, h, NC, P, D), device=U.device, dtype=inc_dtype)
    mch = torch.empty((b, h, NC, 2), device=U.device, dtype=torch.float32)
    bp, up = _f32(B_prev), _f32(U_prev)
    with _lib.guard(U.device):
        _lib.check(_lib.lib().slx_chunk_increment_fwd(
            byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), _lib.ptr(bp), _lib.ptr(up),
            inc.data_ptr(), _lib.dtype_code(inc_dtype), mch.data_ptr(), _lib.stream_ptr(U.device)),
            "chunk_increment")
    return inc, mch


def state_passing_b200(inc, m_chunk, *, initial_states=None, want_starts: bool = True,
                       starts_dtype: torch.dtype = torch.float32):
    """Stage 2 -> ``(chunk_starts, final_state)``.  The recurrence and ``final_state`` are fp32;
    ``chunk_starts`` is stored as ``starts_dtype`` (fp32 like the reference by default; the fused
    op uses the activation dtype where the tensor-core kernels run).  ``want_starts=False``
    returns ``(None, final_state)`` and writes nothing but the final state (half the traffic).
    ``inc`` is read in its own dtype: fp32, or ``starts_dtype`` (what ``chunk_increment_b200`` wrote
    with ``inc_dtype`` set)."""
    if inc.ndim != 5:
        raise ValueError(f"inc must be (batch,heads,chunks,P,2N). Got {tuple(inc.shape)}.")
    b, h, NC, P, D = map(int, inc.shape)
    if D % 2 != 0:
        raise ValueError(f"inc 2N dim must be divisible by 2. Got {D}.")
    if tuple(m_chunk.shape) != (b, h, NC, 2):
        raise ValueError(f"m_chunk must be (batch,heads,chunks,2)={(b, h, NC, 2)}. Got {tuple(m_chunk.shape)}.")
    if initial_states is not None and tuple(initial_states.shape) != (b, h, P, D):
        raise ValueError(f"initial_states must be (batch,heads,P,2N)={(b, h, P, D)}. "
                         f"Got {tuple(initial_states.shape)}.")
    if starts_dtype not in _ACT_DTYPES:
        raise TypeError(f"starts_dtype must be float32, bfloat16 or float16. Got {starts_dtype}.")
    if inc.dtype in _ACT_DTYPES and inc.dtype != torch.float32 and want_starts and inc.dtype != starts_dtype:
        raise TypeError(f"inc must be float32 or starts_dtype={starts_dtype}. Got {inc.dtype}.")
    _require_cuda(inc, m_chunk, initial_states)
    dev = _lib.same_device(inc, m_chunk, initial_states)
    if inc.dtype not in _ACT_DTYPES:
        inc = inc.to(torch.float32)
    inc, m_chunk = _aligned(inc.detach().contiguous()), _f32(m_chunk)
    init = _f32(initial_states)
    starts = torch.empty(inc.shape, device=dev, dtype=starts_dtype) if want_starts else None
    final = torch.empty((b, h, P, D), device=dev, dtype=torch.float32)
    with _lib.guard(dev):
        _lib.check(_lib.lib().slx_state_passing_fwd(
            b * h, NC, P, D // 2, inc.data_ptr(), _lib.dtype_code(inc.dtype), m_chunk.data_ptr(), _lib.ptr(init),
            _lib.ptr(starts), _lib.dtype_code(starts_dtype), final.data_ptr(), _lib.stream_ptr(dev)),
            "state_passing")
    return starts, final


def chunk_scan_b200(U, M, K, B, C, chunk_starts, *, B_prev=None, U_prev=None, chunk_size: int):
    """Stage 3 -> ``Y (b,h,T,P)`` in the activation dtype.  Inputs are checked as the reference
    checks them; ``chunk_starts`` must be ``(b,h,chunks,P,2N)`` for this ``chunk_size``."""
    U, M, K, B, C = _stage_inputs(U, M, K, B, C, B_prev, U_prev)
    b, h, T, P = map(int, U.shape)
    D = int(B.shape[-1])
    L = int(chunk_size)
    if L <= 0:
        raise ValueError(f"chunk_size must be positive. Got {chunk_size}.")
    NC = (T + L - 1) // L
    if tuple(chunk_starts.shape) != (b, h, NC, P, D):
        raise ValueError(f"chunk_starts must be (batch,heads,chunks,P,2N)={(b, h, NC, P, D)}. "
                         f"Got {tuple(chunk_starts.shape)}.")
    _lib.same_device(U, chunk_starts)
    s = _shape(b, h, T, P, D // 2, L, U.dtype)
    chunk_starts = _aligned(_as_starts(chunk_starts, s).contiguous())
    Y = torch.empty_like(U)
    bp, up = _f32(B_prev), _f32(U_prev)
    with _lib.guard(U.device):
        _lib.check(_lib.lib().slx_chunk_scan_fwd(
            byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), C.data_ptr(),
            chunk_starts.data_ptr(), _lib.ptr(bp), _lib.ptr(up), Y.data_ptr(), _lib.stream_ptr(U.device)),
            "chunk_scan")
    return Y


def _as_starts(chunk_starts: torch.Tensor, s: "_lib.ScanShape") -> torch.Tensor:
    """chunk_starts in the dtype the kernels of this shape exchange it in (a conversion pass only
    when the caller's tensor is in another dtype, e.g. fp32 starts from the stage-level API)."""
    want = _lib.starts_dtype(s)
    return chunk_starts if chunk_starts.dtype == want else chunk_starts.to(want)


def _fwd_impl(U, M, K, B, C, init32, bp32, up32, L):
    """Three stages back to back.  Returns (Y, final32, chunk_starts, m_chunk)."""
    b, h, T, P = map(int, U.shape)
    D = int(B.shape[-1])
    NC = (T + L - 1) // L
    s = _shape(b, h, T, P, D // 2, L, U.dtype)
    dev = U.device
    Y = torch.empty_like(U)
    final = torch.empty((b, h, P, D), device=dev, dtype=torch.float32)
    starts = torch.empty((b, h, NC, P, D), device=dev, dtype=_lib.starts_dtype(s))
    mch = torch.empty((b, h, NC, 2), device=dev, dtype=torch.float32)
    # separate increment buffer (stored like the chunk starts): the two-buffer state pass is ~2.5x
    # faster than the in-place one
    inc = torch.empty((b, h, NC, P, D), device=dev, dtype=starts.dtype)
    with _lib.guard(dev):
        _lib.check(_lib.lib().slx_v2x2ssd_fwd(
            byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), C.data_ptr(),
            _lib.ptr(init32), _lib.ptr(bp32), _lib.ptr(up32), Y.data_ptr(), final.data_ptr(),
            starts.data_ptr(), mch.data_ptr(), inc.data_ptr(), _lib.stream_ptr(dev)), "v2x2ssd forward")
    return Y, final, starts, mch


def _bwd_begin(M, C, mch, dY, L, P):
    """First half of the two-call backward: dZ0 into a fresh workspace and the segment's
    d_initial for a zero d_final.  Returns ``(g0, workspace)``; pass the workspace to
    ``_bwd_impl(..., workspace=...)``."""
    b, h, T, D = map(int, C.shape)
    s = _shape(b, h, T, P, D // 2, L, C.dtype)
    dev = C.device
    L_ = _lib.lib()
    nbytes = int(L_.slx_v2x2ssd_bwd_workspace_bytes(byref(s)))
    ws = torch.empty((nbytes,), device=dev, dtype=torch.uint8)
    g0 = torch.empty((b, h, P, D), device=dev, dtype=torch.float32)
    with _lib.guard(dev):
        _lib.check(L_.slx_v2x2ssd_bwd_begin(byref(s), M.data_ptr(), C.data_ptr(), mch.data_ptr(), dY.data_ptr(),
                                            g0.data_ptr(), ws.data_ptr(), nbytes, _lib.stream_ptr(dev)),
                   "v2x2ssd backward (begin)")
    return g0, ws


def _bwd_impl(U, M, K, B, C, bp32, up32, starts, mch, final32, dY, d_final32, L, *,
              want_initial: bool, want_prev: bool, workspace=None):
    b, h, T, P = map(int, U.shape)
    D = int(B.shape[-1])
    s = _shape(b, h, T, P, D // 2, L, U.dtype)
    dev = U.device
    dU, dB, dC = torch.empty_like(U), torch.empty_like(B), torch.empty_like(C)
    dM = torch.empty((b, h, T, 2), device=dev, dtype=torch.float32)
    dK = torch.empty((b, h, T, 2, 2), device=dev, dtype=torch.float32)
    d_init = torch.empty((b, h, P, D), device=dev, dtype=torch.float32) if want_initial else None
    dBp = torch.empty((b, h, D), device=dev, dtype=torch.float32) if want_prev else None
    dUp = torch.empty((b, h, P), device=dev, dtype=torch.float32) if want_prev else None
    L_ = _lib.lib()
    nbytes = int(L_.slx_v2x2ssd_bwd_workspace_bytes(byref(s)))
    starts = _as_starts(starts, s)
    ws = torch.empty((nbytes,), device=dev, dtype=torch.uint8) if workspace is None else workspace
    entry = L_.slx_v2x2ssd_bwd if workspace is None else L_.slx_v2x2ssd_bwd_finish  # dZ0 already there
    with _lib.guard(dev):
        _lib.check(entry(
            byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), C.data_ptr(),
            _lib.ptr(bp32), _lib.ptr(up32), starts.data_ptr(), mch.data_ptr(), final32.data_ptr(),
            dY.data_ptr(), _lib.ptr(d_final32), dU.data_ptr(), dM.data_ptr(), dK.data_ptr(),
            dB.data_ptr(), dC.data_ptr(), _lib.ptr(d_init), _lib.ptr(dBp), _lib.ptr(dUp),
            ws.data_ptr(), nbytes, _lib.stream_ptr(dev)), "v2x2ssd backward")
    return dU, dM, dK, dB, dC, d_init, dBp, dUp


class _V2x2SSDFn(torch.autograd.Function):
    """Autograd node; same inputs/outputs as the reference's
    ``_V2x2SSDCuTeTrainingFn`` (cute/autograd.py:40-266)."""

    @staticmethod
    def forward(ctx, U, M, K, B, C, initial_states, B_prev, U_prev, L, odtype, return_state, residual="keep"):
        init32, bp32, up32 = _f32(initial_states), _f32(B_prev), _f32(U_prev)
        Y, final32, starts, mch = _fwd_impl(U.detach(), M.detach(), K.detach(), B.detach(),
                                            C.detach(), init32, bp32, up32, L)
        ctx.L = L
        ctx.return_state = return_state
        ctx.has_init = initial_states is not None
        ctx.has_prev = B_prev is not None
        ctx.init_dtype = None if initial_states is None else initial_states.dtype
        ctx.prev_dtype = None if B_prev is None else B_prev.dtype
        # What is kept of the chunk-start states (the largest residual, (b,h,NC,P,2N)): "keep" as the
        # kernels exchange them (activation dtype on the tensor-core path, fp32 otherwise);
        # "recompute" nothing: the backward rebuilds them from the inputs with one more
        # chunk-increment and state pass.
        ctx.residual = residual
        if residual == "recompute":
            starts = init32 if init32 is not None else final32.new_empty(0)
        saved = [U, M, K, B, C, mch, starts, final32]
        if ctx.has_prev:
            saved += [bp32, up32]
        ctx.save_for_backward(*[t.detach() for t in saved])
        Y = Y.to(odtype)
        if not return_state:
            return Y
        B_last = B.detach()[:, :, -1, :].to(odtype).contiguous()
        U_last = U.detach()[:, :, -1, :].to(odtype).contiguous()
        return Y, final32.to(odtype), B_last, U_last

    @staticmethod
    def backward(ctx, *grads):
        saved = ctx.saved_tensors
        U, M, K, B, C, mch, starts, final32 = saved[:8]
        bp32, up32 = (saved[8], saved[9]) if ctx.has_prev else (None, None)
        if ctx.return_state:
            dY, d_final, dB_last, dU_last = grads
        else:
            (dY,) = grads
            d_final = dB_last = dU_last = None
        dU = dM = dK = dB = dC = d_init = dBp = dUp = None
        if dY is not None or d_final is not None:
            dYc = (torch.zeros_like(U) if dY is None else _aligned(dY.to(U.dtype).contiguous()))
            dfin = None if d_final is None else d_final.to(torch.float32).contiguous()
            if ctx.residual == "recompute":
                init32 = starts if starts.numel() else None
                b_, h_, T_, P_ = map(int, U.shape)
                sdt = _lib.starts_dtype(_shape(b_, h_, T_, P_, int(B.shape[-1]) // 2, ctx.L, U.dtype))
                inc, _ = chunk_increment_b200(U, M, K, B, B_prev=bp32, U_prev=up32, chunk_size=ctx.L, inc_dtype=sdt)
                starts, _ = state_passing_b200(inc, mch, initial_states=init32, starts_dtype=sdt)
                del inc
            dU, dM, dK, dB, dC, d_init, dBp, dUp = _bwd_impl(
                U, M, K, B, C, bp32, up32, starts, mch, final32, dYc, dfin, ctx.L,
                want_initial=ctx.has_init, want_prev=ctx.has_prev)
        if dB_last is not None:
            if dB is None:
                dB = torch.zeros_like(B)
            dB[:, :, -1, :].add_(dB_last.to(B.dtype))
        if dU_last is not None:
            if dU is None:
                dU = torch.zeros_like(U)
            dU[:, :, -1, :].add_(dU_last.to(U.dtype))
        if d_init is not None:
            d_init = d_init.to(ctx.init_dtype)
        if dBp is not None:
            dBp, dUp = dBp.to(ctx.prev_dtype), dUp.to(ctx.prev_dtype)
        return dU, dM, dK, dB, dC, d_init, dBp, dUp, None, None, None, None


@torch.compiler.disable
def v2x2ssd_b200(U, M, K, B, C, *, chunk_size: int, initial_states=None, B_prev=None, U_prev=None,
                 compute_dtype: Optional[torch.dtype] = None,
                 output_dtype: Optional[torch.dtype] = None, return_state: bool = False,
                 retile: bool = True, strict: bool = False, residual: str = "keep"):
    """Drop-in for ``v2x2ssd_cute`` (cute/api.py:52): returns ``Y`` or
    ``(Y, final_state, B_last, U_last)``; differentiable in all eight inputs.

    ``chunk_size`` only says how the sequence is tiled; none of the returned values depends
    on it beyond rounding.  With ``retile`` (default) half-precision inputs of head dim 64 and
    state width up to 256 are tiled in the 128-token chunks of the tcgen05 kernels whatever
    ``chunk_size`` asks for (the reference's default is 64); ``retile=False`` keeps the
    requested tiling (fp32-exact kernels for anything but 128).

    A transition ``M`` of magnitude exactly 0 makes the reference raise ``ValueError``
    (reference.py:480-485).  The kernels cannot raise: they fill the affected outputs with NaN
    and set a status word (``read_scan_status``).  ``strict=True`` reads that word after the
    forward (one device synchronisation per call) and raises like the reference; it also reads
    the tensor-core kernels' status word (a completion wait that ran out) and raises
    ``RuntimeError`` for it.  The status words are one per device, shared by every stream and
    thread using that device: ``strict`` is meant for one caller at a time per device.

    ``residual`` chooses what autograd keeps of the chunk-start states, the largest residual
    ((batch, heads, chunks, P, 2N); the reference saves it in fp32, cute/autograd.py:98):
    ``"keep"`` (default) as the kernels exchange it (activation dtype on the tensor-core path,
    fp32 otherwise) or ``"recompute"`` (nothing kept; the backward rebuilds it with one more
    chunk-increment and state pass, bitwise the same gradients).
    """
    if residual not in ("keep", "recompute"):
        raise ValueError(f"residual must be 'keep' or 'recompute'. Got {residual!r}.")
    b, h, T, N, P = _validate_inputs(U, M, K, B, C, initial_states, B_prev, U_prev)
    if U.device.type != "cuda":
        raise ValueError("slinoss_b200 v2x2ssd requires CUDA tensors.")
    if chunk_size <= 0:
        raise ValueError(f"chunk_size must be positive. Got {chunk_size}.")
    D = 2 * N
    rdtype, odtype = _resolve_dtypes([U.dtype, M.dtype, K.dtype, B.dtype, C.dtype], compute_dtype,
                                     output_dtype, U.dtype)
    if rdtype != torch.float32:
        raise ValueError("The sm_100a v2x2ssd path supports only float32 compute. "
                         f"Got compute_dtype={rdtype}.")
    if T == 0:
        out = _resolve_empty_outputs(b, h, P, D, U.device, odtype, initial_states, B_prev, U_prev)
        return out if return_state else out[0]
    # the kernels take U, B, C in one activation dtype and M, K in fp32
    act = torch.promote_types(torch.promote_types(U.dtype, B.dtype), C.dtype)
    if act not in _ACT_DTYPES:
        raise TypeError(f"U/B/C must be float32, bfloat16 or float16. Got {act}.")
    if odtype == torch.float32 and act != torch.float32:
        act = torch.float32  # a wider output must not be rounded through the half store
    Ua, Ba, Ca = (t if t.dtype == act else t.to(act) for t in (U, B, C))
    Mf = M if M.dtype == torch.float32 else M.to(torch.float32)
    Kf = K if K.dtype == torch.float32 else K.to(torch.float32)
    Ua, Ba, Ca, Mf, Kf = (_aligned(t) for t in (Ua, Ba, Ca, Mf, Kf))
    if retile and act in (torch.bfloat16, torch.float16) and P == 64 and D % 64 == 0 and D <= 256:
        chunk_size = 128
    needs_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (U, M, K, B, C, initial_states, B_prev, U_prev))
    if strict:
        _lib.read_scan_status(U.device)  # clear what earlier calls on this device may have left
        _lib.read_tc_status(U.device)

    def _checked(out):
        if strict:
            if _lib.read_scan_status(U.device):
                raise ValueError("M has an entry of magnitude exactly 0: the chunked scan needs abs(M) > 0.")
            if _lib.read_tc_status(U.device):
                raise RuntimeError("v2x2ssd: a bounded wait inside a tensor-core kernel ran out; the outputs "
                                   "of the affected chunks are NaN.")
        return out

    if needs_grad:
        return _checked(_V2x2SSDFn.apply(Ua, Mf, Kf, Ba, Ca, initial_states, B_prev, U_prev, int(chunk_size),
                                         odtype, bool(return_state), residual))
    Y, final32, _, _ = _fwd_impl(Ua, Mf, Kf, Ba, Ca, _f32(initial_states), _f32(B_prev),
                                 _f32(U_prev), int(chunk_size))
    Y = Y.to(odtype)
    if not return_state:
        return _checked(Y)
    return _checked((Y, final32.to(odtype), B[:, :, -1, :].to(odtype).contiguous(),
                     U[:, :, -1, :].to(odtype).contiguous()))


__all__ = ["v2x2ssd_b200", "chunk_increment_b200", "state_passing_b200", "chunk_scan_b200"]
