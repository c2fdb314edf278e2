"""Mixer glue on B200: skip connection, ``(b,H,T,P) -> (b,T,H*P)`` re-layout and SiLU gate in one
pass each way (``SLinOSSMixer._apply_gate_skip``, slinoss/layers/mixer.py:585-599, which runs five
elementwise passes and a transposing copy in eager mode)."""

from __future__ import annotations

from ctypes import byref

import torch

from .. import _lib


class _GateSkipFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, u, gate, skip):
        b, H, T, P = map(int, y.shape)
        dev = y.device
        yd, ud = y.detach().contiguous(), u.detach().to(y.dtype).contiguous()
        gd = gate.detach().to(y.dtype)
        if gd.stride(2) != 1 or gd.stride(1) % 8 or gd.stride(0) % 8 or gd.data_ptr() % 16:
            gd = gd.contiguous()
        sk = skip.detach().to(torch.float32).contiguous()
        out = torch.empty((b, T, H * P), device=dev, dtype=y.dtype)
        s = _lib.GlueShape(b, T, H, P, _lib.dtype_code(y.dtype), int(gd.stride(1)), int(gd.stride(0)))
        with _lib.guard(dev):
            _lib.check(_lib.lib().slx_gate_skip_fwd(byref(s), yd.data_ptr(), ud.data_ptr(), gd.data_ptr(),
                                                    sk.data_ptr(), out.data_ptr(), _lib.stream_ptr(dev)),
                       "gate_skip forward")
        ctx.save_for_backward(yd, ud, gd, sk)
        ctx.dtypes = (u.dtype, gate.dtype, skip.dtype)
        return out

    @staticmethod
    def backward(ctx, d_out):
        yd, ud, gd, sk = ctx.saved_tensors
        b, H, T, P = map(int, yd.shape)
        dev = yd.device
        go = d_out.to(yd.dtype).contiguous()
        dy, du = torch.empty_like(yd), torch.empty_like(yd)
        dg = torch.empty((b, T, H * P), device=dev, dtype=yd.dtype)
        dsk = torch.empty((H * P,), device=dev, dtype=torch.float32)
        s = _lib.GlueShape(b, T, H, P, _lib.dtype_code(yd.dtype), int(gd.stride(1)), int(gd.stride(0)))
        L_ = _lib.lib()
        nbytes = int(L_.slx_gate_skip_bwd_workspace_bytes(byref(s)))
        ws = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)
        with _lib.guard(dev):
            _lib.check(L_.slx_gate_skip_bwd(byref(s), yd.data_ptr(), ud.data_ptr(), gd.data_ptr(), sk.data_ptr(),
                                            go.data_ptr(), dy.data_ptr(), du.data_ptr(), dg.data_ptr(),
                                            dsk.data_ptr(), ws.data_ptr(), nbytes, _lib.stream_ptr(dev)),
                       "gate_skip backward")
        u_dt, g_dt, s_dt = ctx.dtypes
        return dy, du.to(u_dt), dg.to(g_dt), dsk.to(s_dt)


@torch.compiler.disable
def gate_skip_b200(scan_y: torch.Tensor, scan_u: torch.Tensor, gate: torch.Tensor, skip: torch.Tensor) -> torch.Tensor:
    """``(scan_y + scan_u * skip)`` re-laid from ``(b,H,T,P)`` to ``(b,T,H*P)`` and multiplied by
    ``silu(gate)``; ``gate (b,T,H*P)`` may be a column slice of the input projection's output,
    ``skip (H*P,)``.  Differentiable in all four."""
    if scan_y.device.type != "cuda":
        raise ValueError("slinoss_b200 gate_skip requires CUDA tensors.")
    if scan_y.ndim != 4 or tuple(scan_u.shape) != tuple(scan_y.shape):
        raise ValueError(f"scan_y and scan_u must be (batch,heads,T,P) and equal. Got {tuple(scan_y.shape)}, "
                         f"{tuple(scan_u.shape)}.")
    b, H, T, P = map(int, scan_y.shape)
    if tuple(gate.shape) != (b, T, H * P):
        raise ValueError(f"gate must be {(b, T, H * P)}. Got {tuple(gate.shape)}.")
    if skip.numel() != H * P:
        raise ValueError(f"skip must have {H * P} entries. Got {tuple(skip.shape)}.")
    if P % 8 != 0:
        raise ValueError(f"head dim must be a multiple of 8. Got {P}.")
    _lib.same_device(scan_y, scan_u, gate, skip)
    if T == 0:
        return scan_y.new_empty((b, 0, H * P))
    return _GateSkipFn.apply(scan_y, scan_u, gate, skip.reshape(-1))


__all__ = ["gate_skip_b200"]
