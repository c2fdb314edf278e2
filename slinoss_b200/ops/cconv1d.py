"""Depthwise causal conv1d on B200 (channel-last, stride-aware).

``cconv1d_b200(x, weight, bias, conv_state)`` is the mixer-facing form
(slinoss/layers/mixer.py:456 ``_apply_cconv_cuda``): ``x (b,T,C)`` -- possibly a
column slice of the input projection -- and ``conv_state (b,C,W-1)`` give
``(y (b,T,C), next_state (b,C,W-1))``.  ``activation="silu"`` fuses the
activation the mixer applies next (mixer.py:562).
"""

from __future__ import annotations

from ctypes import byref
from typing import Optional, Tuple

import torch

from .. import _lib


def _conv_shape(x: torch.Tensor, C: int, W: int, silu: bool) -> _lib.ConvShape:
    b, T = int(x.shape[0]), int(x.shape[1])
    return _lib.ConvShape(b, T, C, W, _lib.dtype_code(x.dtype), 1 if silu else 0,
                          max(int(x.stride(1)), C), int(x.stride(0)))


def _dense_rows(x: torch.Tensor) -> torch.Tensor:
    """Keep a column slice of a wider matrix as it is; copy anything else."""
    ok = x.stride(2) == 1 and (x.shape[1] == 1 or x.stride(1) >= x.shape[2])
    return x if ok else x.contiguous()


class _CConv1dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, conv_state, silu):
        dev = x.device
        b, T, C = map(int, x.shape)
        W = int(weight.shape[1])
        xd = _dense_rows(x.detach())
        w = weight.detach().to(x.dtype).contiguous()
        bs = None if bias is None else bias.detach().to(x.dtype).contiguous()
        st = None if conv_state is None else conv_state.detach().to(x.dtype).contiguous()
        y = torch.empty((b, T, C), device=dev, dtype=x.dtype)
        nxt = torch.empty((b, C, W - 1), device=dev, dtype=x.dtype)
        s = _conv_shape(xd, C, W, silu)
        with _lib.guard(dev):
            _lib.check(_lib.lib().slx_cconv1d_fwd(byref(s), xd.data_ptr(), w.data_ptr(), _lib.ptr(bs),
                                                  _lib.ptr(st), y.data_ptr(), nxt.data_ptr(),
                                                  _lib.stream_ptr(dev)), "cconv1d forward")
        ctx.silu = silu
        ctx.has_bias = bias is not None
        ctx.has_state = conv_state is not None
        ctx.w_dtype = weight.dtype
        ctx.b_dtype = None if bias is None else bias.dtype
        ctx.s_dtype = None if conv_state is None else conv_state.dtype
        ctx.save_for_backward(xd, w, bs if bs is not None else w, st if st is not None else w)
        return y, nxt

    @staticmethod
    def backward(ctx, dy, d_next):
        xd, w, bs, st = ctx.saved_tensors
        if not ctx.has_bias:
            bs = None
        if not ctx.has_state:
            st = None
        dev = xd.device
        b, T, C = map(int, xd.shape)
        W = int(w.shape[1])
        dyc = (torch.zeros((b, T, C), device=dev, dtype=xd.dtype) if dy is None
               else dy.to(xd.dtype).contiguous())
        dn = None if d_next is None else d_next.to(xd.dtype).contiguous()
        dx = torch.empty((b, T, C), device=dev, dtype=xd.dtype)
        dw = torch.empty((C, W), device=dev, dtype=torch.float32)
        db = torch.empty((C,), device=dev, dtype=torch.float32)
        dst = torch.empty((b, C, W - 1), device=dev, dtype=torch.float32) if ctx.has_state else None
        s = _conv_shape(xd, C, W, ctx.silu)
        L_ = _lib.lib()
        nbytes = int(L_.slx_cconv1d_bwd_workspace_bytes(byref(s)))
        ws = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)
        with _lib.guard(dev):
            _lib.check(L_.slx_cconv1d_bwd(byref(s), xd.data_ptr(), w.data_ptr(), _lib.ptr(bs), _lib.ptr(st),
                                          dyc.data_ptr(), _lib.ptr(dn), dx.data_ptr(), dw.data_ptr(),
                                          db.data_ptr(), _lib.ptr(dst), ws.data_ptr(), nbytes,
                                          _lib.stream_ptr(dev)), "cconv1d backward")
        return (dx, dw.to(ctx.w_dtype), db.to(ctx.b_dtype) if ctx.has_bias else None,
                dst.to(ctx.s_dtype) if ctx.has_state else None, None)


@torch.compiler.disable
def cconv1d_b200(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 conv_state: Optional[torch.Tensor] = None, *,
                 activation: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    if x.device.type != "cuda":
        raise ValueError("slinoss_b200 cconv1d requires CUDA tensors.")
    if x.ndim != 3:
        raise ValueError(f"x must be (batch, T, channels). Got {tuple(x.shape)}.")
    b, T, C = map(int, x.shape)
    if weight.ndim != 2 or int(weight.shape[0]) != C:
        raise ValueError(f"weight must be ({C}, width). Got {tuple(weight.shape)}.")
    W = int(weight.shape[1])
    if W not in (2, 3, 4):
        raise ValueError(f"conv width must be 2, 3 or 4. Got {W}.")
    if conv_state is not None and tuple(conv_state.shape) != (b, C, W - 1):
        raise ValueError(f"conv_state must be {(b, C, W - 1)}. Got {tuple(conv_state.shape)}.")
    if T == 0:
        nxt = (torch.zeros((b, C, W - 1), device=x.device, dtype=x.dtype) if conv_state is None
               else conv_state.to(x.dtype))
        return x.new_empty((b, 0, C)), nxt
    return _CConv1dFn.apply(x, weight, bias, conv_state, activation in ("silu", "swish"))


@torch.no_grad()
def cconv1d_update_b200(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                        conv_state: Optional[torch.Tensor] = None, *, activation: Optional[str] = None,
                        inplace: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """One decode token of the depthwise causal conv: the contract of the reference's
    ``causal_conv1d_update`` as ``SLinOSSMixer._apply_causal_depthwise_conv_step`` uses it
    (slinoss/layers/mixer.py:614-676).  ``x (b, C)`` -- possibly a column slice of the input
    projection's one-token output -- and the rolling ``conv_state (b, C, W-1)`` give
    ``(y (b, C), next_state (b, C, W-1))`` with ``y = act(bias + w . [state, x])`` and
    ``next_state = [state[..., 1:], x]``.  ``inplace=True`` rolls ``conv_state`` in place and returns
    it (it must then be contiguous and of ``x``'s dtype).  Inference only (no autograd)."""
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    if x.device.type != "cuda":
        raise ValueError("slinoss_b200 cconv1d requires CUDA tensors.")
    if x.ndim != 2:
        raise ValueError(f"x must be (batch, channels). Got {tuple(x.shape)}.")
    b, C = map(int, x.shape)
    if weight.ndim != 2 or int(weight.shape[0]) != C:
        raise ValueError(f"weight must be ({C}, width). Got {tuple(weight.shape)}.")
    W = int(weight.shape[1])
    if W not in (2, 3, 4):
        raise ValueError(f"conv width must be 2, 3 or 4. Got {W}.")
    if conv_state is not None and tuple(conv_state.shape) != (b, C, W - 1):
        raise ValueError(f"conv_state must be {(b, C, W - 1)}. Got {tuple(conv_state.shape)}.")
    dev = _lib.same_device(x, weight, bias, conv_state)
    if x.stride(1) != 1:
        x = x.contiguous()
    w = weight.to(x.dtype).contiguous()
    bs = None if bias is None else bias.to(x.dtype).contiguous()
    if inplace:
        if conv_state is None or conv_state.dtype != x.dtype or not conv_state.is_contiguous():
            raise ValueError("inplace=True needs a contiguous conv_state of x's dtype.")
        st, nxt = conv_state, conv_state
    else:
        st = None if conv_state is None else conv_state.to(x.dtype).contiguous()
        nxt = torch.empty((b, C, W - 1), device=dev, dtype=x.dtype)
    y = torch.empty((b, C), device=dev, dtype=x.dtype)
    s = _lib.ConvShape(b, 1, C, W, _lib.dtype_code(x.dtype), 1 if activation in ("silu", "swish") else 0,
                       C, int(x.stride(0)))
    with _lib.guard(dev):
        _lib.check(_lib.lib().slx_cconv1d_update(byref(s), x.data_ptr(), w.data_ptr(), _lib.ptr(bs), _lib.ptr(st),
                                                 y.data_ptr(), nxt.data_ptr(), _lib.stream_ptr(dev)),
                   "cconv1d update")
    return y, nxt


__all__ = ["cconv1d_b200", "cconv1d_update_b200"]
