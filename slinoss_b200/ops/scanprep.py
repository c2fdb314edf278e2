"""SLinOSSScanPrep on B200: ``(value, params, bc) -> (U, M, K, B, C)``.

``scanprep_b200`` has the argument list of the reference's ``scanprep_cute``
(slinoss/ops/scanprep/cute/api.py:10) and the results of
``SLinOSSScanPrep._prepare_inputs_reference`` (slinoss/layers/scanprep.py:351).
Inputs may be column slices of the mixer's input projection (only the last
dimension has to be dense); nothing is copied on the host side.
"""

from __future__ import annotations

from ctypes import byref
from typing import Optional

import torch

from .. import _lib
from ..types import ScanInputs

PARAM_DIM = 13
BIAS_SLOTS = (0, 1, 2, 5, 6, 7, 8)  # slinoss/layers/scanprep.py:187-206


def _rows_view(x: torch.Tensor, width: int):
    """(tensor, row stride in elements) of a (b, T, width) tensor whose rows are dense
    and equally spaced over (b, T); copies only when they are not."""
    b, T = int(x.shape[0]), int(x.shape[1])
    if x.stride(2) != 1 or x.stride(1) < width or (b > 1 and x.stride(0) != T * x.stride(1)):
        x = x.contiguous()
    return x, int(x.stride(1))


def _flat_bias(n_heads: int, biases, device) -> torch.Tensor:
    out = torch.zeros((n_heads, PARAM_DIM), device=device, dtype=torch.float32)
    for slot, t in zip(BIAS_SLOTS, biases):
        out[:, slot] = t.detach().to(torch.float32)
    return out


def _prep_shape(value, params, bc, n_heads, d_state, d_head, normalize_bc, hp, vs, ps, bs):
    b, T = int(value.shape[0]), int(value.shape[1])
    return _lib.PrepShape(b, T, n_heads, d_head, d_state, _lib.dtype_code(value.dtype),
                          1 if normalize_bc else 0, hp["dt_min"], hp["dt_max"], hp["r_min"],
                          hp["r_max"], hp["theta_bound"], hp["k_max"], hp["eps"], vs, ps, bs)


class _ScanPrepFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, value, params, bc, dt_bias, gamma_bias, omega_bias, mix_r_bias,
                mix_theta_bias, mix_k_prev_bias, mix_k_curr_bias, b_scale, c_scale, meta):
        n_heads, d_state, d_head, normalize_bc, hp = meta
        dev = value.device
        b, T = int(value.shape[0]), int(value.shape[1])
        v, vs = _rows_view(value.detach(), n_heads * d_head)
        p, ps = _rows_view(params.detach(), n_heads * PARAM_DIM)
        c, bs = _rows_view(bc.detach().reshape(b, T, n_heads * 4 * d_state), n_heads * 4 * d_state)
        bias = _flat_bias(n_heads, (dt_bias, gamma_bias, omega_bias, mix_r_bias, mix_theta_bias,
                                    mix_k_prev_bias, mix_k_curr_bias), dev)
        scale = None
        if normalize_bc:
            scale = torch.cat((b_scale.detach(), c_scale.detach()), dim=1).to(torch.float32).contiguous()
        s = _prep_shape(v, p, c, n_heads, d_state, d_head, normalize_bc, hp, vs, ps, bs)
        dt = value.dtype
        U = torch.empty((b, n_heads, T, d_head), device=dev, dtype=dt)
        Bo = torch.empty((b, n_heads, T, 2 * d_state), device=dev, dtype=dt)
        Co = torch.empty_like(Bo)
        M = torch.empty((b, n_heads, T, 2), device=dev, dtype=torch.float32)
        K = torch.empty((b, n_heads, T, 2, 2), device=dev, dtype=torch.float32)
        with _lib.guard(dev):
            _lib.check(_lib.lib().slx_scanprep_fwd(
                byref(s), v.data_ptr(), p.data_ptr(), c.data_ptr(), bias.data_ptr(), _lib.ptr(scale),
                U.data_ptr(), M.data_ptr(), K.data_ptr(), Bo.data_ptr(), Co.data_ptr(),
                _lib.stream_ptr(dev)), "scanprep forward")
        ctx.meta = meta
        ctx.has_scale = scale is not None
        ctx.bias_dtypes = [t.dtype for t in (dt_bias, gamma_bias, omega_bias, mix_r_bias,
                                             mix_theta_bias, mix_k_prev_bias, mix_k_curr_bias)]
        ctx.scale_dtypes = (None if b_scale is None else b_scale.dtype,
                            None if c_scale is None else c_scale.dtype)
        ctx.bc_shape = tuple(bc.shape)
        ctx.strides = (ps, bs)
        ctx.save_for_backward(p, c, bias, scale if scale is not None else bias)
        return U, M, K, Bo, Co

    @staticmethod
    def backward(ctx, dU, dM, dK, dB, dC):
        n_heads, d_state, d_head, normalize_bc, hp = ctx.meta
        p, c, bias, scale = ctx.saved_tensors
        if not ctx.has_scale:
            scale = None
        dev = p.device
        b, T = int(p.shape[0]), int(p.shape[1])
        dt = p.dtype

        def z(g, shape, dtype):
            return torch.zeros(shape, device=dev, dtype=dtype) if g is None else g.to(dtype).contiguous()

        dU = z(dU, (b, n_heads, T, d_head), dt)
        dB = z(dB, (b, n_heads, T, 2 * d_state), dt)
        dC = z(dC, (b, n_heads, T, 2 * d_state), dt)
        dM = z(dM, (b, n_heads, T, 2), torch.float32)
        dK = z(dK, (b, n_heads, T, 2, 2), torch.float32)
        ps, bs = ctx.strides
        s = _prep_shape(p, p, c, n_heads, d_state, d_head, normalize_bc, hp, n_heads * d_head, ps, bs)
        d_value = torch.empty((b, T, n_heads * d_head), device=dev, dtype=dt)
        d_params = torch.empty((b, T, n_heads * PARAM_DIM), device=dev, dtype=dt)
        d_bc = torch.empty((b, T, n_heads * 4 * d_state), device=dev, dtype=dt)
        d_bias = torch.empty((n_heads, PARAM_DIM), device=dev, dtype=torch.float32)
        d_scale = (torch.empty((n_heads, 4, d_state), device=dev, dtype=torch.float32)
                   if scale is not None else None)
        L_ = _lib.lib()
        nbytes = int(L_.slx_scanprep_bwd_workspace_bytes(byref(s)))
        ws = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)
        with _lib.guard(dev):
            _lib.check(L_.slx_scanprep_bwd(
                byref(s), p.data_ptr(), c.data_ptr(), bias.data_ptr(), _lib.ptr(scale), dU.data_ptr(),
                dM.data_ptr(), dK.data_ptr(), dB.data_ptr(), dC.data_ptr(), d_value.data_ptr(),
                d_params.data_ptr(), d_bc.data_ptr(), d_bias.data_ptr(), _lib.ptr(d_scale),
                ws.data_ptr(), nbytes, _lib.stream_ptr(dev)), "scanprep backward")
        gb = [d_bias[:, slot].to(dtp) for slot, dtp in zip(BIAS_SLOTS, ctx.bias_dtypes)]
        gbs = gcs = None
        if d_scale is not None:
            gbs = d_scale[:, :2].to(ctx.scale_dtypes[0]).contiguous()
            gcs = d_scale[:, 2:].to(ctx.scale_dtypes[1]).contiguous()
        return (d_value, d_params, d_bc.view(ctx.bc_shape), *gb, gbs, gcs, None)


@torch.compiler.disable
def scanprep_b200(value, params, bc, *, n_heads: int, d_state: int, d_head: int,
                  normalize_bc: bool = True, dt_min: float, dt_max: float, r_min: float,
                  r_max: float, theta_bound: float, k_max: float, eps: float, dt_bias, gamma_bias,
                  omega_bias, mix_r_bias, mix_theta_bias, mix_k_prev_bias, mix_k_curr_bias,
                  b_scale: Optional[torch.Tensor] = None,
                  c_scale: Optional[torch.Tensor] = None) -> ScanInputs:
    """Same keyword list as ``scanprep_cute`` (scanprep.py:359-384 shows the call)."""
    for name, t in (("value", value), ("params", params), ("bc", bc)):
        if t.device.type != "cuda":
            raise ValueError(f"slinoss_b200 scanprep requires CUDA tensors ({name} is on {t.device}).")
    if value.ndim != 3 or value.shape[-1] != n_heads * d_head:
        raise ValueError(f"value must be (batch, T, {n_heads * d_head}). Got {tuple(value.shape)}.")
    b, T = int(value.shape[0]), int(value.shape[1])
    if params.ndim != 3 or tuple(params.shape) != (b, T, n_heads * PARAM_DIM):
        raise ValueError(f"params must be (batch, T, {n_heads * PARAM_DIM}). Got {tuple(params.shape)}.")
    if bc.ndim != 5 or tuple(bc.shape) != (b, T, n_heads, 4, d_state):
        raise ValueError(f"bc must be (batch, T, heads, 4, d_state). Got {tuple(bc.shape)}.")
    if not (value.dtype == params.dtype == bc.dtype):
        raise TypeError("value, params and bc must share one dtype.")
    if normalize_bc and (b_scale is None or c_scale is None):
        raise ValueError("b_scale and c_scale are required when normalize_bc is set.")
    if T == 0:
        dev, dt = value.device, value.dtype
        return ScanInputs(U=torch.empty((b, n_heads, 0, d_head), device=dev, dtype=dt),
                          M=torch.empty((b, n_heads, 0, 2), device=dev, dtype=torch.float32),
                          K=torch.empty((b, n_heads, 0, 2, 2), device=dev, dtype=torch.float32),
                          B=torch.empty((b, n_heads, 0, 2 * d_state), device=dev, dtype=dt),
                          C=torch.empty((b, n_heads, 0, 2 * d_state), device=dev, dtype=dt))
    hp = dict(dt_min=float(dt_min), dt_max=float(dt_max), r_min=float(r_min), r_max=float(r_max),
              theta_bound=float(theta_bound), k_max=float(k_max), eps=float(eps))
    meta = (int(n_heads), int(d_state), int(d_head), bool(normalize_bc), hp)
    U, M, K, Bo, Co = _ScanPrepFn.apply(value, params, bc, dt_bias, gamma_bias, omega_bias,
                                        mix_r_bias, mix_theta_bias, mix_k_prev_bias,
                                        mix_k_curr_bias, b_scale, c_scale, meta)
    return ScanInputs(U=U, M=M, K=K, B=Bo, C=Co)


__all__ = ["scanprep_b200"]
