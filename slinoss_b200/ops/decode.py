"""One-token mixer decode step on B200 (inference only).

``mixer_decode_step_b200`` follows the keyword list and return values of the reference's
``mixer_decode_step_cute`` (slinoss/ops/v2x2ssd/cute/decode.py:117-149) without its shape
limits (P = 64, N = 64, batch in {1,2,4,8,16}); the arithmetic is
``SLinOSSMixer._decode_step_reference`` (slinoss/layers/mixer.py:714-748).  The carried
state is kept in fp32; passing ``final_state_out=initial_states`` (and likewise
``b_last_out`` / ``u_last_out``) updates a ``ScanState`` in place.
"""

from __future__ import annotations

from ctypes import byref
from typing import Optional, Tuple

import torch

from .. import _lib
from .scanprep import _flat_bias

_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _like(name: str, t: torch.Tensor, shape, dtype, device) -> torch.Tensor:
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must be {tuple(shape)}. Got {tuple(t.shape)}.")
    if t.device != device:
        raise ValueError(f"{name} must be on {device}.")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}. Got {t.dtype}.")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous; got strides {t.stride()}.")
    return t


@torch.compiler.disable
@torch.no_grad()
def mixer_decode_step_b200(value, params, bc, gate, skip, *, initial_states=None, B_prev=None,
                           U_prev=None, dt_min: float, dt_max: float, r_min: float, r_max: float,
                           theta_bound: float, k_max: float, eps: float, dt_bias, gamma_bias,
                           omega_bias, mix_r_bias, mix_theta_bias, mix_k_prev_bias, mix_k_curr_bias,
                           b_scale: Optional[torch.Tensor] = None,
                           c_scale: Optional[torch.Tensor] = None, normalize_bc: bool = True,
                           output_dtype: Optional[torch.dtype] = None,
                           final_state_out: Optional[torch.Tensor] = None,
                           b_last_out: Optional[torch.Tensor] = None,
                           u_last_out: Optional[torch.Tensor] = None
                           ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``value, gate (b,H,P)``, ``params (b,H,13)``, ``bc (b,H,4,N)``, ``skip (H,P)`` ->
    ``(gated (b, H*P), final_state (b,H,P,2N) fp32, b_last (b,H,2N), u_last (b,H,P))``."""
    if value.device.type != "cuda":
        raise ValueError("slinoss_b200 decode step requires CUDA tensors.")
    if value.ndim != 3:
        raise ValueError(f"value must be (batch, heads, P). Got {tuple(value.shape)}.")
    dev, dt = value.device, value.dtype
    if dt not in _DTYPES:
        raise TypeError(f"value must be float32, bfloat16 or float16. Got {dt}.")
    if output_dtype is not None and output_dtype != dt:
        raise TypeError("the decode step writes its output in the dtype of value.")
    b, H, P = map(int, value.shape)
    if bc.ndim != 4 or tuple(bc.shape[:3]) != (b, H, 4):
        raise ValueError(f"bc must be (batch, heads, 4, N). Got {tuple(bc.shape)}.")
    N = int(bc.shape[-1])
    value = _like("value", value, (b, H, P), dt, dev)
    params = _like("params", params, (b, H, 13), dt, dev)
    bc = _like("bc", bc, (b, H, 4, N), dt, dev)
    gate = _like("gate", gate, (b, H, P), dt, dev)
    skip = skip.detach().reshape(H, P).to(device=dev, dtype=dt).contiguous()
    if normalize_bc and (b_scale is None or c_scale is None):
        raise ValueError("b_scale and c_scale are required when normalize_bc is set.")
    if (B_prev is None) != (U_prev is None):
        raise ValueError("B_prev and U_prev must be passed together (or both omitted).")
    bias = _flat_bias(H, (dt_bias, gamma_bias, omega_bias, mix_r_bias, mix_theta_bias, mix_k_prev_bias,
                          mix_k_curr_bias), dev)
    scale = None
    if normalize_bc:
        scale = torch.cat((b_scale.detach(), c_scale.detach()), dim=1).to(torch.float32).contiguous()
    state_in = None
    if initial_states is not None:
        state_in = _like("initial_states", initial_states, (b, H, P, 2 * N), None, dev)
        if state_in.dtype != torch.float32:
            state_in = state_in.to(torch.float32)
    if B_prev is not None:
        B_prev = _like("B_prev", B_prev, (b, H, 2 * N), None, dev).to(dt)
        U_prev = _like("U_prev", U_prev, (b, H, P), None, dev).to(dt)
    state_out = (torch.empty((b, H, P, 2 * N), device=dev, dtype=torch.float32) if final_state_out is None
                 else _like("final_state_out", final_state_out, (b, H, P, 2 * N), torch.float32, dev))
    b_last = (torch.empty((b, H, 2 * N), device=dev, dtype=dt) if b_last_out is None
              else _like("b_last_out", b_last_out, (b, H, 2 * N), dt, dev))
    u_last = (torch.empty((b, H, P), device=dev, dtype=dt) if u_last_out is None
              else _like("u_last_out", u_last_out, (b, H, P), dt, dev))
    out = torch.empty((b, H * P), device=dev, dtype=dt)
    s = _lib.DecodeShape(b, H, P, N, _lib.dtype_code(dt), 1 if normalize_bc else 0, float(dt_min),
                         float(dt_max), float(r_min), float(r_max), float(theta_bound), float(k_max),
                         float(eps))
    with _lib.guard(dev):
        _lib.check(_lib.lib().slx_decode_step(
            byref(s), value.data_ptr(), params.data_ptr(), bc.data_ptr(), gate.data_ptr(), skip.data_ptr(),
            bias.data_ptr(), _lib.ptr(scale), _lib.ptr(state_in), _lib.ptr(B_prev), _lib.ptr(U_prev),
            out.data_ptr(), state_out.data_ptr(), b_last.data_ptr(), u_last.data_ptr(),
            _lib.stream_ptr(dev)), "decode step")
    return out, state_out, b_last, u_last


__all__ = ["mixer_decode_step_b200"]
