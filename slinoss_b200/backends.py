"""Drop-in backends for the reference's ``SLinOSSMixer`` backend switch.

Each class implements the matching Protocol of slinoss/layers/backend.py
(``ScanBackend`` :238, ``ScanPrepBackend`` :114, ``CConv1dBackend`` :174,
``MixerDecodeBackend`` :251) and is handed to the mixer through its constructor:

    SLinOSSMixer(..., backend=B200ScanBackend(), scanprep_backend=B200ScanPrepBackend(),
                 cconv_backend=B200CConv1dBackend(), decode_backend=B200MixerDecodeBackend())

The classes accept the reference's own ``ScanInputs`` / ``ScanPrepInputs`` /
``ScanState`` objects (only attributes are read) and return this package's
mirror types, which expose the same attributes.
"""

from __future__ import annotations

import types
from typing import Optional, Tuple, Union

import torch

from .ops.cconv1d import cconv1d_b200, cconv1d_update_b200
from .ops.decode import mixer_decode_step_b200
from .ops.glue import gate_skip_b200
from .ops.scanprep import scanprep_b200
from .ops.v2x2ssd import v2x2ssd_b200
from .types import ScanInputs, ScanState


def _default_compute_dtype(dtype: torch.dtype) -> Optional[torch.dtype]:
    # slinoss/layers/backend.py:271-274
    return torch.float32 if dtype in (torch.float16, torch.bfloat16) else None


class B200ScanBackend:
    """``ScanBackend`` running the sm_100a chunked scan (cf. ``CuteScanBackend``,
    backend.py:318-377)."""

    def __init__(self, *, compute_dtype: Optional[torch.dtype] = None, state_cls=ScanState) -> None:
        self.compute_dtype = compute_dtype
        self.state_cls = state_cls

    def __call__(self, inputs, *, chunk_size: int, state=None,
                 return_state: Optional[bool] = None) -> Union[torch.Tensor, Tuple[torch.Tensor, ScanState]]:
        if return_state is None:
            return_state = state is not None
        st = self.state_cls() if state is None else state
        odt = inputs.U.dtype
        cdt = self.compute_dtype if self.compute_dtype is not None else _default_compute_dtype(odt)
        out = v2x2ssd_b200(inputs.U, inputs.M, inputs.K, inputs.B, inputs.C, chunk_size=chunk_size,
                           initial_states=st.state, B_prev=st.b_prev, U_prev=st.u_prev,
                           compute_dtype=cdt, output_dtype=odt, return_state=bool(return_state))
        if not return_state:
            return out
        y, final_state, b_last, u_last = out
        return y, self.state_cls(state=final_state, b_prev=b_last, u_prev=u_last)


class B200ScanPrepBackend:
    """``ScanPrepBackend``: ``owner`` is the ``SLinOSSScanPrep`` module whose
    hyper-parameters and parameters are read (cf. scanprep.py:359-384)."""

    def __init__(self, inputs_cls=ScanInputs) -> None:
        self.inputs_cls = inputs_cls

    def __call__(self, owner, inputs):
        out = scanprep_b200(
            inputs.value, inputs.params, inputs.bc, n_heads=owner.n_heads, d_state=owner.d_state,
            d_head=owner.d_head, normalize_bc=owner.normalize_bc, dt_min=owner.dt_min,
            dt_max=owner.dt_max, r_min=owner.r_min, r_max=owner.r_max, theta_bound=owner.theta_bound,
            k_max=owner.k_max, eps=owner.eps, dt_bias=owner.dt_bias, gamma_bias=owner.gamma_bias,
            omega_bias=owner.omega_bias, mix_r_bias=owner.mix_r_bias,
            mix_theta_bias=owner.mix_theta_bias, mix_k_prev_bias=owner.mix_k_prev_bias,
            mix_k_curr_bias=owner.mix_k_curr_bias, b_scale=owner.b_scale, c_scale=owner.c_scale)
        if self.inputs_cls is ScanInputs:
            return out
        return self.inputs_cls(U=out.U, M=out.M, K=out.K, B=out.B, C=out.C)


class B200CConv1dBackend:
    """``CConv1dBackend``: ``owner`` is the mixer (``dw_weight (C,W)``, ``dw_bias (C)``,
    ``d_conv``); returns ``(y (b,T,C), next_state (b,C,W-1))`` like
    mixer.py:420-454.  Width-1 convolutions are not a kernel case."""

    def __call__(self, owner, x: torch.Tensor, conv_state: Optional[torch.Tensor]):
        if int(owner.d_conv) < 2:
            raise ValueError("B200CConv1dBackend needs d_conv in {2,3,4}.")
        return cconv1d_b200(x, owner.dw_weight, owner.dw_bias, conv_state)


class B200MixerDecodeBackend:
    """``MixerDecodeBackend`` (backend.py:251-268): one token through scan prep, one recurrence
    step, skip and gate.  ``owner`` is the mixer: ``owner.scanprep`` carries the prep parameters
    and hyper-parameters (read as in mixer.py:758-782), ``inputs`` is a ``MixerDecodeInputs``
    (``value, params, bc, gate, skip``), ``state`` a ``ScanState`` whose tensors are updated in
    place when they have the layout the kernel writes (fp32 state, activation-dtype rows)."""

    def __init__(self, *, state_cls=ScanState) -> None:
        self.state_cls = state_cls

    def supports(self, owner, *, batch_size: int, device: torch.device, dtype: torch.dtype) -> bool:
        del batch_size
        return (device.type == "cuda" and dtype in (torch.float32, torch.bfloat16, torch.float16)
                and int(owner.d_state) % 2 == 0 and getattr(owner, "output_norm", None) is None)

    def __call__(self, owner, inputs, state):
        sp = owner.scanprep
        v = inputs.value
        b, H, P = map(int, v.shape)
        N = int(inputs.bc.shape[-1])

        def reuse(t, shape, dtype):
            ok = (t is not None and tuple(t.shape) == shape and t.dtype == dtype and t.is_contiguous()
                  and t.device == v.device)
            return t if ok else None

        gated, fin, b_last, u_last = mixer_decode_step_b200(
            v.contiguous(), inputs.params.contiguous(), inputs.bc.contiguous(), inputs.gate.contiguous(),
            inputs.skip, initial_states=state.state, B_prev=state.b_prev, U_prev=state.u_prev,
            dt_min=sp.dt_min, dt_max=sp.dt_max, r_min=sp.r_min, r_max=sp.r_max, theta_bound=sp.theta_bound,
            k_max=sp.k_max, eps=sp.eps, dt_bias=sp.dt_bias, gamma_bias=sp.gamma_bias, omega_bias=sp.omega_bias,
            mix_r_bias=sp.mix_r_bias, mix_theta_bias=sp.mix_theta_bias, mix_k_prev_bias=sp.mix_k_prev_bias,
            mix_k_curr_bias=sp.mix_k_curr_bias, b_scale=getattr(sp, "b_scale", None),
            c_scale=getattr(sp, "c_scale", None), normalize_bc=bool(getattr(sp, "normalize_bc", True)),
            final_state_out=reuse(state.state, (b, H, P, 2 * N), torch.float32),
            b_last_out=reuse(state.b_prev, (b, H, 2 * N), v.dtype),
            u_last_out=reuse(state.u_prev, (b, H, P), v.dtype))
        return gated, self.state_cls(state=fin, b_prev=b_last, u_prev=u_last)


def _conv_step_b200(self, value_raw: torch.Tensor, conv_state: Optional[torch.Tensor]):
    """Replacement for ``SLinOSSMixer._apply_causal_depthwise_conv_step`` (mixer.py:614-676): the
    conv half of a decode token (conv + SiLU, rolling state) in one ``slx_cconv1d_update`` launch.
    The reference reaches its vendored ``causal_conv1d_update`` directly there, not through a
    backend object, so the method itself is replaced on the instance."""
    if value_raw.ndim != 2 or value_raw.shape[-1] != self.d_inner:
        raise ValueError(f"Expected value_raw shape (batch, {self.d_inner}), got {tuple(value_raw.shape)}.")
    state_len = max(int(self.d_conv) - 1, 0)
    if state_len == 0 or value_raw.device.type != "cuda":
        return type(self)._apply_causal_depthwise_conv_step(self, value_raw, conv_state)
    init = self._validate_conv_state(conv_state, batch=int(value_raw.shape[0]), state_len=state_len,
                                     device=value_raw.device, dtype=value_raw.dtype)
    return cconv1d_update_b200(value_raw, self.dw_weight, self.dw_bias, init, activation="silu")


def _mixer_forward_fused(self, x: torch.Tensor, *, state=None, return_state: bool = False):
    """``SLinOSSMixer.forward`` (mixer.py:534-583) with the elementwise glue folded into the kernels on
    either side of it: the SiLU after the conv (mixer.py:562) runs in the conv kernel's epilogue
    (``activation="silu"``), and skip, re-layout and gate (``_apply_gate_skip``, mixer.py:585-599) run
    as one pass (``gate_skip_b200``).  Same arguments, results and state handling as the original;
    installed on a mixer instance by ``use_b200_backends(..., fuse_glue=True)``."""
    if x.ndim != 3 or x.shape[-1] != self.d_model:
        raise ValueError(f"Expected x shape (batch, T, {self.d_model}), got {tuple(x.shape)}.")
    batch, T, _ = map(int, x.shape)
    if T == 0 or x.device.type != "cuda" or int(self.d_conv) < 2 or int(self.d_head) % 8 != 0:
        return type(self).forward(self, x, state=state, return_state=return_state)
    proj = self.in_proj(x)
    gate, value_raw, params, bc_flat = torch.split(
        proj, [self.d_inner, self.d_inner, self.param_proj_dim, self.bc_proj_dim], dim=-1)
    conv_state_in = None if state is None else state.conv
    if conv_state_in is not None:
        conv_state_in = self._validate_conv_state(conv_state_in, batch=batch, state_len=int(self.d_conv) - 1,
                                                  device=x.device, dtype=value_raw.dtype)
    value, conv_state = cconv1d_b200(value_raw, self.dw_weight, self.dw_bias, conv_state_in, activation="silu")
    bc = self._reshape_bc(bc_flat, batch, T)
    scan_inputs = self._build_scan_inputs(value=value, params=params, bc=bc)
    scan_state_in = None if state is None else state.scan
    scan_result = self._run_scan_backend(scan_inputs, scan_state_in, return_state)
    scan_y, scan_state = scan_result if return_state else (scan_result, None)
    gated = gate_skip_b200(scan_y, scan_inputs.U, gate, self.skip)
    if self.output_norm is not None:
        gated = self.output_norm(gated)
    out = self.out_proj(gated)
    if not return_state:
        return out
    return out, _mixer_state(conv_state, scan_state)


def _mixer_state(conv_state, scan_state):
    from slinoss.layers.state import SLinOSSMixerState

    return SLinOSSMixerState(conv=conv_state, scan=scan_state)


def _padded_linear_forward(self, x: torch.Tensor) -> torch.Tensor:
    """``nn.Linear.forward`` for a projection whose output width is not a multiple of 8 half values
    (e.g. the mixer's input projection at d_model 768, 12 heads, d_state 64: 2*768 + 12*13 + 4*12*64 =
    4764).  With such a width every row of the output starts on an odd 8-byte boundary, the library GEMM
    falls back to its 4-byte-aligned kernels (measured 0.46 ms against 0.13 ms per product at 16384 x 768 x
    4764, bf16) and every consumer of the row slices loses its 16-byte accesses.  The weight is padded with
    zero rows to the next multiple of 8 for the product (a 7 MB copy per call) and the extra columns are
    sliced off again: same values, rows 16-byte aligned.  The parameters themselves are untouched."""
    pad = (-int(self.out_features)) % 8
    if pad == 0 or x.device.type != "cuda" or x.dtype == torch.float32:
        return torch.nn.functional.linear(x, self.weight, self.bias)
    w = torch.nn.functional.pad(self.weight, (0, 0, 0, pad))
    b = None if self.bias is None else torch.nn.functional.pad(self.bias, (0, pad))
    return torch.nn.functional.linear(x, w, b)[..., : self.out_features]


def use_b200_backends(model, *, decode_conv: bool = True, fuse_glue: bool = False,
                      align_projection: bool = True) -> int:
    """Point every ``SLinOSSMixer`` inside ``model`` (a mixer, a block, a whole ``NextCharLM``) at
    the four B200 backends, the way the reference's own workload builder swaps backends
    (scripts/perf/_nextchar.py:101-127: ``module.backend``, ``module.scanprep.backend``,
    ``module.cconv_backend``, ``module.decode_backend``).  With ``decode_conv`` the one-token conv
    step of each mixer (not behind a backend object in the reference) is replaced as well; with
    ``fuse_glue`` each mixer's ``forward`` is replaced by ``_mixer_forward_fused`` (same results; the
    SiLU after the conv and the skip / re-layout / gate pass run inside kernels); with
    ``align_projection`` an input projection whose width is not a multiple of 8 runs its product on a
    zero-padded weight (``_padded_linear_forward``).  The
    reference package must be importable; its own ``ScanInputs`` / ``ScanState`` classes are used
    for the values handed back to the mixer.  Returns the number of mixers switched."""
    from slinoss.layers import SLinOSSMixer
    from slinoss.layers.backend import ScanInputs as RefScanInputs
    from slinoss.layers.state import ScanState as RefScanState

    scan = B200ScanBackend(state_cls=RefScanState)
    prep = B200ScanPrepBackend(inputs_cls=RefScanInputs)
    conv = B200CConv1dBackend()
    dec = B200MixerDecodeBackend(state_cls=RefScanState)
    n = 0
    for module in model.modules():
        if isinstance(module, SLinOSSMixer):
            module.backend = scan
            module.scanprep.backend = prep
            module.cconv_backend = conv
            module.decode_backend = dec
            if decode_conv:
                module._apply_causal_depthwise_conv_step = types.MethodType(_conv_step_b200, module)
            if fuse_glue:
                module.forward = types.MethodType(_mixer_forward_fused, module)
            if align_projection and int(module.in_proj.out_features) % 8 != 0:
                module.in_proj.forward = types.MethodType(_padded_linear_forward, module.in_proj)
            n += 1
    return n


__all__ = ["B200ScanBackend", "B200ScanPrepBackend", "B200CConv1dBackend", "B200MixerDecodeBackend",
           "use_b200_backends"]
