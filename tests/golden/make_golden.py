"""Generate the golden fixtures in this directory from the reference.

Run in a container that has the reference checked out (it is imported, never
copied):

    PYTHONPATH=/path/to/reference python tests/golden/make_golden.py

The fixtures pin the CPU oracle (oracle/) and are compared directly with the
CUDA path in the GPU tests; the GPU box never needs the reference itself.

Fixtures
--------
scan_small_f64.npz   tiny ragged case (T not a multiple of the chunk), streaming
                     inputs + initial state, float64 compute: forward, the three
                     stage outputs, and all eight gradients.
scan_cfg0_f32.npz    b2 H4 T256 P32 N16 chunk 64, fp32, scan inputs produced by
                     a seeded default-init SLinOSSScanPrep from N(0,1)
                     activations; forward + gradients (seeded dY).
scan_bf16.npz        b1 H2 T192 P64 N32 chunk 64, bf16 inputs / fp32 compute.
prep_f32.npz         SLinOSSScanPrep forward + gradients incl. all parameters.
conv_f64.npz         depthwise causal conv (width 4 and 2), with/without state.
decode_f32.npz       one-token mixer decode step (SLinOSSMixer._decode_step_reference):
                     scan prep of one token, one recurrence step from a carried
                     state, skip and gate; inputs, parameters, outputs, next state.
"""

from __future__ import annotations

import math
import sys
from pathlib import Path

import numpy as np
import torch

from slinoss.layers import SLinOSSScanPrep  # type: ignore
from slinoss.layers.backend import ReferenceScanPrepBackend, ScanPrepInputs  # type: ignore
from slinoss.ops.v2x2ssd.reference import (  # type: ignore
    chunk_increment,
    chunk_scan,
    state_passing,
    v2x2ssd,
    v2x2ssm,
)

OUT = Path(__file__).resolve().parent


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach()
    if t.dtype == torch.bfloat16:
        t = t.float()
    return t.cpu().numpy()


def _rand_scan_inputs(b, h, T, N, P, dtype, *, streaming, with_init, gen):
    """Same distributions as the reference's own tests
    (tests/test_v2x2ssd_cute.py:25-67)."""
    radius = 0.6 + 0.35 * torch.rand((b, h, T), generator=gen)
    angle = (2.0 * math.pi) * torch.rand((b, h, T), generator=gen) - math.pi
    M = torch.view_as_real(torch.polar(radius, angle)).to(torch.float32).contiguous()
    K = (torch.randn((b, h, T, 2, 2), generator=gen) * 0.1).to(torch.float32)
    U = torch.randn((b, h, T, P), generator=gen).to(dtype)
    B = (torch.randn((b, h, T, 2 * N), generator=gen) * 0.1).to(dtype)
    C = (torch.randn((b, h, T, 2 * N), generator=gen) * 0.1).to(dtype)
    init = (torch.randn((b, h, P, 2 * N), generator=gen)).to(dtype) if with_init else None
    Bp = (torch.randn((b, h, 2 * N), generator=gen) * 0.1).to(dtype) if streaming else None
    Up = torch.randn((b, h, P), generator=gen).to(dtype) if streaming else None
    return U, M, K, B, C, init, Bp, Up


def _scan_case(name, *, b, h, T, N, P, L, dtype, compute_dtype, streaming, with_init,
               seed, stages):
    gen = torch.Generator().manual_seed(seed)
    U, M, K, B, C, init, Bp, Up = _rand_scan_inputs(
        b, h, T, N, P, dtype, streaming=streaming, with_init=with_init, gen=gen)
    if compute_dtype == torch.float64:
        U, M, K, B, C = (x.double() for x in (U, M, K, B, C))
        init, Bp, Up = (None if x is None else x.double() for x in (init, Bp, Up))
    leaves = [U, M, K, B, C] + [x for x in (init, Bp, Up) if x is not None]
    for x in leaves:
        x.requires_grad_(True)
    odt = U.dtype
    Y, fin, b_last, u_last = v2x2ssd(U, M, K, B, C, chunk_size=L, initial_states=init,
                                     B_prev=Bp, U_prev=Up, compute_dtype=compute_dtype,
                                     output_dtype=odt)
    dY = torch.randn(Y.shape, generator=gen).to(Y.dtype)
    dfin = torch.randn(fin.shape, generator=gen).to(fin.dtype) * 0.1
    grads = torch.autograd.grad([Y, fin], leaves, [dY, dfin])
    out = dict(chunk_size=np.int64(L), U=_np(U), M=_np(M), K=_np(K), B=_np(B), C=_np(C),
               Y=_np(Y), final_state=_np(fin), dY=_np(dY), d_final=_np(dfin))
    names = ["dU", "dM", "dK", "dB", "dC"]
    if init is not None:
        out["initial_states"] = _np(init)
        names.append("d_initial")
    if Bp is not None:
        out["B_prev"], out["U_prev"] = _np(Bp), _np(Up)
        names += ["dB_prev", "dU_prev"]
    for n, g in zip(names, grads):
        out[n] = _np(g)
    with torch.no_grad():
        y_seq, fin_seq, _, _ = v2x2ssm(U, M, K, B, C, initial_states=init, B_prev=Bp,
                                       U_prev=Up, compute_dtype=compute_dtype,
                                       output_dtype=odt)
        out["Y_sequential"] = _np(y_seq)
        if stages:
            inc, mch = chunk_increment(U, M, K, B, B_prev=Bp, U_prev=Up, T=T,
                                       chunk_size=L, compute_dtype=compute_dtype)
            starts, fin2 = state_passing(inc, mch, initial_states=init,
                                         compute_dtype=compute_dtype)
            y3 = chunk_scan(U, M, K, B, C, starts, B_prev=Bp, U_prev=Up, T=T,
                            chunk_size=L, output_dtype=odt, compute_dtype=compute_dtype)
            out.update(inc=_np(inc), m_chunk=_np(mch), chunk_starts=_np(starts),
                       Y_stage3=_np(y3))
    np.savez_compressed(OUT / name, **out)
    print(name, {k: v.shape for k, v in out.items() if hasattr(v, "shape")})


def _prep_module(H, N, P, seed, randomize):
    torch.manual_seed(seed)
    prep = SLinOSSScanPrep(n_heads=H, d_state=N, d_head=P,
                           backend=ReferenceScanPrepBackend())
    if randomize:
        with torch.no_grad():
            for p in prep.parameters():
                p.add_(0.3 * torch.randn_like(p))
    return prep


PREP_PARAM_NAMES = ("dt_bias", "gamma_bias", "omega_bias", "mix_r_bias", "mix_theta_bias",
                    "mix_k_prev_bias", "mix_k_curr_bias", "b_scale", "c_scale")


def _cfg0():
    """Smallest reference shape (b2 H4 T256 P32 N16): scan inputs from a seeded default-init prep."""
    torch.manual_seed(0)
    b, T, H, P, N, L = 2, 256, 4, 32, 16, 64
    prep = _prep_module(H, N, P, seed=0, randomize=False)
    value = torch.randn(b, T, H * P)
    params = torch.randn(b, T, H * 13)
    bc = torch.randn(b, T, H, 4, N)
    with torch.no_grad():
        si = prep(value, params, bc)
    U, M, K, B, C = (x.detach().clone().requires_grad_(True)
                     for x in (si.U, si.M, si.K, si.B, si.C))
    Y, fin, _, _ = v2x2ssd(U, M, K, B, C, chunk_size=L)
    gen = torch.Generator().manual_seed(1)
    dY = torch.randn(Y.shape, generator=gen)
    grads = torch.autograd.grad(Y, [U, M, K, B, C], dY)
    out = dict(chunk_size=np.int64(L), U=_np(U), M=_np(M), K=_np(K), B=_np(B), C=_np(C),
               Y=_np(Y), final_state=_np(fin), dY=_np(dY))
    for n, g in zip(["dU", "dM", "dK", "dB", "dC"], grads):
        out[n] = _np(g)
    np.savez_compressed(OUT / "scan_cfg0_f32.npz", **out)
    print("scan_cfg0_f32.npz", "abs(M) in", float(M.detach().norm(dim=-1).min()),
          float(M.detach().norm(dim=-1).max()))


def _prep_case():
    b, T, H, P, N = 2, 48, 3, 8, 16
    prep = _prep_module(H, N, P, seed=3, randomize=True)
    gen = torch.Generator().manual_seed(4)
    value = torch.randn(b, T, H * P, generator=gen).requires_grad_(True)
    params = (1.5 * torch.randn(b, T, H * 13, generator=gen)).requires_grad_(True)
    bc = torch.randn(b, T, H, 4, N, generator=gen).requires_grad_(True)
    si = prep._prepare_inputs_reference(ScanPrepInputs(value=value, params=params, bc=bc))
    outs = [si.U, si.M, si.K, si.B, si.C]
    gouts = [torch.randn(o.shape, generator=gen) for o in outs]
    plist = [getattr(prep, n) for n in PREP_PARAM_NAMES]
    grads = torch.autograd.grad(outs, [value, params, bc] + plist, gouts)
    out = dict(value=_np(value), params=_np(params), bc=_np(bc))
    for n in PREP_PARAM_NAMES:
        out[n] = _np(getattr(prep, n))
    for n, o, g in zip("UMKBC", outs, gouts):
        out[n] = _np(o)
        out["g" + n] = _np(g)
    for n, g in zip(["d_value", "d_params", "d_bc"] + ["d_" + n for n in PREP_PARAM_NAMES],
                    grads):
        out[n] = _np(g)
    for n in ("dt_min", "dt_max", "r_min", "r_max", "theta_bound", "k_max", "eps"):
        out["hp_" + n] = np.float64(getattr(prep, n))
    # closed-form anchor of the reference's own test (tests/test_scanprep.py:45-56)
    from slinoss.ops.scanprep import foh_taps_from_polar  # type: ignore
    kp, kc = foh_taps_from_polar(torch.tensor([0.05]), torch.tensor([1.0]),
                                 torch.tensor([0.0]), eps=1e-8)
    out["anchor_foh_r1_theta0"] = np.stack([_np(kp), _np(kc)])
    np.savez_compressed(OUT / "prep_f32.npz", **out)
    print("prep_f32.npz written")


def _conv_case():
    import torch.nn.functional as F

    out = {}
    gen = torch.Generator().manual_seed(5)
    for tag, (b, T, C, W, with_state) in {
        "w4_state": (2, 37, 24, 4, True),
        "w4_nostate": (2, 5, 24, 4, False),
        "w2_state": (1, 9, 8, 2, True),
        "w4_short": (2, 2, 16, 4, True),
    }.items():
        x = torch.randn(b, T, C, generator=gen, dtype=torch.float64, requires_grad=True)
        w = torch.randn(C, W, generator=gen, dtype=torch.float64, requires_grad=True)
        bias = torch.randn(C, generator=gen, dtype=torch.float64, requires_grad=True)
        st = (torch.randn(b, C, W - 1, generator=gen, dtype=torch.float64, requires_grad=True)
              if with_state else None)
        # the mixer's reference conv: slinoss/layers/mixer.py:443-454
        prefix = torch.zeros(b, C, W - 1, dtype=torch.float64) if st is None else st
        cat = torch.cat([prefix, x.transpose(1, 2)], dim=-1)
        y = F.conv1d(cat, w.unsqueeze(1), bias, groups=C).transpose(1, 2)
        nxt = cat[..., -(W - 1):]
        dy = torch.randn(y.shape, generator=gen, dtype=torch.float64)
        dn = torch.randn(nxt.shape, generator=gen, dtype=torch.float64)
        leaves = [x, w, bias] + ([st] if st is not None else [])
        grads = torch.autograd.grad([y, nxt], leaves, [dy, dn], retain_graph=True)
        ysilu = F.silu(y)
        gs = torch.autograd.grad(ysilu, leaves[:3], dy)
        d = dict(x=x, w=w, bias=bias, y=y, next_state=nxt, dy=dy, d_next=dn, dx=grads[0],
                 dw=grads[1], dbias=grads[2], y_silu=ysilu, dx_silu=gs[0], dw_silu=gs[1],
                 dbias_silu=gs[2])
        if st is not None:
            d["state"], d["dstate"] = st, grads[3]
        for k, v in d.items():
            out[f"{tag}.{k}"] = _np(v)
    np.savez_compressed(OUT / "conv_f64.npz", **out)
    print("conv_f64.npz written")


def _decode_case():
    """b3 H2 P8 N16, fp32: two consecutive decode steps of a randomised mixer."""
    from slinoss.layers import SLinOSSMixer  # type: ignore
    from slinoss.layers.backend import (MixerDecodeInputs, ReferenceCConv1dBackend,  # type: ignore
                                        ReferenceScanBackend)
    from slinoss.layers.state import ScanState  # type: ignore

    b, H, P, N = 3, 2, 8, 16
    torch.manual_seed(21)
    mixer = SLinOSSMixer(d_model=H * P, d_state=N, expand=1, d_head=P, d_conv=4, chunk_size=16,
                         backend=ReferenceScanBackend(), scanprep_backend=ReferenceScanPrepBackend(),
                         cconv_backend=ReferenceCConv1dBackend())
    with torch.no_grad():
        for prm in mixer.scanprep.parameters():
            prm.add_(0.3 * torch.randn_like(prm))
        mixer.skip.add_(0.5 * torch.randn_like(mixer.skip))
    gen = torch.Generator().manual_seed(22)
    state = ScanState(state=torch.randn(b, H, P, 2 * N, generator=gen),
                      b_prev=torch.randn(b, H, 2 * N, generator=gen),
                      u_prev=torch.randn(b, H, P, generator=gen))
    out = dict(state0=_np(state.state), b_prev0=_np(state.b_prev), u_prev0=_np(state.u_prev),
               skip=_np(mixer.skip.reshape(H, P)))
    for n in PREP_PARAM_NAMES:
        out[n] = _np(getattr(mixer.scanprep, n))
    for n in ("dt_min", "dt_max", "r_min", "r_max", "theta_bound", "k_max", "eps"):
        out["hp_" + n] = np.float64(getattr(mixer.scanprep, n))
    with torch.no_grad():
        for step in range(2):
            inp = MixerDecodeInputs(value=torch.randn(b, H, P, generator=gen),
                                    params=1.5 * torch.randn(b, H, 13, generator=gen),
                                    bc=torch.randn(b, H, 4, N, generator=gen),
                                    gate=torch.randn(b, H, P, generator=gen),
                                    skip=mixer.skip.reshape(H, P))
            y, state = mixer._decode_step_reference(inp, state)
            out.update({f"value{step}": _np(inp.value), f"params{step}": _np(inp.params),
                        f"bc{step}": _np(inp.bc), f"gate{step}": _np(inp.gate), f"y{step}": _np(y),
                        f"state{step + 1}": _np(state.state), f"b_prev{step + 1}": _np(state.b_prev),
                        f"u_prev{step + 1}": _np(state.u_prev)})
    np.savez_compressed(OUT / "decode_f32.npz", **out)
    print("decode_f32.npz written")


def main() -> int:
    torch.set_num_threads(8)
    if "--only-decode" in sys.argv:
        _decode_case()
        return 0
    _scan_case("scan_small_f64.npz", b=1, h=2, T=37, N=3, P=5, L=16, dtype=torch.float32,
               compute_dtype=torch.float64, streaming=True, with_init=True, seed=11,
               stages=True)
    _scan_case("scan_bf16.npz", b=1, h=2, T=192, N=32, P=64, L=64, dtype=torch.bfloat16,
               compute_dtype=torch.float32, streaming=False, with_init=False, seed=12,
               stages=False)
    _cfg0()
    _prep_case()
    _conv_case()
    _decode_case()
    return 0


if __name__ == "__main__":
    sys.exit(main())
