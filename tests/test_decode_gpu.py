"""One-token decode step on the GPU (through the C ABI) against the golden fixture generated
from the reference and against the float64 oracle."""

from __future__ import annotations

import types

import numpy as np
import pytest
import torch

from util import golden, rel_err

pytestmark = pytest.mark.gpu

HP = ("dt_min", "dt_max", "r_min", "r_max", "theta_bound", "k_max", "eps")
BIASES = ("dt_bias", "gamma_bias", "omega_bias", "mix_r_bias", "mix_theta_bias", "mix_k_prev_bias",
          "mix_k_curr_bias")


def _t(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).cuda()


def _np(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def test_decode_matches_reference_fixture():
    import slinoss_b200 as sb

    g = golden("decode_f32.npz")
    kw = {k: float(g["hp_" + k]) for k in HP}
    kw.update({k: _t(g[k]) for k in BIASES})
    kw.update(b_scale=_t(g["b_scale"]), c_scale=_t(g["c_scale"]))
    st, bp, up = _t(g["state0"]), _t(g["b_prev0"]), _t(g["u_prev0"])
    for step in range(2):
        y, st, bp, up = sb.mixer_decode_step_b200(
            _t(g[f"value{step}"]), _t(g[f"params{step}"]), _t(g[f"bc{step}"]), _t(g[f"gate{step}"]),
            _t(g["skip"]), initial_states=st, B_prev=bp, U_prev=up, **kw)
        # the reference's fp32 taps carry cancellation noise (see the oracle pin of the same fixture)
        assert rel_err(_np(y), g[f"y{step}"]) < 1e-4
        assert rel_err(_np(st), g[f"state{step + 1}"]) < 1e-4
        assert rel_err(_np(bp), g[f"b_prev{step + 1}"]) < 2e-6
        assert torch.equal(up.cpu(), torch.from_numpy(g[f"u_prev{step + 1}"]))


def _random_case(b, H, P, N, dtype, seed):
    from oracle import prep as oprep

    gen = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=gen)
    case = dict(value=r(b, H, P).to(dtype), params=(1.5 * r(b, H, 13)).to(dtype), bc=r(b, H, 4, N).to(dtype),
                gate=r(b, H, P).to(dtype), skip=r(H, P).to(dtype), state=r(b, H, P, 2 * N),
                b_prev=r(b, H, 2 * N).to(dtype), u_prev=r(b, H, P).to(dtype),
                b_scale=1 + 0.1 * r(H, 2, N), c_scale=1 + 0.1 * r(H, 2, N))
    biases = {k: 0.3 * r(H) for k in BIASES}
    cfg = oprep.PrepConfig(n_heads=H, d_state=N, d_head=P)
    return case, biases, cfg


@pytest.mark.parametrize("b,H,P,N,dtype,tol", [
    (5, 3, 64, 128, torch.bfloat16, 2e-2),
    (2, 2, 64, 64, torch.float16, 5e-3),
    (3, 2, 24, 10, torch.float32, 1e-5),      # odd sizes: rows and items not multiples of the warp tiling
])
def test_decode_vs_oracle_and_in_place(b, H, P, N, dtype, tol):
    import slinoss_b200 as sb
    from oracle import decode as odec
    from oracle import prep as oprep

    case, biases, cfg = _random_case(b, H, P, N, dtype, seed=b * 100 + N)
    hp = {k: getattr(cfg, k) for k in HP}
    dev = {k: v.cuda() for k, v in case.items()}
    kw = dict(hp, **{k: v.cuda() for k, v in biases.items()}, b_scale=dev["b_scale"], c_scale=dev["c_scale"])
    y, st, bl, ul = sb.mixer_decode_step_b200(dev["value"], dev["params"], dev["bc"], dev["gate"], dev["skip"],
                                              initial_states=dev["state"], B_prev=dev["b_prev"],
                                              U_prev=dev["u_prev"], **kw)
    bias = oprep.flat_bias(*(_np(biases[k]) for k in BIASES))
    scale = np.concatenate([_np(case["b_scale"]), _np(case["c_scale"])], axis=1)
    yo, sto, blo, ulo = odec.decode_step(_np(case["value"]), _np(case["params"]), _np(case["bc"]),
                                         _np(case["gate"]), _np(case["skip"]), bias, scale, cfg,
                                         state=_np(case["state"]), b_prev=_np(case["b_prev"]),
                                         u_prev=_np(case["u_prev"]))
    # the oracle does not round b, c to the activation dtype: for half inputs that is inside tol
    assert rel_err(_np(y), yo) < tol
    assert rel_err(_np(st), sto) < max(tol, 1e-6)
    assert rel_err(_np(bl), blo) < max(tol, 1e-6)
    assert torch.equal(ul, dev["value"])
    # in-place update of the carried tensors gives the same bits
    st2, bp2, up2 = dev["state"].clone(), dev["b_prev"].clone(), dev["u_prev"].clone()
    y2, st2o, bl2, ul2 = sb.mixer_decode_step_b200(dev["value"], dev["params"], dev["bc"], dev["gate"],
                                                   dev["skip"], initial_states=st2, B_prev=bp2, U_prev=up2,
                                                   final_state_out=st2, b_last_out=bp2, u_last_out=up2, **kw)
    assert st2o.data_ptr() == st2.data_ptr()
    assert torch.equal(y2, y) and torch.equal(st2, st) and torch.equal(bp2, bl) and torch.equal(up2, ul)
    # no carried state at all: zero state, no previous token
    y0, st0, _, _ = sb.mixer_decode_step_b200(dev["value"], dev["params"], dev["bc"], dev["gate"], dev["skip"], **kw)
    yo0, sto0, _, _ = odec.decode_step(_np(case["value"]), _np(case["params"]), _np(case["bc"]), _np(case["gate"]),
                                       _np(case["skip"]), bias, scale, cfg, state=None, b_prev=None, u_prev=None)
    assert rel_err(_np(y0), yo0) < tol and rel_err(_np(st0), sto0) < max(tol, 1e-6)


def test_decode_backend_protocol():
    """B200MixerDecodeBackend against a stand-in owner with the attributes the mixer exposes."""
    import slinoss_b200 as sb

    b, H, P, N = 4, 2, 64, 32
    case, biases, cfg = _random_case(b, H, P, N, torch.bfloat16, seed=9)
    dev = {k: v.cuda() for k, v in case.items()}
    prep = types.SimpleNamespace(**{k: getattr(cfg, k) for k in HP}, **{k: v.cuda() for k, v in biases.items()},
                                 b_scale=dev["b_scale"], c_scale=dev["c_scale"], normalize_bc=True)
    owner = types.SimpleNamespace(scanprep=prep, d_state=N, d_head=P, output_norm=None)
    inputs = types.SimpleNamespace(value=dev["value"], params=dev["params"], bc=dev["bc"], gate=dev["gate"],
                                   skip=dev["skip"])
    state = sb.ScanState(state=dev["state"].clone(), b_prev=dev["b_prev"].clone(), u_prev=dev["u_prev"].clone())
    be = sb.B200MixerDecodeBackend()
    assert be.supports(owner, batch_size=b, device=dev["value"].device, dtype=torch.bfloat16)
    assert not be.supports(owner, batch_size=b, device=torch.device("cpu"), dtype=torch.bfloat16)
    y, nxt = be(owner, inputs, state)
    assert tuple(y.shape) == (b, H * P) and nxt.state.data_ptr() == state.state.data_ptr()
    y_ref, st_ref, _, _ = sb.mixer_decode_step_b200(
        dev["value"], dev["params"], dev["bc"], dev["gate"], dev["skip"], initial_states=dev["state"],
        B_prev=dev["b_prev"], U_prev=dev["u_prev"], **{k: getattr(cfg, k) for k in HP},
        **{k: v.cuda() for k, v in biases.items()}, b_scale=dev["b_scale"], c_scale=dev["c_scale"])
    assert torch.equal(y, y_ref) and torch.equal(nxt.state, st_ref)
    with pytest.raises(ValueError):
        sb.mixer_decode_step_b200(dev["value"].cpu(), dev["params"], dev["bc"], dev["gate"], dev["skip"],
                                  **{k: getattr(cfg, k) for k in HP}, **{k: v.cuda() for k, v in biases.items()},
                                  b_scale=dev["b_scale"], c_scale=dev["c_scale"])
