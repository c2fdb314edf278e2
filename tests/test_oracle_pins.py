"""Pins the CPU oracle (oracle/) against fixtures generated from the reference
(tests/golden/make_golden.py).  CPU only."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import prep as oprep
from oracle import scan as oscan
from util import golden, rel_err

SCAN_GRADS = ("dU", "dM", "dK", "dB", "dC", "d_initial", "dB_prev", "dU_prev")


def _scan_kwargs(g):
    return dict(initial_states=g.get("initial_states"), B_prev=g.get("B_prev"),
                U_prev=g.get("U_prev"))


def test_scan_small_f64_forward_and_stages():
    g = golden("scan_small_f64.npz")
    L = int(g["chunk_size"])
    kw = _scan_kwargs(g)
    Y, fin = oscan.v2x2ssm_fwd(g["U"], g["M"], g["K"], g["B"], g["C"], **kw)
    assert rel_err(Y, g["Y_sequential"]) < 1e-12
    assert rel_err(Y, g["Y"]) < 1e-11
    assert rel_err(fin, g["final_state"]) < 1e-11
    inc, mch = oscan.chunk_increment(g["U"], g["M"], g["K"], g["B"], B_prev=g["B_prev"],
                                     U_prev=g["U_prev"], chunk_size=L)
    assert rel_err(inc, g["inc"]) < 1e-12
    assert rel_err(mch, g["m_chunk"]) < 1e-12
    starts, fin2 = oscan.state_passing(inc, mch, initial_states=g["initial_states"])
    assert rel_err(starts, g["chunk_starts"]) < 1e-12
    assert rel_err(fin2, g["final_state"]) < 1e-12
    Y3 = oscan.chunk_scan(g["U"], g["M"], g["K"], g["B"], g["C"], starts,
                          B_prev=g["B_prev"], U_prev=g["U_prev"], chunk_size=L)
    assert rel_err(Y3, g["Y_stage3"]) < 1e-12
    Y4, fin4, st4, m4 = oscan.v2x2ssd_fwd(g["U"], g["M"], g["K"], g["B"], g["C"],
                                          chunk_size=L, **kw)
    assert rel_err(Y4, g["Y"]) < 1e-12 and rel_err(st4, g["chunk_starts"]) < 1e-12


def test_scan_small_f64_gradients():
    g = golden("scan_small_f64.npz")
    out = oscan.v2x2ssm_bwd(g["U"], g["M"], g["K"], g["B"], g["C"], dY=g["dY"],
                            d_final=g["d_final"], **_scan_kwargs(g))
    for name in SCAN_GRADS:
        assert rel_err(out[name], g[name]) < 1e-11, name


def test_scan_cfg0_f32():
    g = golden("scan_cfg0_f32.npz")
    L = int(g["chunk_size"])
    Y, fin, _, _ = oscan.v2x2ssd_fwd(g["U"], g["M"], g["K"], g["B"], g["C"], chunk_size=L)
    # the fixture was computed by the reference in fp32; the oracle is fp64
    assert rel_err(Y, g["Y"]) < 5e-6
    assert rel_err(fin, g["final_state"]) < 5e-6
    out = oscan.v2x2ssm_bwd(g["U"], g["M"], g["K"], g["B"], g["C"], dY=g["dY"])
    for name in ("dU", "dM", "dK", "dB", "dC"):
        assert rel_err(out[name], g[name]) < 2e-5, name


def test_scan_bf16_fixture():
    g = golden("scan_bf16.npz")
    Y, fin = oscan.v2x2ssm_fwd(g["U"], g["M"], g["K"], g["B"], g["C"])
    # reference output is rounded to bf16 (2^-9 relative per element)
    assert rel_err(Y, g["Y"]) < 4e-3
    out = oscan.v2x2ssm_bwd(g["U"], g["M"], g["K"], g["B"], g["C"], dY=g["dY"],
                            d_final=g["d_final"])
    for name in ("dU", "dB", "dC"):
        assert rel_err(out[name], g[name]) < 4e-3, name
    for name in ("dM", "dK"):
        assert rel_err(out[name], g[name]) < 1e-4, name


def test_exact_zero_transition_rejected():
    g = golden("scan_small_f64.npz")
    M = g["M"].copy()
    M[0, 0, 3] = 0.0
    with pytest.raises(ValueError):
        oscan.v2x2ssd_fwd(g["U"], M, g["K"], g["B"], g["C"], chunk_size=16)


def _prep_cfg(g, n_heads=None, d_state=None, d_head=None):
    H, _, N = g["b_scale"].shape
    P = d_head if d_head is not None else g["value"].shape[-1] // H
    return oprep.PrepConfig(n_heads=H, d_state=N, d_head=P,
                            **{k[3:]: float(v) for k, v in g.items() if k.startswith("hp_")})


def _prep_tables(g):
    bias = oprep.flat_bias(*(g[n] for n in ("dt_bias", "gamma_bias", "omega_bias",
                                             "mix_r_bias", "mix_theta_bias",
                                             "mix_k_prev_bias", "mix_k_curr_bias")))
    scale = np.concatenate([g["b_scale"], g["c_scale"]], axis=1)
    return bias, scale


def test_prep_forward():
    g = golden("prep_f32.npz")
    cfg = _prep_cfg(g)
    bias, scale = _prep_tables(g)
    b, T, _ = g["value"].shape
    p4 = g["params"].reshape(b, T, cfg.n_heads, 13)
    M, K = oprep.coefficients_fwd(p4, bias, cfg)
    assert rel_err(M, g["M"]) < 2e-6
    # the reference evaluates (rho-1)/z and (rho(z-1)+1)/z^2 in fp32, which cancels
    # for small |z|; the float64 oracle is the more accurate of the two
    assert rel_err(K, g["K"]) < 1e-4
    Bm, Cm = oprep.pack_bc_fwd(g["bc"], scale, cfg)
    assert rel_err(Bm, g["B"]) < 2e-6 and rel_err(Cm, g["C"]) < 2e-6
    assert np.array_equal(oprep.pack_u_fwd(g["value"], cfg).astype(np.float32), g["U"])


def test_prep_backward():
    g = golden("prep_f32.npz")
    cfg = _prep_cfg(g)
    bias, scale = _prep_tables(g)
    b, T, _ = g["value"].shape
    p4 = g["params"].reshape(b, T, cfg.n_heads, 13)
    dp, dbias = oprep.coefficients_bwd(p4, bias, cfg, g["gM"], g["gK"])
    # fp32 cancellation in the reference's FOH-tap formulas limits the agreement;
    # the analytic VJP itself matches float64 autograd of the same map to 3e-15
    assert rel_err(dp.reshape(b, T, -1), g["d_params"]) < 1e-4
    for slot, name in zip(oprep.BIAS_SLOTS, ("dt_bias", "gamma_bias", "omega_bias",
                                             "mix_r_bias", "mix_theta_bias",
                                             "mix_k_prev_bias", "mix_k_curr_bias")):
        # a bias gradient is a signed sum over all tokens of fp32-noisy terms:
        # bound the mismatch by the sum of magnitudes, not by the (cancelling) sum
        mag = np.abs(dp[..., slot]).sum(axis=(0, 1))
        floor = 5e-6 * b * T  # fp32 noise floor of the reference per token (O(1) upstream)
        assert np.all(np.abs(dbias[:, slot] - g["d_" + name]) <= 1e-4 * mag + floor), name
    dbc, dscale = oprep.pack_bc_bwd(g["bc"], scale, cfg, g["gB"], g["gC"])
    assert rel_err(dbc, g["d_bc"]) < 2e-5
    assert rel_err(dscale[:, :2], g["d_b_scale"]) < 2e-5
    assert rel_err(dscale[:, 2:], g["d_c_scale"]) < 2e-5
    assert rel_err(oprep.pack_u_bwd(g["gU"]), g["d_value"]) < 1e-7


def test_prep_closed_form_anchor():
    """FOH taps at r=1, theta=0 are dt/2 each (reference tests/test_scanprep.py:45-56)."""
    g = golden("prep_f32.npz")
    ref = g["anchor_foh_r1_theta0"]
    assert np.allclose(ref[:, 0, 0], 0.025, atol=1e-7) and np.allclose(ref[:, 0, 1], 0, atol=1e-7)


@pytest.mark.parametrize("tag", ["w4_state", "w4_nostate", "w2_state", "w4_short"])
def test_conv(tag):
    g = {k.split(".", 1)[1]: v for k, v in golden("conv_f64.npz").items()
         if k.startswith(tag + ".")}
    st = g.get("state")
    y, nxt, _ = oprep.cconv1d_fwd(g["x"], g["w"], g["bias"], st)
    assert rel_err(y, g["y"]) < 1e-12 and rel_err(nxt, g["next_state"]) < 1e-12
    dx, dw, db, dst = oprep.cconv1d_bwd(g["x"], g["w"], g["bias"], st, g["dy"],
                                        d_next_state=g["d_next"])
    assert rel_err(dx, g["dx"]) < 1e-12 and rel_err(dw, g["dw"]) < 1e-12
    assert rel_err(db, g["dbias"]) < 1e-12
    if st is not None:
        assert rel_err(dst, g["dstate"]) < 1e-12
    ys, _, _ = oprep.cconv1d_fwd(g["x"], g["w"], g["bias"], st, silu=True)
    assert rel_err(ys, g["y_silu"]) < 1e-12
    dxs, dws, dbs, _ = oprep.cconv1d_bwd(g["x"], g["w"], g["bias"], st, g["dy"], silu=True)
    assert rel_err(dxs, g["dx_silu"]) < 1e-12 and rel_err(dws, g["dw_silu"]) < 1e-12
    assert rel_err(dbs, g["dbias_silu"]) < 1e-12


def test_prep_coefficient_vjp_matches_float64_autograd():
    """The hand-written VJP equals torch.autograd of the same map in float64
    (removes the fp32 noise of the reference fixture from the comparison)."""
    import math

    import torch

    torch.manual_seed(0)
    H = 3
    cfg = oprep.PrepConfig(n_heads=H, d_state=4, d_head=4)
    params = (1.5 * torch.randn(2, 7, H, 13, dtype=torch.float64)).requires_grad_(True)
    bias = torch.randn(H, 13, dtype=torch.float64) * 0.3
    sg = torch.sigmoid
    p = params.permute(0, 2, 1, 3) + bias[None, :, None, :]
    dt = cfg.dt_min + (cfg.dt_max - cfg.dt_min) * sg(p[..., 0])
    gamma = torch.nn.functional.softplus(p[..., 1])
    rs = cfg.r_min + (cfg.r_max - cfg.r_min) * torch.exp(-gamma * dt)
    ths = p[..., 2] * dt
    rd = cfg.r_min + (cfg.r_max - cfg.r_min) * sg(p[..., 3])
    thd = cfg.theta_bound * torch.tanh(p[..., 4])
    r = torch.lerp(rd, rs, sg(p[..., 5]))
    th = torch.remainder(torch.lerp(thd, ths, sg(p[..., 6])) + math.pi, 2 * math.pi) - math.pi
    rho = torch.polar(r, th)
    z = torch.complex(torch.log(r), th)
    k1 = (rho - 1) / z
    k2 = (rho * (z - 1) + 1) / (z * z)
    kps = dt * k2
    kcs = dt * k1 - kps
    kpl = cfg.k_max * torch.complex(torch.tanh(p[..., 9]), torch.tanh(p[..., 10]))
    kcl = cfg.k_max * torch.complex(torch.tanh(p[..., 11]), torch.tanh(p[..., 12]))
    kp = kpl + sg(p[..., 7]) * (kps - kpl)
    kc = kcl + sg(p[..., 8]) * (kcs - kcl)
    M = torch.view_as_real(rho)
    K = torch.stack([torch.view_as_real(kp), torch.view_as_real(kc)], -2)
    gM, gK = torch.randn_like(M), torch.randn_like(K)
    (gp,) = torch.autograd.grad([M, K], [params], [gM, gK])
    dp, _ = oprep.coefficients_bwd(params.detach().numpy(), bias.numpy(), cfg,
                                   gM.numpy(), gK.numpy())
    M2, K2 = oprep.coefficients_fwd(params.detach().numpy(), bias.numpy(), cfg)
    assert rel_err(M2, M.detach().numpy()) < 1e-13 and rel_err(K2, K.detach().numpy()) < 1e-13
    assert rel_err(dp, gp.numpy()) < 1e-12


def test_decode_step_two_tokens():
    """One-token decode step against SLinOSSMixer._decode_step_reference, two steps chained."""
    from oracle import decode as odec

    g = golden("decode_f32.npz")
    cfg = _prep_cfg(g, n_heads=g["skip"].shape[0], d_state=g["bc0"].shape[-1], d_head=g["skip"].shape[1])
    bias, scale = _prep_tables(g)
    st, bp, up = g["state0"], g["b_prev0"], g["u_prev0"]
    for step in range(2):
        y, st, bp, up = odec.decode_step(g[f"value{step}"], g[f"params{step}"], g[f"bc{step}"],
                                         g[f"gate{step}"], g["skip"], bias, scale, cfg,
                                         state=st, b_prev=bp, u_prev=up)
        # the taps carry the reference's fp32 cancellation noise (see test_prep_forward)
        assert rel_err(y, g[f"y{step}"]) < 1e-4
        assert rel_err(st, g[f"state{step + 1}"]) < 1e-4
        assert rel_err(bp, g[f"b_prev{step + 1}"]) < 2e-6
        assert rel_err(up, g[f"u_prev{step + 1}"]) < 1e-7
