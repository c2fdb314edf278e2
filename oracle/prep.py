"""numpy float64 restatement of SLinOSSScanPrep and the depthwise causal conv
-- TEST INFRASTRUCTURE ONLY (never imported by the shipped library).

Parity status: PINNED against fixtures generated from the reference
(tests/golden/make_golden.py; checked in tests/test_oracle_pins.py).

Forward maps follow the reference line by line; the backward maps are the
analytic vector-Jacobian products of those forwards (the reference obtains them
from torch.autograd), written out by hand so that they can be compared with the
reference's autograd output in the pin tests.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

# slots of the 13-wide parameter row that carry a per-head bias
# (slinoss/layers/scanprep.py:187-206)
BIAS_SLOTS = (0, 1, 2, 5, 6, 7, 8)


@dataclass
class PrepConfig:
    """Hyper-parameters of SLinOSSScanPrep (slinoss/layers/scanprep.py:50-66)."""

    n_heads: int
    d_state: int
    d_head: int
    normalize_bc: bool = True
    dt_min: float = 1e-4
    dt_max: float = 1e-1
    r_min: float = 0.9
    r_max: float = 1.0
    theta_bound: float = math.pi
    k_max: float = 0.5
    eps: float = 1e-8


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def _softplus(x):
    return np.logaddexp(0.0, x)


def principal_angle(theta):
    """slinoss/ops/scanprep/reference.py:12-16."""
    return np.remainder(theta + math.pi, 2.0 * math.pi) - math.pi


def _z_threshold(eps: float) -> float:
    # slinoss/ops/scanprep/reference.py:37
    return float(max(1.0e-4, math.sqrt(max(float(eps), 1.0e-12))))


def coefficients_fwd(params, bias, cfg: PrepConfig, *, want_ctx: bool = False):
    """(b,T,H,13) params + (H,13) bias -> M (b,H,T,2), K (b,H,T,2,2).

    slinoss/layers/scanprep.py:208-286 and
    slinoss/ops/scanprep/reference.py:26-57 (_foh_taps_from_normalized).
    """
    p = np.transpose(np.asarray(params, dtype=np.float64), (0, 2, 1, 3))
    p = p + np.asarray(bias, dtype=np.float64)[None, :, None, :]
    d_dt = cfg.dt_max - cfg.dt_min
    d_r = cfg.r_max - cfg.r_min
    dt_u = _sigmoid(p[..., 0])
    dt = cfg.dt_min + d_dt * dt_u
    gamma = _softplus(p[..., 1])
    omega = p[..., 2]
    e_gdt = np.exp(-gamma * dt)
    r_struct = cfg.r_min + d_r * e_gdt
    th_struct = omega * dt
    r_dir_u = _sigmoid(p[..., 3])
    r_direct = cfg.r_min + d_r * r_dir_u
    th_t = np.tanh(p[..., 4])
    th_direct = cfg.theta_bound * th_t
    mix_r = _sigmoid(p[..., 5])
    mix_th = _sigmoid(p[..., 6])
    mix_kp = _sigmoid(p[..., 7])
    mix_kc = _sigmoid(p[..., 8])
    tk = np.tanh(p[..., 9:13])
    kpl = cfg.k_max * (tk[..., 0] + 1j * tk[..., 1])
    kcl = cfg.k_max * (tk[..., 2] + 1j * tk[..., 3])

    r = r_direct + mix_r * (r_struct - r_direct)
    theta = principal_angle(th_direct + mix_th * (th_struct - th_direct))
    log_r = np.log(r)
    rho = r * np.exp(1j * theta)
    z = log_r + 1j * theta
    thr = _z_threshold(cfg.eps)
    small = (log_r ** 2 + theta ** 2) < thr * thr
    zs = np.where(small, 1.0 + 0j, z)
    k1 = (rho - 1.0) / zs
    k2 = (rho * (zs - 1.0) + 1.0) / (zs * zs)
    k1_t = 1.0 + 0.5 * z + z * z / 6.0 + z ** 3 / 24.0
    k2_t = 0.5 + z / 3.0 + z * z / 8.0 + z ** 3 / 30.0
    k1 = np.where(small, k1_t, k1)
    k2 = np.where(small, k2_t, k2)
    kps = dt * k2
    kcs = dt * k1 - kps
    k_prev = kpl + mix_kp * (kps - kpl)
    k_curr = kcl + mix_kc * (kcs - kcl)

    M = np.stack([rho.real, rho.imag], axis=-1)
    K = np.stack(
        [np.stack([k_prev.real, k_prev.imag], -1), np.stack([k_curr.real, k_curr.imag], -1)],
        axis=-2,
    )
    if not want_ctx:
        return M, K
    ctx = dict(p=p, dt_u=dt_u, dt=dt, gamma=gamma, omega=omega, e_gdt=e_gdt,
               r_struct=r_struct, th_struct=th_struct, r_dir_u=r_dir_u,
               r_direct=r_direct, th_t=th_t, th_direct=th_direct, mix_r=mix_r,
               mix_th=mix_th, mix_kp=mix_kp, mix_kc=mix_kc, tk=tk, kpl=kpl, kcl=kcl,
               r=r, theta=theta, rho=rho, z=z, zs=zs, small=small, k1=k1, k2=k2,
               kps=kps, kcs=kcs)
    return M, K, ctx


def coefficients_bwd(params, bias, cfg: PrepConfig, dM, dK):
    """VJP of coefficients_fwd.  Returns (dparams (b,T,H,13), dbias (H,13))."""
    _, _, c = coefficients_fwd(params, bias, cfg, want_ctx=True)
    dM = np.asarray(dM, dtype=np.float64)
    dK = np.asarray(dK, dtype=np.float64)
    dm = dM[..., 0] + 1j * dM[..., 1]
    dkp = dK[..., 0, 0] + 1j * dK[..., 0, 1]
    dkc = dK[..., 1, 0] + 1j * dK[..., 1, 1]
    d_dt = cfg.dt_max - cfg.dt_min
    d_r = cfg.r_max - cfg.r_min

    def rdot(a, g):  # real inner product of two complex numbers seen as 2-vectors
        return (np.conj(a) * g).real

    dkps = c["mix_kp"] * dkp
    dkpl = (1.0 - c["mix_kp"]) * dkp
    dmix_kp = rdot(c["kps"] - c["kpl"], dkp)
    dkcs = c["mix_kc"] * dkc
    dkcl = (1.0 - c["mix_kc"]) * dkc
    dmix_kc = rdot(c["kcs"] - c["kcl"], dkc)

    dt, k1, k2, z, rho = c["dt"], c["k1"], c["k2"], c["z"], c["rho"]
    dk2 = dt * (dkps - dkcs)
    dk1 = dt * dkcs
    ddt = rdot(k2, dkps) + rdot(k1 - k2, dkcs)
    zs = c["zs"]
    k1p = np.where(c["small"], 0.5 + z / 3.0 + z * z / 8.0, k2)
    k2p = np.where(c["small"], 1.0 / 3.0 + z / 4.0 + z * z / 10.0, (rho - 2.0 * k2) / zs)
    dz = np.conj(k1p) * dk1 + np.conj(k2p) * dk2 + np.conj(rho) * dm
    dlog_r = dz.real
    dtheta = dz.imag
    dr = dlog_r / c["r"]

    dth_d = (1.0 - c["mix_th"]) * dtheta
    dth_s = c["mix_th"] * dtheta
    dmix_th = (c["th_struct"] - c["th_direct"]) * dtheta
    dr_d = (1.0 - c["mix_r"]) * dr
    dr_s = c["mix_r"] * dr
    dmix_r = (c["r_struct"] - c["r_direct"]) * dr

    dgamma = dr_s * d_r * c["e_gdt"] * (-dt)
    ddt = ddt + dr_s * d_r * c["e_gdt"] * (-c["gamma"])
    domega = dth_s * dt
    ddt = ddt + dth_s * c["omega"]

    def dsig(s):
        return s * (1.0 - s)

    dp = np.zeros_like(c["p"])
    dp[..., 0] = ddt * d_dt * dsig(c["dt_u"])
    dp[..., 1] = dgamma * _sigmoid(c["p"][..., 1])
    dp[..., 2] = domega
    dp[..., 3] = dr_d * d_r * dsig(c["r_dir_u"])
    dp[..., 4] = dth_d * cfg.theta_bound * (1.0 - c["th_t"] ** 2)
    dp[..., 5] = dmix_r * dsig(c["mix_r"])
    dp[..., 6] = dmix_th * dsig(c["mix_th"])
    dp[..., 7] = dmix_kp * dsig(c["mix_kp"])
    dp[..., 8] = dmix_kc * dsig(c["mix_kc"])
    one_m = 1.0 - c["tk"] ** 2
    dp[..., 9] = cfg.k_max * one_m[..., 0] * dkpl.real
    dp[..., 10] = cfg.k_max * one_m[..., 1] * dkpl.imag
    dp[..., 11] = cfg.k_max * one_m[..., 2] * dkcl.real
    dp[..., 12] = cfg.k_max * one_m[..., 3] * dkcl.imag
    dbias = dp.sum(axis=(0, 2))
    mask = np.zeros(13)
    mask[list(BIAS_SLOTS)] = 1.0
    return np.transpose(dp, (0, 2, 1, 3)), dbias * mask[None, :]


def pack_bc_fwd(bc, scale, cfg: PrepConfig, *, want_ctx: bool = False):
    """bc (b,T,H,4,N) -> B,C (b,H,T,2N).

    RMS-norm over N (eps 1e-5) times per-head scale (H,4,N) (rows 0,1 = b_scale,
    rows 2,3 = c_scale), then interleave rows (0,1)->B, (2,3)->C.
    slinoss/layers/scanprep.py:297-336.
    """
    x = np.asarray(bc, dtype=np.float64)
    if cfg.normalize_bc:
        rstd = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + 1e-5)
        xhat = x * rstd
        y = xhat * np.asarray(scale, dtype=np.float64)[None, None]
    else:
        rstd, xhat, y = None, None, x
    yt = np.transpose(y, (0, 2, 1, 4, 3))  # (b,H,T,N,4)
    b, H, T, N, _ = yt.shape
    Bm = yt[..., :2].reshape(b, H, T, 2 * N)
    Cm = yt[..., 2:].reshape(b, H, T, 2 * N)
    if want_ctx:
        return Bm, Cm, dict(rstd=rstd, xhat=xhat)
    return Bm, Cm


def pack_bc_bwd(bc, scale, cfg: PrepConfig, dB, dC):
    """VJP of pack_bc_fwd.  Returns (dbc (b,T,H,4,N), dscale (H,4,N) or None)."""
    _, _, c = pack_bc_fwd(bc, scale, cfg, want_ctx=True)
    dB = np.asarray(dB, dtype=np.float64)
    dC = np.asarray(dC, dtype=np.float64)
    b, H, T, D = dB.shape
    N = D // 2
    dyt = np.concatenate([dB.reshape(b, H, T, N, 2), dC.reshape(b, H, T, N, 2)], axis=-1)
    dy = np.transpose(dyt, (0, 2, 1, 4, 3))  # (b,T,H,4,N)
    if not cfg.normalize_bc:
        return dy, None
    s = np.asarray(scale, dtype=np.float64)[None, None]
    dscale = (dy * c["xhat"]).sum(axis=(0, 1))
    g = dy * s
    dx = c["rstd"] * (g - c["xhat"] * (g * c["xhat"]).mean(axis=-1, keepdims=True))
    return dx, dscale


def pack_u_fwd(value, cfg: PrepConfig):
    """value (b,T,H*P) -> U (b,H,T,P).  slinoss/layers/scanprep.py:302-311."""
    v = np.asarray(value, dtype=np.float64)
    b, T, _ = v.shape
    return np.ascontiguousarray(
        np.transpose(v.reshape(b, T, cfg.n_heads, cfg.d_head), (0, 2, 1, 3)))


def pack_u_bwd(dU):
    dU = np.asarray(dU, dtype=np.float64)
    b, H, T, P = dU.shape
    return np.ascontiguousarray(np.transpose(dU, (0, 2, 1, 3)).reshape(b, T, H * P))


def flat_bias(dt_bias, gamma_bias, omega_bias, mix_r_bias, mix_theta_bias,
              mix_k_prev_bias, mix_k_curr_bias):
    """(H,13) bias table.  slinoss/layers/scanprep.py:187-206."""
    H = len(dt_bias)
    out = np.zeros((H, 13))
    for slot, v in zip(BIAS_SLOTS, (dt_bias, gamma_bias, omega_bias, mix_r_bias,
                                    mix_theta_bias, mix_k_prev_bias, mix_k_curr_bias)):
        out[:, slot] = np.asarray(v, dtype=np.float64)
    return out


# --------------------------------------------------------------------------- #
# depthwise causal conv1d
# --------------------------------------------------------------------------- #

def cconv1d_fwd(x, weight, bias, conv_state=None, *, silu: bool = False):
    """x (b,T,C), weight (C,W), bias (C,) or None, conv_state (b,C,W-1) or None.

    Returns (y (b,T,C), next_state (b,C,W-1)).  slinoss/layers/mixer.py:420-454
    (cross-correlation over [state, x]); optional SiLU as in
    slinoss/ops/cconv1d.py:288.
    """
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(weight, dtype=np.float64)
    b, T, C = x.shape
    W = w.shape[1]
    st = np.zeros((b, C, W - 1)) if conv_state is None else np.asarray(conv_state, np.float64)
    cat = np.concatenate([np.transpose(st, (0, 2, 1)), x], axis=1)  # (b, W-1+T, C)
    y = np.zeros((b, T, C))
    for j in range(W):
        y += cat[:, j:j + T, :] * w[None, None, :, j]
    if bias is not None:
        y += np.asarray(bias, dtype=np.float64)[None, None, :]
    pre = y
    if silu:
        y = y * _sigmoid(y)
    nxt = np.transpose(cat[:, cat.shape[1] - (W - 1):, :], (0, 2, 1)) if W > 1 else np.zeros((b, C, 0))
    return y, np.ascontiguousarray(nxt), pre


def cconv1d_bwd(x, weight, bias, conv_state, dy, *, d_next_state=None, silu: bool = False):
    """VJP of cconv1d_fwd.  Returns (dx, dweight, dbias, dstate)."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(weight, dtype=np.float64)
    dy = np.asarray(dy, dtype=np.float64)
    b, T, C = x.shape
    W = w.shape[1]
    st = np.zeros((b, C, W - 1)) if conv_state is None else np.asarray(conv_state, np.float64)
    cat = np.concatenate([np.transpose(st, (0, 2, 1)), x], axis=1)
    if silu:
        _, _, pre = cconv1d_fwd(x, weight, bias, conv_state)
        s = _sigmoid(pre)
        dy = dy * (s * (1.0 + pre * (1.0 - s)))
    dcat = np.zeros_like(cat)
    dw = np.zeros_like(w)
    for j in range(W):
        dcat[:, j:j + T, :] += dy * w[None, None, :, j]
        dw[:, j] = (dy * cat[:, j:j + T, :]).sum(axis=(0, 1))
    if d_next_state is not None and W > 1:
        dcat[:, cat.shape[1] - (W - 1):, :] += np.transpose(
            np.asarray(d_next_state, np.float64), (0, 2, 1))
    dbias = dy.sum(axis=(0, 1))
    dx = dcat[:, W - 1:, :]
    dstate = np.transpose(dcat[:, :W - 1, :], (0, 2, 1))
    return dx, dw, dbias, np.ascontiguousarray(dstate)
