"""float64 restatement of the one-token mixer decode step -- TEST INFRASTRUCTURE ONLY
(never imported by the shipped library).

Follows SLinOSSMixer._decode_step_reference (slinoss/layers/mixer.py:714-748): scan prep of
the single token (scanprep.py:351), one step of the sequential recurrence from the carried
state (ops/v2x2ssd/reference.py:704), then skip and gate (mixer.py:585-599).

Parity status: PINNED against tests/golden/decode_f32.npz, generated from the reference by
tests/golden/make_golden.py (checked in tests/test_oracle_pins.py).
"""

from __future__ import annotations

import numpy as np

from . import prep as oprep
from . import scan as oscan


def decode_step(value, params, bc, gate, skip, bias, scale, cfg: oprep.PrepConfig, *,
                state, b_prev, u_prev):
    """value (b,H,P), params (b,H,13), bc (b,H,4,N), gate (b,H,P), skip (H,P), bias (H,13),
    scale (H,4,N); state (b,H,P,2N), b_prev (b,H,2N), u_prev (b,H,P).

    Returns (gated (b,H*P), next_state (b,H,P,2N), b_last (b,H,2N), u_last (b,H,P)).
    """
    value, params, bc, gate = (np.asarray(x, dtype=np.float64) for x in (value, params, bc, gate))
    b, H, P = value.shape
    M, K = oprep.coefficients_fwd(params[:, None], bias, cfg)              # (b,H,1,2), (b,H,1,2,2)
    B, C = oprep.pack_bc_fwd(bc[:, None], scale, cfg)                      # (b,H,1,2N)
    U = value[:, :, None, :]                                               # (b,H,1,P)
    Y, nxt = oscan.v2x2ssm_fwd(U, M, K, B, C, initial_states=state, B_prev=b_prev, U_prev=u_prev)
    y = Y[:, :, 0, :] + U[:, :, 0, :] * np.asarray(skip, dtype=np.float64)[None]
    gated = y * (gate / (1.0 + np.exp(-gate)))
    return gated.reshape(b, H * P), nxt, B[:, :, 0, :], U[:, :, 0, :]
