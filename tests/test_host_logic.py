"""Host-side behaviour that needs no GPU: validation, T == 0 semantics, the
"no CPU fallback" rule and backend plumbing (with a fake op, as the reference's
tests/test_cute_backend.py:36-142 does)."""

from __future__ import annotations

import pytest
import torch

import slinoss_b200
from slinoss_b200 import backends
from slinoss_b200.ops import v2x2ssd as op
from slinoss_b200.types import ScanInputs, ScanState


def _inputs(b=1, h=2, T=8, P=4, N=3, dtype=torch.float32):
    g = torch.Generator().manual_seed(0)
    U = torch.randn(b, h, T, P, generator=g, dtype=dtype)
    M = torch.randn(b, h, T, 2, generator=g)
    K = torch.randn(b, h, T, 2, 2, generator=g)
    B = torch.randn(b, h, T, 2 * N, generator=g, dtype=dtype)
    C = torch.randn(b, h, T, 2 * N, generator=g, dtype=dtype)
    return U, M, K, B, C


def test_cpu_tensors_are_rejected_not_emulated():
    U, M, K, B, C = _inputs()
    with pytest.raises(ValueError, match="requires CUDA"):
        slinoss_b200.v2x2ssd_b200(U, M, K, B, C, chunk_size=16)
    with pytest.raises(ValueError, match="requires CUDA"):
        slinoss_b200.cconv1d_b200(torch.zeros(1, 4, 8), torch.zeros(8, 4))


def test_shape_validation_matches_reference_messages():
    U, M, K, B, C = _inputs()
    with pytest.raises(ValueError, match="must be contiguous"):
        slinoss_b200.v2x2ssd_b200(U.transpose(2, 3).contiguous().transpose(2, 3), M, K, B, C, chunk_size=16)
    with pytest.raises(ValueError, match=r"M must be \(batch,heads,T,2\)"):
        slinoss_b200.v2x2ssd_b200(U, M[..., :1].contiguous(), K, B, C, chunk_size=16)
    with pytest.raises(ValueError, match="C must match B exactly"):
        slinoss_b200.v2x2ssd_b200(U, M, K, B, C[..., :4].contiguous(), chunk_size=16)
    with pytest.raises(ValueError, match="passed together"):
        slinoss_b200.v2x2ssd_b200(U, M, K, B, C, chunk_size=16, B_prev=torch.zeros(1, 2, 6))
    with pytest.raises(ValueError, match="initial_states must be"):
        slinoss_b200.v2x2ssd_b200(U, M, K, B, C, chunk_size=16, initial_states=torch.zeros(1, 2, 4, 4))


def test_empty_sequence_semantics():
    """T == 0: reference.py:670-701."""
    init = torch.randn(1, 2, 4, 6)
    bp, up = torch.randn(1, 2, 6), torch.randn(1, 2, 4)
    Y, fin, bl, ul = op._resolve_empty_outputs(1, 2, 4, 6, torch.device("cpu"), torch.float32, init, bp, up)
    assert Y.shape == (1, 2, 0, 4) and torch.equal(fin, init) and torch.equal(bl, bp) and torch.equal(ul, up)
    Y, fin, bl, ul = op._resolve_empty_outputs(1, 2, 4, 6, torch.device("cpu"), torch.float32, None, None, None)
    assert fin.abs().sum() == 0 and bl.shape == (1, 2, 6) and ul.shape == (1, 2, 4)


def test_dtype_resolution():
    assert op._resolve_dtypes([torch.bfloat16, torch.float32], None, None, torch.bfloat16) == (
        torch.float32, torch.bfloat16)
    assert op._resolve_dtypes([torch.bfloat16], None, None, torch.bfloat16)[0] == torch.float32
    with pytest.raises(ValueError):
        op._resolve_dtypes([torch.float32], torch.float16, None, torch.float32)


def test_scan_backend_threads_state_through(monkeypatch):
    seen = {}

    def fake(U, M, K, B, C, **kw):
        seen.update(kw)
        y = torch.zeros_like(U)
        if kw["return_state"]:
            return y, torch.ones(1), torch.full((1,), 2.0), torch.full((1,), 3.0)
        return y

    monkeypatch.setattr(backends, "v2x2ssd_b200", fake)
    U, M, K, B, C = _inputs(dtype=torch.bfloat16)
    be = backends.B200ScanBackend()
    st = ScanState(state=torch.zeros(1), b_prev=torch.zeros(1), u_prev=torch.zeros(1))
    y, nxt = be(ScanInputs(U, M, K, B, C), chunk_size=64, state=st)
    assert seen["chunk_size"] == 64 and seen["compute_dtype"] == torch.float32
    assert seen["output_dtype"] == torch.bfloat16 and seen["initial_states"] is st.state
    assert float(nxt.state) == 1 and float(nxt.b_prev) == 2 and float(nxt.u_prev) == 3
    y2 = be(ScanInputs(U, M, K, B, C), chunk_size=32)
    assert isinstance(y2, torch.Tensor) and seen["return_state"] is False


def test_unsupported_chunk_is_a_value_error():
    with pytest.raises(ValueError, match="chunk_size must be one of"):
        op._shape(1, 1, 8, 4, 2, 48, torch.float32)


def test_decode_step_host_checks():
    """The decode step raises on CPU tensors and on mismatched shapes before any launch."""
    import types

    kw = dict(dt_min=1e-4, dt_max=1e-1, r_min=0.9, r_max=1.0, theta_bound=3.14, k_max=0.5, eps=1e-8,
              b_scale=torch.ones(2, 2, 4), c_scale=torch.ones(2, 2, 4),
              **{k: torch.zeros(2) for k in ("dt_bias", "gamma_bias", "omega_bias", "mix_r_bias", "mix_theta_bias",
                                             "mix_k_prev_bias", "mix_k_curr_bias")})
    v, p, bc, g, sk = (torch.zeros(1, 2, 8), torch.zeros(1, 2, 13), torch.zeros(1, 2, 4, 4), torch.zeros(1, 2, 8),
                       torch.zeros(2, 8))
    with pytest.raises(ValueError, match="requires CUDA"):
        slinoss_b200.mixer_decode_step_b200(v, p, bc, g, sk, **kw)
    be = backends.B200MixerDecodeBackend()
    owner = types.SimpleNamespace(d_state=4, output_norm=None)
    assert not be.supports(owner, batch_size=1, device=torch.device("cpu"), dtype=torch.float32)
    assert be.supports(owner, batch_size=300, device=torch.device("cuda", 0), dtype=torch.bfloat16)
    assert not be.supports(types.SimpleNamespace(d_state=5, output_norm=None), batch_size=1,
                           device=torch.device("cuda", 0), dtype=torch.bfloat16)
    assert not be.supports(types.SimpleNamespace(d_state=4, output_norm=object()), batch_size=1,
                           device=torch.device("cuda", 0), dtype=torch.bfloat16)
