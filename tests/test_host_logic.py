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


def test_device_guard_enters_the_tensors_device(monkeypatch):
    """Every library call runs under ``_lib.guard(device)``: with another device current the guard
    switches to the tensors' device for the duration of the call and back afterwards."""
    from slinoss_b200 import _lib

    events = []

    class FakeCtx:
        def __init__(self, idx):
            self.idx = idx

        def __enter__(self):
            events.append(("enter", self.idx))

        def __exit__(self, *exc):
            events.append(("exit", self.idx))
            return False

    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(torch.cuda, "device", FakeCtx)
    with _lib.guard(torch.device("cuda", 1)):
        events.append("call")
    assert events == [("enter", 1), "call", ("exit", 1)]
    events.clear()
    with _lib.guard(torch.device("cuda", 0)):   # already current: nothing to switch
        events.append("call")
    assert events == ["call"]
    with pytest.raises(ValueError, match="CUDA"):
        with _lib.guard(torch.device("cpu")):
            pass


def test_ops_wrap_their_library_calls_in_the_guard():
    """Source-level check that no op reaches the library outside a guard: every ``_lib.check(`` of
    the op modules sits inside a ``with _lib.guard(`` block."""
    import inspect

    from slinoss_b200 import context_parallel
    from slinoss_b200.ops import cconv1d, decode, scanprep, v2x2ssd

    for mod in (cconv1d, decode, scanprep, v2x2ssd, context_parallel):
        lines = inspect.getsource(mod).splitlines()
        for i, line in enumerate(lines):
            if "_lib.check(" in line and "def " not in line:
                indent = len(line) - len(line.lstrip())
                j = i - 1
                while j >= 0 and (not lines[j].strip() or len(lines[j]) - len(lines[j].lstrip()) >= indent):
                    j -= 1
                assert "with _lib.guard(" in lines[j], f"{mod.__name__}:{i + 1} is outside a device guard"


def test_same_device_rejects_mixed_devices():
    from slinoss_b200 import _lib

    class T:
        def __init__(self, dev):
            self.device = torch.device(dev)

    assert _lib.same_device(T("cuda:1"), None, T("cuda:1")) == torch.device("cuda:1")
    with pytest.raises(ValueError, match="same device"):
        _lib.same_device(T("cuda:0"), T("cuda:1"))


def test_stage_entry_points_validate_like_the_fused_op():
    """The stage functions hand raw pointers to the kernels, so they run the fused op's checks first
    (contiguity, shapes, dtypes); a time slice of a longer tensor must be made contiguous."""
    U, M, K, B, C = _inputs(T=16)
    sl = slice(4, 12)
    with pytest.raises(ValueError, match="must be contiguous"):
        slinoss_b200.chunk_increment_b200(U[:, :, sl], M[:, :, sl], K[:, :, sl], B[:, :, sl], chunk_size=16)
    with pytest.raises(ValueError, match=r"M must be \(batch,heads,T,2\)"):
        slinoss_b200.chunk_increment_b200(U, M[..., :1].contiguous(), K, B, chunk_size=16)
    with pytest.raises(ValueError, match="requires CUDA"):
        slinoss_b200.chunk_increment_b200(U, M, K, B, chunk_size=16)
    with pytest.raises(ValueError, match="C must match B"):
        slinoss_b200.chunk_scan_b200(U, M, K, B, C[..., :4].contiguous(), torch.zeros(1, 2, 1, 4, 6), chunk_size=16)
    inc = torch.zeros(1, 2, 3, 4, 6)
    with pytest.raises(ValueError, match="requires CUDA"):
        slinoss_b200.state_passing_b200(inc, torch.zeros(1, 2, 3, 2))
    with pytest.raises(ValueError, match=r"inc must be \(batch,heads,chunks,P,2N\)"):
        slinoss_b200.state_passing_b200(inc[0], torch.zeros(2, 3, 2))
    # half-precision increments go with chunk starts of the same dtype only
    with pytest.raises(TypeError, match="inc must be float32 or starts_dtype"):
        slinoss_b200.state_passing_b200(inc.to(torch.bfloat16), torch.zeros(1, 2, 3, 2))
    with pytest.raises(TypeError, match="inc_dtype must be"):
        slinoss_b200.chunk_increment_b200(U, M, K, B, chunk_size=16, inc_dtype=torch.float64)


def test_context_parallel_rejects_non_contiguous_slices():
    import torch.distributed as dist

    from slinoss_b200.context_parallel import v2x2ssd_context_parallel

    U, M, K, B, C = _inputs(T=16)
    import os

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29547")
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        with pytest.raises(ValueError, match="must be contiguous"):
            v2x2ssd_context_parallel(U[:, :, 4:12], M[:, :, 4:12], K[:, :, 4:12], B[:, :, 4:12], C[:, :, 4:12],
                                     chunk_size=8)
    finally:
        dist.destroy_process_group()


def test_use_b200_backends_switches_every_mixer_and_leaves_cpu_math_alone():
    """``use_b200_backends`` on the reference's own mixer: the four backend slots are replaced, an input
    projection whose width is not a multiple of 8 gets the padded forward, and that forward is the plain
    ``nn.Linear`` for tensors it does not apply to (CPU, fp32)."""
    from ref_util import import_reference

    import_reference()
    from slinoss.layers import SLinOSSMixer

    import slinoss_b200 as sb

    torch.manual_seed(0)
    mixer = SLinOSSMixer(96, d_state=16, expand=1, d_head=32, d_conv=4, chunk_size=32)
    width = int(mixer.in_proj.out_features)
    assert width == 2 * 96 + 3 * 13 + 4 * 3 * 16 and width % 8 != 0
    x = torch.randn(2, 5, 96)
    before = mixer.in_proj(x)
    assert sb.use_b200_backends(mixer) == 1
    assert isinstance(mixer.backend, sb.B200ScanBackend) and isinstance(mixer.scanprep.backend, sb.B200ScanPrepBackend)
    assert isinstance(mixer.cconv_backend, sb.B200CConv1dBackend)
    assert isinstance(mixer.decode_backend, sb.B200MixerDecodeBackend)
    assert "forward" in vars(mixer.in_proj) and "_apply_causal_depthwise_conv_step" in vars(mixer)
    assert "forward" not in vars(mixer)                       # the fused forward is opt-in
    assert torch.equal(mixer.in_proj(x), before)              # CPU tensors: the stock product
    other = SLinOSSMixer(96, d_state=16, expand=1, d_head=32, d_conv=4, chunk_size=32)
    assert sb.use_b200_backends(other, fuse_glue=True, align_projection=False, decode_conv=False) == 1
    assert "forward" in vars(other) and "forward" not in vars(other.in_proj)
    assert "_apply_causal_depthwise_conv_step" not in vars(other)
